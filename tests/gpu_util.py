"""Helpers shared by the GPU parity tests."""

import torch

from oracle import ops

DEV = "cuda"


def to_dev(*tensors):
    return tuple(None if t is None else t.to(DEV) for t in tensors)


def check(actual, expected, dtype, table=None):
    rtol, atol, frac = (table or ops.TOLERANCE)[dtype]
    ops.assert_close_with_outliers(actual, expected, rtol=rtol, atol=atol, max_outlier_fraction=frac)


def device_status_clean(like):
    from custom_cuda_kernals_b200 import _native
    return _native.take_device_status(like) == 0
