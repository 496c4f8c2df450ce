"""GPU: the C ABI called directly through ctypes with raw device pointers - the way a
non-Python host (the reference's Rust layer, cgo, JNI) would bind it."""

import ctypes
import pathlib

import pytest
import torch

from oracle import ops
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu
LIB = pathlib.Path(__file__).resolve().parent.parent / "custom_cuda_kernals_b200" / "libcustom_cuda_b200.so"


@pytest.fixture(scope="module")
def lib():
    handle = ctypes.CDLL(str(LIB))
    for name in ("launch_swiglu_fwd", "launch_rmsnorm_residual_fwd", "launch_fp8_quant_token_fwd",
                 "launch_matmul_add_bias_fwd", "launch_fp8_quant_tensor_fwd"):
        getattr(handle, name).restype = ctypes.c_int32
    return handle


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_swiglu_and_rmsnorm_through_ctypes(lib):
    g = torch.Generator().manual_seed(0)
    gate = torch.randn(3, 1000, generator=g).to(torch.bfloat16)
    up = torch.randn(3, 1000, generator=g).to(torch.bfloat16)
    gd, ud = gate.to(DEV), up.to(DEV)
    y = torch.empty_like(gd)
    assert lib.launch_swiglu_fwd(_p(gd), _p(ud), _p(y), ctypes.c_int64(gd.numel()), ctypes.c_int32(2), _stream()) == 0
    ops.assert_close_with_outliers(y, ops.swiglu(gate, up), rtol=1e-2, atol=1e-2, max_outlier_fraction=1e-5)

    x = torch.randn(6, 512, generator=g)
    r = torch.randn(6, 512, generator=g)
    w = torch.randn(512, generator=g)
    xd, rd, wd = x.to(DEV), r.to(DEV), w.to(DEV)
    yo, ro = torch.empty_like(xd), torch.empty_like(xd)
    rc = lib.launch_rmsnorm_residual_fwd(_p(xd), _p(rd), _p(wd), _p(yo), _p(ro), ctypes.c_int64(6),
                                         ctypes.c_int64(512), ctypes.c_float(1e-5), ctypes.c_int32(0), _stream())
    assert rc == 0
    want_y, want_ro = ops.rmsnorm_residual(x, r, w, 1e-5)
    torch.testing.assert_close(ro.cpu(), want_ro, rtol=0, atol=0)
    torch.testing.assert_close(yo.cpu(), want_y, rtol=1e-4, atol=1e-4)


def test_error_codes_and_empty_problems(lib):
    x = torch.zeros(16, device=DEV)
    assert lib.launch_swiglu_fwd(_p(x), _p(x), _p(x), ctypes.c_int64(0), ctypes.c_int32(0), _stream()) == 0
    assert lib.launch_swiglu_fwd(_p(x), _p(x), _p(x), ctypes.c_int64(16), ctypes.c_int32(9), _stream()) == 1  # cudaErrorInvalidValue
    assert lib.launch_matmul_add_bias_fwd(_p(x), _p(x), None, _p(x), ctypes.c_int64(0), ctypes.c_int64(4),
                                          ctypes.c_int64(4), ctypes.c_int32(0), _stream()) == 0
    torch.cuda.synchronize()


def test_fp8_token_and_tensor_through_ctypes(lib):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    xd = x.to(DEV)
    codes = torch.empty(64, 256, dtype=torch.uint8, device=DEV)
    scale = torch.empty(64, device=DEV)
    rc = lib.launch_fp8_quant_token_fwd(_p(xd), _p(codes), _p(scale), ctypes.c_int64(64), ctypes.c_int64(256),
                                        ctypes.c_int32(2), ctypes.c_int32(3), _stream())
    assert rc == 0
    want_codes, want_scale = ops.fp8_quant(x, "e4m3", "token")
    assert torch.equal(codes.cpu(), want_codes.view(torch.uint8))
    assert torch.equal(scale.cpu(), want_scale.reshape(-1))
    amax = torch.zeros(1, dtype=torch.int32, device=DEV)
    s1 = torch.empty(1, device=DEV)
    rc = lib.launch_fp8_quant_tensor_fwd(_p(xd), _p(codes), _p(s1), _p(amax), ctypes.c_int64(64), ctypes.c_int64(256),
                                         ctypes.c_int32(2), ctypes.c_int32(4), _stream())
    assert rc == 0
    want_codes, want_scale = ops.fp8_quant(x, "e5m2", "tensor")
    assert torch.equal(codes.cpu(), want_codes.view(torch.uint8)) and s1.item() == want_scale.item()


def test_pair_kernel_is_available_on_this_gpu(lib):
    """The two-CTA (cta_group::2) GEMM is the default tensor-core path: at least 64 CTA pairs
    fit a B200 (148 SMs = 74 TPCs)."""
    lib.cck_gemm_pair_capacity.restype = ctypes.c_int32
    torch.zeros(1, device=DEV)
    assert lib.cck_gemm_pair_capacity() >= 64
