"""GPU: a bounded device-side wait that runs out gives up and reports; nothing faults or hangs.

Every mbarrier wait of the tensor-core kernels polls the GPU's global timer and gives up after
the device's wait limit (2 s by default).  These tests shorten the limit to a millisecond and
launch ONE tile of a real GEMM kernel whose "stage full" barrier can never complete (the host
builds the A tensor map with half the rows the kernel counts on, so too few bytes arrive and no
MMA is ever issued).  Expected: the kernel returns by itself within milliseconds, the output is
untouched, bit 0 of the status word is set, tensor memory was freed (the next GEMMs run and are
correct) and the context is still healthy."""

import time

import pytest
import torch

from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu

VARIANTS = {0: "single-CTA gemm_kernel", 1: "CTA-pair gemm_pair_kernel", 2: "cluster split-K kernel"}


@pytest.fixture
def short_limit():
    from custom_cuda_kernals_b200 import _native
    like = torch.empty(1, device=DEV)
    previous = _native.set_wait_limit_ns(like, 1_000_000)          # 1 ms
    yield
    assert _native.set_wait_limit_ns(like, previous) == 1_000_000
    assert _native.set_wait_limit_ns(like, previous) == previous


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_wait_runs_out_kernel_gives_up_and_reports(short_limit, variant):
    from custom_cuda_kernals_b200 import _native
    from custom_cuda_kernals_b200.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator(device=DEV).manual_seed(variant)
    a = torch.randn(256, 64, device=DEV, generator=g).to(torch.bfloat16)
    b = torch.randn(256, 64, device=DEV, generator=g).to(torch.bfloat16)
    y = torch.full((256, 256), 7.0, device=DEV, dtype=torch.bfloat16)
    assert _native.take_device_status(y) == 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _native.wait_limit_selftest(a, b, y, variant)
    torch.cuda.synchronize()                                        # returns: the kernel did not hang
    elapsed = time.perf_counter() - t0
    assert elapsed < 1.0, f"{VARIANTS[variant]} took {elapsed:.3f} s to give up with a 1 ms limit"
    assert _native.take_device_status(y) & 1 == 1                   # the give-up was reported ...
    assert _native.take_device_status(y) == 0                       # ... and reading it cleared it
    assert torch.all(y == 7.0)                                      # no epilogue ran on garbage
    # tensor memory was freed and the context is healthy: the same kernels run and are right
    for m in (128, 1024):                                           # narrow-tile kernel, CTA-pair kernel
        x = torch.randn(m, 512, device=DEV, generator=g).to(torch.bfloat16)
        w = torch.randn(768, 512, device=DEV, generator=g).to(torch.bfloat16)
        got = matmul_add_bias(x, w)
        torch.testing.assert_close(got.float(), x.float() @ w.float().T, rtol=1e-2, atol=2e-1)
    assert _native.take_device_status(y) == 0


def test_wait_limit_is_clamped_and_restored():
    from custom_cuda_kernals_b200 import _native
    like = torch.empty(1, device=DEV)
    default = _native.set_wait_limit_ns(like, 5)                    # below the 1 us floor
    assert default == 2_000_000_000
    assert _native.set_wait_limit_ns(like, 10 ** 12) == 1000        # was clamped up to 1 us; now above the 10 s cap
    assert _native.set_wait_limit_ns(like, default) == 10_000_000_000
