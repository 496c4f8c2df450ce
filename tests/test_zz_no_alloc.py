"""GPU: the allocation-free cross-entropy entry point, called through the C ABI.

launch_linear_cross_entropy_fwd_noalloc serves hosts that cannot give the library a
workspace (all device memory already belongs to their own pool, or cudaMalloc's
device-wide synchronisation is not acceptable where they call from).  It must return
exactly what launch_linear_cross_entropy_fwd returns, call after call, although every
call reuses one fixed device array that still holds the previous call's partials, and
it must refuse problems that do not fit that array.
"""

import ctypes
import pathlib

import pytest
import torch

pytestmark = pytest.mark.gpu
LIB = pathlib.Path(__file__).resolve().parent.parent / "custom_cuda_kernals_b200" / "libcustom_cuda_b200.so"
I64, I32, VP = ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p


def _lib():
    lib = ctypes.CDLL(str(LIB))
    lib.cck_lce_workspace_bytes.restype = I64
    lib.cck_lce_workspace_bytes.argtypes = [I64, I64]
    lib.cck_lce_noalloc_max_workspace_bytes.restype = I64
    lib.launch_linear_cross_entropy_fwd.restype = I32
    lib.launch_linear_cross_entropy_fwd.argtypes = [VP, VP, VP, I64, I64, I64, I64, VP, VP, I64, I32, VP]
    lib.launch_linear_cross_entropy_fwd_noalloc.restype = I32
    lib.launch_linear_cross_entropy_fwd_noalloc.argtypes = [VP, VP, VP, I64, I64, I64, I64, VP, I32, VP]
    return lib


def _inputs(n, h, v, seed, dev="cuda"):
    g = torch.Generator().manual_seed(seed)
    hid = torch.randn(n, h, generator=g).to(torch.bfloat16).to(dev)
    w = (0.05 * torch.randn(v, h, generator=g)).to(torch.bfloat16).to(dev)
    t = torch.randint(0, v, (n,), generator=g).to(dev)
    return hid, w, t


def _two_calls_in_a_row(dev):
    lib = _lib()
    BF16 = 2
    with torch.cuda.device(dev):
        stream = VP(torch.cuda.current_stream().cuda_stream)
        # the second problem is smaller, so most of the array still holds the first call's partials
        for call, (n, h, v, v_start, seed) in enumerate([(1000, 256, 5000, 0, 1), (300, 128, 1100, 640, 2)]):
            hid, w, t = _inputs(n, h, v, seed, dev)
            need = lib.cck_lce_workspace_bytes(n, v)
            assert 0 < need <= lib.cck_lce_noalloc_max_workspace_bytes()
            ws = torch.empty(need, dtype=torch.uint8, device=dev)
            want = torch.full((3, n), float("nan"), device=dev)
            got = torch.full((3, n), float("nan"), device=dev)
            rc = lib.launch_linear_cross_entropy_fwd(hid.data_ptr(), w.data_ptr(), t.data_ptr(), v_start, n, h, v,
                                                     want.data_ptr(), ws.data_ptr(), need, BF16, stream)
            assert rc == 0
            torch.cuda.synchronize()
            # "allocates nothing", seen from the driver: the device's free memory (cudaMemGetInfo) covers
            # allocations by ANY library in the process, torch's caching allocator only its own.  The first
            # call on a device may load the kernels' module, so free memory is compared around the second.
            before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
            rc = lib.launch_linear_cross_entropy_fwd_noalloc(hid.data_ptr(), w.data_ptr(), t.data_ptr(), v_start, n, h,
                                                             v, got.data_ptr(), BF16, stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            if call > 0:
                assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.equal(got, want)            # same kernels, same order of operations: bit for bit
            # and the statistics are right: row loss against an fp64 evaluation on the CPU
            logits = hid.cpu().double() @ w.cpu().double().T
            lse = torch.logsumexp(logits, dim=1)
            mine = (got[0].double() + got[1].double().log()).cpu()
            torch.testing.assert_close(mine, lse, rtol=1e-4, atol=1e-5)


def test_noalloc_matches_workspace_entry_point_two_calls_in_a_row():
    _two_calls_in_a_row(torch.device("cuda", 0))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_noalloc_on_a_second_device_uses_that_devices_array():
    """The array's address is looked up per device: the same two calls on cuda:1."""
    _two_calls_in_a_row(torch.device("cuda", 1))


def test_noalloc_refuses_problems_beyond_its_fixed_array():
    lib = _lib()
    n, v = 1 << 20, 1 << 16
    assert lib.cck_lce_workspace_bytes(n, v) > lib.cck_lce_noalloc_max_workspace_bytes()
    dummy = torch.zeros(16, device="cuda")
    rc = lib.launch_linear_cross_entropy_fwd_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, n, 64, v,
                                                     dummy.data_ptr(), 2, VP(torch.cuda.current_stream().cuda_stream))
    assert rc == 1     # cudaErrorInvalidValue, nothing launched
    torch.cuda.synchronize()
