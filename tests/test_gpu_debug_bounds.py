"""GPU: the -DCC_DEBUG_BOUNDS build of the bandwidth-bound kernels (stand-in for a memory checker).

In that build every global access through the shared load / store helpers is checked against the
address ranges the host registered, skipped and counted when outside.  The tests register exactly
the tensors of a call, launch ragged shapes (vector tails, scalar fallbacks, odd head dims) through
the C ABI of the debug library, and require zero violations and results identical to the release
library's.  Nothing here launches an out-of-range access on purpose."""

import ctypes
import pathlib

import pytest
import torch

pytestmark = pytest.mark.gpu
PKG = pathlib.Path(__file__).resolve().parent.parent / "custom_cuda_kernals_b200"
I64, I32, VP, F32 = ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_float
TAG = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


@pytest.fixture(scope="module")
def dbg():
    path = PKG / "libcustom_cuda_b200_dbg.so"
    assert path.exists(), "build first: python -m custom_cuda_kernals_b200._build"
    return ctypes.CDLL(str(path))


def _register(lib, tag, tensors):
    n = len(tensors)
    base = (VP * n)(*[t.data_ptr() for t in tensors])
    size = (I64 * n)(*[t.numel() * t.element_size() for t in tensors])
    assert getattr(lib, f"cck_dbg_set_ranges_{tag}")(base, size, I32(n)) == 0


def _violations(lib, tag):
    out = ctypes.c_uint32(123)
    assert getattr(lib, f"cck_dbg_take_violations_{tag}")(ctypes.byref(out)) == 0
    return out.value


@pytest.mark.parametrize("n", [1, 7, 8, 129, 1000, 4096 * 3 + 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_touches_only_its_tensors(dbg, n, dtype):
    from custom_cuda_kernals_b200.kernels.swiglu import swiglu
    g = torch.Generator(device="cuda").manual_seed(n)
    a = torch.randn(n, device="cuda", generator=g).to(dtype)
    b = torch.randn(n, device="cuda", generator=g).to(dtype)
    y = torch.empty_like(a)
    _register(dbg, "swiglu", [a, b, y])
    rc = dbg.launch_swiglu_fwd(VP(a.data_ptr()), VP(b.data_ptr()), VP(y.data_ptr()), I64(n), I32(TAG[dtype]),
                               VP(torch.cuda.current_stream().cuda_stream))
    assert rc == 0 and _violations(dbg, "swiglu") == 0
    assert torch.equal(y, swiglu(a, b))


@pytest.mark.parametrize("rows,cols", [(3, 8), (5, 100), (4, 4096), (2, 4100), (7, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_rmsnorm_residual_touches_only_its_tensors(dbg, rows, cols, dtype):
    from custom_cuda_kernals_b200.kernels.rmsnorm_residual import rmsnorm_residual
    g = torch.Generator(device="cuda").manual_seed(rows * cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
    r = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
    w = torch.randn(cols, device="cuda", generator=g).to(dtype)
    y, ro = torch.empty_like(x), torch.empty_like(x)
    _register(dbg, "rmsnorm", [x, r, w, y, ro])
    dbg.launch_rmsnorm_residual_fwd.argtypes = [VP, VP, VP, VP, VP, I64, I64, F32, I32, VP]
    rc = dbg.launch_rmsnorm_residual_fwd(x.data_ptr(), r.data_ptr(), w.data_ptr(), y.data_ptr(), ro.data_ptr(), rows,
                                         cols, 1e-5, TAG[dtype], torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and _violations(dbg, "rmsnorm") == 0
    want_y, want_ro = rmsnorm_residual(x, r, w, 1e-5)
    assert torch.equal(y, want_y) and torch.equal(ro, want_ro)


@pytest.mark.parametrize("shape", [(2, 5, 4, 2, 64), (1, 3, 3, 1, 6), (3, 7, 8, 8, 128), (1, 1, 1, 1, 10)])
def test_rope_touches_only_its_tensors(dbg, shape):
    from custom_cuda_kernals_b200.kernels.rope import rope
    from custom_cuda_kernals_b200.llama_block import rope_tables
    b, s, hq, hkv, d = shape
    g = torch.Generator(device="cuda").manual_seed(d)
    q = torch.randn(b, s, hq, d, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(b, s, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
    cos, sin = rope_tables(s, d, 10000.0, "cuda")
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    _register(dbg, "rope", [q, k, cos, sin, qo, ko])
    dbg.launch_rope_fwd.argtypes = [VP, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, I32, VP]
    rc = dbg.launch_rope_fwd(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), qo.data_ptr(), ko.data_ptr(),
                             b, s, hq, hkv, d, 2, torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and _violations(dbg, "rope") == 0
    wq, wk = rope(q, k, cos, sin)
    assert torch.equal(qo, wq) and torch.equal(ko, wk)


def test_unregistered_tensor_is_counted_and_left_alone(dbg):
    """The checker itself works: with the OUTPUT left out of the table a correct launch is counted as
    violations and the output is never written (the access is skipped, not performed)."""
    a = torch.randn(1000, device="cuda")
    b = torch.randn(1000, device="cuda")
    y = torch.full((1000,), 7.0, device="cuda")
    _register(dbg, "swiglu", [a, b])
    rc = dbg.launch_swiglu_fwd(VP(a.data_ptr()), VP(b.data_ptr()), VP(y.data_ptr()), I64(1000), I32(0),
                               VP(torch.cuda.current_stream().cuda_stream))
    assert rc == 0 and _violations(dbg, "swiglu") > 0
    assert torch.all(y == 7.0)
    assert _violations(dbg, "swiglu") == 0          # reading the count cleared it
