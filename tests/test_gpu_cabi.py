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


def test_moe_entry_points_through_ctypes(lib):
    """launch_moe_router_fwd / launch_token_gather_fwd / launch_token_combine_fwd with raw pointers,
    as the reference's own Rust layer declares them (src/kernels/moe_router.rs:11-23,
    src/kernels/token_permute.rs)."""
    for name in ("launch_moe_router_fwd", "launch_token_gather_fwd", "launch_token_combine_fwd"):
        getattr(lib, name).restype = ctypes.c_int32
    g = torch.Generator().manual_seed(2)
    logits = torch.randn(100, 16, generator=g)
    ld = logits.to(DEV)
    w = torch.empty(100, 4, device=DEV)
    idx = torch.empty(100, 4, dtype=torch.long, device=DEV)
    rc = lib.launch_moe_router_fwd(_p(ld), _p(w), _p(idx), ctypes.c_int64(100), ctypes.c_int64(16), ctypes.c_int64(4),
                                   ctypes.c_int32(0), ctypes.c_int32(1), _stream())
    assert rc == 0
    want_w, want_i = ops.moe_router(logits, 4, True)
    assert torch.equal(idx.cpu(), want_i)
    torch.testing.assert_close(w.cpu(), want_w, rtol=1e-5, atol=1e-6)
    assert lib.launch_moe_router_fwd(_p(ld), _p(w), _p(idx), ctypes.c_int64(100), ctypes.c_int64(300), ctypes.c_int64(4),
                                     ctypes.c_int32(0), ctypes.c_int32(1), _stream()) == 1       # more than 256 experts
    x = torch.randn(100, 64, generator=g).to(torch.bfloat16).to(DEV)
    perm = torch.argsort(idx.reshape(-1), stable=True) // 4
    rows = torch.empty(400, 64, dtype=torch.bfloat16, device=DEV)
    assert lib.launch_token_gather_fwd(_p(x), _p(perm), _p(rows), ctypes.c_int64(400), ctypes.c_int64(64),
                                       ctypes.c_int32(2), _stream()) == 0
    assert torch.equal(rows, x[perm])
    inv = torch.empty(400, dtype=torch.long, device=DEV)
    inv[torch.argsort(idx.reshape(-1), stable=True)] = torch.arange(400, device=DEV)
    out = torch.empty(100, 64, dtype=torch.bfloat16, device=DEV)
    assert lib.launch_token_combine_fwd(_p(rows), _p(inv), _p(w), _p(out), ctypes.c_int64(100), ctypes.c_int64(4),
                                        ctypes.c_int64(64), ctypes.c_int32(2), _stream()) == 0
    torch.testing.assert_close(out.float(), x.float(), rtol=2 ** -7, atol=1e-6)      # renormalised weights sum to 1


def test_gradient_entry_points_through_ctypes(lib):
    for name in ("launch_swiglu_bwd", "launch_rmsnorm_residual_bwd", "launch_transpose_2byte"):
        getattr(lib, name).restype = ctypes.c_int32
    lib.cck_rmsnorm_bwd_workspace_bytes.restype = ctypes.c_int64
    g = torch.Generator().manual_seed(3)
    gate, up, dy = (torch.randn(40, 256, generator=g).to(DEV) for _ in range(3))
    dg, du = torch.empty_like(gate), torch.empty_like(up)
    assert lib.launch_swiglu_bwd(_p(gate), _p(up), _p(dy), _p(dg), _p(du), ctypes.c_int64(gate.numel()), ctypes.c_int32(0),
                                 _stream()) == 0
    g32, u32 = gate.cpu().requires_grad_(True), up.cpu().requires_grad_(True)
    (torch.nn.functional.silu(g32) * u32).backward(dy.cpu())
    torch.testing.assert_close(dg.cpu(), g32.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(du.cpu(), u32.grad, rtol=1e-4, atol=1e-5)
    ro, w = torch.randn(40, 256, generator=g).to(DEV), (1 + 0.1 * torch.randn(256, generator=g)).to(DEV)
    dx, dw = torch.empty_like(ro), torch.empty_like(w)
    need = lib.cck_rmsnorm_bwd_workspace_bytes(ctypes.c_int64(40), ctypes.c_int64(256))
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    rc = lib.launch_rmsnorm_residual_bwd(_p(dy), None, _p(ro), _p(w), _p(dx), _p(dw), _p(ws), ctypes.c_int64(need),
                                         ctypes.c_int64(40), ctypes.c_int64(256), ctypes.c_float(1e-5), ctypes.c_int32(0), _stream())
    assert rc == 0
    r32, w32 = ro.cpu().requires_grad_(True), w.cpu().requires_grad_(True)
    (r32 * torch.rsqrt(r32.pow(2).mean(-1, keepdim=True) + 1e-5) * w32).backward(dy.cpu())
    torch.testing.assert_close(dx.cpu(), r32.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dw.cpu(), w32.grad, rtol=1e-4, atol=1e-4)
    assert lib.launch_rmsnorm_residual_bwd(_p(dy), None, _p(ro), _p(w), _p(dx), _p(dw), _p(ws), ctypes.c_int64(8),
                                           ctypes.c_int64(40), ctypes.c_int64(256), ctypes.c_float(1e-5), ctypes.c_int32(0),
                                           _stream()) == 1                                       # workspace too small
    a = torch.randn(30, 64, generator=g).to(torch.bfloat16).to(DEV)
    at = torch.full((64, 32), 9.0, dtype=torch.bfloat16, device=DEV)
    assert lib.launch_transpose_2byte(_p(a), ctypes.c_int64(30), ctypes.c_int64(64), _p(at), ctypes.c_int64(32), _stream()) == 0
    assert torch.equal(at[:, :30], a.t()) and torch.all(at[:, 30:] == 0)
