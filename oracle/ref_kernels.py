"""ctypes access to the reference project's own CUDA kernels recompiled for sm_100a
(``oracle/_ref/libcustom_cuda_ref.so``, built by ``oracle/build_ref.py``).  Test and
measurement infrastructure only.

Each function does what the reference's Python wrapper does - allocate the outputs, call the
launcher on torch's current stream (custom_cuda/kernels/*.py) - so that tests can compare this
library's kernels with the reference's on the same GPU and the benchmark can time them side by
side.  ``available()`` is False when the library has not been built.
"""

from __future__ import annotations

import ctypes
import math
import pathlib

import torch

LIB_PATH = pathlib.Path(__file__).resolve().parent / "_ref" / "libcustom_cuda_ref.so"
_TAG = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_FP8 = {"e4m3": (3, torch.float8_e4m3fn), "e5m2": (4, torch.float8_e5m2)}
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(LIB_PATH))      # RTLD_LOCAL: its launch_* names do not shadow ours
        for name in ("launch_rmsnorm_residual_fwd", "launch_swiglu_fwd", "launch_rope_fwd",
                     "launch_fp8_quant_block_fwd", "launch_fp8_quant_tensor_fwd", "launch_matmul_add_bias_fwd",
                     "launch_linear_ce_chunk_update", "launch_moe_router_fwd", "launch_token_gather_fwd",
                     "launch_token_combine_fwd"):
            if not hasattr(_lib, name):          # a library built before the MoE kernels were added
                continue
            getattr(_lib, name).restype = ctypes.c_int32
    return _lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _s():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _i(v):
    return ctypes.c_int64(v)


def _ok(rc, name):
    if rc != 0:
        raise RuntimeError(f"reference {name} failed, cudaError_t = {rc}")


def rmsnorm_residual(x, residual, weight, eps=1e-6):
    """custom_cuda/kernels/rmsnorm_residual.py:17-28"""
    y, ro = torch.empty_like(x), torch.empty_like(x)
    cols = x.shape[-1]
    _ok(lib().launch_rmsnorm_residual_fwd(_p(x), _p(residual), _p(weight), _p(y), _p(ro), _i(x.numel() // cols),
                                          _i(cols), ctypes.c_float(eps), ctypes.c_int32(_TAG[x.dtype]), _s()), "rmsnorm")
    return y, ro


def swiglu(gate, up):
    """custom_cuda/kernels/swiglu.py:16-20"""
    y = torch.empty_like(gate)
    _ok(lib().launch_swiglu_fwd(_p(gate), _p(up), _p(y), _i(gate.numel()), ctypes.c_int32(_TAG[gate.dtype]), _s()), "swiglu")
    return y


def rope(q, k, cos, sin):
    """custom_cuda/kernels/rope.py:16-28"""
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    b, s, hq, d = q.shape
    _ok(lib().launch_rope_fwd(_p(q), _p(k), _p(cos), _p(sin), _p(qo), _p(ko), _i(b), _i(s), _i(hq), _i(k.shape[2]),
                              _i(d), ctypes.c_int32(_TAG[q.dtype]), _s()), "rope")
    return qo, ko


def fp8_quant(x, fp8_format="e4m3", granularity="block"):
    """custom_cuda/kernels/fp8_quant.py:28-63"""
    tag, dt = _FP8[fp8_format]
    m, n = x.shape
    codes = torch.empty((m, n), dtype=dt, device=x.device)
    if granularity == "block":
        scale = torch.empty(math.ceil(m / 128), math.ceil(n / 128), dtype=torch.float32, device=x.device)
        _ok(lib().launch_fp8_quant_block_fwd(_p(x), _p(codes), _p(scale), _i(m), _i(n), ctypes.c_int32(_TAG[x.dtype]),
                                             ctypes.c_int32(tag), _s()), "fp8 block")
        return codes, scale
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.zeros(1, dtype=torch.int32, device=x.device)
    _ok(lib().launch_fp8_quant_tensor_fwd(_p(x), _p(codes), _p(scale), _p(scratch), _i(m), _i(n),
                                          ctypes.c_int32(_TAG[x.dtype]), ctypes.c_int32(tag), _s()), "fp8 tensor")
    return codes, scale


def matmul_add_bias(x, weight, bias=None):
    """custom_cuda/kernels/matmul_add_bias.py:16-26"""
    m, k = x.shape
    n = weight.shape[0]
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    _ok(lib().launch_matmul_add_bias_fwd(_p(x), _p(weight), _p(bias), _p(y), _i(m), _i(k), _i(n),
                                         ctypes.c_int32(_TAG[x.dtype]), _s()), "matmul_add_bias")
    return y


def linear_cross_entropy(hidden, weight, targets, ignore_index=-100, reduction="mean", chunk_size=4096):
    """custom_cuda/kernels/linear_cross_entropy.py:32-82: a loop over vocabulary chunks, each
    chunk's logits from torch's matmul (cuBLAS), folded in by the reference's chunk-update kernel."""
    n, v = hidden.shape[0], weight.shape[0]
    dev = hidden.device
    mx = torch.full((n,), float("-inf"), device=dev)
    sm, tg = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    for v0 in range(0, v, chunk_size):
        v1 = min(v0 + chunk_size, v)
        logits = (hidden @ weight[v0:v1].T).contiguous()
        _ok(lib().launch_linear_ce_chunk_update(_p(logits), _p(targets), _i(v0), _i(n), _i(v1 - v0), _p(mx), _p(sm),
                                                _p(tg), ctypes.c_int32(_TAG[logits.dtype]), _s()), "lce chunk")
    loss = mx + torch.log(sm) - tg
    keep = targets != ignore_index
    loss = torch.where(keep, loss, torch.zeros_like(loss))
    if reduction == "none":
        return loss
    return loss.sum() if reduction == "sum" else loss.sum() / keep.sum().float()


def has_moe() -> bool:
    return available() and hasattr(lib(), "launch_moe_router_fwd")


def moe_router(logits, k, renormalize=True):
    """custom_cuda/kernels/moe_router.py:18-30"""
    t, e = logits.shape
    w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(t, k, dtype=torch.long, device=logits.device)
    _ok(lib().launch_moe_router_fwd(_p(logits), _p(w), _p(idx), _i(t), _i(e), _i(k), ctypes.c_int32(_TAG[logits.dtype]),
                                    ctypes.c_int32(1 if renormalize else 0), _s()), "moe_router")
    return w, idx


def token_gather(src, indices):
    """custom_cuda/kernels/token_permute.py:18-26"""
    dst = torch.empty(indices.shape[0], src.shape[1], dtype=src.dtype, device=src.device)
    _ok(lib().launch_token_gather_fwd(_p(src), _p(indices), _p(dst), _i(indices.shape[0]), _i(src.shape[1]),
                                      ctypes.c_int32(_TAG[src.dtype]), _s()), "token_gather")
    return dst


def token_combine(expert_output, unpermute_index, weights):
    """custom_cuda/kernels/token_permute.py:29-42"""
    t, k = unpermute_index.shape
    out = torch.empty(t, expert_output.shape[1], dtype=expert_output.dtype, device=expert_output.device)
    _ok(lib().launch_token_combine_fwd(_p(expert_output), _p(unpermute_index), _p(weights), _p(out), _i(t), _i(k),
                                       _i(expert_output.shape[1]), ctypes.c_int32(_TAG[expert_output.dtype]), _s()),
        "token_combine")
    return out
