"""Llama-3 style decoder block forward built from this library's ops.

Host-side mirror of the reference's integration example
(examples/llama_block.py:83-204, ``CustomCUDA_LlamaBlock``): pre-norm, GQA,
RoPE, SwiGLU FFN, with the same op order

    norm -> q/k/v projections -> rope -> causal attention -> o_proj
         -> norm(+residual) -> gate/up -> swiglu -> down -> + residual

The reference swaps in its three bandwidth-bound kernels and leaves every
projection to ``nn.Linear`` (cuBLAS); here the seven projections also run on this
library's tcgen05 GEMM (``matmul_add_bias`` with no bias), and by default two of
them carry the neighbouring elementwise op in their epilogue - gate/up + SwiGLU in
one GEMM, o_proj and down_proj + their residual adds in two more (so both norms read
one tensor instead of two) - and q, k, v come from one
projection that applies RoPE to its q / k columns in the epilogue (heads of 128;
otherwise, or with ``rope_in_gemm=False``, a rope kernel reads the q / k column ranges
in place); results are identical to the unfused chain (``fused=False`` runs that chain).  The attention core stays
``torch.nn.functional.scaled_dot_product_attention`` as in the reference.
Forward only, no autograd.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.nn.functional as F

from .kernels.fp8_quant import fp8_quant
from .kernels.fused import (GATE_UP_BLOCK, fp8_quant_token_from_amax, interleave_gate_up, matmul_add_bias_residual,
                            matmul_add_bias_residual_fp8, matmul_add_bias_rope, matmul_add_bias_rope_fp8, matmul_swiglu,
                            matmul_swiglu_fp8, rmsnorm_fp8_quant)
from .kernels.matmul_add_bias import matmul_add_bias, matmul_add_bias_fp8
from .kernels.rmsnorm_residual import rmsnorm, rmsnorm_residual
from .kernels.rope import rope, rope_strided
from .kernels.swiglu import swiglu

__all__ = ["LlamaBlock", "LlamaBlockFP8", "rope_tables", "OpTimer", "PARAM_NAMES", "host_pipeline_groups",
           "host_pipeline_items", "HostStep"]

PARAM_NAMES = ("input_layernorm_weight", "post_attention_layernorm_weight", "q_proj", "k_proj", "v_proj",
               "o_proj", "gate_proj", "up_proj", "down_proj")


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos, sin [seq_len, head_dim/2]`` (baselines/rope.py:103-115)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    angle = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv_freq)
    return angle.cos().contiguous(), angle.sin().contiguous()


class OpTimer:
    """Optional per-op CUDA-event timing inside a forward pass.

    ``forward(x, timer=t)`` records an event pair around every op on the current
    stream; ``t.totals()`` (after a synchronize) returns milliseconds and call
    counts per op kind.  Recording costs about a microsecond per event.
    """

    def __init__(self):
        self.spans: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []

    def run(self, kind: str, fn: Callable, *args, **kwargs):
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn(*args, **kwargs)
        b.record()
        self.spans.append((kind, a, b))
        return out

    def totals(self) -> dict[str, dict[str, float]]:
        out: dict[str, dict[str, float]] = {}
        for kind, a, b in self.spans:
            slot = out.setdefault(kind, {"ms": 0.0, "calls": 0})
            slot["ms"] += a.elapsed_time(b)
            slot["calls"] += 1
        return out


class _NoTimer:
    @staticmethod
    def run(kind, fn, *args, **kwargs):
        return fn(*args, **kwargs)


def host_pipeline_groups(batch: int, chunks: int | None = None) -> list[tuple[int, int]]:
    """Sequence ranges ``[b0, b1)`` of the host pipeline's groups, in execution order.

    Three resources work in parallel - the copy-in engine, the SMs, the copy-out engine - each
    handling the groups in order.  A sequence takes about half as long to copy (one way) as to
    compute, so the schedule stays compute-bound exactly when (a) a group's copy-in fits behind the
    previous group's compute - a group may be at most twice as large as the one before it - and
    (b) a group's copy-out fits behind the NEXT group's compute - at most twice as large as the one
    after it.  Only the first group's copy-in and the last group's copy-out are exposed, so both
    are one sequence.  Default: ``1, 2, 2, ..., 2, 1`` (an odd remainder as an extra single
    sequence before the last), e.g. 8 -> 1 2 2 2 1: modelled 6.1 ms for the 8 x 2048 step where
    ``1 3 3 1`` gave 6.8 (its three-sequence copy-in cannot hide behind one sequence of compute).
    ``chunks`` asks for that many equal groups instead."""
    if batch <= 0:
        return []
    if chunks is not None:
        n = max(1, min(batch, chunks))
        return [(batch * i // n, batch * (i + 1) // n) for i in range(n)]
    if batch <= 3:
        return [(i, i + 1) for i in range(batch)]
    sizes = [1] + [2] * ((batch - 2) // 2) + [1] * ((batch - 2) % 2) + [1]
    bounds, at = [], 0
    for size in sizes:
        bounds.append((at, at + size))
        at += size
    return bounds


_LOWER_RIGHT_OK = True


def _continuation_attention(q, k, v, gqa: bool):
    """Attention of ``L`` new queries over ``S >= L`` keys whose last ``L`` are the queries' own
    positions: causal mask aligned bottom-right.  Uses torch's fused kernels through
    ``causal_lower_right``; where this torch build has no fused kernel for that mask on the
    device, an explicit boolean mask gives the same result (slower)."""
    global _LOWER_RIGHT_OK
    seq_q, seq_k = q.shape[-2], k.shape[-2]
    if seq_q == 1:       # a single new position sees every key: no mask at all
        return F.scaled_dot_product_attention(q, k, v, enable_gqa=gqa)
    if _LOWER_RIGHT_OK:
        try:
            from torch.nn.attention.bias import causal_lower_right
            return F.scaled_dot_product_attention(q, k, v, attn_mask=causal_lower_right(seq_q, seq_k), enable_gqa=gqa)
        except (RuntimeError, TypeError, ValueError):
            _LOWER_RIGHT_OK = False
    mask = torch.ones(seq_q, seq_k, dtype=torch.bool, device=q.device).tril(diagonal=seq_k - seq_q)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=gqa)


def host_pipeline_items(batch: int, seq: int, chunks: int | None = None, seq_pieces: int | None = None,
                        min_piece: int = 512) -> list[tuple[int, int, int, int]]:
    """Work items ``(b0, b1, s0, s1)`` of the host pipeline: sequences ``[b0, b1)``, positions
    ``[s0, s1)``, in execution order.  The groups of ``host_pipeline_groups``; the first and the
    last group, when they are one sequence, are cut into ``seq_pieces`` equal runs of positions, so
    that only the first piece's copy-in and the last piece's copy-out stay exposed.  With at most
    three sequences every group is a single sequence and every one is cut.

    Default: two pieces when the call holds ONE sequence (one sequence per rank, where nothing
    else can overlap the copies), none otherwise.  Measured on one B200 (PCIe uncontended), 2048
    tokens: 1 sequence 1.39 ms whole, 1.35 ms in 2 pieces, 1.71 ms in 4; 2 sequences 2.19 / 2.41 /
    3.29 ms; 8 sequences 6.73 / 6.91 / 8.00 ms - a piece of 512 tokens runs ten launches whose
    host-side cost (~0.3 ms) exceeds their device time, so finer cuts turn the pipeline
    launch-bound.  Eight ranks sharing the host's PCIe root stretch the copies, which favours the
    cut at one sequence per rank."""
    groups = host_pipeline_groups(batch, chunks)
    if seq_pieces is None:
        seq_pieces = 2 if (batch == 1 and seq >= 2 * min_piece) else 1
    seq_pieces = max(1, min(seq_pieces, seq))
    items = []
    for i, (b0, b1) in enumerate(groups):
        ends = i == 0 or i == len(groups) - 1 or batch <= 3
        if seq_pieces > 1 and b1 - b0 == 1 and ends and chunks is None:
            cuts = [seq * j // seq_pieces for j in range(seq_pieces + 1)]
            items += [(b0, b1, lo, hi) for lo, hi in zip(cuts[:-1], cuts[1:]) if hi > lo]
        else:
            items.append((b0, b1, 0, seq))
    return items


class HostStep:
    """One step enqueued by ``LlamaBlock.forward_host_async``: ``input_consumed`` fires when the
    step's input has been copied to the device, ``landed`` when its output is complete in
    ``out_host``; ``wait()`` blocks the host on the latter and returns ``out_host``."""

    __slots__ = ("out_host", "input_consumed", "landed")

    def __init__(self, out_host: torch.Tensor, input_consumed: torch.cuda.Event, landed: torch.cuda.Event):
        self.out_host, self.input_consumed, self.landed = out_host, input_consumed, landed

    def wait(self) -> torch.Tensor:
        self.landed.synchronize()
        return self.out_host


class LlamaBlock:
    """One decoder block; ``weights`` maps PARAM_NAMES to CUDA tensors
    (projections as ``[out_features, in_features]``, the nn.Linear layout)."""

    def __init__(self, weights: dict[str, torch.Tensor], n_heads: int = 32, n_kv_heads: int = 8,
                 eps: float = 1e-5, theta: float = 500000.0, max_seq_len: int = 2048, fused: bool = True,
                 rope_in_gemm: bool = True):
        missing = [n for n in PARAM_NAMES if n not in weights]
        if missing:
            raise ValueError(f"missing block parameters: {missing}")
        self.w = {n: weights[n] for n in PARAM_NAMES}
        for name, t in self.w.items():
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"parameter '{name}' must be a contiguous CUDA tensor")
        self.hidden = self.w["q_proj"].shape[1]
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.head_dim = self.w["q_proj"].shape[0] // n_heads
        self.eps = eps
        dev = self.device = self.w["q_proj"].device
        self.cos, self.sin = rope_tables(max_seq_len, self.head_dim, theta, dev)
        ffn, dt = self.w["gate_proj"].shape[0], self.w["gate_proj"].dtype
        self.fused = bool(fused and ffn % GATE_UP_BLOCK == 0 and self.hidden % 8 == 0 and ffn % 8 == 0
                          and dt in (torch.float16, torch.bfloat16))
        if self.fused:      # one-time re-layout; the separate q/k/v and gate/up weights are not kept
            self.w_gate_up = interleave_gate_up(self.w["gate_proj"], self.w["up_proj"])
            self.w_qkv = torch.cat([self.w["q_proj"], self.w["k_proj"], self.w["v_proj"]], dim=0).contiguous()
            self.q_cols = self.w["q_proj"].shape[0]
            self.kv_cols = self.w["k_proj"].shape[0]
            self.ffn = ffn
            for name in ("gate_proj", "up_proj", "q_proj", "k_proj", "v_proj"):
                del self.w[name]
        #: the rotary embedding rides in the epilogue of the q/k/v projection (heads of 128 only)
        self.rope_in_gemm = bool(self.fused and self.head_dim == 128 and rope_in_gemm)
        #: kernels of this library launched per forward call: 2 norms, rope, and either
        #: q + k + v + o + gate + up + swiglu + down (unfused: 11 in all) or
        #: qkv + o + gate-up-swiglu + down-residual (fused: 7 in all, 6 with the rope in the qkv GEMM)
        self.launches_per_forward = (6 if self.rope_in_gemm else 7) if self.fused else 11

    def forward(self, x: torch.Tensor, timer: OpTimer | None = None, pos_offset: int = 0,
                kv_cache: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
        """x ``[B, S, hidden]`` -> ``[B, S, hidden]``.  ``pos_offset`` shifts the RoPE positions:
        ``x[:, i]`` is rotated as position ``pos_offset + i`` (attention stays causal within
        the ``S`` tokens given).

        With ``kv_cache = (k, v)``, two ``[B, max_len, n_kv_heads, head_dim]`` buffers that hold the
        rotated keys and the values of positions ``0 .. pos_offset - 1`` of the same sequences, the
        ``S`` tokens are a continuation: their keys / values are appended to the cache and they
        attend causally to everything up to themselves.  Feeding a sequence piece by piece this
        way computes the same function as one call on the whole sequence (every other op of the
        block works on tokens independently)."""
        t = timer if timer is not None else _NoTimer
        w = self.w
        b, s, hid = x.shape
        if pos_offset + s > self.cos.shape[0]:
            raise ValueError(f"sequence positions {pos_offset}..{pos_offset + s - 1} exceed the RoPE table "
                             f"({self.cos.shape[0]} rows)")
        x2 = x.view(b * s, hid)
        if self.fused:       # x + 0 is x: the norm alone, and x itself is the residual stream
            h, res = t.run("rmsnorm", rmsnorm, x2, w["input_layernorm_weight"], self.eps), x2
        else:
            zero = t.run("fill", torch.zeros_like, x2)
            h, res = t.run("rmsnorm", rmsnorm_residual, x2, zero, w["input_layernorm_weight"], self.eps)
        cos, sin = self.cos[pos_offset:pos_offset + s], self.sin[pos_offset:pos_offset + s]
        if self.fused:       # one projection for q, k and v
            qc, kc = self.q_cols, self.kv_cols
            # ... with the rotary embedding applied in its epilogue - except for decode-sized calls
            # (at most 128 tokens), where the plain projection runs on the weight-streaming decode
            # kernel, three times as fast as full-width tiles there, and a rope kernel follows
            rope_in_gemm = self.rope_in_gemm and b * s > 128
            if rope_in_gemm:
                qkv = t.run("gemm_rope", matmul_add_bias_rope, h, self.w_qkv, None, cos, sin, qc + kc).view(b, s, -1)
            else:
                qkv = t.run("gemm", matmul_add_bias, h, self.w_qkv).view(b, s, -1)
            q = qkv[..., :qc].unflatten(-1, (self.n_heads, self.head_dim))
            k = qkv[..., qc:qc + kc].unflatten(-1, (self.n_kv_heads, self.head_dim))
            v = qkv[..., qc + kc:].unflatten(-1, (self.n_kv_heads, self.head_dim))
            if not rope_in_gemm:         # rope reads its q / k column ranges in place
                q, k = t.run("rope", rope_strided, q, k, cos, sin)
        else:
            q = t.run("gemm", matmul_add_bias, h, w["q_proj"]).view(b, s, self.n_heads, self.head_dim)
            k = t.run("gemm", matmul_add_bias, h, w["k_proj"]).view(b, s, self.n_kv_heads, self.head_dim)
            v = t.run("gemm", matmul_add_bias, h, w["v_proj"]).view(b, s, self.n_kv_heads, self.head_dim)
            q, k = t.run("rope", rope, q, k, cos, sin)
        gqa = self.n_heads != self.n_kv_heads
        if kv_cache is None:
            att = t.run("sdpa", F.scaled_dot_product_attention, q.transpose(1, 2), k.transpose(1, 2),
                        v.transpose(1, 2), is_causal=True, enable_gqa=gqa)
        else:
            k_all, v_all = kv_cache
            end = pos_offset + s
            if k_all.shape[0] != b or end > k_all.shape[1]:
                raise ValueError(f"kv_cache of shape {tuple(k_all.shape)} cannot hold positions up to {end} of {b} sequences")
            k_all[:, pos_offset:end].copy_(k)
            v_all[:, pos_offset:end].copy_(v)
            if pos_offset == 0:
                att = t.run("sdpa", F.scaled_dot_product_attention, q.transpose(1, 2), k_all[:, :end].transpose(1, 2),
                            v_all[:, :end].transpose(1, 2), is_causal=True, enable_gqa=gqa)
            else:        # the new queries sit at the END of the key range: causal mask aligned bottom-right
                att = t.run("sdpa", _continuation_attention, q.transpose(1, 2), k_all[:, :end].transpose(1, 2),
                            v_all[:, :end].transpose(1, 2), gqa)
        att = t.run("copy", lambda a: a.transpose(1, 2).contiguous().view(b * s, hid), att)
        if self.fused:       # o_proj adds the residual in its epilogue; the norm reads that sum once
            res2 = t.run("gemm_residual", matmul_add_bias_residual, att, w["o_proj"], None, res)
            h2 = t.run("rmsnorm", rmsnorm, res2, w["post_attention_layernorm_weight"], self.eps)
        else:
            att = t.run("gemm", matmul_add_bias, att, w["o_proj"])
            h2, res2 = t.run("rmsnorm", rmsnorm_residual, att, res, w["post_attention_layernorm_weight"], self.eps)
        if self.fused:
            act = t.run("gemm_swiglu", matmul_swiglu, h2, self.w_gate_up)
            out = t.run("gemm_residual", matmul_add_bias_residual, act, w["down_proj"], None, res2)
        else:
            gate = t.run("gemm", matmul_add_bias, h2, w["gate_proj"])
            up = t.run("gemm", matmul_add_bias, h2, w["up_proj"])
            act = t.run("swiglu", swiglu, gate, up)
            mlp = t.run("gemm", matmul_add_bias, act, w["down_proj"])
            out = t.run("add", torch.add, mlp, res2)
        return out.view(b, s, hid)

    __call__ = forward

    def capture(self, x: torch.Tensor, pos_offset: int = 0,
                kv_cache: tuple[torch.Tensor, torch.Tensor] | None = None) -> Callable[[], torch.Tensor]:
        """Record ``forward(x, pos_offset=..., kv_cache=...)`` into a CUDA graph and return a
        function that replays it: every call re-runs the block on whatever ``x`` (and the cache)
        hold at that moment and returns the same output tensor, overwritten in place.  For steps
        that are short enough for launch overhead to show - a decode step of 16 sequences x 1 token
        takes 162 us launched op by op and 139 us replayed - keep ``x`` as a staging buffer and copy
        each step's input into it.  ``pos_offset`` and the cache length are frozen at capture time:
        capture one graph per position bucket, or pad.  Three eager warm-up calls run first, on a
        side stream as graph capture requires, so the captured step has appended to the cache four
        times when this returns; the keys / values it writes are the same every time."""
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(3):
                self.forward(x, pos_offset=pos_offset, kv_cache=kv_cache)
        torch.cuda.current_stream(self.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(graph):
            out = self.forward(x, pos_offset=pos_offset, kv_cache=kv_cache)

        def replay() -> torch.Tensor:
            graph.replay()
            return out

        replay.graph = graph          # keeps the graph (and its memory pool) alive with the function
        return replay

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, chunks: int | None = None,
                     seq_pieces: int | None = None) -> torch.Tensor:
        """Host-buffer entry point: ``x_host`` / ``out_host`` are pinned CPU tensors
        ``[B, S, hidden]``.  The work is cut into items that flow through three streams - copy-in,
        compute (the current stream) and copy-out - so the PCIe transfers of one item overlap the
        kernels of another.  Items are groups of whole sequences (``host_pipeline_groups``); a
        group that is a single sequence at either end of the schedule - the only places where a
        copy cannot hide behind compute, and at one sequence per rank the whole job - is further
        cut into ``seq_pieces`` runs of positions that are fed through ``forward(..., kv_cache=)``
        one after the other (``host_pipeline_items``).  ``seq_pieces=1`` keeps sequences whole.
        Returns ``out_host`` once every item has landed in it."""
        self.forward_host_async(x_host, out_host, chunks, seq_pieces).wait()
        return out_host

    def forward_host_async(self, x_host: torch.Tensor, out_host: torch.Tensor, chunks: int | None = 2,
                           seq_pieces: int | None = 1) -> "HostStep":
        """``forward_host`` without the final wait: enqueues the copies and kernels of one step and
        returns a ``HostStep`` at once.  ``step.wait()`` blocks the host until ``out_host`` is
        complete; ``step.input_consumed`` is the event after which ``x_host`` may be overwritten.
        Steps enqueued back to back overlap across the step boundary - the next step's copy-in runs
        under this step's kernels, this step's copy-out under the next step's - which is what hides
        the transfers when a step is a single sequence (one sequence per rank at 8 GPUs) and
        nothing inside the step can.  Give every step in flight its own ``out_host``; two in
        flight are enough to keep all three streams busy.  By default the step is cut into two
        halves of its sequences (``chunks=2``) and sequences stay whole (``seq_pieces=1``): with the
        neighbouring steps to overlap with, finer cuts only shrink the GEMMs and add launches, while
        two halves cost nothing in the steady state and halve what is exposed when the pipeline
        starts and drains (the first copy-in, the last copy-out).  Measured on one B200, per step:
        one 2048-token sequence 0.78 ms whole and 1.01 ms in two runs of positions, against 0.72 ms
        of kernels and 1.32 ms for the blocking call; eight sequences 6.1 ms as one item or two,
        6.3-6.5 ms as four or as the blocking call's 1-2-2-2-1 plan, against 5.7 ms of kernels and
        6.7 ms for the blocking call.  ``chunks=None`` / ``seq_pieces=None`` select the blocking
        call's plan."""
        dev = self.device
        b, seq = x_host.shape[0], x_host.shape[1]
        if not hasattr(self, "_copy_in"):
            self._copy_in, self._copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        compute = torch.cuda.current_stream(dev)
        items = host_pipeline_items(b, seq, chunks, seq_pieces if self.fused else 1)
        staged = []
        with torch.cuda.stream(self._copy_in):
            for b0, b1, s0, s1 in items:
                xd = x_host[b0:b1, s0:s1].to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._copy_in)
                staged.append((xd, ev))
        consumed = staged[-1][1]
        cache = None
        for (b0, b1, s0, s1), (xd, ev) in zip(items, staged):
            compute.wait_event(ev)
            xd.record_stream(compute)
            if s0 == 0 and s1 == seq:
                y = self.forward(xd)
            else:
                if s0 == 0:
                    shape = (b1 - b0, seq, self.n_kv_heads, self.head_dim)
                    cache = (torch.empty(shape, dtype=xd.dtype, device=dev), torch.empty(shape, dtype=xd.dtype, device=dev))
                y = self.forward(xd, pos_offset=s0, kv_cache=cache)
            done = torch.cuda.Event()
            done.record(compute)
            self._copy_out.wait_event(done)
            y.record_stream(self._copy_out)
            with torch.cuda.stream(self._copy_out):
                out_host[b0:b1, s0:s1].copy_(y, non_blocking=True)
        landed = torch.cuda.Event()
        landed.record(self._copy_out)
        return HostStep(out_host, consumed, landed)

    def gemm_flops(self, tokens: int) -> int:
        """2*M*K*N summed over the seven projections for ``tokens`` rows."""
        shapes = [self.w[n].shape for n in ("o_proj", "down_proj")]
        shapes += ([self.w_gate_up.shape, self.w_qkv.shape] if self.fused else
                   [self.w[n].shape for n in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")])
        return sum(2 * tokens * o * i for o, i in shapes)


class LlamaBlockFP8:
    """The same decoder block with every projection on the FP8 tensor-core path (e4m3 operands,
    fp32 accumulation): weights quantised once per output channel, activations per token on the
    fly.  An addition - the reference's block and this library's ``LlamaBlock`` compute in
    bfloat16 - for serving stacks that accept FP8 projections; the residual stream, RoPE, the
    attention core and both norms' arithmetic stay in bfloat16 / fp32.  The quantisers are folded
    into their neighbours so no activation makes an extra trip through HBM:

        x --[rmsnorm + quant, one pass]--> qkv GEMM (fp8) --> rope, SDPA (bf16)
          --[per-token quant]--> o_proj GEMM (fp8) + residual epilogue
          --[rmsnorm + quant, one pass]--> gate-up GEMM (fp8) + SwiGLU epilogue, which also leaves
            each row's maxima per 128 columns --[quant from those maxima]--> down GEMM (fp8) +
            residual epilogue

    ``fused=False`` runs the same arithmetic as separate kernels (norm, quantise, GEMM, swiglu,
    add); the two give identical results."""

    def __init__(self, weights: dict[str, torch.Tensor], n_heads: int = 32, n_kv_heads: int = 8, eps: float = 1e-5,
                 theta: float = 500000.0, max_seq_len: int = 2048, fused: bool = True):
        missing = [n for n in PARAM_NAMES if n not in weights]
        if missing:
            raise ValueError(f"missing block parameters: {missing}")
        for name in PARAM_NAMES:
            if not weights[name].is_cuda or not weights[name].is_contiguous():
                raise ValueError(f"parameter '{name}' must be a contiguous CUDA tensor")
        self.hidden = weights["q_proj"].shape[1]
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.head_dim = weights["q_proj"].shape[0] // n_heads
        self.eps, self.fused = eps, fused
        self.device = weights["q_proj"].device
        self.ffn = weights["gate_proj"].shape[0]
        if self.ffn % GATE_UP_BLOCK or self.hidden % 16 or self.ffn % 16:
            raise ValueError("the FP8 block needs hidden and FFN sizes that are multiples of 16 (FFN of 128)")
        self.cos, self.sin = rope_tables(max_seq_len, self.head_dim, theta, self.device)
        self.w_in, self.w_post = weights["input_layernorm_weight"], weights["post_attention_layernorm_weight"]
        self.q_cols, self.kv_cols = weights["q_proj"].shape[0], weights["k_proj"].shape[0]
        quant = lambda w: fp8_quant(w.contiguous(), "e4m3", "token")            # one scale per output channel
        self.qkv = quant(torch.cat([weights["q_proj"], weights["k_proj"], weights["v_proj"]], dim=0))
        self.o = quant(weights["o_proj"])
        self.gate_up = quant(interleave_gate_up(weights["gate_proj"], weights["up_proj"]))
        self.gate, self.up = quant(weights["gate_proj"]), quant(weights["up_proj"])
        self.down = quant(weights["down_proj"])
        if fused:
            del self.gate, self.up
        #: this library's kernels per forward: 2 norm+quant, 2 quantisers, 4 GEMMs, and a rope kernel
        #: unless the heads are 128 wide (the rotation then rides in the QKV epilogue)
        self.launches_per_forward = (8 if self.head_dim == 128 else 9) if fused else 15

    def forward(self, x: torch.Tensor, timer: OpTimer | None = None) -> torch.Tensor:
        t = timer if timer is not None else _NoTimer
        b, s, hid = x.shape
        x2 = x.view(b * s, hid)
        if self.fused:
            h8, hs = t.run("rmsnorm_quant", rmsnorm_fp8_quant, x2, self.w_in, self.eps)
        else:
            h8, hs = fp8_quant(rmsnorm(x2, self.w_in, self.eps), "e4m3", "token")
        qc, kc = self.q_cols, self.kv_cols
        rope_in_gemm = self.fused and self.head_dim == 128
        if rope_in_gemm:
            qkv = t.run("gemm_fp8_rope", matmul_add_bias_rope_fp8, h8, hs, *self.qkv, None, self.cos[:s], self.sin[:s],
                        qc + kc).view(b, s, -1)
        else:
            qkv = t.run("gemm_fp8", matmul_add_bias_fp8, h8, hs, *self.qkv).view(b, s, -1)
        q = qkv[..., :qc].unflatten(-1, (self.n_heads, self.head_dim))
        k = qkv[..., qc:qc + kc].unflatten(-1, (self.n_kv_heads, self.head_dim))
        v = qkv[..., qc + kc:].unflatten(-1, (self.n_kv_heads, self.head_dim))
        if not rope_in_gemm:
            q, k = t.run("rope", rope_strided, q, k, self.cos[:s], self.sin[:s])
        att = t.run("sdpa", F.scaled_dot_product_attention, q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                    is_causal=True, enable_gqa=self.n_heads != self.n_kv_heads)
        att = att.transpose(1, 2).contiguous().view(b * s, hid)
        a8, a_s = t.run("quant", fp8_quant, att, "e4m3", "token")
        if self.fused:
            res2 = t.run("gemm_fp8_residual", matmul_add_bias_residual_fp8, a8, a_s, *self.o, None, x2)
            h28, h2s = t.run("rmsnorm_quant", rmsnorm_fp8_quant, res2, self.w_post, self.eps)
            act, amax = t.run("gemm_fp8_swiglu", matmul_swiglu_fp8, h28, h2s, *self.gate_up, amax=True)
            act8, act_s = t.run("quant", fp8_quant_token_from_amax, act, amax)
            out = t.run("gemm_fp8_residual", matmul_add_bias_residual_fp8, act8, act_s, *self.down, None, res2)
        else:
            res2 = matmul_add_bias_fp8(a8, a_s, *self.o) + x2
            h28, h2s = fp8_quant(rmsnorm(res2, self.w_post, self.eps), "e4m3", "token")
            act = swiglu(matmul_add_bias_fp8(h28, h2s, *self.gate), matmul_add_bias_fp8(h28, h2s, *self.up))
            act8, act_s = fp8_quant(act, "e4m3", "token")
            out = matmul_add_bias_fp8(act8, act_s, *self.down) + res2
        return out.view(b, s, hid)

    __call__ = forward

    def gemm_flops(self, tokens: int) -> int:
        shapes = [self.qkv[0].shape, self.o[0].shape, self.gate_up[0].shape, self.down[0].shape]
        return sum(2 * tokens * o * i for o, i in shapes)
