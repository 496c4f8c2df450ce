"""GPU parity: the Llama decoder block (examples/llama_block.py:158-173 structure) built
from this library's ops, against the CPU oracle block with the same weights.

The oracle block is pinned bit for bit to the reference's own BaselineLlamaBlock on CPU
(tests/golden/make_golden.py, pin_report.json "block").  A seven-GEMM bf16 chain cannot be
compared bit for bit across machines: torch's own eager bf16 block on GPU and on CPU differ on
2.2 % (192-token sequences) to 5.9 % (2048-token sequences) of the elements at the reference's
block tolerance (rtol 1e-2, atol 2e-2; examples/llama_block.py:271-283 compares two blocks that
share cuBLAS and SDPA, so only its three fused ops differ).  The bars, each the value measured
on B200 plus a stated margin:

  (1) against an fp32 evaluation of the same block, the GPU result is as accurate as the
      oracle's bf16 result (rms error ratio <= 1.25; at full size also against torch's own bf16
      GPU ops, ratio <= 1.1);
  (2) elementwise against the CPU oracle at the reference's tolerance: no further from it than
      torch's own GPU ops are (<= 1.1 x their outlier fraction + 1e-3), and in absolute terms
      <= 3 % at 192 tokens (measured 2.21 %), <= 7.5 % at 2048 tokens (measured 5.93-6.02 %);
  (3) against the same block written with torch's own GPU ops (F.linear, SDPA, eager norm /
      rope / swiglu), where only accumulation order differs: <= 2e-3 at 192 tokens (measured
      4.5e-4 to 6.7e-4), <= 1.2e-2 at 2048 tokens (measured 5.8e-3 to 8.4e-3 per sequence)."""

import pytest
import torch
import torch.nn.functional as F

from oracle import ops, workloads
from tests.gpu_util import DEV, device_status_clean

pytestmark = pytest.mark.gpu


def _gpu_eager_block(x, w, n_heads, n_kv, eps, theta):
    b, s, hid = x.shape
    d = hid // n_heads
    cos, sin = ops.rope_tables(s, d, theta)
    cos, sin = cos.to(x.device), sin.to(x.device)
    h, res = ops.rmsnorm_residual(x, torch.zeros_like(x), w["input_layernorm_weight"], eps)
    q = F.linear(h, w["q_proj"]).view(b, s, n_heads, d)
    k = F.linear(h, w["k_proj"]).view(b, s, n_kv, d)
    v = F.linear(h, w["v_proj"]).view(b, s, n_kv, d)
    q, k = ops.rope(q, k, cos, sin)
    att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                         is_causal=True, enable_gqa=n_heads != n_kv)
    att = F.linear(att.transpose(1, 2).contiguous().view(b, s, hid), w["o_proj"])
    h2, res2 = ops.rmsnorm_residual(att, res, w["post_attention_layernorm_weight"], eps)
    return F.linear(ops.swiglu(F.linear(h2, w["gate_proj"]), F.linear(h2, w["up_proj"])), w["down_proj"]) + res2


def _outside(a, b):
    """Fraction of elements outside the reference's block tolerance (examples/llama_block.py:271-283)."""
    return float(((a - b).abs() > 2e-2 + 1e-2 * b.abs()).float().mean())


def _check(cfg, batch, seq):
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    w = workloads.block_weights(cfg)
    x = workloads.block_input(batch, seq, cfg["hidden"])
    kw = dict(n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], eps=cfg["eps"], theta=cfg["theta"])
    with torch.no_grad():
        want = ops.llama_block(x, w, **kw).float()
        truth = ops.llama_block(x.float(), {k: v.float() for k, v in w.items()}, **kw)
        wd = {k: v.to(DEV) for k, v in w.items()}
        block = LlamaBlock(dict(wd), cfg["n_heads"], cfg["n_kv_heads"], cfg["eps"], cfg["theta"], max_seq_len=seq)
        got_dev = block(x.to(DEV))
        # the fused epilogues (gate-up + SwiGLU, down + residual) change nothing, bit for bit
        unfused = LlamaBlock(dict(wd), cfg["n_heads"], cfg["n_kv_heads"], cfg["eps"], cfg["theta"], max_seq_len=seq,
                             fused=False)
        assert block.fused == (cfg["ffn"] % 128 == 0) and not unfused.fused
        assert torch.equal(got_dev, unfused(x.to(DEV)))
        eager_dev = _gpu_eager_block(x.to(DEV), wd, cfg["n_heads"], cfg["n_kv_heads"], cfg["eps"], cfg["theta"])
    assert got_dev.shape == x.shape and got_dev.dtype == torch.bfloat16
    got = got_dev.cpu().float()
    rms = lambda t: float(t.pow(2).mean().sqrt())
    assert rms(got - truth) <= 1.25 * rms(want - truth)
    eager = eager_dev.cpu().float()
    assert _outside(got, want) <= min(0.03, 1.1 * _outside(eager, want) + 1e-3)
    assert _outside(got, eager) <= 2e-3
    assert device_status_clean(got_dev)


def test_block_llama3_8b_shapes_short_sequences():
    """Benchmark config 4's architecture at batch 2 x seq 192 (the CPU oracle costs ~0.9 GFLOP per token)."""
    _check(dict(workloads.LLAMA3_8B), 2, 192)


def test_block_small_config_ragged_tokens():
    """hidden 512, 8 q / 2 kv heads, FFN 1408, 3 x 77 tokens: partial GEMM tiles everywhere."""
    cfg = dict(workloads.LLAMA3_8B, hidden=512, ffn=1408, n_heads=8, n_kv_heads=2, head_dim=64)
    _check(cfg, 3, 77)


def test_block_is_deterministic_and_batch_independent():
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    cfg = dict(workloads.LLAMA3_8B, hidden=1024, ffn=2816, n_heads=8, n_kv_heads=2, head_dim=128)
    wd = {k: v.to(DEV) for k, v in workloads.block_weights(cfg).items()}
    block = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256)
    x = workloads.block_input(4, 256, 1024).to(DEV)
    with torch.no_grad():
        full = block(x)
        assert torch.equal(full, block(x))
        # sequences are independent: a rank that holds only sequences 2..3 gets the same rows
        part = block(x[2:4].contiguous())
    assert torch.equal(part, full[2:4])
    # the host-buffer entry point (pinned in, pinned out, groups pipelined over three streams)
    x_host = x.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    with torch.no_grad():
        for chunks in (None, 1, 3):
            out_host.zero_()
            block.forward_host(x_host, out_host, chunks=chunks)
            assert torch.equal(out_host, full.cpu())
        # several steps in flight (submit, then wait for the step before), different inputs, own outputs
        inputs = [x_host, (x * 0.5).cpu().pin_memory(), x.flip(0).contiguous().cpu().pin_memory()]
        wants = [full.cpu(), block(x * 0.5).cpu(), block(x.flip(0).contiguous()).cpu()]
        outs = [torch.zeros_like(x_host).pin_memory() for _ in inputs]
        steps = [block.forward_host_async(xi, oi) for xi, oi in zip(inputs, outs)]
        assert steps[0].input_consumed is not steps[0].landed
        for step, out, want in zip(steps, outs, wants):
            assert step.wait() is out and torch.equal(out, want)
        steps[-1].input_consumed.synchronize()


def test_decode_sized_steps_through_a_kv_cache_match_the_whole_sequence():
    """One new token per sequence against a filled KV cache (the decode-sized path: plain QKV
    projection and projection + residual on the weight-streaming kernel, a rope kernel on views
    with one position per sequence) gives the rows the whole-sequence call gives, to the block
    tolerance.  The unfused chain agrees to that tolerance as well, not bit for bit: at these sizes
    its gate / up projections split K over a cluster while the fused gate-up GEMM does not."""
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    cfg = dict(workloads.LLAMA3_8B, hidden=1024, ffn=2816, n_heads=8, n_kv_heads=2, head_dim=128)
    wd = {k: v.to(DEV) for k, v in workloads.block_weights(cfg).items()}
    block = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256)
    chain = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256, fused=False)
    x = workloads.block_input(3, 200, 1024).to(DEV)
    with torch.no_grad():
        whole = block(x)
        caches = [tuple(torch.zeros(3, 256, 2, 128, dtype=torch.bfloat16, device=DEV) for _ in range(2)) for _ in range(2)]
        first = block(x[:, :197].contiguous(), kv_cache=caches[0])
        chain(x[:, :197].contiguous(), kv_cache=caches[1])
        assert torch.equal(first, whole[:, :197])
        for pos in (197, 198, 199):
            step = block(x[:, pos:pos + 1].contiguous(), pos_offset=pos, kv_cache=caches[0])
            same = chain(x[:, pos:pos + 1].contiguous(), pos_offset=pos, kv_cache=caches[1])
            assert step.shape == (3, 1, 1024)
            ops.assert_close_with_outliers(step, same, rtol=1e-2, atol=2e-2, max_outlier_fraction=0.01)
            ops.assert_close_with_outliers(step, whole[:, pos:pos + 1], rtol=1e-2, atol=2e-2, max_outlier_fraction=0.01)


def test_rope_in_the_qkv_epilogue_equals_the_rope_kernel_path():
    """The block with RoPE in the QKV GEMM's epilogue (default for heads of 128), with the rope
    kernel on the QKV buffer's column ranges (``rope_in_gemm=False``) and the unfused chain give the
    same bits; heads of 64 take the rope-kernel path by themselves."""
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    cfg = dict(workloads.LLAMA3_8B, hidden=1024, ffn=2816, n_heads=8, n_kv_heads=2, head_dim=128)
    wd = {k: v.to(DEV) for k, v in workloads.block_weights(cfg).items()}
    x = workloads.block_input(2, 160, 1024).to(DEV)
    with torch.no_grad():
        a = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256)
        b = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256, rope_in_gemm=False)
        c = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256, fused=False)
        assert a.rope_in_gemm and not b.rope_in_gemm and a.launches_per_forward == 6 and b.launches_per_forward == 7
        ya = a(x)
        assert torch.equal(ya, b(x)) and torch.equal(ya, c(x))
        d = LlamaBlock(wd, 16, 4, cfg["eps"], cfg["theta"], max_seq_len=256)          # the same weights read as heads of 64
        e = LlamaBlock(wd, 16, 4, cfg["eps"], cfg["theta"], max_seq_len=256, fused=False)
        assert not d.rope_in_gemm and torch.equal(d(x), e(x))
    assert device_status_clean(x)


def test_captured_block_replays_the_eager_result_on_new_inputs():
    """``LlamaBlock.capture`` returns a CUDA-graph replay of the forward call: after new data is
    copied into the staging input it gives, bit for bit, what the eager call gives - for a whole
    sequence and for a decode-sized step against a KV cache."""
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    cfg = dict(workloads.LLAMA3_8B, hidden=1024, ffn=2816, n_heads=8, n_kv_heads=2, head_dim=128)
    wd = {k: v.to(DEV) for k, v in workloads.block_weights(cfg).items()}
    block = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=256)
    x = workloads.block_input(2, 200, 1024).to(DEV)
    stage = torch.zeros(2, 192, 1024, dtype=x.dtype, device=DEV)
    replay = block.capture(stage)
    with torch.no_grad():
        for lo in (0, 8):
            stage.copy_(x[:, lo:lo + 192])
            assert torch.equal(replay(), block(x[:, lo:lo + 192].contiguous()))
        cache = tuple(torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        block(x[:, :199].contiguous(), kv_cache=cache)
        want = block(x[:, 199:200].contiguous(), pos_offset=199, kv_cache=cache)
        token = torch.zeros(2, 1, 1024, dtype=x.dtype, device=DEV)
        step = block.capture(token, pos_offset=199, kv_cache=cache)
        token.copy_(x[:, 199:200])
        assert torch.equal(step(), want)
    assert device_status_clean(x)


def test_block_config4_full_size():
    """Benchmark config 4 at full size (batch 8 x seq 2048), all 16384 tokens: against the CPU
    oracle block, against the same block on torch's own GPU ops (bf16, and fp32 as the common
    truth), and sequence independence (the rows a rank would compute for sequences 6..7 are the
    same rows).  Bars as listed at the top of this file."""
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    cfg = dict(workloads.LLAMA3_8B)
    w = workloads.block_weights(cfg)
    x = workloads.block_input(8, 2048, cfg["hidden"])
    kw = dict(n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], eps=cfg["eps"], theta=cfg["theta"])
    arch = (cfg["n_heads"], cfg["n_kv_heads"], cfg["eps"], cfg["theta"])
    with torch.no_grad():
        want = ops.llama_block(x, w, **kw).float()
        wd = {k: v.to(DEV) for k, v in w.items()}
        block = LlamaBlock(dict(wd), *arch, max_seq_len=2048)
        xd = x.to(DEV)
        got_dev = block(xd)
        part = block(xd[6:8].contiguous())
        eager = _gpu_eager_block(xd, wd, *arch).cpu().float()
        w32 = {k: v.float() for k, v in wd.items()}
        truth = torch.cat([_gpu_eager_block(xd[i:i + 1].float(), w32, *arch).cpu() for i in range(8)])
    got = got_dev.cpu().float()
    rms = lambda t: float(t.pow(2).mean().sqrt())
    assert rms(got - truth) <= 1.1 * rms(eager - truth)             # as accurate as torch's bf16 GPU ops ...
    assert rms(got - truth) <= 1.25 * rms(want - truth)             # ... and as the CPU oracle
    assert _outside(got, want) <= min(0.075, 1.1 * _outside(eager, want) + 1e-3)
    per_sequence = [_outside(got[i], eager[i]) for i in range(8)]
    assert max(per_sequence) <= 1.2e-2, per_sequence
    assert torch.equal(part, got_dev[6:8])
    assert device_status_clean(got_dev)


@pytest.mark.parametrize("cfg,batch,seq", [
    (dict(workloads.LLAMA3_8B), 2, 192),
    (dict(workloads.LLAMA3_8B, hidden=512, ffn=1408, n_heads=8, n_kv_heads=2, head_dim=64), 3, 77)])
def test_fp8_block_fused_equals_its_unfused_chain_and_tracks_the_bf16_block(cfg, batch, seq):
    """The FP8 variant of the block (an addition; the reference computes in bfloat16): with the
    quantisers folded into the norms and the GEMM epilogues it returns, bit for bit, what the same
    arithmetic gives as separate kernels (norm, per-token quantiser, FP8 GEMM, swiglu, add - each
    checked against the oracle on its own), and it stays within FP8 accuracy of the bfloat16
    block: relative rms difference below 20 % (measured 13.8 % at 192 tokens, 14.9 % at 2048: e4m3
    keeps 3 mantissa bits, so every product carries two roundings of up to 6 % each, four
    projections deep, with a norm in between that rescales the small attention branch)."""
    from custom_cuda_kernals_b200.llama_block import LlamaBlock, LlamaBlockFP8
    w = {k: v.to(DEV) for k, v in workloads.block_weights(cfg).items()}
    g = torch.Generator().manual_seed(3)
    for key in ("input_layernorm_weight", "post_attention_layernorm_weight"):
        w[key] = (1 + 0.1 * torch.randn(cfg["hidden"], generator=g)).to(torch.bfloat16).to(DEV)
    x = workloads.block_input(batch, seq, cfg["hidden"]).to(DEV)
    arch = (cfg["n_heads"], cfg["n_kv_heads"], cfg["eps"], cfg["theta"])
    with torch.no_grad():
        fused = LlamaBlockFP8(dict(w), *arch, max_seq_len=seq)(x)
        chain = LlamaBlockFP8(dict(w), *arch, max_seq_len=seq, fused=False)(x)
        bf16 = LlamaBlock(dict(w), *arch, max_seq_len=seq)(x)
    assert fused.shape == x.shape and fused.dtype == torch.bfloat16
    assert torch.equal(fused, chain)
    rel = float((fused.float() - bf16.float()).norm() / bf16.float().norm())
    assert rel < 0.2, rel
    assert device_status_clean(fused)


def test_sequence_fed_in_pieces_through_a_kv_cache_matches_the_whole_sequence():
    """Chunked prefill: positions fed piece by piece with ``kv_cache`` compute the same function as
    one call (every op but attention is token-wise; attention sees the same keys).  The attention
    core runs a different kernel for a continuation (bottom-right causal mask over a longer key
    range), so the comparison is the block tolerance with the outlier budget of test (3) at the top
    of this file, not bit equality; the first piece (no history yet) is bit-equal.  Then the host
    pipeline that uses it: ``forward_host`` with sequences cut into position pieces."""
    from custom_cuda_kernals_b200.llama_block import LlamaBlock, host_pipeline_items
    cfg = dict(workloads.LLAMA3_8B, hidden=1024, ffn=2816, n_heads=8, n_kv_heads=2, head_dim=128)
    wd = {k: v.to(DEV) for k, v in workloads.block_weights(cfg).items()}
    block = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=1024)
    x = workloads.block_input(2, 1024, 1024).to(DEV)
    with torch.no_grad():
        whole = block(x)
        cache = tuple(torch.empty(2, 1024, 2, 128, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        cuts = [0, 256, 300, 768, 1024]                         # ragged pieces
        parts = [block(x[:, a:b].contiguous(), pos_offset=a, kv_cache=cache) for a, b in zip(cuts[:-1], cuts[1:])]
        small = tuple(torch.empty(2, 512, 2, 128, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        with pytest.raises(ValueError, match="kv_cache of shape"):
            block(x[:, :8].contiguous(), pos_offset=510, kv_cache=small)
    pieced = torch.cat(parts, dim=1)
    assert torch.equal(pieced[:, :256], whole[:, :256])
    assert _outside(pieced.float().cpu(), whole.float().cpu()) <= 2e-3
    # keys and values in the cache are those of the whole-sequence pass
    assert host_pipeline_items(1, 1024) == [(0, 1, 0, 512), (0, 1, 512, 1024)]      # one sequence: cut in two
    x_host = x.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    with torch.no_grad():
        block.forward_host(x_host, out_host, seq_pieces=1)
        assert torch.equal(out_host, whole.cpu())
        for pieces in (None, 2, 4):
            out_host.zero_()
            block.forward_host(x_host, out_host, seq_pieces=pieces)
            assert _outside(out_host.float(), whole.float().cpu()) <= 2e-3
    assert device_status_clean(whole)
