"""GPU parity: matmul_add_bias (tensor-core and CUDA-core paths) and the FP8 GEMM
against the CPU oracle (baselines/matmul_add_bias.py cases and tolerances)."""

import pytest
import torch

from oracle import cases, ops, workloads
from tests.gpu_util import DEV, check, device_status_clean, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", cases.GEMM_CASES, ids=lambda c: c.name)
def test_matmul_add_bias_cases(case):
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    x, w, b = cases.gemm_inputs(case)
    y = matmul_add_bias(*to_dev(x, w, b))
    assert y.shape == (case.m, case.n) and y.dtype == case.dtype
    if case.m == 0:
        return
    check(y.double(), ops.matmul_add_bias_fp64(x, w, b), case.dtype, ops.TOLERANCE_GEMM)
    if case.m * case.k * case.n <= 2048 * 4096 * 4096 or case.dtype != torch.float32:
        check(y, ops.matmul_add_bias(x, w, b), case.dtype, ops.TOLERANCE_GEMM)
    assert device_status_clean(y)


def test_none_bias_equals_zero_bias():
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(384, 512, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    w = (torch.randn(640, 512, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    a = matmul_add_bias(x, w, None)
    b = matmul_add_bias(x, w, torch.zeros(640, dtype=torch.bfloat16, device=DEV))
    assert torch.equal(a, b)


@pytest.mark.parametrize("shape", [(128, 64, 256), (129, 72, 257), (300, 200, 520), (1000, 4096, 264),
                                   (4, 512, 1024), (2048, 8, 512), (131, 1032, 777)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tensor_core_path_ragged_shapes(shape, dtype):
    """K a multiple of 8 goes to the tcgen05 kernel: partial tiles in M, N and K are
    zero-filled by TMA and masked in the epilogue; N not a multiple of 8 takes scalar stores."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    m, k, n = shape
    g = torch.Generator().manual_seed(m * 7 + n)
    x = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
    w = (torch.randn(n, k, generator=g) * 0.05).to(dtype)
    b = torch.randn(n, generator=g).to(dtype)
    y = matmul_add_bias(*to_dev(x, w, b))
    check(y.double(), ops.matmul_add_bias_fp64(x, w, b), dtype, ops.TOLERANCE_GEMM)
    assert device_status_clean(y)


@pytest.mark.parametrize("shape", [(128, 4096, 4096), (16, 4096, 11008), (256, 1024, 4096), (100, 512, 1000),
                                   (512, 4096, 4096), (128, 4096, 72), (1, 8192, 4096), (16, 4096, 4096),
                                   (17, 1024, 2048), (64, 4096, 4096), (5, 256, 520), (33, 11008, 4096)])
def test_small_m_narrow_tiles_match_oracle(shape):
    """Decode-sized batches (few 128 x 256 tiles) run on 128 x 64 tiles: same results as the
    oracle's bf16 chain and as an fp32 evaluation, ragged column counts included."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    m, k, n = shape
    g = torch.Generator().manual_seed(m + k + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    b = (0.02 * torch.randn(n, generator=g)).to(torch.bfloat16)
    y = matmul_add_bias(*to_dev(x, w, b))
    check(y.double(), ops.matmul_add_bias_fp64(x, w, b), torch.bfloat16, ops.TOLERANCE_GEMM)
    exact = x.float() @ w.float().T + b.float()
    assert (y.float().cpu() - exact).abs().max() <= 2 ** -8 * exact.abs().max() + 1e-3
    assert device_status_clean(y)


def test_row_and_column_shards_are_bitwise_slices_of_the_whole_at_small_sizes():
    """The default kernels (full-width and 128 x 64 tiles) add a row's products in one order
    whatever the problem size: shards of more than 128 rows reproduce the whole exactly.  Batches of
    at most 128 rows split K over a cluster by default (decode-sized problems), which adds in
    another order: those agree to the GEMM tolerance, not bit for bit."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator().manual_seed(8)
    x = torch.randn(768, 1024, generator=g).to(torch.bfloat16).to(DEV)
    w = (0.05 * torch.randn(1536, 1024, generator=g)).to(torch.bfloat16).to(DEV)
    whole = matmul_add_bias(x, w)
    assert torch.equal(matmul_add_bias(x[:256].contiguous(), w), whole[:256])
    assert torch.equal(matmul_add_bias(x[300:429].contiguous(), w), whole[300:429])
    assert torch.equal(matmul_add_bias(x[470:749].contiguous(), w), whole[470:749])
    for lo, hi in ((300, 316), (700, 749), (0, 128), (300, 396)):
        check(matmul_add_bias(x[lo:hi].contiguous(), w), whole[lo:hi], torch.bfloat16, ops.TOLERANCE_GEMM)
    assert torch.equal(matmul_add_bias(x, w[512:1024].contiguous()), whole[:, 512:1024])


def test_large_problem_rows_do_not_depend_on_how_many_rows_are_computed_together():
    """8192 x 512 x 1792 (224 CTA-pair tiles, a ragged last wave) equals, bit for bit, the same
    rows computed as two 4096-row problems, and matches the oracle; ragged edges included."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator().manual_seed(77)
    x = torch.randn(8192, 512, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(1792, 512, generator=g)).to(torch.bfloat16)
    b = (0.05 * torch.randn(1792, generator=g)).to(torch.bfloat16)
    xd, wd, bd = to_dev(x, w, b)
    y = matmul_add_bias(xd, wd, bd)
    halves = torch.cat([matmul_add_bias(xd[:4096].contiguous(), wd, bd), matmul_add_bias(xd[4096:].contiguous(), wd, bd)])
    assert torch.equal(y, halves)
    check(y[:1024], ops.matmul_add_bias(x[:1024], w, b), torch.bfloat16, ops.TOLERANCE_GEMM)
    check(y[-512:], ops.matmul_add_bias(x[-512:], w, b), torch.bfloat16, ops.TOLERANCE_GEMM)
    # ragged edges: 8000 rows, 1800 columns
    y2 = matmul_add_bias(xd[:8000].contiguous(), torch.cat([wd, wd[:8]]), torch.cat([bd, bd[:8]]))
    assert torch.equal(y2[:, :1792], y[:8000]) and torch.equal(y2[:, 1792:], y[:8000, :8])
    assert device_status_clean(y)


_SPLITK_CHILD = r"""
import torch
from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
from custom_cuda_kernals_b200 import _native
dev = torch.device("cuda", 0)
for (m, k, n) in [(128, 4096, 4096), (16, 4096, 4096), (256, 1024, 4096), (100, 512, 1000), (128, 4096, 72),
                  (1, 8192, 4096), (128, 11008, 4096), (77, 4096, 520)]:
    g = torch.Generator().manual_seed(m + k + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    b = (0.02 * torch.randn(n, generator=g)).to(torch.bfloat16)
    y = matmul_add_bias(x.to(dev), w.to(dev), b.to(dev))
    exact = x.double() @ w.double().T + b.double()
    err = (y.cpu().double() - exact).abs().max().item()
    assert err <= 2 ** -8 * exact.abs().max().item() + 1e-3, (m, k, n, err)
    again = matmul_add_bias(x.to(dev), w.to(dev), b.to(dev))
    assert torch.equal(y, again), "split-K must be deterministic"
    y16 = matmul_add_bias(x.to(dev).half(), w.to(dev).half(), None)
    assert (y16.cpu().double() - x.half().double() @ w.half().double().T).abs().max().item() <= 2e-2
assert _native.take_device_status(y) == 0
print("SPLITK_OK")
"""


def test_cluster_split_k_mode_matches_fp64_and_is_deterministic():
    """CCK_GEMM_SPLITK=1 (read once per process, so a child process): decode-sized problems run
    on clusters of 2-8 CTAs per tile that split K and reduce through distributed shared memory."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, CCK_GEMM_SPLITK="1", PYTHONPATH=os.pathsep.join([os.getcwd(), os.environ.get("PYTHONPATH", "")]))
    out = subprocess.run([sys.executable, "-c", _SPLITK_CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "SPLITK_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_matmul_identity_is_exact():
    """x @ I + 0 reproduces x bit for bit (every product is exact, one addend per sum)."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator().manual_seed(2)
    x = torch.randn(512, 1024, generator=g).to(torch.bfloat16).to(DEV)
    eye = torch.eye(1024, dtype=torch.bfloat16, device=DEV)
    assert torch.equal(matmul_add_bias(x, eye, None), x)


def test_matmul_config3_full_size():
    """Benchmark config 3: A [8192,4096], W [14336,4096], bias [14336], bf16."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    a, w, b = workloads.gemm_bf16()
    y = matmul_add_bias(*to_dev(a, w, b))
    rows = torch.arange(0, 8192, 61)           # every 61st row through the fp64 oracle
    check(y[rows.to(DEV)].double(), ops.matmul_add_bias_fp64(a[rows], w, b), torch.bfloat16, ops.TOLERANCE_GEMM)
    check(y, ops.matmul_add_bias(a, w, b), torch.bfloat16, ops.TOLERANCE_GEMM)
    # linearity in x: (2x) W^T + b - (x W^T + b) == x W^T, on the whole output
    y2 = matmul_add_bias((a * 2).to(DEV), w.to(DEV), b.to(DEV))
    y0 = matmul_add_bias(a.to(DEV), w.to(DEV), None)
    torch.testing.assert_close((y2.float() - y.float()), y0.float(), rtol=2e-2, atol=4e-2)
    assert device_status_clean(y)


FP8_SHAPES = [(256, 512, 512), (1024, 4096, 1792), (200, 144, 300),
              # shapes the 16-bit entry point accepts and this one used to refuse: decode-sized M (narrow
              # tensor-core tiles), N and K below one tile, K not a multiple of 16 and tiny problems (CUDA cores)
              (16, 4096, 4096), (1, 4096, 1024), (128, 4096, 64), (8, 128, 1000), (300, 64, 2048), (64, 48, 100),
              (130, 100, 70), (257, 129, 513), (1, 1, 1), (3, 16, 5), (2048, 24, 512)]


@pytest.mark.parametrize("shape", FP8_SHAPES)
def test_fp8_gemm_matches_oracle(shape):
    """e4m3 A with per-token scales x e4m3 W with per-channel scales, both from the per-token
    quantiser; oracle = dequantise, fp32 matmul, + bias (unpinned by the reference).  Every
    shape runs, as the reference's launcher guarantees for its dtypes
    (csrc/kernels/matmul_add_bias.cu:170-180)."""
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias_fp8
    m, k, n = shape
    g = torch.Generator().manual_seed(k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    b = (0.02 * torch.randn(n, generator=g)).to(torch.bfloat16)
    a8, a_s = fp8_quant(a.to(DEV), "e4m3", "token")
    w8, w_s = fp8_quant(w.to(DEV), "e4m3", "token")
    y = matmul_add_bias_fp8(a8, a_s, w8, w_s, b.to(DEV))
    want = ops.matmul_add_bias_fp8(a8.cpu(), a_s.cpu(), w8.cpu(), w_s.cpu(), b)
    check(y, want, torch.bfloat16, ops.TOLERANCE_GEMM)
    # and it approximates the unquantised product to FP8 accuracy
    full = ops.matmul_add_bias_fp64(a, w, b)
    rel = (y.cpu().double() - full).norm() / full.norm()
    assert rel < 0.08, rel
    # no bias == zero bias, float16 output
    y0 = matmul_add_bias_fp8(a8, a_s, w8, w_s, None)
    assert torch.equal(y0, matmul_add_bias_fp8(a8, a_s, w8, w_s, torch.zeros(n, dtype=torch.bfloat16, device=DEV)))
    yh = matmul_add_bias_fp8(a8, a_s, w8, w_s, b.to(DEV).half(), out_dtype=torch.float16)
    check(yh, ops.matmul_add_bias_fp8(a8.cpu(), a_s.cpu(), w8.cpu(), w_s.cpu(), b.half(), out_dtype=torch.float16),
          torch.float16, ops.TOLERANCE_GEMM)
    assert device_status_clean(y)


def test_fp8_gemm_config3_full_size():
    """Benchmark config 3 in FP8 (8192 x 4096 x 14336): A and W through the per-token quantiser
    (W per output channel), every 61st row through the dequantise-fp32 oracle, the whole output
    against the bf16 GEMM of the unquantised operands to FP8 accuracy, and row-shard invariance
    (the rows a rank would own come out bit-identical)."""
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias, matmul_add_bias_fp8
    a, w, b = workloads.gemm_bf16()
    ad, wd, bd = to_dev(a, w, b)
    a8, a_s = fp8_quant(ad, "e4m3", "token")
    w8, w_s = fp8_quant(wd, "e4m3", "token")
    y = matmul_add_bias_fp8(a8, a_s, w8, w_s, bd)
    rows = torch.arange(0, 8192, 61)
    rd = rows.to(DEV)
    want = ops.matmul_add_bias_fp8(a8[rd].cpu(), a_s[rd].cpu(), w8.cpu(), w_s.cpu(), b)
    check(y[rd], want, torch.bfloat16, ops.TOLERANCE_GEMM)
    full = matmul_add_bias(ad, wd, bd).float()
    rel = float((y.float() - full).norm() / full.norm())
    assert rel < 0.05, rel                                     # measured 0.036: two e4m3 roundings per product
    part = matmul_add_bias_fp8(a8[4096:6144].contiguous(), a_s[4096:6144].contiguous(), w8, w_s, bd)
    assert torch.equal(part, y[4096:6144])
    assert device_status_clean(y)


@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 1024, 1408), (130, 72, 384), (4096, 4096, 14336)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_gate_up_swiglu_equals_unfused_chain(shape, dtype):
    """One GEMM over the interleaved gate/up weight with the SwiGLU in its epilogue gives, bit
    for bit, what matmul_add_bias x 2 followed by swiglu gives (same roundings in the same
    places), and so inherits their parity with the oracle."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda.kernels.swiglu import swiglu
    from custom_cuda_kernals_b200.kernels.fused import interleave_gate_up, matmul_swiglu
    m, k, f = shape
    g = torch.Generator().manual_seed(f + m)
    x = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    wg = (0.05 * torch.randn(f, k, generator=g)).to(dtype).to(DEV)
    wu = (0.05 * torch.randn(f, k, generator=g)).to(dtype).to(DEV)
    fused = matmul_swiglu(x, interleave_gate_up(wg, wu))
    chain = swiglu(matmul_add_bias(x, wg), matmul_add_bias(x, wu))
    assert torch.equal(fused, chain)
    if m * k * f <= 1 << 31:
        want = ops.swiglu(ops.matmul_add_bias(x.cpu(), wg.cpu()), ops.matmul_add_bias(x.cpu(), wu.cpu()))
        check(fused, want, dtype, ops.TOLERANCE_GEMM)
    assert device_status_clean(fused)


@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 1408, 1024), (131, 72, 777), (4096, 14336, 4096),
                                   (16, 4096, 4096), (100, 1032, 520), (128, 512, 1024), (1, 14336, 4096)])   # the last four: decode kernel
@pytest.mark.parametrize("with_bias", [False, True])
def test_fused_residual_add_equals_unfused_chain(shape, with_bias):
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda_kernals_b200.kernels.fused import matmul_add_bias_residual
    m, k, n = shape
    g = torch.Generator().manual_seed(n + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (0.05 * torch.randn(n, k, generator=g)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(torch.bfloat16).to(DEV) if with_bias else None
    r = torch.randn(m, n, generator=g).to(torch.bfloat16).to(DEV)
    fused = matmul_add_bias_residual(x, w, b, r)
    assert torch.equal(fused, matmul_add_bias(x, w, b) + r)
    assert device_status_clean(fused)


@pytest.mark.parametrize("cfg", [
    # (batch, seq, hidden, q heads, kv heads, with_bias)
    (2, 192, 1024, 8, 2, False),      # two heads per 256-column tile
    (3, 100, 264, 2, 1, True),        # ragged rows and K; the last tile holds one k head (rotated) and one v head (not)
    (1, 2048, 4096, 32, 8, False),    # one Llama-3-8B sequence
    (2, 77, 512, 3, 3, True),         # odd head counts: tiles that start inside q, k and v
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_qkv_projection_with_rope_equals_unfused_chain(cfg, dtype):
    """One projection for q, k and v with the rotary embedding in its epilogue gives, bit for bit,
    what matmul_add_bias followed by the rope kernel on the q / k column ranges gives, and leaves the
    v columns as projected."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda_kernals_b200.kernels.fused import matmul_add_bias_rope
    from custom_cuda_kernals_b200.kernels.rope import rope_strided
    from custom_cuda_kernals_b200.llama_block import rope_tables
    b, s, hidden, hq, hkv, with_bias = cfg
    qc, kc = hq * 128, hkv * 128
    n = qc + 2 * kc
    g = torch.Generator().manual_seed(hidden + s)
    x = torch.randn(b * s, hidden, generator=g).to(dtype).to(DEV)
    w = (0.05 * torch.randn(n, hidden, generator=g)).to(dtype).to(DEV)
    bias = torch.randn(n, generator=g).to(dtype).to(DEV) if with_bias else None
    cos, sin = rope_tables(s + 5, 128, 10000.0, DEV)
    cos, sin = cos[5:], sin[5:]                                   # a slice of positions, as a continuation passes it
    fused = matmul_add_bias_rope(x, w, bias, cos, sin, qc + kc).view(b, s, n)
    plain = matmul_add_bias(x, w, bias).view(b, s, n)
    q, k = rope_strided(plain[..., :qc].unflatten(-1, (hq, 128)), plain[..., qc:qc + kc].unflatten(-1, (hkv, 128)), cos, sin)
    assert torch.equal(fused[..., :qc], q.flatten(-2))
    assert torch.equal(fused[..., qc:qc + kc], k.flatten(-2))
    assert torch.equal(fused[..., qc + kc:], plain[..., qc + kc:])
    assert not torch.equal(fused[..., :qc], plain[..., :qc])
    assert device_status_clean(fused)


@pytest.mark.parametrize("cfg", [(2, 192, 1024, 8, 2, False), (3, 100, 272, 2, 1, True), (1, 2048, 4096, 32, 8, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_fp8_qkv_projection_with_rope_equals_unfused_chain(cfg, dtype):
    """The same with e4m3 operands: FP8 projection with RoPE in its epilogue == matmul_add_bias_fp8
    followed by the rope kernel on the q / k column ranges, bit for bit."""
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias_fp8
    from custom_cuda_kernals_b200.kernels.fused import matmul_add_bias_rope_fp8
    from custom_cuda_kernals_b200.kernels.rope import rope_strided
    from custom_cuda_kernals_b200.llama_block import rope_tables
    b, s, hidden, hq, hkv, with_bias = cfg
    qc, kc = hq * 128, hkv * 128
    n = qc + 2 * kc
    g = torch.Generator().manual_seed(hidden + s)
    x = torch.randn(b * s, hidden, generator=g).to(torch.bfloat16).to(DEV)
    w = (0.05 * torch.randn(n, hidden, generator=g)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(n, generator=g).to(dtype).to(DEV) if with_bias else None
    a8, a_s = fp8_quant(x, "e4m3", "token")
    w8, w_s = fp8_quant(w, "e4m3", "token")
    cos, sin = rope_tables(s, 128, 10000.0, DEV)
    fused = matmul_add_bias_rope_fp8(a8, a_s, w8, w_s, bias, cos, sin, qc + kc, out_dtype=dtype).view(b, s, n)
    plain = matmul_add_bias_fp8(a8, a_s, w8, w_s, bias, out_dtype=dtype).view(b, s, n)
    q, k = rope_strided(plain[..., :qc].unflatten(-1, (hq, 128)), plain[..., qc:qc + kc].unflatten(-1, (hkv, 128)), cos, sin)
    assert torch.equal(fused[..., :qc], q.flatten(-2))
    assert torch.equal(fused[..., qc:qc + kc], k.flatten(-2))
    assert torch.equal(fused[..., qc + kc:], plain[..., qc + kc:])
    assert device_status_clean(fused)


def test_fused_qkv_rope_rejects_what_it_cannot_run():
    from custom_cuda_kernals_b200.kernels.fused import matmul_add_bias_rope
    from custom_cuda_kernals_b200.llama_block import rope_tables
    x = torch.randn(256, 512, device=DEV).to(torch.bfloat16)
    w = torch.randn(512, 512, device=DEV).to(torch.bfloat16)
    cos, sin = rope_tables(128, 128, 10000.0, DEV)
    with pytest.raises(ValueError, match="multiples of 128"):
        matmul_add_bias_rope(x, w[:500].contiguous(), None, cos, sin, 256)
    with pytest.raises(ValueError, match="multiples of 128"):
        matmul_add_bias_rope(x, w, None, cos, sin, 640)
    with pytest.raises(ValueError, match="multiple of seq_len"):
        matmul_add_bias_rope(x[:200].contiguous(), w, None, cos, sin, 256)
    with pytest.raises(ValueError, match="seq_len, 64"):
        matmul_add_bias_rope(x, w, None, cos[:, :32].contiguous(), sin[:, :32].contiguous(), 256)
    with pytest.raises(ValueError, match="fp32"):
        matmul_add_bias_rope(x, w, None, cos.half(), sin.half(), 256)
    with pytest.raises(ValueError, match="fused path"):
        matmul_add_bias_rope(x.float(), w.float(), None, cos, sin, 256)


def test_fused_ops_reject_what_they_cannot_run():
    from custom_cuda_kernals_b200.kernels.fused import interleave_gate_up, matmul_add_bias_residual, matmul_swiglu
    x = torch.randn(16, 64, device=DEV)
    with pytest.raises(ValueError):
        matmul_swiglu(x, torch.randn(256, 64, device=DEV))                 # float32
    with pytest.raises(ValueError):
        interleave_gate_up(torch.randn(100, 64), torch.randn(100, 64))     # F not a multiple of 128
    xb = x.to(torch.bfloat16)
    with pytest.raises(ValueError):
        matmul_swiglu(xb, torch.randn(128, 64, device=DEV).to(torch.bfloat16))   # rows not a multiple of 256
    with pytest.raises(ValueError):
        matmul_add_bias_residual(xb, torch.randn(32, 64, device=DEV).to(torch.bfloat16), None,
                                 torch.randn(16, 31, device=DEV).to(torch.bfloat16))


GENERAL_SHAPES = [(256, 512, 512), (1000, 1024, 1408), (130, 72, 384), (64, 200, 264), (4096, 1000, 1024),
                  (8, 8, 8), (300, 77, 136), (2048, 8192, 512)]


@pytest.mark.parametrize("shape", GENERAL_SHAPES)
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_matmul_general_reads_transposed_operands_as_stored(shape, a_t, b_t, dtype):
    """``A @ B.T`` with A stored [M,K] or [K,M] and B stored [N,K] or [K,N] (MN-major tensor-core
    descriptors, no transposed copies): equal bit for bit to this library's GEMM on explicitly
    transposed copies (same products, same accumulation order), and within the GEMM tolerance of an
    fp64 product.  Ragged M, N and K (K = 77, 200, 1000: partial last slab, zero-filled by TMA)."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda_kernals_b200.kernels.fused import matmul_general
    m, k, n = shape
    if (a_t and m % 8) or (not a_t and k % 8) or (b_t and n % 8) or (not b_t and k % 8):
        pytest.skip("the contiguous dimension of an operand must be a multiple of 8")
    g = torch.Generator(device=DEV).manual_seed(m + k + n)
    a = torch.randn(m, k, device=DEV, generator=g).to(dtype)
    b = (k ** -0.5 * torch.randn(n, k, device=DEV, generator=g)).to(dtype)
    a_st = a.t().contiguous() if a_t else a
    b_st = b.t().contiguous() if b_t else b
    y = matmul_general(a_st, b_st, a_t, b_t)
    want = matmul_add_bias(a, b)
    if 2 * m * n * k >= 1 << 22 and k % 8 == 0:      # both on the tensor cores: identical arithmetic
        assert torch.equal(y, want)
    check(y.double().cpu(), a.double().cpu() @ b.double().cpu().T, dtype, ops.TOLERANCE_GEMM)
    # accumulating form: out (fp32) += product, twice
    acc = torch.full((m, n), 0.5, device=DEV)
    matmul_general(a_st, b_st, a_t, b_t, out=acc, accumulate=True)
    matmul_general(a_st, b_st, a_t, b_t, out=acc, accumulate=True)
    torch.testing.assert_close(acc.double().cpu(), 0.5 + 2 * (a.double().cpu() @ b.double().cpu().T), rtol=1e-3, atol=1e-3)
    assert device_status_clean(y)


def test_matmul_general_rejects_bad_arguments():
    from custom_cuda_kernals_b200.kernels.fused import matmul_general
    a = torch.zeros(64, 32, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="contraction lengths differ"):
        matmul_general(a, torch.zeros(16, 48, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="multiple of 8"):
        matmul_general(torch.zeros(64, 36, device=DEV, dtype=torch.bfloat16), torch.zeros(16, 36, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="float16 or bfloat16"):
        matmul_general(a.float(), a.float())
    with pytest.raises(ValueError, match="accumulate=True needs"):
        matmul_general(a, a, accumulate=True)
    with pytest.raises(ValueError, match="must be float32"):
        matmul_general(a, a, out=torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16), accumulate=True)


@pytest.mark.parametrize("m", [1, 16, 64, 100, 128])
def test_decode_sized_batches_split_k_by_default(m):
    """M <= 128 rows: K is split over a thread-block cluster by default (the weight matrix then
    streams through every SM).  Against the fp64 oracle at the GEMM tolerance, identical run to
    run, and - documented - not bit-identical to the rows of a larger batch, whose kernels add a
    row's products in one order."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator().manual_seed(m)
    a = torch.randn(256, 4096, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(4096, 4096, generator=g)).to(torch.bfloat16)
    b = (0.02 * torch.randn(4096, generator=g)).to(torch.bfloat16)
    ad, wd, bd = to_dev(a, w, b)
    y = matmul_add_bias(ad[:m].contiguous(), wd, bd)
    check(y.double().cpu(), ops.matmul_add_bias_fp64(a[:m], w, b), torch.bfloat16, ops.TOLERANCE_GEMM)
    assert torch.equal(y, matmul_add_bias(ad[:m].contiguous(), wd, bd))
    whole = matmul_add_bias(ad, wd, bd)[:m]
    check(y, whole, torch.bfloat16, ops.TOLERANCE_GEMM)        # same values up to summation order
    assert device_status_clean(y)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (7, 1032, 520), (16, 72, 136), (17, 4096, 1000), (32, 2048, 6144),
                                   (33, 512, 264), (48, 11008, 4096), (64, 4096, 14336), (3, 8192, 72), (64, 64, 4096),
                                   (65, 4096, 4096), (128, 4096, 4096), (100, 1032, 520), (128, 14336, 4096), (97, 72, 136)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_kernel_ragged_shapes(shape, dtype):
    """Batches of at most 128 tokens: the weight rows sit on the M side of the tensor-core instruction,
    the tokens on the N side (16 / 32 / 64 / 128), K split over a cluster.  Ragged token counts, feature
    counts that are not multiples of 128 or 8, K that ends inside a 64-element slab, with and
    without bias; against the fp64 oracle at the GEMM tolerance, and identical run to run."""
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    m, k, n = shape
    g = torch.Generator().manual_seed(m * 31 + n)
    x = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
    w = (torch.randn(n, k, generator=g) * k ** -0.5).to(dtype)
    b = torch.randn(n, generator=g).to(dtype)
    xd, wd, bd = to_dev(x, w, b)
    y = matmul_add_bias(xd, wd, bd)
    assert y.shape == (m, n) and y.dtype == dtype
    check(y.double(), ops.matmul_add_bias_fp64(x, w, b), dtype, ops.TOLERANCE_GEMM)
    assert torch.equal(y, matmul_add_bias(xd, wd, bd))
    y0 = matmul_add_bias(xd, wd, None)
    check(y0.double(), ops.matmul_add_bias_fp64(x, w, None), dtype, ops.TOLERANCE_GEMM)
    assert device_status_clean(y)
