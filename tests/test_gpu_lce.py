"""GPU parity: linear_cross_entropy (fused tensor-core path, chunk-loop path and the
chunk-update entry point) against the CPU oracle (baselines/linear_cross_entropy.py)."""

import pytest
import torch

from oracle import cases, ops, workloads
from tests.gpu_util import DEV, device_status_clean, to_dev

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-4, 1e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-2, 2e-2)}


@pytest.mark.parametrize("case", cases.LCE_CASES, ids=lambda c: c.name)
def test_lce_cases(case):
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    h, w, t = cases.lce_inputs(case)
    got = linear_cross_entropy(*to_dev(h, w, t), reduction=case.reduction)
    assert got.dtype == torch.float32
    assert got.shape == ((case.n_tokens,) if case.reduction == "none" else ())
    assert got.grad_fn is None and not got.requires_grad
    if case.n_tokens == 0:
        return
    heavy = case.n_tokens * case.hidden_dim * case.vocab_size > 1 << 32
    want64 = ops.linear_cross_entropy_rowblocked(h, w, t, reduction=case.reduction, rows_per_block=128,
                                                 wide=torch.float32 if heavy else torch.float64)
    if case.name.startswith("all_ignored"):
        assert torch.isnan(got).all() if case.reduction == "mean" else True
        return
    # the reference's own bar: against the eager loss in the storage dtype.  On the CPU a 16-bit
    # F.cross_entropy also accumulates its mean in 16 bits, so 16-bit cases are compared row by row.
    if not heavy:
        if case.dtype == torch.float32 or case.reduction == "none":
            eager = ops.linear_cross_entropy(h, w, t, reduction=case.reduction).float()
            torch.testing.assert_close(got.cpu(), eager, rtol=TOL[case.dtype][0], atol=TOL[case.dtype][1])
        else:
            rows = linear_cross_entropy(*to_dev(h, w, t), reduction="none").cpu()
            eager = ops.linear_cross_entropy(h, w, t, reduction="none").float()
            torch.testing.assert_close(rows, eager, rtol=TOL[case.dtype][0], atol=TOL[case.dtype][1])
    # the stricter bar: fp32 logits never rounded, so 1e-4 relative against fp64 on the same inputs
    torch.testing.assert_close(got.cpu().double(), want64, rtol=1e-4, atol=1e-6)
    assert device_status_clean(got)


@pytest.mark.parametrize("chunk_size", [1, 3, 7, 500, 1000, 10_000])
def test_chunk_loop_path_is_chunk_size_invariant(chunk_size):
    """fp32 inputs take the chunk loop (tests/test_linear_cross_entropy_kernel.py:76-87)."""
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    case = cases.LceCase("chunk_sweep", 64, 64, 1000, torch.float32)
    h, w, t = cases.lce_inputs(case)
    got = linear_cross_entropy(*to_dev(h, w, t), chunk_size=chunk_size)
    torch.testing.assert_close(got.cpu(), ops.linear_cross_entropy(h, w, t), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("chunk_v", [5, 64, 1000, 4096, 9000])
def test_chunk_update_entry_point(dtype, chunk_v):
    """launch_linear_ce_chunk_update on materialised logits: register path, two-pass path, ragged widths."""
    from custom_cuda import _native
    g = torch.Generator().manual_seed(chunk_v)
    n = 37
    logits = (torch.randn(n, 2 * chunk_v, generator=g) * 4).to(dtype)
    t = torch.randint(0, 2 * chunk_v, (n,), generator=g)
    mx = torch.full((n,), float("-inf"), device=DEV)
    sm = torch.zeros(n, device=DEV)
    tg = torch.zeros(n, device=DEV)
    td = t.to(DEV)
    for c0 in (chunk_v, 0):      # any chunk order
        _native.linear_ce_chunk_update(logits[:, c0:c0 + chunk_v].contiguous().to(DEV), td, c0, mx, sm, tg)
    loss = (mx + sm.log() - tg).cpu()
    want = torch.nn.functional.cross_entropy(logits.float(), t, reduction="none")
    torch.testing.assert_close(loss, want, rtol=1e-4, atol=1e-4)


def test_out_of_range_target_gives_zero_target_logit():
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    g = torch.Generator().manual_seed(5)
    h = torch.randn(130, 64, generator=g).to(torch.bfloat16)
    w = torch.randn(300, 64, generator=g).to(torch.bfloat16)
    t = torch.full((130,), 100000, dtype=torch.long)
    got = linear_cross_entropy(*to_dev(h, w, t), reduction="none").cpu()
    lse = torch.logsumexp(h.double() @ w.double().T, dim=1)
    torch.testing.assert_close(got.double(), lse, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("shards", [2, 8])
def test_vocab_sharded_stats_merge_equals_single_shot(shards):
    """Each shard owns whole 128-row vocabulary tiles; merging the per-shard
    (max, sumexp, target) statistics gives the single-shot loss."""
    from custom_cuda.kernels.linear_cross_entropy import (lce_loss_from_stats, lce_row_stats,
                                                          linear_cross_entropy)
    g = torch.Generator().manual_seed(11)
    n, hdim, v = 300, 256, 128256 // 16
    h = torch.randn(n, hdim, generator=g).to(torch.bfloat16).to(DEV)
    w = (0.05 * torch.randn(v, hdim, generator=g)).to(torch.bfloat16).to(DEV)
    t = torch.randint(0, v, (n,), generator=g)
    t[::7] = -100
    t = t.to(DEV)
    tiles = -(-v // 128)
    cuts = [min(v, (tiles * i // shards) * 128) for i in range(shards)] + [v]
    stats = torch.stack([lce_row_stats(h, w[a:b], t, a) for a, b in zip(cuts[:-1], cuts[1:])])
    merged = lce_loss_from_stats(stats, t, -100, "mean")
    single = linear_cross_entropy(h, w, t)
    torch.testing.assert_close(merged, single, rtol=1e-6, atol=1e-6)
    want = ops.linear_cross_entropy_fp64(h.cpu(), w.cpu(), t.cpu())
    torch.testing.assert_close(single.cpu().double(), want, rtol=1e-4, atol=1e-6)


def test_lce_config5_shapes_sampled_rows():
    """Benchmark config 5 at full H and V with 2048 of the 16384 rows (the CPU oracle
    needs ~1 GFLOP per row); fp32-upcast oracle, 1e-4 relative on the mean loss."""
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    h, w, t = workloads.lce_bf16(tokens=2048)
    got = linear_cross_entropy(*to_dev(h, w, t))
    want = ops.linear_cross_entropy_rowblocked(h, w, t, rows_per_block=256, wide=torch.float32)
    assert abs(got.item() - want.item()) / want.item() < 1e-4
    per_row = linear_cross_entropy(*to_dev(h, w, t), reduction="none").cpu()
    rows = torch.arange(0, 2048, 64)
    want_rows = ops.linear_cross_entropy_fp64(h[rows], w, t[rows], reduction="none")
    torch.testing.assert_close(per_row[rows].double(), want_rows, rtol=1e-4, atol=1e-5)
    assert device_status_clean(got)


def test_lce_config5_full_size_properties():
    """Benchmark config 5 at full size (16384 x 4096 x 128256, 5 % ignored): the mean equals the
    masked mean of the per-row losses, eight vocabulary shards merge to the single-shot result,
    and 64 sampled rows match the fp64 oracle to 1e-4."""
    from custom_cuda.kernels.linear_cross_entropy import (lce_loss_from_stats, lce_row_stats,
                                                          linear_cross_entropy)
    from custom_cuda_kernals_b200 import dist
    h, w, t = workloads.lce_bf16()
    hd, wd, td = to_dev(h, w, t)
    mean = linear_cross_entropy(hd, wd, td)
    rows = linear_cross_entropy(hd, wd, td, reduction="none")
    total = linear_cross_entropy(hd, wd, td, reduction="sum")
    keep = td != -100
    assert torch.all(rows[~keep] == 0)
    torch.testing.assert_close(total, rows.double().sum().float(), rtol=1e-5, atol=0)
    torch.testing.assert_close(mean, (rows.double().sum() / keep.sum()).float(), rtol=1e-5, atol=0)
    stats = torch.stack([lce_row_stats(hd, wd[a:b], td, a)
                         for a, b in (dist.vocab_range(w.shape[0], r, 8) for r in range(8))])
    torch.testing.assert_close(lce_loss_from_stats(stats, td, -100, "mean"), mean, rtol=1e-6, atol=0)
    pick = torch.arange(5, 16384, 256)
    want = ops.linear_cross_entropy_fp64(h[pick], w, t[pick], reduction="none")
    torch.testing.assert_close(rows[pick.to(DEV)].cpu().double(), want, rtol=1e-4, atol=1e-5)
    assert device_status_clean(mean)


def _grad_close(got, want, what):
    got, want = got.float().cpu(), want.float().cpu()
    scale = want.abs().max().item()
    err = (got - want).abs()
    assert err.max().item() <= 3e-2 * scale + 1e-9, (what, err.max().item(), scale)
    assert (err.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item() <= 1e-2, what


@pytest.mark.parametrize("shape", [(300, 256, 5000), (1000, 512, 9000), (130, 64, 264), (77, 64, 1000)])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("mode", ["chunks", "one_chunk", "recompute"])
def test_lce_gradients_match_autograd(shape, reduction, mode):
    """d_hidden and d_weight against torch autograd on fp32 copies of the same bf16 inputs:
    several row chunks (128 rows each, ragged last chunk), one chunk over all rows (a row count
    that is not a multiple of 8 among them), and the variant that recomputes the logits
    instead of storing them; 20 % ignored rows."""
    kw = {"chunks": dict(rows_per_chunk=128), "one_chunk": dict(rows_per_chunk=8192),
          "recompute": dict(rows_per_chunk=128, recompute=True)}[mode]
    from custom_cuda_kernals_b200.kernels.linear_cross_entropy import (linear_cross_entropy_fwd_bwd,
                                                                          linear_cross_entropy_trainable)
    n, hdim, v = shape
    g = torch.Generator().manual_seed(n + v)
    h = torch.randn(n, hdim, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(v, hdim, generator=g)).to(torch.bfloat16)
    t = torch.randint(0, v, (n,), generator=g)
    t[::5] = -100
    h32 = h.float().requires_grad_(True)
    w32 = w.float().requires_grad_(True)
    want = torch.nn.functional.cross_entropy(h32 @ w32.T, t, ignore_index=-100, reduction=reduction)
    want.backward()
    loss, dh, dw = linear_cross_entropy_fwd_bwd(*to_dev(h, w, t), reduction=reduction, **kw)
    torch.testing.assert_close(loss.cpu(), want.detach(), rtol=1e-4, atol=1e-5)
    _grad_close(dh, h32.grad, "d_hidden")
    _grad_close(dw, w32.grad, "d_weight")
    assert torch.all(dh[::5] == 0)                         # ignored rows get no gradient
    # the autograd wrapper hands the same gradients to .backward(), scaled by the upstream gradient
    hd = h.to(DEV).requires_grad_(True)
    wd = w.to(DEV).requires_grad_(True)
    out = linear_cross_entropy_trainable(hd, wd, t.to(DEV), reduction=reduction, rows_per_chunk=128)
    assert out.grad_fn is not None
    (2.0 * out).backward()
    _grad_close(hd.grad, 2.0 * h32.grad, "autograd d_hidden")
    _grad_close(wd.grad, 2.0 * w32.grad, "autograd d_weight")
    assert device_status_clean(out)


@pytest.mark.parametrize("ignore_index", [-100, 0, 5])
@pytest.mark.parametrize("recompute", [False, True])
def test_vocab_sharded_gradients_with_a_pad_id_inside_the_vocabulary(ignore_index, recompute):
    """Two vocabulary shards emulated as consecutive calls on one GPU (the shards do not wait on
    each other), against torch autograd.  With ``ignore_index`` 0 or 5 (a pad id) the shard that
    starts at column 384 holds real targets whose local index equals ``ignore_index``; they must
    get their gradient, and rows whose GLOBAL target is the pad id must get none."""
    from custom_cuda_kernals_b200.kernels import linear_cross_entropy as lce
    n, hdim, v, cut = 200, 128, 768, 384
    g = torch.Generator().manual_seed(11 + ignore_index)
    h = torch.randn(n, hdim, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(v, hdim, generator=g)).to(torch.bfloat16)
    t = torch.randint(0, v, (n,), generator=g)
    t[::6] = ignore_index
    t[1::9] = cut + ignore_index if ignore_index >= 0 else cut     # local index in shard 1 == ignore_index
    h32, w32 = h.float().requires_grad_(True), w.float().requires_grad_(True)
    want = torch.nn.functional.cross_entropy(h32 @ w32.T, t, ignore_index=ignore_index)
    want.backward()
    hd, wd, td_ = to_dev(h, w, t)
    shards = [(0, cut), (cut, v)]
    stats_all = torch.stack([lce.lce_row_stats(hd, wd[a:b].contiguous(), td_, a) for a, b in shards])
    scale = lce.lce_grad_scale(td_, ignore_index, "mean")
    dh, dws = torch.zeros(n, hdim, device=DEV), []
    for a, b in shards:
        _, dh_part, dw_part = lce.lce_stats_and_gradients(hd, wd[a:b].contiguous(), td_, scale, a, ignore_index,
                                                          gather=lambda st: stats_all, recompute=recompute)
        dh += dh_part.float()
        dws.append(dw_part)
    loss = lce.lce_loss_from_stats(stats_all, td_, ignore_index, "mean")
    torch.testing.assert_close(loss.cpu(), want.detach(), rtol=1e-4, atol=1e-5)
    _grad_close(dh, h32.grad, "d_hidden")
    _grad_close(torch.cat(dws), w32.grad, "d_weight")
    assert torch.all(dh[t == ignore_index] == 0) and torch.all(dh[1::9][t[1::9] != ignore_index].abs().sum(1) > 0)


@pytest.mark.parametrize("n,v", [(64, 64), (200, 1000), (77, 332), (1, 8), (513, 4100)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dlogits_from_logits_row_major_and_transposed(n, v, dtype):
    """The bandwidth pass alone: both layouts hold the same values, and they are the rounded
    (softmax - onehot) * scale of the stored logits; padding columns of the transpose stay
    untouched; ragged tiles in both directions."""
    from custom_cuda_kernals_b200 import _native
    g = torch.Generator().manual_seed(n * 7 + v)
    logits = 3.0 * torch.randn(n, v, generator=g)
    t = torch.randint(0, v, (n,), generator=g)
    t[::4] = -100
    if n > 2:
        t[2] = -1                                            # matches no column, row still counted
    lse = torch.logsumexp(logits, dim=1)
    width = (n + 7) // 8 * 8
    dl = torch.empty(n, v, dtype=dtype, device=DEV)
    dl_t = torch.full((v, width), 7.0, dtype=dtype, device=DEV)
    _native.lce_dlogits_from_logits(logits.to(DEV), t.to(DEV), lse.to(DEV), -100, 0.25, dl, dl_t)
    want = torch.exp(logits - lse[:, None])
    hit = t >= 0
    want[hit.nonzero().squeeze(1), t[hit]] -= 1.0
    want = want * 0.25 * (t != -100)[:, None]
    torch.testing.assert_close(dl.float().cpu(), want, rtol=2 ** -8 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-6)
    assert torch.equal(dl_t[:, :n].cpu(), dl.t().cpu())
    assert torch.all(dl_t[:, n:] == 7.0)


@pytest.mark.parametrize("rows,cols,width", [(64, 128, 64), (77, 332, 80), (1, 4, 4), (1000, 4096, 1000), (130, 260, 136)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_transpose_2byte_is_exact_and_zero_pads(rows, cols, width, dtype):
    from custom_cuda_kernals_b200 import _native
    x = torch.randn(rows, cols, generator=torch.Generator().manual_seed(rows + cols)).to(dtype).to(DEV)
    out = torch.full((cols, width), 3.0, dtype=dtype, device=DEV)
    _native.transpose_2byte(x, out)
    assert torch.equal(out[:, :rows], x.t())
    assert torch.all(out[:, rows:] == 0)
