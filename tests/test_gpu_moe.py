"""GPU: the mixture-of-experts neighbours (router, token gather, weighted combine) against
the CPU oracle on the reference's own case tables and the committed golden vectors
(reference tests: tests/test_moe_router_kernel.py, tests/test_token_permute_kernel.py)."""

import pathlib

import pytest
import torch

from custom_cuda_kernals_b200.kernels.moe_router import moe_router
from custom_cuda_kernals_b200.kernels.token_permute import compute_permutation, token_combine, token_gather
from oracle import cases, ops
from tests.gpu_util import DEV, check, to_dev

pytestmark = pytest.mark.gpu
golden = torch.load(pathlib.Path(__file__).parent / "golden" / "golden_small.pt")

ROUTER_TOL = {torch.float32: (1e-4, 1e-4, 0.0), torch.float16: (1e-2, 1e-2, 0.0), torch.bfloat16: (1e-2, 2e-2, 1e-5)}


def _same_selection(logits, got_idx, want_idx, k):
    """Expert sets equal per token, except where the k-th and (k+1)-th logits tie exactly -
    there any of the tied experts is a correct choice (torch.topk leaves the order of equal
    values unspecified)."""
    got, want = torch.sort(got_idx, dim=-1)[0], torch.sort(want_idx, dim=-1)[0]
    rows = (got != want).any(dim=-1).nonzero().squeeze(1)
    for r in rows.tolist():
        lg = logits[r].float()
        kth = torch.sort(lg, descending=True)[0][k - 1]
        only_got = set(got[r].tolist()) - set(want[r].tolist())
        only_want = set(want[r].tolist()) - set(got[r].tolist())
        assert all(lg[e] == kth for e in only_got | only_want), (r, only_got, only_want)
    assert torch.all((got_idx >= 0) & (got_idx < logits.shape[1]))
    assert all(len(set(row)) == k for row in got_idx.tolist()[:64])          # no expert twice


@pytest.mark.parametrize("case", cases.ROUTER_CASES, ids=lambda c: c.name)
def test_router_matches_oracle(case):
    logits = cases.router_inputs(case)
    want_w, want_i = ops.moe_router(logits, case.k, case.renormalize)
    got_w, got_i = moe_router(logits.to(DEV), case.k, case.renormalize)
    assert got_w.shape == (case.n_tokens, case.k) and got_w.dtype == torch.float32
    assert got_i.shape == (case.n_tokens, case.k) and got_i.dtype == torch.int64
    if case.n_tokens == 0:
        return
    check(got_w.cpu(), want_w, case.dtype, ROUTER_TOL)
    _same_selection(logits, got_i.cpu(), want_i, case.k)
    if case.dtype == torch.float32:                       # no ties to speak of: positions match too
        assert (got_i.cpu() == want_i).float().mean() > 0.9999
    # descending weights, and with renormalisation they sum to one
    assert torch.all(got_w[:, :-1] >= got_w[:, 1:])
    if case.renormalize:
        torch.testing.assert_close(got_w.sum(-1).cpu(), torch.ones(case.n_tokens), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("router/")])
def test_router_golden(key):
    case = cases.by_name(cases.ROUTER_CASES, key.split("/")[1])
    logits = cases.router_inputs(case)
    got_w, got_i = moe_router(logits.to(DEV), case.k, case.renormalize)
    check(got_w.cpu(), golden[key]["weights"], case.dtype, ROUTER_TOL)
    _same_selection(logits, got_i.cpu(), golden[key]["indices"], case.k)


def test_router_ties_go_to_the_lower_expert():
    logits = torch.zeros(3, 12, device=DEV)
    logits[1, 7] = 1.0
    w, i = moe_router(logits, 3, renormalize=False)
    assert i[0].tolist() == [0, 1, 2] and i[1].tolist() == [7, 0, 1]
    torch.testing.assert_close(w[0], torch.full((3,), 1 / 12, device=DEV))


def test_router_rejects_what_the_reference_rejects():
    with pytest.raises(ValueError):
        moe_router(torch.randn(4, 8), k=2)                                   # CPU tensor
    with pytest.raises(RuntimeError):
        moe_router(torch.randn(4, 8, device=DEV), k=16)                      # k > experts, as torch.topk
    with pytest.raises(ValueError):
        moe_router(torch.randn(4, 300, device=DEV), k=2)                     # more than 256 experts
    with pytest.raises(ValueError):
        moe_router(torch.randn(4, 8, device=DEV).t(), k=2)                   # not contiguous


@pytest.mark.parametrize("case", cases.GATHER_CASES, ids=lambda c: c.name)
def test_gather_is_exact(case):
    src, idx = cases.gather_inputs(case)
    got = token_gather(*to_dev(src, idx))
    assert got.shape == (case.n_dst_rows, case.hidden_dim) and got.dtype == case.dtype
    assert torch.equal(got.cpu(), ops.token_gather(src, idx))


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("gather/")])
def test_gather_golden(key):
    case = cases.by_name(cases.GATHER_CASES, key.split("/")[1])
    assert torch.equal(token_gather(*to_dev(*cases.gather_inputs(case))).cpu(), golden[key]["dst"])


def test_gather_unaligned_view_takes_the_scalar_path():
    base = torch.randn(65 * 24 + 1, device=DEV, dtype=torch.bfloat16)
    src = base[1:].view(65, 24)                                             # 2-byte aligned only
    idx = torch.randint(0, 65, (200,), device=DEV)
    assert torch.equal(token_gather(src, idx), src.index_select(0, idx))


@pytest.mark.parametrize("case", cases.COMBINE_CASES, ids=lambda c: c.name)
def test_combine_matches_oracle(case):
    eo, idx, w = cases.combine_inputs(case)
    got = token_combine(*to_dev(eo, idx, w))
    assert got.shape == (case.n_tokens, case.hidden_dim) and got.dtype == case.dtype
    if case.n_tokens:
        check(got.cpu(), ops.token_combine(eo, idx, w), case.dtype, ROUTER_TOL)
        # one rounding of the fp32 sum: within half an ulp-ish of the fp64 result
        wide = ops.token_combine(eo, idx, w, wide=True)
        ulp = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[case.dtype]
        assert ((got.cpu().double() - wide).abs() <= ulp * wide.abs() + 1e-6).all()


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("combine/") and "permutation" not in k])
def test_combine_golden(key):
    case = cases.by_name(cases.COMBINE_CASES, key.split("/")[1])
    got = token_combine(*to_dev(*cases.combine_inputs(case)))
    check(got.cpu(), golden[key]["combined"], case.dtype, ROUTER_TOL)


def test_dispatch_round_trip_full_size():
    """Router -> permutation -> gather -> identity experts -> combine at a Mixtral-sized
    layer: with renormalised weights the combine returns the input rows (up to one rounding of
    a sum of k scaled copies)."""
    t, e, k, h = 8192, 8, 2, 4096
    g = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(t, h, device=DEV, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, device=DEV, generator=g).to(torch.bfloat16)
    w, idx = moe_router(logits, k)
    perm, unperm = compute_permutation(idx)
    g0 = golden["combine/compute_permutation"]
    p0, u0 = compute_permutation(g0["topk"].to(DEV))
    assert torch.equal(p0.cpu(), g0["permute_index"]) and torch.equal(u0.cpu(), g0["unpermute_index"])
    rows = token_gather(x, perm)
    experts_sorted = idx.reshape(-1)[torch.argsort(idx.reshape(-1), stable=True)]
    assert torch.all(experts_sorted.diff() >= 0)
    assert torch.equal(rows, x[perm])
    back = token_combine(rows, unperm, w)
    torch.testing.assert_close(back.float(), x.float(), rtol=2 ** -7, atol=1e-6)


def test_gather_and_combine_reject_what_the_reference_rejects():
    src = torch.randn(8, 16, device=DEV)
    idx = torch.zeros(4, dtype=torch.long, device=DEV)
    with pytest.raises(ValueError):
        token_gather(torch.randn(8, 16), torch.zeros(4, dtype=torch.long))       # CPU tensors
    with pytest.raises(ValueError):
        token_gather(src, idx.int())                                              # indices not int64
    with pytest.raises(ValueError):
        token_gather(src.t(), idx)                                                # not contiguous
    rows = torch.randn(8, 16, device=DEV, dtype=torch.bfloat16)
    u = torch.arange(8, device=DEV).reshape(4, 2)
    with pytest.raises(ValueError):
        token_combine(rows, u, torch.rand(4, 2, device=DEV, dtype=torch.bfloat16))   # weights must be float32
    with pytest.raises(ValueError):
        token_combine(rows, u, torch.rand(4, 3, device=DEV))                      # weights shape
    from custom_cuda_kernals_b200 import _native
    with pytest.raises(ValueError):
        _native.token_combine_fwd(rows, u, torch.rand(4, 2, device=DEV), torch.empty(4, 16, device=DEV))  # dtype mismatch


@pytest.mark.parametrize("hidden", [8, 24, 100, 257, 4096 + 8])
def test_combine_vector_tail_and_scalar_fallback(hidden):
    """Row widths around the vector width: whole vectors, ragged (scalar path), and a slab that
    is only partly filled (reference: test_combine_vectorization_tail_and_fallback_path)."""
    g = torch.Generator().manual_seed(hidden)
    rows = torch.randn(60, hidden, generator=g).to(torch.bfloat16)
    u = torch.randperm(60, generator=g).reshape(20, 3)
    w = torch.rand(20, 3, generator=g)
    got = token_combine(*to_dev(rows, u, w))
    check(got.cpu(), ops.token_combine(rows, u, w), torch.bfloat16, ROUTER_TOL)
    assert torch.equal(token_gather(rows.to(DEV), u.reshape(-1).to(DEV)).cpu(), rows[u.reshape(-1)])
