"""Expert-parallel token exchange: the planning arithmetic on CPU for several emulated ranks, the
kernels on one GPU with the ranks' buffers side by side (the kernels never wait on one another,
so the ranks can run one after the other), and the real thing on two GPUs."""

import os
import socket

import pytest
import torch

from custom_cuda_kernals_b200 import ep


def _setup(world, experts, t, k, hidden, seed, device="cpu", dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(t + r, hidden, generator=g).to(dtype).to(device) for r in range(world)]      # ragged token counts
    idx = [torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(t + r)]).to(device) for r in range(world)]
    w = [torch.rand(t + r, k, generator=g).to(device) for r in range(world)]
    counts = torch.stack([torch.bincount(i.reshape(-1).cpu(), minlength=experts) for i in idx]).to(device)
    return xs, idx, w, counts


def _expert(rows, expert_ids):
    return (rows.float() * (0.25 + 0.125 * expert_ids.float())[:, None]).to(rows.dtype)


def _expected(x, idx, w):
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for j in range(idx.shape[1]):
        acc += w[:, j:j + 1] * _expert(x, idx[:, j]).float()
    return acc


@pytest.mark.parametrize("world,experts,k", [(1, 4, 2), (2, 8, 2), (4, 8, 3), (8, 16, 1)])
def test_plans_fill_every_receive_buffer_exactly_and_in_order(world, experts, k):
    epr = experts // world
    xs, idx, w, counts = _setup(world, experts, 17, k, 8, seed=world * 10 + k)
    cap = int(counts.reshape(world, world, epr).sum(-1).sum(0).max())
    recv = [torch.full((cap, 8), float("nan")) for _ in range(world)]
    tag = [torch.full((cap, 3), -1, dtype=torch.long) for _ in range(world)]          # (source, expert, token)
    plans = [ep.plan_dispatch(idx[r], counts, r, epr) for r in range(world)]
    for r, p in enumerate(plans):
        experts_sorted = idx[r].reshape(-1)[torch.argsort(idx[r].reshape(-1), stable=True)]
        for i in range(p.src_row.numel()):
            d, row = int(p.dst_rank[i]), int(p.dst_row[i])
            assert tag[d][row, 0] == -1, "two rows sent to one slot"
            recv[d][row] = xs[r][p.src_row[i]]
            tag[d][row] = torch.tensor([r, int(experts_sorted[i]), int(p.src_row[i])])
    outs = []
    for r in range(world):
        n_rows, expert_of_row = ep.plan_receive(counts, r, epr)
        assert (tag[r][:n_rows, 0] >= 0).all() and (tag[r][n_rows:, 0] == -1).all()   # dense, nothing beyond
        assert torch.equal(tag[r][:n_rows, 1], expert_of_row)                          # the ids the receiver derives
        keys = tag[r][:n_rows, 0] * 10 ** 6 + tag[r][:n_rows, 1] * 10 ** 3
        assert (keys.diff() >= 0).all()                                                # source-major, expert-minor
        assert torch.div(expert_of_row, epr, rounding_mode="floor").eq(r).all()
        outs.append(_expert(recv[r][:n_rows], expert_of_row))
        # the way back: every received row returns to its source rank, into the slot it was sent from
        home, slot = ep.plan_return(counts, r, epr)
        assert torch.equal(home, tag[r][:n_rows, 0])
        for i in range(n_rows):
            p = plans[int(home[i])]
            assert int(p.dst_rank[slot[i]]) == r and int(p.dst_row[slot[i]]) == i
    for r, p in enumerate(plans):
        got = torch.zeros_like(xs[r])
        for j in range(k):
            slot = p.slot_of[:, j]
            rows = torch.stack([outs[int(p.dst_rank[s])][int(p.dst_row[s])] for s in slot])
            got += w[r][:, j:j + 1] * rows
        torch.testing.assert_close(got, _expected(xs[r], idx[r], w[r]), rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("world,experts,k,hidden,dtype", [(4, 8, 2, 256, torch.bfloat16), (8, 32, 4, 1024, torch.bfloat16),
                                                          (2, 4, 1, 64, torch.float32), (3, 6, 2, 4096, torch.float16)])
def test_kernels_with_the_ranks_side_by_side_on_one_gpu(world, experts, k, hidden, dtype):
    from custom_cuda_kernals_b200 import _native
    dev = torch.device("cuda", 0)
    epr = experts // world
    xs, idx, w, counts = _setup(world, experts, 200, k, hidden, seed=world + hidden, device=dev, dtype=dtype)
    cap = int(counts.reshape(world, world, epr).sum(-1).sum(0).max()) + 5
    recv = [torch.full((cap, hidden), 7.0, dtype=dtype, device=dev) for _ in range(world)]
    out = [torch.zeros(cap, hidden, dtype=dtype, device=dev) for _ in range(world)]
    recv_bases = torch.tensor([b.data_ptr() for b in recv], dtype=torch.int64, device=dev)
    out_bases = torch.tensor([b.data_ptr() for b in out], dtype=torch.int64, device=dev)
    plans = [ep.plan_dispatch(idx[r], counts, r, epr) for r in range(world)]
    for r, p in enumerate(plans):
        _native.token_dispatch_fwd(xs[r], p.src_row, p.dst_rank, p.dst_row, recv_bases, cap)
    for r in range(world):
        n_rows, expert_of_row = ep.plan_receive(counts, r, epr)
        assert torch.all(recv[r][n_rows:] == 7.0)                                       # nothing written past the plan
        out[r][:n_rows] = _expert(recv[r][:n_rows], expert_of_row)
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    for r, p in enumerate(plans):
        combined = torch.empty(xs[r].shape[0], hidden, dtype=dtype, device=dev)
        _native.token_combine_remote_fwd(out_bases, cap, p.dst_rank[p.slot_of].contiguous(), p.dst_row[p.slot_of].contiguous(),
                                         w[r], combined)
        torch.testing.assert_close(combined.float(), _expected(xs[r], idx[r], w[r]), rtol=tol, atol=tol)
    assert _native.take_device_status(xs[0]) == 0
    # a route outside the table or the buffers is skipped and reported, not followed
    bad_rank = plans[0].dst_rank.clone()
    bad_rank[0] = world
    bad_row = plans[0].dst_row.clone()
    bad_row[1] = cap
    _native.token_dispatch_fwd(xs[0], plans[0].src_row, bad_rank, bad_row, recv_bases, cap)
    torch.cuda.synchronize()
    assert _native.take_device_status(xs[0]) & 4
    assert _native.take_device_status(xs[0]) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("world,experts,k,tokens", [(1, 4, 2, 50), (2, 8, 2, 1000), (4, 8, 3, 700), (8, 256, 8, 513),
                                                    (8, 64, 6, 4096), (3, 6, 1, 1), (32, 256, 2, 300)])
def test_planning_kernel_equals_the_index_arithmetic(world, experts, k, tokens):
    """One launch gives exactly the routes of plan_dispatch (a stable sort by expert) for every
    emulated rank: 1024-pair chunks that end mid-way, 256 experts, one thread per expert."""
    from custom_cuda_kernals_b200 import _native
    dev = torch.device("cuda", 0)
    epr = experts // world
    _, idx, _, counts = _setup(world, experts, tokens, k, 8, seed=world + experts + tokens, device=dev)
    per_rank = counts.reshape(world, world, epr).sum(-1)
    for r in range(world):
        want = ep.plan_dispatch(idx[r], counts, r, epr)
        src_row, dst_rank, dst_row, pull_rank, pull_row, meta = ep.plan_on_device(idx[r], counts, r)
        assert torch.equal(src_row, want.src_row) and torch.equal(dst_rank, want.dst_rank) and torch.equal(dst_row, want.dst_row)
        assert torch.equal(pull_rank, want.dst_rank[want.slot_of]) and torch.equal(pull_row, want.dst_row[want.slot_of])
        assert meta.tolist() == [int(per_rank[:, r].sum()), int(per_rank.sum(0).max())]
    assert _native.take_device_status(counts) == 0
    bad = idx[0].clone()
    bad[0, 0] = experts                                          # an expert id that does not exist
    out = ep.plan_on_device(bad, counts, 0)
    torch.cuda.synchronize()
    assert _native.take_device_status(counts) & 4 and out[3][0, 0] == -1 and out[4][0, 0] == -1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_rank(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as td
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    td.init_process_group("nccl", device_id=dev)
    from custom_cuda_kernals_b200 import _native
    experts, k, hidden, t = 8, 2, 1024, 300
    xs, idx, w, counts = _setup(world, experts, t, k, hidden, seed=5, device="cpu", dtype=torch.bfloat16)
    x, i, wt = xs[rank].to(dev), idx[rank].to(dev), w[rank].to(dev)
    cap = 2 * world * (t + world) * k // world + 64
    layer = ep.ExpertParallel(experts, hidden, capacity_rows=cap, device=dev)
    got = layer.forward(x, wt, i, _expert)
    again = layer.forward(x, wt, i, _expert)                    # buffers are reusable call after call
    pushed = ep.ExpertParallel(experts, hidden, capacity_rows=cap, max_local_rows=(t + world) * k, device=dev,
                               return_mode="push").forward(x, wt, i, _expert)
    torch.cuda.synchronize()
    ok = bool(torch.allclose(got.float(), _expected(x, i, wt), rtol=1.6e-2, atol=1.6e-2) and torch.equal(got, again)
              and torch.equal(got, pushed) and _native.take_device_status(x) == 0)
    try:
        tiny = ep.ExpertParallel(experts, hidden, capacity_rows=8, device=dev)
        tiny.forward(x, wt, i, _expert)
        refused = False
    except ValueError:
        refused = True                                          # every rank refuses before anything is sent
    torch.save({"ok": ok, "refused": refused}, os.path.join(out_dir, f"ep{rank}.pt"))
    td.barrier()
    td.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_two_ranks_exchange_rows_over_peer_memory(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_ep_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"ep{r}.pt")
        assert res["ok"] and res["refused"]


def test_plans_are_a_bijection_onto_dense_buffers_for_random_routings():
    """Property check over random (world, experts per rank, k, tokens): every (source, slot) maps
    to a distinct (rank, row), the rows of a rank are exactly 0..n_rows-1, the receiver's expert
    ids match what was sent, and plan_return inverts plan_dispatch."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=40, deadline=None)
    @given(st.integers(1, 8), st.integers(1, 5), st.integers(1, 4), st.integers(0, 60), st.integers(0, 10 ** 6))
    def check(world, epr, k, tokens, seed):
        experts = world * epr
        k = min(k, experts)
        g = torch.Generator().manual_seed(seed)
        idx = [torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens + r % 3)]).reshape(-1, k)
               if tokens + r % 3 else torch.empty(0, k, dtype=torch.long) for r in range(world)]
        counts = torch.stack([torch.bincount(i.reshape(-1), minlength=experts) for i in idx])
        plans = [ep.plan_dispatch(idx[r], counts, r, epr) for r in range(world)]
        for d in range(world):
            n_rows, expert_of_row = ep.plan_receive(counts, d, epr)
            rows, sent_experts, sources, slots = [], [], [], []
            for r, p in enumerate(plans):
                mask = p.dst_rank == d
                rows.append(p.dst_row[mask])
                sent_experts.append(idx[r].reshape(-1)[torch.argsort(idx[r].reshape(-1), stable=True)][mask])
                sources.append(torch.full((int(mask.sum()),), r))
                slots.append(mask.nonzero().squeeze(1))
            rows, sent_experts = torch.cat(rows), torch.cat(sent_experts)
            assert rows.numel() == n_rows and torch.equal(torch.sort(rows)[0], torch.arange(n_rows))
            assert torch.equal(expert_of_row[rows], sent_experts)
            home, slot = ep.plan_return(counts, d, epr)
            assert torch.equal(home[rows], torch.cat(sources)) and torch.equal(slot[rows], torch.cat(slots))

    check()


def test_forward_refuses_rows_that_do_not_match_the_exchange_buffers():
    """The exchange kernels take the row pitch from the tensor they are handed while capacity is
    counted in buffer rows, so a wider, differently typed or strided ``x`` (or expert output) must
    be refused on the host before any row is sent.  Checked on a layer object without buffers:
    the checks run before anything touches them."""
    layer = object.__new__(ep.ExpertParallel)
    layer.hidden, layer.dtype, layer.device = 64, torch.bfloat16, torch.device("cpu")
    layer.return_mode, layer.max_local = "pull", 0
    idx = torch.zeros(10, 2, dtype=torch.long)
    w = torch.rand(10, 2)
    good = torch.zeros(10, 64, dtype=torch.bfloat16)
    for bad, what in [(torch.zeros(10, 128, dtype=torch.bfloat16), r"must be \[10, 64\]"),
                      (torch.zeros(9, 64, dtype=torch.bfloat16), r"must be \[10, 64\]"),
                      (torch.zeros(10, 64, dtype=torch.float16), "exchange buffers are"),
                      (torch.zeros(10, 128, dtype=torch.bfloat16)[:, ::2], "contiguous"),
                      (torch.zeros(640, dtype=torch.bfloat16), r"must be \[10, 64\]")]:
        with pytest.raises(ValueError, match=what):
            layer.forward(bad, w, idx, _expert)
    with pytest.raises(ValueError, match="topk_weights shape"):
        layer.forward(good, torch.rand(10, 3), idx, _expert)
    with pytest.raises(ValueError, match=r"topk_indices must be \[T, k\]"):
        layer.forward(good, w, idx.reshape(-1), _expert)
    with pytest.raises(ValueError, match="expert_fn's output"):
        layer._check_rows("expert_fn's output", torch.zeros(7, 32, dtype=torch.bfloat16), 7, contiguous=False)
