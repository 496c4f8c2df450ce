"""CPU: the multi-rank host logic - partition arithmetic, and the vocabulary-parallel
statistics exchange run as two gloo ranks (no GPU involved; the per-rank statistics
come from the oracle, the collective and the merge contract are what is tested)."""

import os
import socket

import pytest
import torch
import torch.distributed as td
import torch.multiprocessing as mp

from custom_cuda_kernals_b200 import dist
from oracle import cases, ops


def test_ranges_cover_and_align():
    for total, world, mult in [(128256, 8, 128), (128256, 4, 128), (1009, 3, 128), (14336, 8, 8), (10, 4, 1), (3, 8, 1)]:
        spans = [dist._even_range(total, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans[:-1], spans[1:]):
            assert b == c and a <= b and a % mult == 0
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 2 * mult


def test_vocab_range_llama3_at_8_ranks():
    spans = [dist.vocab_range(128256, r, 8) for r in range(8)]
    tiles = [(b - a) // 128 for a, b in spans]
    assert sorted(set(tiles)) == [125, 126] and sum(tiles) == 1002


def test_column_and_sequence_ranges():
    assert [dist.column_range(14336, r, 8) for r in (0, 7)] == [(0, 1792), (12544, 14336)]
    assert [dist.sequence_range(8, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        dist.sequence_range(8, 0, 3)
    with pytest.raises(ValueError):
        dist.row_range(8, 4, 4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    r, w, _ = dist.init_from_env(timeout_s=60)
    assert (r, w) == (rank, world) and td.get_backend() == "gloo"
    case = cases.by_name(cases.LCE_CASES, "with_ignored_float32")
    h, wt, t = cases.lce_inputs(case)                       # replicated inputs, same seed on every rank
    v0, v1 = dist.vocab_range(case.vocab_size, rank, world)
    mx, sm, tg = ops.lce_partials(h, wt[v0:v1], t, v0)      # stand-in for the GPU kernel's row statistics
    stats = torch.stack([mx, sm, tg]).float()
    gathered = dist.gather_row_stats(stats)                 # the one collective
    assert gathered.shape == (world, 3, case.n_tokens)
    per_row = ops.lce_merge([(g[0].double(), g[1].double(), g[2].double()) for g in gathered])
    keep = t != -100
    loss = per_row[keep].sum() / keep.sum()
    slowest = dist.max_over_ranks(float(rank + 1))
    torch.save({"loss": loss, "slowest": slowest, "range": (v0, v1)}, os.path.join(out_dir, f"r{rank}.pt"))
    td.destroy_process_group()


def test_vocab_parallel_exchange_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    case = cases.by_name(cases.LCE_CASES, "with_ignored_float32")
    want = ops.linear_cross_entropy_fp64(*cases.lce_inputs(case))
    for o in outs:
        torch.testing.assert_close(o["loss"], want, rtol=1e-5, atol=1e-6)
        assert o["slowest"] == float(world)
    assert outs[0]["loss"] == outs[1]["loss"]               # every rank computes the identical loss
    assert outs[0]["range"][1] == outs[1]["range"][0]


def _grad_rank_main(rank, world, port, out_dir, scatter, ignore_index=-100):
    """The vocabulary-parallel gradient path on two gloo ranks.  The three GPU kernels it
    calls are replaced by fp32 torch stand-ins; the target localisation, the log-sum-exp
    merge, the gradient scale and both collectives are the library's own."""
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_from_env(timeout_s=60)
    from custom_cuda_kernals_b200.kernels import linear_cross_entropy as lce

    def loss_from_stats(stats, t, ignore_index=-100, reduction="mean"):
        per_row = ops.lce_merge([(g[0].double(), g[1].double(), g[2].double()) for g in stats])
        keep = t != ignore_index
        total = per_row[keep].sum()
        return (total / keep.sum() if reduction == "mean" else total).float()

    def stats_and_gradients(h, w, t, scale, v_start=0, ignore_index=-100, rows_per_chunk=8192, weight_t=None,
                            gather=None, recompute=False):
        stats = gather(torch.stack(ops.lce_partials(h, w, t, v_start)).float())
        lse = lce.lce_lse_from_stats(stats)
        # like the dlogits kernels: a row is ignored when its LOCAL target equals the marker the
        # library passes along with the local targets - nothing here looks at the global ids
        local, local_ignore = lce._local_targets(t, v_start, w.shape[0], ignore_index)
        keep = local != local_ignore
        dl = torch.exp(h.float() @ w.float().T - lse[:, None])
        hit = (local >= 0) & (local < w.shape[0]) & keep
        dl[hit.nonzero().squeeze(1), local[hit]] -= 1.0
        dl = dl * scale * keep[:, None]
        return stats, dl @ w.float(), dl.T @ h.float()

    lce.lce_loss_from_stats, lce.lce_stats_and_gradients = loss_from_stats, stats_and_gradients
    g = torch.Generator().manual_seed(5)
    n, hd, v = 64, 32, 384
    h = torch.randn(n, hd, generator=g)
    w = 0.2 * torch.randn(v, hd, generator=g)
    t = torch.randint(0, v, (n,), generator=g)
    t[::7] = ignore_index
    # a real target whose index WITHIN shard 1 equals ignore_index: must not be ignored there
    t[1] = dist.vocab_range(v, 1, world)[0] + ignore_index
    v0, v1 = dist.vocab_range(v, rank, world)
    loss, dh, dw = dist.vocab_parallel_linear_cross_entropy_fwd_bwd(h, w[v0:v1], t, v0, ignore_index=ignore_index,
                                                                    scatter_rows=scatter)
    torch.save({"loss": loss, "dh": dh, "dw": dw, "range": (v0, v1)}, os.path.join(out_dir, f"g{rank}.pt"))
    td.destroy_process_group()


@pytest.mark.parametrize("ignore_index", [-100, 0])
def test_vocab_parallel_gradients_two_gloo_ranks(tmp_path, ignore_index):
    """``ignore_index`` 0 is a pad id inside the vocabulary: the first column of shard 1 has local
    index 0 and is a real target there."""
    world = 2
    mp.spawn(_grad_rank_main, args=(world, _free_port(), str(tmp_path), False, ignore_index), nprocs=world, join=True)
    g = torch.Generator().manual_seed(5)
    n, hd, v = 64, 32, 384
    h = torch.randn(n, hd, generator=g).requires_grad_(True)
    w = (0.2 * torch.randn(v, hd, generator=g)).requires_grad_(True)
    t = torch.randint(0, v, (n,), generator=g)
    t[::7] = ignore_index
    t[1] = dist.vocab_range(v, 1, world)[0] + ignore_index
    want = torch.nn.functional.cross_entropy(h @ w.T, t, ignore_index=ignore_index)
    want.backward()
    outs = [torch.load(tmp_path / f"g{r}.pt") for r in range(world)]
    for o in outs:
        torch.testing.assert_close(o["loss"], want.detach(), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(o["dh"], h.grad, rtol=1e-4, atol=1e-6)       # all-reduced: whole d_hidden
        v0, v1 = o["range"]
        torch.testing.assert_close(o["dw"], w.grad[v0:v1], rtol=1e-4, atol=1e-6)  # own rows, no exchange


def _rank_that_loses_its_peer(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_from_env(timeout_s=10)
    if rank == 1:
        return                      # leaves between steps, with no collective in flight, and never joins the next one
    outcome = "completed"
    try:
        dist.gather_row_stats(torch.zeros(3, 16))
    except Exception as e:          # the survivor must get an error, not hang
        outcome = type(e).__name__
    with open(os.path.join(out_dir, "r0.txt"), "w") as f:
        f.write(outcome)


def test_a_rank_that_never_joins_surfaces_as_an_error_on_the_survivor(tmp_path):
    """Failure detection on the host: rank 1 exits before the statistics exchange; rank 0's
    all-gather ends with an exception within the process-group timeout instead of waiting forever."""
    mp.spawn(_rank_that_loses_its_peer, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "r0.txt").read_text() != "completed"


def test_local_targets_decide_ignored_on_global_ids():
    from custom_cuda_kernals_b200.kernels.linear_cross_entropy import _local_targets
    t = torch.tensor([0, 5, 128, 133, 300, 0])
    local, marker = _local_targets(t, 128, 128, 0)            # shard [128, 256), pad id 0
    assert marker == -1 and local.tolist() == [-1, -2, 0, 5, -2, -1]
    local, marker = _local_targets(t, 0, 128, 0)              # first shard: local ids are the global ids
    assert marker == 0 and local is t
    local, marker = _local_targets(torch.tensor([-100, 28, 200]), 128, 128, -100)
    assert marker == -1 and local.tolist() == [-1, -2, 72]


def _phase_rank(rank, world, port, out_dir, leaver):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_from_env(timeout_s=8)
    from custom_cuda_kernals_b200.ep import PhaseBarrier
    barrier = PhaseBarrier("cpu")
    outcome = "completed"
    try:
        barrier()                   # after "dispatch": every rank is there
        if rank == leaver:
            return                  # raises / leaves between the phases, nothing in flight
        barrier()                   # after "expert outputs": the leaver never arrives
    except Exception as e:
        outcome = type(e).__name__
    with open(os.path.join(out_dir, f"phase{rank}.txt"), "w") as f:
        f.write(f"{outcome} {barrier.passed}")


def test_phase_barrier_completes_and_surfaces_a_rank_that_left_between_phases(tmp_path):
    """The expert-parallel exchange separates its phases with PhaseBarrier.  Two healthy ranks
    pass both barriers; when one rank leaves after the first phase, the survivor's second barrier
    ends with an exception inside the process-group timeout - it does not wait forever."""
    mp.spawn(_phase_rank, args=(2, _free_port(), str(tmp_path), -1), nprocs=2, join=True)
    assert [(tmp_path / f"phase{r}.txt").read_text() for r in range(2)] == ["completed 2", "completed 2"]
    mp.spawn(_phase_rank, args=(2, _free_port(), str(tmp_path), 1), nprocs=2, join=True)
    outcome, passed = (tmp_path / "phase0.txt").read_text().split()
    assert outcome != "completed" and passed == "1"


def test_single_process_needs_no_group():
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    assert dist.init_from_env() == (0, 1, 0)
    s = torch.zeros(3, 5)
    assert dist.gather_row_stats(s).shape == (1, 3, 5)
    assert dist.max_over_ranks(3.5) == 3.5


def test_host_pipeline_groups_cover_the_batch_with_single_sequence_ends():
    from custom_cuda_kernals_b200.llama_block import host_pipeline_groups
    for batch in range(0, 20):
        groups = host_pipeline_groups(batch)
        assert [g for g in groups if g[1] <= g[0]] == []
        assert sum(b1 - b0 for b0, b1 in groups) == batch
        assert all(a[1] == b[0] for a, b in zip(groups[:-1], groups[1:]))
        if batch >= 4:      # only the first copy-in and the last copy-out are exposed: keep them small
            assert groups[0] == (0, 1) and groups[-1] == (batch - 1, batch)
            sizes = [b1 - b0 for b0, b1 in groups]
            # a copy-in hides behind the previous group's compute, a copy-out behind the next group's
            assert all(b <= 2 * a for a, b in zip(sizes[:-1], sizes[1:]))
            assert all(a <= 2 * b for a, b in zip(sizes[:-1], sizes[1:]))
    assert [b1 - b0 for b0, b1 in host_pipeline_groups(8)] == [1, 2, 2, 2, 1]
    assert [b1 - b0 for b0, b1 in host_pipeline_groups(7)] == [1, 2, 2, 1, 1]
    assert [b1 - b0 for b0, b1 in host_pipeline_groups(4)] == [1, 2, 1]
    assert host_pipeline_groups(8, 4) == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert host_pipeline_groups(3, 8) == [(0, 1), (1, 2), (2, 3)]


def test_host_pipeline_items_cut_single_sequence_ends_into_position_pieces():
    from custom_cuda_kernals_b200.llama_block import host_pipeline_items
    for batch in range(0, 12):
        for seq in (1, 300, 1024, 2048, 4096):
            for pieces in (None, 1, 2, 4):
                items = host_pipeline_items(batch, seq, seq_pieces=pieces)
                covered = torch.zeros(batch, seq, dtype=torch.int32)
                for b0, b1, s0, s1 in items:
                    assert b1 > b0 and s1 > s0
                    if (s0, s1) != (0, seq):
                        assert b1 - b0 == 1                      # only single sequences are cut
                    covered[b0:b1, s0:s1] += 1
                assert torch.all(covered == 1)                   # every token exactly once
                order = [(b0, s0) for b0, _, s0, _ in items]
                assert order == sorted(order)                    # pieces of a sequence in position order
    # default: one sequence per call is cut in two, everything else stays whole
    assert host_pipeline_items(1, 2048) == [(0, 1, 0, 1024), (0, 1, 1024, 2048)]
    assert host_pipeline_items(1, 512) == [(0, 1, 0, 512)]
    assert host_pipeline_items(2, 2048) == [(0, 1, 0, 2048), (1, 2, 0, 2048)]
    assert host_pipeline_items(8, 2048) == [(0, 1, 0, 2048), (1, 3, 0, 2048), (3, 5, 0, 2048), (5, 7, 0, 2048), (7, 8, 0, 2048)]
    assert host_pipeline_items(1, 2048, seq_pieces=4) == [(0, 1, 0, 512), (0, 1, 512, 1024), (0, 1, 1024, 1536), (0, 1, 1536, 2048)]
    assert [i for i in host_pipeline_items(8, 2048, seq_pieces=4) if i[3] - i[2] == 2048] == [(1, 3, 0, 2048), (3, 5, 0, 2048), (5, 7, 0, 2048)]
    assert host_pipeline_items(8, 2048, chunks=4) == [(0, 2, 0, 2048), (2, 4, 0, 2048), (4, 6, 0, 2048), (6, 8, 0, 2048)]
