"""Expert-parallel token exchange: the all-to-all around the expert FFNs of a mixture-of-experts
layer, done by the row movers themselves over peer memory.

The reference stops at one GPU (its token_permute kernels gather and combine rows locally:
csrc/kernels/token_permute.cu, baselines/token_permute.py:58-72).  With the experts spread over
the ranks of one NVLink/NVSwitch box, the same two steps become the dispatch and combine
all-to-all - and instead of packing rows, calling a collective and unpacking, the dispatch kernel
writes each token row straight into the owning rank's receive buffer (peer memory), and after the
experts ran, the combine kernel reads each token's k output rows straight out of the ranks that
produced them, weighting and summing as it goes ("pull", the default: one pass, 0.56 ms of
device time per layer call at 8 GPUs for 8192 tokens x top-2 x 4096 bf16 per rank).  The other
way back ("push": the dispatch kernel writes every output row into its token's home rank, then
the local combine runs) is there for comparison; it measured slower (0.72 ms).  The kernels only
push or pull and never wait on another GPU; the phases are separated by ``PhaseBarrier``, a
stream-ordered one-element all-reduce of the process group, so a peer that left or raised between
two phases surfaces on the others as an exception within the group's timeout instead of a GPU
spinning on a flag.  The only other communication is one all-gather of per-expert counts (world x
experts ints).

Receive layout on rank r: blocks in source-rank order; inside a block the rows are sorted by
expert (ascending) and inside an expert keep the sender's token order - so every sender can
compute where its rows land from the count matrix alone.

``plan_dispatch`` / ``plan_receive`` / ``plan_return`` are pure index arithmetic (any device,
testable without a GPU); ``plan_on_device`` gets the same routes from one kernel launch;
``ExpertParallel`` owns the symmetric buffers and runs the phases.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _native

__all__ = ["DispatchPlan", "plan_dispatch", "plan_receive", "plan_return", "plan_on_device", "PhaseBarrier",
           "ExpertParallel"]


class PhaseBarrier:
    """Separates two phases of the exchange on the current stream: a one-element all-reduce of the
    process group.  When it completes on a rank, every rank's kernels launched before its own call
    have finished (their peer-memory stores are visible: a kernel's writes are released at its
    end, and the collective cannot finish without every rank's contribution, which each rank
    sends only after its earlier work on the stream).  Unlike a spin on a peer's flag it is
    covered by the process group's timeout and watchdog: a rank that never arrives turns into an
    exception (or an aborted communicator) on the others, not a kernel that waits forever.
    Works on any backend (NCCL on GPUs, gloo on CPU for the tests)."""

    def __init__(self, device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.passed = 0

    def __call__(self) -> None:
        dist.all_reduce(self.token, group=self.group)
        self.passed += 1


@dataclass
class DispatchPlan:
    src_row: torch.Tensor        # [T*k] source token of every slot of the expert-sorted order
    dst_rank: torch.Tensor       # [T*k] rank that owns the slot's expert
    dst_row: torch.Tensor        # [T*k] row in that rank's receive buffer
    slot_of: torch.Tensor        # [T, k] slot of every (token, choice): where its output row comes back to


def plan_dispatch(topk_indices: torch.Tensor, counts: torch.Tensor, rank: int, experts_per_rank: int) -> DispatchPlan:
    """Where this rank's rows go.  ``topk_indices``: ``[T, k]`` expert ids of the local tokens;
    ``counts``: ``[world, experts]``, ``counts[s, e]`` = number of (token, choice) pairs of rank
    ``s`` routed to expert ``e`` (the all-gathered bincounts)."""
    t, k = topk_indices.shape
    world = counts.shape[0]
    flat = topk_indices.reshape(-1)
    order = torch.argsort(flat, stable=True)
    experts_sorted = flat[order]
    dst_rank = torch.div(experts_sorted, experts_per_rank, rounding_mode="floor")
    per_rank = counts.reshape(world, world, experts_per_rank).sum(-1)           # [source, destination]
    seg_start = per_rank[:rank].sum(0)                                          # rows of lower sources, per destination
    first = torch.cumsum(per_rank[rank], 0) - per_rank[rank]                    # start of each destination in my sorted order
    slots = torch.arange(t * k, device=flat.device)
    dst_row = seg_start[dst_rank] + (slots - first[dst_rank])
    slot_of = torch.empty_like(order)
    slot_of[order] = slots
    return DispatchPlan(torch.div(order, k, rounding_mode="floor"), dst_rank, dst_row, slot_of.reshape(t, k))


def plan_receive(counts: torch.Tensor, rank: int, experts_per_rank: int) -> tuple[int, torch.Tensor]:
    """What arrives at ``rank``: the number of rows and the expert id of every row, in buffer order."""
    mine = counts[:, rank * experts_per_rank:(rank + 1) * experts_per_rank]     # [source, my experts]
    ids = torch.arange(rank * experts_per_rank, (rank + 1) * experts_per_rank, device=counts.device)
    expert_of_row = torch.repeat_interleave(ids.repeat(counts.shape[0]), mine.reshape(-1))
    return int(mine.sum().item()), expert_of_row


def plan_return(counts: torch.Tensor, rank: int, experts_per_rank: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Where the rows received at ``rank`` go back to, in buffer order: the source rank of every
    row and its slot in that rank's expert-sorted order (the index ``DispatchPlan.slot_of`` uses)."""
    world = counts.shape[0]
    per_rank = counts.reshape(world, world, experts_per_rank).sum(-1)           # [source, destination]
    rows_from = per_rank[:, rank]                                               # block sizes, source order
    home = torch.repeat_interleave(torch.arange(world, device=counts.device), rows_from)
    block_start = torch.cumsum(rows_from, 0) - rows_from
    first_in_source = per_rank[:, :rank].sum(1)                                 # where my segment starts in each source's order
    n_rows = int(rows_from.sum().item())
    slot = first_in_source[home] + (torch.arange(n_rows, device=counts.device) - block_start[home])
    return home, slot


def plan_on_device(topk_indices: torch.Tensor, counts: torch.Tensor, rank: int):
    """``plan_dispatch`` and the combine's routes by ONE kernel launch instead of ~25 small
    PyTorch ops (at most 256 experts, 32 ranks).  Returns ``(src_row, dst_rank, dst_row,
    pull_rank [T, k], pull_row [T, k], meta)``; ``meta`` is a device tensor ``[rows this rank
    receives, most rows any rank receives]``."""
    t, k = topk_indices.shape
    dev = topk_indices.device
    routes = torch.empty(5, t * k, dtype=torch.int64, device=dev)
    meta = torch.empty(2, dtype=torch.int64, device=dev)
    _native.ep_plan(topk_indices, counts, rank, routes[0], routes[1], routes[2], routes[3], routes[4], meta)
    return routes[0], routes[1], routes[2], routes[3].view(t, k), routes[4].view(t, k), meta


class ExpertParallel:
    """Dispatch / expert / combine over the ranks of one process group (one process per GPU).

    ``capacity_rows`` bounds the rows one rank can receive per call (its experts' share of
    ``world * T * k`` in the worst case); a call that would exceed it raises ``ValueError`` on
    every rank before anything is sent.  Buffers are symmetric memory: allocated once, mapped
    into every peer."""

    def __init__(self, n_experts: int, hidden: int, capacity_rows: int, max_local_rows: int = 0,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | None = None, group=None,
                 return_mode: str = "pull"):
        """``capacity_rows``: rows this rank can receive per call.  ``return_mode`` "pull" (the
        combine reads peers' output buffers) or "push" (outputs are written back to the tokens'
        ranks; needs ``max_local_rows`` >= the largest ``T * k`` of a call)."""
        import torch.distributed._symmetric_memory as symm_mem
        if return_mode not in ("pull", "push"):
            raise ValueError(f"return_mode must be 'pull' or 'push', got {return_mode!r}")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if n_experts % self.world:
            raise ValueError(f"n_experts ({n_experts}) must be divisible by the world size ({self.world})")
        self.n_experts, self.experts_per_rank = n_experts, n_experts // self.world
        self.hidden, self.capacity, self.max_local, self.dtype = hidden, capacity_rows, max_local_rows, dtype
        self.return_mode = return_mode
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())

        def symmetric(rows):
            buf = symm_mem.empty((rows, hidden), dtype=dtype, device=self.device)
            handle = symm_mem.rendezvous(buf, self.group.group_name)
            return buf, handle, torch.tensor(list(handle.buffer_ptrs), dtype=torch.int64, device=self.device)

        self.barrier = PhaseBarrier(self.device, self.group)
        self.recv, self._recv_h, self.recv_bases = symmetric(capacity_rows)
        # the second buffer: expert outputs where they were computed (pull), or returned rows at home (push)
        self.ret, self._ret_h, self.ret_bases = symmetric(capacity_rows if return_mode == "pull" else max(1, max_local_rows))

    def exchange_counts(self, topk_indices: torch.Tensor) -> torch.Tensor:
        mine = torch.bincount(topk_indices.reshape(-1), minlength=self.n_experts).to(torch.int64)
        counts = torch.empty(self.world, self.n_experts, dtype=torch.int64, device=mine.device)
        dist.all_gather_into_tensor(counts, mine, group=self.group)
        return counts

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_indices: torch.Tensor, expert_fn) -> torch.Tensor:
        """``combined[t] = sum_j topk_weights[t, j] * expert_fn(x[t], expert topk_indices[t, j])``
        with the experts evaluated on the ranks that own them.  ``expert_fn(rows, expert_ids)``
        maps this rank's received rows ``[R, hidden]`` (with the expert id of every row) to
        ``[R, hidden]``."""
        from .kernels.token_permute import token_combine
        if topk_indices.dim() != 2:
            raise ValueError(f"topk_indices must be [T, k], got {tuple(topk_indices.shape)}")
        t, k = topk_indices.shape
        self._check_rows("x", x, t)
        if tuple(topk_weights.shape) != (t, k):
            raise ValueError(f"topk_weights shape {tuple(topk_weights.shape)} must match topk_indices' {(t, k)}")
        for name, tensor in (("topk_weights", topk_weights), ("topk_indices", topk_indices)):
            if tensor.device != self.device:
                raise ValueError(f"{name} is on {tensor.device}, the exchange buffers on {self.device}")
        push = self.return_mode == "push"
        if push and t * k > self.max_local:
            raise ValueError(f"T * k = {t * k} exceeds max_local_rows = {self.max_local}")
        counts = self.exchange_counts(topk_indices)
        on_device = self.n_experts <= 256 and self.world <= 32 and not push
        if on_device:
            src_row, dst_rank, dst_row, pull_rank, pull_row, meta = plan_on_device(topk_indices, counts, self.rank)
            n_rows, worst = meta.tolist()                    # the call's one host read
        else:
            per_rank = counts.reshape(self.world, self.world, self.experts_per_rank).sum(-1)
            worst = int(per_rank.sum(0).max().item())
        if worst > self.capacity:
            raise ValueError(f"a rank would receive {worst} rows, more than capacity_rows = {self.capacity}")
        if not on_device:
            plan = plan_dispatch(topk_indices, counts, self.rank, self.experts_per_rank)
            src_row, dst_rank, dst_row = plan.src_row, plan.dst_rank, plan.dst_row
        _native.token_dispatch_fwd(x, src_row, dst_rank, dst_row, self.recv_bases, self.capacity)
        self.barrier()                                       # every rank's pushes have landed
        if on_device:
            mine = counts[:, self.rank * self.experts_per_rank:(self.rank + 1) * self.experts_per_rank]
            ids = torch.arange(self.rank * self.experts_per_rank, (self.rank + 1) * self.experts_per_rank, device=self.device)
            expert_of_row = torch.repeat_interleave(ids.repeat(self.world), mine.reshape(-1), output_size=n_rows)
        else:
            n_rows, expert_of_row = plan_receive(counts, self.rank, self.experts_per_rank)
        if n_rows:
            y = expert_fn(self.recv[:n_rows], expert_of_row)
            self._check_rows("expert_fn's output", y, n_rows, contiguous=False)
            if push:
                home, slot = plan_return(counts, self.rank, self.experts_per_rank)
                _native.token_dispatch_fwd(y.contiguous(), torch.arange(n_rows, device=self.device), home, slot,
                                           self.ret_bases, self.max_local)
            else:
                self.ret[:n_rows].copy_(y)
        self.barrier()                                       # outputs are where the combine looks for them
        if push:
            # the next call's first barrier keeps peers from overwriting `ret` before this combine ran
            return token_combine(self.ret[:t * k], plan.slot_of, topk_weights)
        combined = torch.empty(t, self.hidden, dtype=self.dtype, device=self.device)
        if not on_device:
            pull_rank, pull_row = plan.dst_rank[plan.slot_of].contiguous(), plan.dst_row[plan.slot_of].contiguous()
        _native.token_combine_remote_fwd(self.ret_bases, self.capacity, pull_rank, pull_row, topk_weights, combined)
        self.barrier()                                       # nobody still reads the buffers the next call overwrites
        return combined

    def _check_rows(self, name, rows, n_rows, contiguous=True):
        """The exchange kernels take the row pitch from the tensor they are given, while the
        receive buffers' capacity is counted in rows of ``hidden`` elements of ``dtype``: a wider
        or differently typed row would be written past a peer's buffer, so refuse it here."""
        if rows.dim() != 2 or tuple(rows.shape) != (n_rows, self.hidden):
            raise ValueError(f"{name} must be [{n_rows}, {self.hidden}], got {tuple(rows.shape)}")
        if rows.dtype != self.dtype:
            raise ValueError(f"{name} is {rows.dtype}, the exchange buffers are {self.dtype}")
        if rows.device != self.device:
            raise ValueError(f"{name} is on {rows.device}, the exchange buffers on {self.device}")
        if contiguous and not rows.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
