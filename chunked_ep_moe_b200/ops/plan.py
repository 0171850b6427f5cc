"""Slice planning for chunked expert-parallel dispatch (integer bookkeeping, plain torch).

Notation: P EP ranks, E experts, L = E / P local experts per rank (rank-major:
global expert e = r * L + l), K top-k, T tokens per rank, S slice rows.

Sender view. A rank stably sorts its T*K token copies by global expert id
("send order"); copies for (receiver r, local expert l) are contiguous there,
starting at `send_start[s, r*L + l]`.

Receiver view. Rank r lays out what it receives as ONE packed expert-major
stream: all copies for its local expert 0 (from source 0, then source 1, ...),
then expert 1, ... Segment (s, l) starts at `recv_start[r, l, s]`; the stream
has `R[r] = sum_{s,l} counts[s, r, l]` rows and no padding.

Slices. Slice j is stream rows `[j*S, (j+1)*S)`. Every rank loops
`max_r ceil(R[r] / S)` times; a rank with a shorter stream sends and receives
nothing in the tail.

Semantics follow the reference planner (src/chunked_moe/plan.py:60-163). This
module is the oracle for the device-side plan kernels and is what the
torch/gloo/NCCL layer paths run on.
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch
import torch.distributed as dist


class DispatchPlan(NamedTuple):
    """Per-layer routing bookkeeping, identical in forward and backward."""

    order: torch.Tensor  # [T*K] int64: flat assignment index t*K+k at each send-order position
    counts: torch.Tensor  # [P, P, L] copies routed from source s to local expert l of rank r
    send_start: torch.Tensor  # [P, P*L] exclusive prefix sums of counts[s].reshape(-1)
    recv_start: torch.Tensor  # [P, L, P] start of segment (source s, expert l) in rank r's stream
    expert_start: torch.Tensor  # [P, L] start of expert l's rows in rank r's stream
    expert_rows: torch.Tensor  # [P, L] rows of expert l in rank r's stream
    num_slices: int  # slice iterations, the same on every rank
    rank: int  # this rank's index on the EP axis
    num_ranks: int


class SliceArgs(NamedTuple):
    """Arguments of one ragged exchange, flat `[peer * L + l]`."""

    input_offsets: torch.Tensor
    send_sizes: torch.Tensor
    output_offsets: torch.Tensor
    recv_sizes: torch.Tensor


def _exclusive_cumsum(x: torch.Tensor, dim: int) -> torch.Tensor:
    return torch.cumsum(x, dim=dim) - x


def sort_and_count(expert_ids: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Stable sort of the T*K copies by expert id, and the per-expert histogram."""
    flat = expert_ids.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    my_counts = torch.bincount(flat, minlength=num_experts)
    if my_counts.numel() != num_experts:
        raise ValueError(f"expert id out of range: ids reach {my_counts.numel() - 1}, num_experts={num_experts}")
    return order, my_counts


def gather_traffic_matrix(my_counts: torch.Tensor, num_ranks: int, group: Optional[dist.ProcessGroup]) -> torch.Tensor:
    """All-gathers each rank's `[P, L]` counts into the `[P(s), P(r), L]` traffic matrix (the plan's only collective)."""
    local = my_counts.numel() // num_ranks
    mine = my_counts.reshape(num_ranks, local).contiguous()
    if num_ranks == 1:
        return mine[None]
    out = torch.empty((num_ranks * num_ranks * local,), dtype=mine.dtype, device=mine.device)
    dist.all_gather_into_tensor(out, mine.reshape(-1), group=group)
    return out.reshape(num_ranks, num_ranks, local)


def plan_from_counts(order: torch.Tensor, counts: torch.Tensor, slice_size: int, rank: int) -> DispatchPlan:
    """Everything after the all-gather: pure prefix sums on the `[P, P, L]` traffic matrix."""
    num_ranks, _, local = counts.shape
    counts = counts.to(torch.int64)
    send_start = _exclusive_cumsum(counts.reshape(num_ranks, num_ranks * local), dim=1)
    per_receiver = counts.permute(1, 2, 0)  # [r, l, s]
    expert_rows = per_receiver.sum(dim=2)  # [r, l]
    expert_start = _exclusive_cumsum(expert_rows, dim=1)
    recv_start = expert_start[:, :, None] + _exclusive_cumsum(per_receiver, dim=2)  # [r, l, s]
    stream_rows = expert_rows.sum(dim=1)
    num_slices = int((int(stream_rows.max()) + slice_size - 1) // slice_size)
    return DispatchPlan(order, counts, send_start, recv_start.contiguous(), expert_start, expert_rows, num_slices,
                        rank, num_ranks)


def make_plan(expert_ids: torch.Tensor, num_experts: int, slice_size: int,
              group: Optional[dist.ProcessGroup] = None, *, rank: Optional[int] = None,
              num_ranks: Optional[int] = None) -> DispatchPlan:
    """Builds the dispatch plan from this rank's `[T, K]` expert ids."""
    if num_ranks is None:
        initialised = dist.is_available() and dist.is_initialized()
        num_ranks = dist.get_world_size(group) if initialised else 1
        rank = dist.get_rank(group) if initialised else 0
    if num_experts % num_ranks:
        raise ValueError(f"num_experts={num_experts} is not divisible by the EP size {num_ranks}")
    order, my_counts = sort_and_count(expert_ids, num_experts)
    counts = gather_traffic_matrix(my_counts, num_ranks, group)
    return plan_from_counts(order, counts, slice_size, rank)


def _overlap(lo: int, hi: int, start: torch.Tensor, size: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Intersection of `[lo, hi)` with `[start, start+size)` as (first row, length)."""
    end = start + size
    first = torch.minimum(torch.clamp(start, min=lo), end)
    last = torch.minimum(torch.clamp(start, min=hi), end)
    return first, last - first


def dispatch_args(plan: DispatchPlan, j: int, slice_size: int) -> SliceArgs:
    """Arguments that move slice j from senders' send order into receivers' S-row slice buffers."""
    me, num_ranks = plan.rank, plan.num_ranks
    local = plan.counts.shape[2]
    lo, hi = j * slice_size, (j + 1) * slice_size
    # As a sender: one segment per (receiver r, local expert l).
    seg_start = plan.recv_start[:, :, me]  # [r, l] where my segment starts in r's stream
    seg_size = plan.counts[me]  # [r, l]
    first, size = _overlap(lo, hi, seg_start, seg_size)
    input_offsets = plan.send_start[me].reshape(num_ranks, local) + (first - seg_start)
    output_offsets = first - lo
    # As a receiver: one segment per (source s, my local expert l).
    in_start = plan.recv_start[me].transpose(0, 1)  # [s, l]
    in_size = plan.counts[:, me, :]
    _, recv_sizes = _overlap(lo, hi, in_start, in_size)
    flat = lambda a: a.reshape(-1).contiguous()
    return SliceArgs(flat(input_offsets), flat(size), flat(output_offsets), flat(recv_sizes))


def combine_args(plan: DispatchPlan, j: int, slice_size: int) -> SliceArgs:
    """The exact reverse of `dispatch_args`: slice j's rows go back to their place in the senders' send order."""
    me, num_ranks = plan.rank, plan.num_ranks
    local = plan.counts.shape[2]
    lo, hi = j * slice_size, (j + 1) * slice_size
    in_start = plan.recv_start[me].transpose(0, 1)  # [s, l]
    in_size = plan.counts[:, me, :]
    first, size = _overlap(lo, hi, in_start, in_size)
    input_offsets = first - lo
    source_send_start = plan.send_start.reshape(num_ranks, num_ranks, local)[:, me, :]  # [s, l]
    output_offsets = source_send_start + (first - in_start)
    seg_start = plan.recv_start[:, :, me]
    _, recv_sizes = _overlap(lo, hi, seg_start, plan.counts[me])
    flat = lambda a: a.reshape(-1).contiguous()
    return SliceArgs(flat(input_offsets), flat(size), flat(output_offsets), flat(recv_sizes))


def slice_group_sizes(plan: DispatchPlan, j: int, slice_size: int) -> torch.Tensor:
    """`[L]` rows of each local expert inside this rank's slice j (contiguous, in expert order)."""
    lo = j * slice_size
    _, rows = _overlap(lo, lo + slice_size, plan.expert_start[plan.rank], plan.expert_rows[plan.rank])
    return rows


def stream_rows(plan: DispatchPlan) -> torch.Tensor:
    """`[P]` rows R[r] of every rank's receive stream."""
    return plan.expert_rows.sum(dim=1)


def plan_stats(plan: DispatchPlan, slice_size: int) -> dict:
    """Load statistics that fall out of the plan for free (rows per rank, padding, imbalance)."""
    rows = stream_rows(plan)
    mine = int(rows[plan.rank])
    per_expert = plan.expert_rows.reshape(-1).float()
    mean = float(per_expert.mean()) if per_expert.numel() else 0.0
    return {
        "num_slices": plan.num_slices,
        "stream_rows": [int(v) for v in rows.tolist()],
        "my_stream_rows": mine,
        "my_active_slices": -(-mine // slice_size),
        "my_padding_rows": (-(-mine // slice_size)) * slice_size - mine,
        "max_expert_rows": int(per_expert.max()) if per_expert.numel() else 0,
        "mean_expert_rows": mean,
        "imbalance": (float(per_expert.max()) / mean) if mean > 0 else 0.0,
        "rows_sent_remote": int(plan.counts[plan.rank].sum() - plan.counts[plan.rank, plan.rank].sum()),
    }
