"""Host-side routing plan of the collective (torch.distributed) layer paths.

Notation: P expert-parallel ranks, E experts, L = E / P experts per rank (global expert e = r * L + l lives on rank
r), K choices per token, T tokens per rank, S rows per slice.

The only thing ranks have to tell each other is the traffic matrix `counts[s, r, l]`: how many of source s's T*K token
copies go to expert l of rank r. It is tiny (P*P*L integers), so this planner brings it to the host ONCE per layer pass
and derives everything else there with numpy, for all slices at once:

  * source s keeps its copies sorted by global expert ("send order"); the block for (r, l) starts at
    `send_begin[s, r, l]`;
  * rank r receives one packed stream, expert after expert and inside an expert source after source; the block of
    (l, s) starts at `stream_begin[r, l, s]`. The stream has `rows[r] = counts[:, r, :].sum()` rows: no padding.
  * slice j is stream rows [j*S, (j+1)*S). Every rank runs `num_slices = ceil(max_r rows[r] / S)` iterations, so
    the loops stay in step; a rank whose stream is shorter simply has nothing to receive in the tail.

`dispatch_spec(j)` / `combine_spec(j)` return the segment lists of one exchange as host arrays (offsets, sizes and the
per-peer totals the collective needs), so an exchange never has to read a size back from the device: one device
synchronisation per pass (the traffic matrix) instead of several per exchange.

The semantics are the reference planner's (src/chunked_moe/plan.py:60-163); the device-side plan kernel
(csrc/plan/plan_tables.cuh) is tested against this module.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ExchangeSpec:
    """One ragged exchange as seen by one rank: P*L outgoing and P*L incoming segments, index `peer * L + l`.

    Outgoing segment i is `operand[src_offset[i] : src_offset[i] + send_rows[i]]` and lands at row `dst_offset[i]`
    of peer `i // L`'s output buffer. Incoming segment i (`recv_rows[i]` rows from peer `i // L`) lands at row
    `land_offset[i]` of MY output buffer: every rank holds the whole traffic matrix, so a receiver knows where the
    sender aims (`land_offset` here equals the sender's `dst_offset` there) and no offsets have to travel.
    """

    src_offset: np.ndarray
    send_rows: np.ndarray
    dst_offset: np.ndarray
    recv_rows: np.ndarray
    land_offset: np.ndarray
    num_ranks: int

    def _per_peer(self, rows: np.ndarray) -> list[int]:
        return rows.reshape(self.num_ranks, -1).sum(axis=1).tolist()

    @property
    def send_splits(self) -> list[int]:
        return self._per_peer(self.send_rows)

    @property
    def recv_splits(self) -> list[int]:
        return self._per_peer(self.recv_rows)


def _exclusive_scan(a: np.ndarray) -> np.ndarray:
    """Exclusive prefix sum over the last axis."""
    return np.cumsum(a, axis=-1) - a


class RoutingPlan:
    """Everything a layer pass needs to know about where rows go, for every slice, as host arrays."""

    def __init__(self, order: torch.Tensor, counts, slice_size: int, rank: int):
        counts = np.asarray(counts.cpu() if isinstance(counts, torch.Tensor) else counts, dtype=np.int64)
        if counts.ndim != 3 or counts.shape[0] != counts.shape[1]:
            raise ValueError(f"traffic matrix must be [P, P, L], got {counts.shape}")
        if slice_size <= 0:
            raise ValueError("slice_size must be positive")
        self.order = order  # [T*K] flat assignment index t*K+k at each send-order position (stays on its device)
        self.counts = counts
        self.slice_size = int(slice_size)
        self.rank = int(rank)
        self.num_ranks, _, self.local_experts = counts.shape
        P, L = self.num_ranks, self.local_experts

        self.send_begin = _exclusive_scan(counts.reshape(P, P * L)).reshape(P, P, L)  # [s, r, l]
        by_receiver = counts.transpose(1, 2, 0)  # [r, l, s]: the order blocks take in r's stream
        self.stream_begin = _exclusive_scan(by_receiver.reshape(P, L * P)).reshape(P, L, P)
        self.expert_rows = by_receiver.sum(axis=2)  # [r, l]
        self.expert_begin = self.stream_begin[:, :, 0]
        self.rows = self.expert_rows.sum(axis=1)  # [r] stream length
        self.num_slices = int(-(-int(self.rows.max()) // self.slice_size)) if self.rows.size else 0

        # Windows of all slices at once (one spare slice: the loops prefetch slice j+1 and it must come out empty).
        n = self.num_slices + 1
        lo = (np.arange(n, dtype=np.int64) * self.slice_size)[:, None, None]
        hi = lo + self.slice_size
        me = self.rank

        def clip(begin, size):  # rows of [begin, begin+size) inside each window -> (first row, how many)
            first = np.minimum(np.maximum(begin[None], lo), (begin + size)[None])
            last = np.minimum(np.maximum(begin[None], hi), (begin + size)[None])
            return first, last - first

        out_begin = self.stream_begin[:, :, me]  # [r, l] where my block starts in r's stream
        self._out_first, self._out_rows = clip(out_begin, counts[me])  # [j, r, l]
        self._out_begin = out_begin
        in_begin = self.stream_begin[me].T  # [s, l] where s's block for my expert l starts in my stream
        self._in_first, self._in_rows = clip(in_begin, counts[:, me, :])  # [j, s, l]
        self._in_begin = in_begin
        _, self._group_rows = clip(self.expert_begin[me][None], self.expert_rows[me][None])  # [j, 1, l]
        self._lo = lo

    # ---- one exchange -------------------------------------------------------------------------------------
    def _slice(self, j: int) -> int:
        if j < 0:
            raise IndexError("negative slice index")
        return j

    def _empty(self) -> ExchangeSpec:
        z = np.zeros(self.num_ranks * self.local_experts, dtype=np.int64)
        return ExchangeSpec(z, z, z, z, z, self.num_ranks)

    def dispatch_spec(self, j: int) -> ExchangeSpec:
        """Send-order rows -> the receivers' S-row slice buffers, slice j."""
        j = self._slice(j)
        if j > self.num_slices:
            return self._empty()
        first, rows = self._out_first[j], self._out_rows[j]
        src = self.send_begin[self.rank] + (first - self._out_begin)
        dst = first - self._lo[j]
        land = self._in_first[j] - self._lo[j]
        return ExchangeSpec(src.reshape(-1), rows.reshape(-1), dst.reshape(-1), self._in_rows[j].reshape(-1),
                            land.reshape(-1), self.num_ranks)

    def combine_spec(self, j: int) -> ExchangeSpec:
        """Slice j's rows -> back to where they sit in their sources' send order (the dispatch run backwards)."""
        j = self._slice(j)
        if j > self.num_slices:
            return self._empty()
        first, rows = self._in_first[j], self._in_rows[j]
        src = first - self._lo[j]
        dst = self.send_begin[:, self.rank, :] + (first - self._in_begin)
        land = self.send_begin[self.rank] + (self._out_first[j] - self._out_begin)
        return ExchangeSpec(src.reshape(-1), rows.reshape(-1), dst.reshape(-1), self._out_rows[j].reshape(-1),
                            land.reshape(-1), self.num_ranks)

    def group_rows(self, j: int) -> np.ndarray:
        """`[L]` rows of each local expert inside this rank's slice j (contiguous, in expert order)."""
        j = self._slice(j)
        if j > self.num_slices:
            return np.zeros(self.local_experts, dtype=np.int64)
        return self._group_rows[j, 0]

    # ---- statistics ---------------------------------------------------------------------------------------
    def stats(self) -> dict:
        """Load statistics that fall out of the plan for free (rows per rank, padding, imbalance)."""
        S = self.slice_size
        mine = int(self.rows[self.rank])
        per_expert = self.expert_rows.reshape(-1).astype(np.float64)
        mean = float(per_expert.mean()) if per_expert.size else 0.0
        active = -(-mine // S)
        return {
            "num_slices": self.num_slices,
            "stream_rows": [int(v) for v in self.rows],
            "my_stream_rows": mine,
            "my_active_slices": active,
            "my_padding_rows": active * S - mine,
            "max_expert_rows": int(per_expert.max()) if per_expert.size else 0,
            "mean_expert_rows": mean,
            "imbalance": (float(per_expert.max()) / mean) if mean > 0 else 0.0,
            "rows_sent_remote": int(self.counts[self.rank].sum() - self.counts[self.rank, self.rank].sum()),
        }


def sort_and_count(expert_ids: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Stable sort of the T*K copies by expert id, and the per-expert histogram (on the ids' device)."""
    flat = expert_ids.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    hist = torch.bincount(flat, minlength=num_experts)
    if hist.numel() != num_experts:
        raise ValueError(f"expert id out of range: ids reach {hist.numel() - 1}, num_experts={num_experts}")
    return order, hist


def gather_traffic_matrix(hist: torch.Tensor, num_ranks: int, group: Optional[dist.ProcessGroup]) -> torch.Tensor:
    """All-gathers every rank's `[P, L]` histogram into `counts[s, r, l]` (the plan's only collective)."""
    mine = hist.reshape(num_ranks, -1).contiguous()
    if num_ranks == 1:
        return mine[None]
    out = torch.empty((num_ranks,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
    dist.all_gather_into_tensor(out.reshape(-1), mine.reshape(-1), group=group)
    return out


def make_plan(expert_ids: torch.Tensor, num_experts: int, slice_size: int,
              group: Optional[dist.ProcessGroup] = None, *, rank: Optional[int] = None,
              num_ranks: Optional[int] = None) -> RoutingPlan:
    """Sort, exchange the histograms, and build the plan on the host (one device->host copy: the traffic matrix)."""
    if num_ranks is None:
        initialised = dist.is_available() and dist.is_initialized()
        num_ranks = dist.get_world_size(group) if initialised else 1
        rank = dist.get_rank(group) if initialised else 0
    if num_experts % num_ranks:
        raise ValueError(f"num_experts={num_experts} is not divisible by the EP size {num_ranks}")
    order, hist = sort_and_count(expert_ids, num_experts)
    counts = gather_traffic_matrix(hist, num_ranks, group)
    return RoutingPlan(order, counts, slice_size, rank)
