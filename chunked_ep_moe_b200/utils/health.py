"""Host-side failure detection between steps.

The fused kernels bound every device-side wait and report through a status block, but the cheapest place to
learn that a peer is gone is the host, *between* steps, before anything is launched that would wait for it.
`RankHealth` is a heartbeat over the job's c10d store: before a step every rank publishes the step number it is
about to run and checks (with a deadline) that every other rank has published it too. A rank that raised,
exited or never joined is named in the `PeerFailure` the survivors get, and no kernel or collective is in
flight when that happens. The reference has no failure detection (its semaphore waits are unbounded,
src/chunked_moe/transport/nvshmem.py:144-177).
"""

from __future__ import annotations

import time
from typing import Iterable, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    """Raised on the surviving ranks when a peer did not reach a step in time."""

    def __init__(self, step: int, missing: Iterable[int], waited_s: float):
        self.step, self.missing, self.waited_s = step, sorted(missing), waited_s
        super().__init__(f"ranks {self.missing} did not reach step {step} within {waited_s:.1f} s")


class PlanMismatch(RuntimeError):
    """Raised when the ranks of a group do not agree on a routing plan (corrupted or stale traffic matrix)."""


class RankHealth:
    def __init__(self, store, rank: int, world: int, prefix: str = "cem/health", timeout_s: float = 30.0,
                 poll_s: float = 0.02, store_host: int = 0):
        self.store, self.rank, self.world = store, rank, world
        self.prefix, self.timeout_s, self.poll_s = prefix, timeout_s, poll_s
        self.store_host = store_host  # the rank whose process serves the store: if the store dies, that rank is gone

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def announce(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(step))

    def mark_failed(self, reason: str) -> None:
        """Lets a rank that caught an exception tell the others why it is leaving."""
        self.store.set(self._key(self.rank), f"failed:{reason[:200]}")

    def _peer_step(self, rank: int) -> Optional[int]:
        key = self._key(rank)
        if not self.store.check([key]):
            return None
        value = self.store.get(key).decode()
        if value.startswith("failed:"):
            return -1
        return int(value)

    def check_peers(self, step: int) -> None:
        """Returns once every rank has announced `step` (or later); raises `PeerFailure` at the deadline."""
        deadline = time.monotonic() + self.timeout_s
        start = time.monotonic()
        missing = set(range(self.world)) - {self.rank}
        while missing:
            for r in list(missing):
                try:
                    s = self._peer_step(r)
                except PeerFailure:
                    raise
                except Exception:  # noqa: BLE001 - the store itself stopped answering: its host has left
                    if self.rank == self.store_host:
                        raise
                    raise PeerFailure(step, [self.store_host], time.monotonic() - start) from None
                if s is not None and s >= step:
                    missing.discard(r)
                elif s == -1:
                    raise PeerFailure(step, [r], time.monotonic() - start)
            if not missing:
                break
            if time.monotonic() > deadline:
                raise PeerFailure(step, missing, time.monotonic() - start)
            time.sleep(self.poll_s)

    def step_barrier(self, step: int) -> None:
        self.announce(step)
        self.check_peers(step)


def verify_plan_agreement(counts, my_counts, rank: int, group=None) -> None:
    """Cheap consistency checks of an all-gathered `[P, P, L]` traffic matrix before anything is dispatched.

    * this rank's row must be what this rank contributed (a stale or corrupted gather shows up here);
    * every rank must hold the same matrix (compared through a checksum all-reduce MIN/MAX).
    """
    import torch

    if not torch.equal(counts[rank].reshape(-1).to(my_counts.dtype), my_counts.reshape(-1)):
        raise PlanMismatch(f"rank {rank}: the gathered traffic matrix does not contain this rank's own counts")
    if (counts < 0).any():
        raise PlanMismatch(f"rank {rank}: negative entry in the traffic matrix")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        weights = torch.arange(1, counts.numel() + 1, device=counts.device, dtype=torch.int64)
        checksum = (counts.reshape(-1).to(torch.int64) * weights).sum().reshape(1)
        lo, hi = checksum.clone(), checksum.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
        if int(lo) != int(hi):
            raise PlanMismatch(f"rank {rank}: ranks disagree on the traffic matrix (checksums {int(lo)} .. {int(hi)})")
