"""Device-side timing: CUDA events on the launching stream, reduced as the max over ranks."""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class DeviceTimer:
    """`start()` ... `stop()` -> milliseconds between two CUDA events; `stop(world, group)` takes the max over ranks."""

    def __init__(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._stop = torch.cuda.Event(enable_timing=True)

    def start(self) -> None:
        self._start.record()

    def stop(self, world: int = 1, group: Optional[dist.ProcessGroup] = None) -> float:
        self._stop.record()
        self._stop.synchronize()
        ms = self._start.elapsed_time(self._stop)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            ms = float(t[0])
        return ms


def time_device(fn, iters: int, warmup: int = 3, world: int = 1, group=None) -> float:
    """Mean milliseconds per call of `fn` after `warmup` calls, with a synchronise (and barrier) on both sides."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group=group)
        torch.cuda.synchronize()
    timer = DeviceTimer()
    timer.start()
    for _ in range(iters):
        fn()
    return timer.stop(world, group) / iters
