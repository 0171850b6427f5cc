"""Symmetric arenas: one `cudaMalloc` block per rank, mapped into every peer with CUDA IPC.

Every rank allocates the same layout (slice buffers, return buffer, arrival counters, credits,
traffic matrix, ...; offsets come from the extension), exports one IPC handle, all-gathers the
handles over the expert-parallel process group and opens its peers' handles. After that a buffer
on rank r is `peer_base[r] + offset` for everyone on the NVLink domain; kernels only ever *store*
to peers and *load* locally. This replaces the reference's NVSHMEM / XLA collective-metadata peer
references (src/chunked_moe/transport/nvshmem.py:125-177). NCCL is only used to exchange the
64-byte handles once.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _build


class SymmetricArena:
    """This rank's arena plus the mapped base address of every peer's arena."""

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None, solo: bool = False):
        ext = _build.load()
        self._ext = ext
        self.nbytes = int(nbytes)
        self.group = group
        initialised = dist.is_available() and dist.is_initialized() and not solo
        self.world = dist.get_world_size(group) if initialised else 1
        self.rank = dist.get_rank(group) if initialised else 0
        self.local = ext.arena_alloc(self.nbytes)
        self.peers = [0] * self.world
        self.peers[self.rank] = self.local
        self._opened = []
        if self.world > 1:
            handle = ext.arena_export(self.local)
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            for r, h in enumerate(handles):
                if r != self.rank:
                    ptr = ext.arena_import(h)
                    self.peers[r] = ptr
                    self._opened.append(ptr)
            dist.barrier(group=group)  # nobody stores into an arena before everyone has mapped it

    def close(self) -> None:
        """Unmaps the peers and frees the local arena. Collective: peers must have stopped storing into it."""
        if self.local == 0:
            return
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        for ptr in self._opened:
            self._ext.arena_close(ptr)
        self._opened = []
        self._ext.arena_free(self.local)
        self.local = 0


class LocalArenas:
    """P arenas on ONE device, for the single-device lockstep harness (no IPC, plain pointers)."""

    def __init__(self, nbytes: int, world: int):
        ext = _build.load()
        self._ext = ext
        self.nbytes = int(nbytes)
        self.world = world
        self.bases = [ext.arena_alloc(self.nbytes) for _ in range(world)]

    def close(self) -> None:
        torch.cuda.synchronize()
        for ptr in self.bases:
            self._ext.arena_free(ptr)
        self.bases = []
