"""Single-device lockstep harness: P expert-parallel ranks emulated on ONE GPU, in one process.

Each virtual rank gets its own arena and executor; their pointer tables point at each other's
arenas on the same device. The harness launches every rank's step in a fixed order on one stream
(all puts of a slice, then all computes of that slice), so every arrival counter and credit a
kernel looks at has already been written when it starts: nothing ever spins, which is what makes
it safe to run kernels that would otherwise wait on one another on a single device. It exercises
exactly the kernels, tables and protocol of the multi-GPU path; only the launch order differs.
"""

from __future__ import annotations

import math

import torch

from .. import _build
from ..config import ChunkedMoEConfig
from .symm import LocalArenas


class LockstepWorld:
    def __init__(self, cfg: ChunkedMoEConfig, world: int, hidden: int, ffn: int, tokens_per_rank: int,
                 spin_limit: int = 1 << 16, cta_pairs: bool = True):
        if cfg.num_experts % world:
            raise ValueError(f"num_experts={cfg.num_experts} is not divisible by world={world}")
        ext = _build.load()
        self.cfg, self.world = cfg, world
        self.local = cfg.num_experts // world
        self.hidden, self.ffn = hidden, ffn
        self.tk = tokens_per_rank * cfg.top_k
        self.max_slices = max(1, math.ceil(world * self.tk / cfg.slice_size)) + 1
        fp8 = cfg.comm_dtype == "float8_e4m3fn"
        nbytes = ext.arena_bytes(world, self.local, cfg.slice_size, hidden, self.tk, fp8)
        self.arenas = LocalArenas(nbytes, world)
        self.ranks = [
            ext.FusedRank(P=world, L=self.local, me=r, S=cfg.slice_size, D=hidden, F=ffn, K=cfg.top_k,
                          stripe=cfg.stripe_width, tk_cap=self.tk, max_slices=self.max_slices, num_sms=cfg.num_sms,
                          fp8=fp8, arena=self.arenas.bases[r], peer_arenas=self.arenas.bases, use_comm_stream=False,
                          spin_limit=spin_limit, put_blocks=8, cta_pairs=cta_pairs, tgmm_pairs=cta_pairs)
            for r in range(world)
        ]
        self.plan_ints = self.ranks[0].plan_ints()

    def close(self) -> None:
        self.ranks = []
        self.arenas.close()

    def forward(self, xs, ids, weights, w_ups, w_downs):
        """Per-rank lists in, per-rank outputs and saved state out."""
        P, dev = self.world, xs[0].device
        n_exp = self.cfg.num_experts
        counts = torch.zeros(P, n_exp, dtype=torch.int32, device=dev)
        plans, orders, invs = [], [], []
        for r in range(P):
            order = torch.empty(ids[r].numel(), dtype=torch.int32, device=dev)
            inv = torch.empty_like(order)
            self.ranks[r].sort_only(ids[r].to(torch.int32).contiguous(), order, inv, counts[r])
            orders.append(order)
            invs.append(inv)
        counts_flat = counts.reshape(-1).contiguous()  # [s][r*L+l] is exactly the [P, P, L] traffic matrix
        slices = []
        for r in range(P):
            plan = torch.empty(self.plan_ints, dtype=torch.int32, device=dev)
            slices.append(self.ranks[r].begin_forward(ids[r].to(torch.int32).contiguous(), plan, orders[r], invs[r],
                                                      counts_flat, True))
            plans.append(plan)
        assert len(set(slices)) == 1, f"ranks disagree on the slice count: {slices}"
        n = slices[0]
        w_flats = [w.detach().float().reshape(-1).contiguous() for w in weights]
        for j in range(n):
            for r in range(P):
                self.ranks[r].put(j, plans[r], orders[r], xs[r], None, w_flats[r])
            for r in range(P):
                self.ranks[r].compute_forward(j, plans[r], w_ups[r], w_downs[r])
        outs = []
        for r in range(P):
            out = torch.empty_like(xs[r])
            self.ranks[r].finish_forward(invs[r], out)
            outs.append(out)
        for rk in self.ranks:
            rk.check_status()
        return outs, (plans, orders, invs, w_flats, n)

    def backward(self, xs, gs, w_ups, w_downs, saved):
        plans, orders, invs, w_flats, _ = saved
        P, dev = self.world, xs[0].device
        slices = [self.ranks[r].begin_backward(plans[r]) for r in range(P)]
        n = slices[0]
        dw_ups = [torch.empty_like(w) for w in w_ups]
        dw_downs = [torch.empty_like(w) for w in w_downs]
        for j in range(n):
            for r in range(P):
                self.ranks[r].put(j, plans[r], orders[r], xs[r], gs[r], w_flats[r])
            for r in range(P):
                self.ranks[r].compute_backward(j, plans[r], w_ups[r], w_downs[r], dw_ups[r], dw_downs[r])
        dxs, dws = [], []
        for r in range(P):
            dx = torch.empty_like(xs[r])
            dw = torch.empty(w_flats[r].numel(), dtype=torch.float32, device=dev)
            self.ranks[r].finish_backward(invs[r], dx, dw)
            dxs.append(dx)
            dws.append(dw)
        for rk in self.ranks:
            rk.check_status()
        return dxs, dws, dw_ups, dw_downs
