"""`expert_compute="fused"` behind the per-slice expert MLP signatures, for collective transports.

The reference lets either expert backend run under either transport (`_expert_fns` and `_exchange_fn` are
independent, src/chunked_moe/moe.py:31-53; fused wrappers: src/chunked_moe/kernels/fused_expert.py:355-366).
Here the fused kernels normally run inside the NVLink path; this module serves the remaining combination
(`transport="ragged_a2a"` or `"emulated"` on GPU with `expert_compute="fused"`): the slice a collective
delivered is pushed through the same sm_100a kernels on a 1-rank world (rows are already expert-major, so
the plan is the identity, K = 1 and every router weight is 1).

The backward recomputes the slice's forward inside the kernels, so `ForwardResiduals` only carries what
the caller's `d_weight` needs (`y` is returned by `expert_forward`).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..config import ChunkedMoEConfig
from . import fused
from .expert import ExpertGrads, ForwardResiduals


def _solo_cfg(num_local: int, rows: int, stripe: int) -> ChunkedMoEConfig:
    # One slice holds the whole input: the caller already cut the stream into slices.
    return ChunkedMoEConfig(num_experts=num_local, top_k=1, slice_size=max(8, -(-rows // 8) * 8), transport="nvshmem",
                            expert_compute="fused", stripe_width=stripe)


def _row_experts(group_sizes: torch.Tensor) -> torch.Tensor:
    sizes = group_sizes.to(torch.int64)
    return torch.repeat_interleave(torch.arange(sizes.numel(), device=sizes.device), sizes).to(torch.int32)[:, None]


def expert_forward(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, group_sizes: torch.Tensor, *,
                   stripe: int, need_residuals: bool = True) -> tuple[torch.Tensor, Optional[ForwardResiduals]]:
    ids = _row_experts(group_sizes)
    rows = ids.shape[0]
    y = torch.zeros_like(x)
    if rows:
        cfg = _solo_cfg(w_up.shape[0], x.shape[0], stripe)
        ones = torch.ones(rows, 1, device=x.device, dtype=torch.float32)
        y[:rows] = fused._ChunkedMoEFused.apply(x[:rows].contiguous(), ids, ones, w_up, w_down, cfg, fused.SOLO)
    # h / act stay inside the kernels (the backward recomputes them); the tuple is kept for API compatibility.
    return y, (ForwardResiduals(h=x.new_empty(0), act=x.new_empty(0)) if need_residuals else None)


def expert_backward(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, group_sizes: torch.Tensor,
                    res: ForwardResiduals, dy: torch.Tensor, *, stripe: int) -> ExpertGrads:
    del res
    ids = _row_experts(group_sizes)
    rows = ids.shape[0]
    dx = torch.zeros_like(x)
    if not rows:
        return ExpertGrads(dx, torch.zeros_like(w_up, dtype=torch.float32), torch.zeros_like(w_down, dtype=torch.float32))
    cfg = _solo_cfg(w_up.shape[0], x.shape[0], stripe)
    xs = x[:rows].detach().contiguous().requires_grad_(True)
    ones = torch.ones(rows, 1, device=x.device, dtype=torch.float32)
    us, ds = w_up.detach().requires_grad_(True), w_down.detach().requires_grad_(True)
    with torch.enable_grad():
        y = fused._ChunkedMoEFused.apply(xs, ids, ones, us, ds, cfg, fused.SOLO)
    y.backward(dy[:rows].contiguous())
    dx[:rows] = xs.grad
    return ExpertGrads(dx, us.grad, ds.grad)
