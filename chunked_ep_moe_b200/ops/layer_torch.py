"""Layer orchestration on collective transports: the slice loops in plain torch.

This is the backend-agnostic restatement of the reference's forward loop and
single fused remat+backward loop (src/chunked_moe/moe.py:96-119, :148-206). It
runs with any collective exchange (`emulated` over gloo for the CPU oracle,
`ragged_a2a` over NCCL for the GPU baseline) and either expert backend. The
fused NVLink path has its own executor (`ops/fused.py`) and is checked against
this one.

  forward:   plan -> gather rows into send order -> loop over slices:
               dispatch slice j+1 | expert MLP on slice j | return slice j
             -> weighted K-way sum per token
  backward:  one loop over slices that re-dispatches x, g and the router
             weights, recomputes the slice's forward and runs its backward at
             once. Only the inputs and the integer plan are kept between passes.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..config import ChunkedMoEConfig
from . import expert as expert_torch
from . import plan as plan_lib
from .quant import dequantize_rows, quantize_rows


def expert_fns(cfg: ChunkedMoEConfig) -> tuple[Callable, Callable]:
    """(expert_forward, expert_backward) for `cfg.expert_compute` on a collective-transport path."""
    if cfg.expert_compute == "reference":
        module = expert_torch
    elif cfg.expert_compute == "fused":
        from . import fused_expert as module  # sm_100a kernels behind the same signatures
    else:
        raise ValueError(f"unknown expert_compute {cfg.expert_compute!r}")

    def fwd(x, w_up, w_down, group_sizes, need_residuals=True):
        return module.expert_forward(x, w_up, w_down, group_sizes, stripe=cfg.stripe_width,
                                     need_residuals=need_residuals)

    def bwd(x, w_up, w_down, group_sizes, res, dy):
        return module.expert_backward(x, w_up, w_down, group_sizes, res, dy, stripe=cfg.stripe_width)

    return fwd, bwd


class Dispatcher:
    """Moves rows from this rank's send order into S-row slice buffers, optionally quantised on the wire."""

    def __init__(self, cfg: ChunkedMoEConfig, plan: plan_lib.DispatchPlan, exchange: Callable,
                 group: Optional[dist.ProcessGroup], rows: torch.Tensor, compute_dtype: torch.dtype,
                 quantize: bool = True):
        self.cfg, self.plan, self.exchange, self.group = cfg, plan, exchange, group
        self.compute_dtype = compute_dtype
        self.values, self.scales = quantize_rows(rows, cfg.comm_dtype if quantize else None)
        self.wire_dtype = self.values.dtype
        if self.scales is not None:
            self.values = self.values.view(torch.uint8)  # collectives move raw bytes

    def __call__(self, j: int) -> torch.Tensor:
        s = self.cfg.slice_size
        args = plan_lib.dispatch_args(self.plan, j, s)
        values = self.exchange(self.values, self.values.new_zeros((s,) + tuple(self.values.shape[1:])), args,
                               self.group)
        if self.scales is None:
            return values
        scales = self.exchange(self.scales, self.scales.new_zeros((s, self.scales.shape[1])), args, self.group)
        return dequantize_rows(values.view(self.wire_dtype), scales, self.compute_dtype)


def forward_loop(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor,
                 w_down: torch.Tensor, cfg: ChunkedMoEConfig, group: Optional[dist.ProcessGroup],
                 exchange: Callable) -> tuple[torch.Tensor, plan_lib.DispatchPlan]:
    num_tokens, hidden = x.shape
    k, s = cfg.top_k, cfg.slice_size
    fwd, _ = expert_fns(cfg)

    plan = plan_lib.make_plan(expert_ids, cfg.num_experts, s, group)
    token_of_row = plan.order // k
    dispatch = Dispatcher(cfg, plan, exchange, group, x[token_of_row], x.dtype)

    ret = x.new_zeros((num_tokens * k, hidden))
    cur = dispatch(0)
    for j in range(plan.num_slices):
        nxt = dispatch(j + 1)  # independent of this slice's compute
        y, _ = fwd(cur, w_up, w_down, plan_lib.slice_group_sizes(plan, j, s), need_residuals=False)
        ret = exchange(y, ret, plan_lib.combine_args(plan, j, s), group)
        cur = nxt

    row_weights = weights.reshape(-1)[plan.order].float()
    out = torch.zeros((num_tokens, hidden), dtype=torch.float32, device=x.device)
    out.index_add_(0, token_of_row, ret.float() * row_weights[:, None])
    return out.to(x.dtype), plan


def backward_loop(x: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                  plan: plan_lib.DispatchPlan, g_out: torch.Tensor, cfg: ChunkedMoEConfig,
                  group: Optional[dist.ProcessGroup], exchange: Callable):
    num_tokens, hidden = x.shape
    k, s = cfg.top_k, cfg.slice_size
    fwd, bwd = expert_fns(cfg)
    accum = getattr(torch, cfg.accum_dtype)

    token_of_row = plan.order // k
    row_weights = weights.reshape(-1)[plan.order].float()[:, None]
    dispatch_x = Dispatcher(cfg, plan, exchange, group, x[token_of_row], x.dtype)
    dispatch_g = Dispatcher(cfg, plan, exchange, group, g_out.to(x.dtype)[token_of_row], x.dtype)
    dispatch_w = Dispatcher(cfg, plan, exchange, group, row_weights, torch.float32, quantize=False)

    dx_rows = x.new_zeros((num_tokens * k, hidden))
    dw_rows = torch.zeros((num_tokens * k, 1), dtype=torch.float32, device=x.device)
    dw_up = torch.zeros(w_up.shape, dtype=accum, device=x.device)
    dw_down = torch.zeros(w_down.shape, dtype=accum, device=x.device)

    cur = (dispatch_x(0), dispatch_g(0), dispatch_w(0))
    for j in range(plan.num_slices):
        nxt = (dispatch_x(j + 1), dispatch_g(j + 1), dispatch_w(j + 1))
        cur_x, cur_g, cur_w = cur
        group_sizes = plan_lib.slice_group_sizes(plan, j, s)

        # Recompute this slice's forward, then run its backward in the same iteration.
        y, res = fwd(cur_x, w_up, w_down, group_sizes)
        dy = (cur_w * cur_g.float()).to(x.dtype)
        d_weight = (cur_g.float() * y.float()).sum(dim=-1, keepdim=True)
        grads = bwd(cur_x, w_up, w_down, group_sizes, res, dy)

        back = plan_lib.combine_args(plan, j, s)
        dx_rows = exchange(grads.dx, dx_rows, back, group)
        dw_rows = exchange(d_weight, dw_rows, back, group)
        dw_up.add_(grads.dw_up)  # accumulates in `accum` whatever dtype the grouped GEMM returned
        dw_down.add_(grads.dw_down)
        cur = nxt

    dx = torch.zeros((num_tokens, hidden), dtype=torch.float32, device=x.device)
    dx.index_add_(0, token_of_row, dx_rows.float())
    d_weights = torch.zeros((num_tokens * k,), dtype=torch.float32, device=x.device)
    d_weights[plan.order] = dw_rows[:, 0]
    return (dx.to(x.dtype), d_weights.reshape(weights.shape).to(weights.dtype), dw_up.to(w_up.dtype),
            dw_down.to(w_down.dtype))
