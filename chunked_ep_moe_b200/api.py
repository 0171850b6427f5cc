"""Public entry point: `chunked_moe` as a `torch.autograd.Function`.

Per rank (one process per GPU, `group` is the expert-parallel process group):

    out = chunked_moe(x, expert_ids, router_weights, w_up, w_down, cfg, group)

  x              [T, D]   this rank's tokens
  expert_ids     [T, K]   global expert ids from the router (rank-major: e = r*L + l)
  router_weights [T, K]   combine weights (differentiable)
  w_up           [L, D, 2F] this rank's experts' striped gate/up weights
  w_down         [L, F, D]  this rank's experts' down weights

Same surface and gradient set as the reference's `custom_vjp`
(src/chunked_moe/moe.py:122-209): gradients flow to x, router_weights, w_up and
w_down; the backward is communicating (every rank of the group must call it).
Only the inputs and the integer routing plan are saved between the passes.

Backend selection: `transport="nvshmem"` + `expert_compute="fused"` runs the
fused sm_100a executor; every other combination runs the torch slice loops on
a collective transport. Shapes the kernels do not cover (D or F not a multiple
of 256, other stripe widths, non-bf16 tensors) fall back to the collective
path with a warning.
"""

from __future__ import annotations

import dataclasses
import warnings
from typing import Optional

import torch
import torch.distributed as dist

from .config import ChunkedMoEConfig
from .ops import layer_torch
from .parallel.exchange import exchange_fn


class _ChunkedMoECollective(torch.autograd.Function):
    """Slice loops on a collective transport (gloo/NCCL)."""

    @staticmethod
    def forward(ctx, x, expert_ids, weights, w_up, w_down, cfg, group):
        exchange = exchange_fn(cfg.transport)
        with torch.no_grad():
            out, plan = layer_torch.forward_pass(x, expert_ids, weights, w_up, w_down, cfg, group, exchange)
        ctx.save_for_backward(x, weights, w_up, w_down)
        ctx.plan, ctx.cfg, ctx.group = plan, cfg, group
        ctx.mark_non_differentiable(expert_ids)
        return out

    @staticmethod
    def backward(ctx, g_out):
        x, weights, w_up, w_down = ctx.saved_tensors
        exchange = exchange_fn(ctx.cfg.transport)
        with torch.no_grad():
            dx, d_weights, dw_up, dw_down = layer_torch.backward_pass(
                x, weights, w_up, w_down, ctx.plan, g_out.contiguous(), ctx.cfg, ctx.group, exchange)
        return dx, None, d_weights, dw_up, dw_down, None, None


def _check_inputs(x, expert_ids, weights, w_up, w_down, cfg: ChunkedMoEConfig, group) -> None:
    if x.dim() != 2:
        raise ValueError(f"x must be [T, D], got {tuple(x.shape)}")
    t, d = x.shape
    if tuple(expert_ids.shape) != (t, cfg.top_k) or tuple(weights.shape) != (t, cfg.top_k):
        raise ValueError(f"expert_ids/router_weights must be [T={t}, K={cfg.top_k}], got "
                         f"{tuple(expert_ids.shape)} and {tuple(weights.shape)}")
    world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    if cfg.num_experts % world:
        raise ValueError(f"num_experts={cfg.num_experts} is not divisible by the EP size {world}")
    local = cfg.num_experts // world
    if w_up.dim() != 3 or w_up.shape[0] != local or w_up.shape[1] != d or w_up.shape[2] % 2:
        raise ValueError(f"w_up must be [L={local}, D={d}, 2F], got {tuple(w_up.shape)}")
    ffn = w_up.shape[2] // 2
    if tuple(w_down.shape) != (local, ffn, d):
        raise ValueError(f"w_down must be [L={local}, F={ffn}, D={d}], got {tuple(w_down.shape)}")
    if ffn % cfg.stripe_width:
        raise ValueError(f"F={ffn} is not a multiple of stripe_width={cfg.stripe_width}")


def chunked_moe(x: torch.Tensor, expert_ids: torch.Tensor, router_weights: torch.Tensor, w_up: torch.Tensor,
                w_down: torch.Tensor, cfg: ChunkedMoEConfig,
                group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Dropless chunked MoE over the expert-parallel `group`; returns `[T, D]` for this rank's tokens."""
    _check_inputs(x, expert_ids, router_weights, w_up, w_down, cfg, group)
    if cfg.transport == "nvshmem":
        from .ops import fused  # needs the sm_100a extension

        return fused.chunked_moe_fused(x, expert_ids, router_weights, w_up, w_down, cfg, group)
    return _ChunkedMoECollective.apply(x, expert_ids, router_weights, w_up, w_down, cfg, group)
