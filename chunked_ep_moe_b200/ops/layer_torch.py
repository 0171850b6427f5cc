"""The layer on collective transports (gloo / NCCL): slice pipeline in plain torch.

This is the CPU oracle (`transport="emulated"` over gloo, fp32) and the GPU baseline the fused NVLink path is
measured against (`transport="ragged_a2a"` over NCCL + library grouped GEMMs). What it computes is fixed by the
reference's forward loop and single remat+backward loop (src/chunked_moe/moe.py:96-119, :148-206); how it is
organised here:

  * the routing plan lives on the host (`ops/plan.RoutingPlan`): one device->host copy per pass, after which every
    split size, offset and group size of every slice is a host value, so no exchange or grouped GEMM ever has to wait
    for the device to tell it a size;
  * `SliceFeed` owns one row stream (x, the output gradient, or the router weights): it is put into send order and
    quantised ONCE, and `_lookahead` asks every feed for slice j+1 before slice j is consumed, which is the overlap
    the collective backends can give;
  * rows come back into send order; the K copies of a token are then combined by un-permuting to `[T, K, D]` and
    summing over K in fp32 (fixed order, no atomics), for the output, dX and d(router weights) alike.

Only the inputs and the integer plan are kept between forward and backward.
"""

from __future__ import annotations

from typing import Callable, Iterator, Optional, Sequence

import torch
import torch.distributed as dist

from ..config import ChunkedMoEConfig
from . import expert as expert_torch
from .plan import RoutingPlan, make_plan
from .quant import dequantize_rows, quantize_rows


def expert_fns(cfg: ChunkedMoEConfig) -> tuple[Callable, Callable]:
    """(expert_forward, expert_backward) for `cfg.expert_compute` on a collective-transport path."""
    if cfg.expert_compute == "reference":
        module = expert_torch
    elif cfg.expert_compute == "fused":
        from . import fused_expert as module  # sm_100a kernels behind the same signatures
    else:
        raise ValueError(f"unknown expert_compute {cfg.expert_compute!r}")

    def fwd(x, w_up, w_down, group_rows, need_residuals=True):
        return module.expert_forward(x, w_up, w_down, group_rows, stripe=cfg.stripe_width,
                                     need_residuals=need_residuals)

    def bwd(x, w_up, w_down, group_rows, res, dy):
        return module.expert_backward(x, w_up, w_down, group_rows, res, dy, stripe=cfg.stripe_width)

    return fwd, bwd


class SliceFeed:
    """One row stream of this rank, delivered slice by slice to the ranks that own the rows' experts.

    `rows` is `[T*K, width]` already in send order. With a wire dtype the stream is quantised here, once per pass
    (values and per-block scales then travel as two exchanges per slice and are expanded on arrival).
    """

    def __init__(self, plan: RoutingPlan, exchange: Callable, group: Optional[dist.ProcessGroup], rows: torch.Tensor,
                 compute_dtype: torch.dtype, comm_dtype: Optional[str]):
        self.plan, self.exchange, self.group = plan, exchange, group
        self.compute_dtype = compute_dtype
        self.values, self.scales = quantize_rows(rows, comm_dtype)
        self.wire_dtype = self.values.dtype
        if self.scales is not None:
            self.values = self.values.view(torch.uint8)  # collectives move raw bytes

    def _receive(self, stream: torch.Tensor, spec) -> torch.Tensor:
        landing = stream.new_zeros((self.plan.slice_size,) + tuple(stream.shape[1:]))
        return self.exchange(stream, landing, spec, self.group)

    def fetch(self, j: int) -> torch.Tensor:
        """This rank's S-row slice j of the stream (rows past the slice's valid rows are zero)."""
        spec = self.plan.dispatch_spec(j)
        values = self._receive(self.values, spec)
        if self.scales is None:
            return values
        return dequantize_rows(values.view(self.wire_dtype), self._receive(self.scales, spec), self.compute_dtype)


def _lookahead(plan: RoutingPlan, feeds: Sequence[SliceFeed]) -> Iterator[tuple[int, tuple[torch.Tensor, ...]]]:
    """Yields (j, this slice's buffers) with slice j+1 already requested from every feed."""
    ahead = tuple(f.fetch(0) for f in feeds)
    for j in range(plan.num_slices):
        current, ahead = ahead, tuple(f.fetch(j + 1) for f in feeds)
        yield j, current


def _sum_over_choices(rows_in_send_order: torch.Tensor, inverse_order: torch.Tensor, num_tokens: int, top_k: int,
                      weights: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """`[T*K, D]` rows in send order -> `[T, D]`: each token's K rows, (weighted and) summed in fp32 in k order."""
    hidden = rows_in_send_order.shape[1]
    out = torch.empty((num_tokens, hidden), dtype=out_dtype, device=rows_in_send_order.device)
    step = max(1, (1 << 24) // max(hidden * top_k, 1))  # bound the fp32 temporary to ~64 MB
    for t0 in range(0, num_tokens, step):
        t1 = min(num_tokens, t0 + step)
        picked = rows_in_send_order[inverse_order[t0 * top_k:t1 * top_k]].float().reshape(t1 - t0, top_k, hidden)
        if weights is not None:
            picked = picked * weights[t0:t1].float()[:, :, None]
        out[t0:t1] = picked.sum(dim=1).to(out_dtype)
    return out


def _inverse(order: torch.Tensor) -> torch.Tensor:
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device, dtype=order.dtype)
    return inverse


def forward_pass(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor,
                 w_down: torch.Tensor, cfg: ChunkedMoEConfig, group: Optional[dist.ProcessGroup],
                 exchange: Callable) -> tuple[torch.Tensor, RoutingPlan]:
    num_tokens, hidden = x.shape
    fwd, _ = expert_fns(cfg)
    plan = make_plan(expert_ids, cfg.num_experts, cfg.slice_size, group)
    token_of_row = plan.order // cfg.top_k
    feed = SliceFeed(plan, exchange, group, x[token_of_row], x.dtype, cfg.comm_dtype)

    returned = x.new_zeros((num_tokens * cfg.top_k, hidden))
    for j, (rows,) in _lookahead(plan, (feed,)):
        y, _ = fwd(rows, w_up, w_down, plan.group_rows(j), need_residuals=False)
        exchange(y, returned, plan.combine_spec(j), group)
    out = _sum_over_choices(returned, _inverse(plan.order), num_tokens, cfg.top_k, weights, x.dtype)
    return out, plan


def backward_pass(x: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, plan: RoutingPlan,
                  g_out: torch.Tensor, cfg: ChunkedMoEConfig, group: Optional[dist.ProcessGroup], exchange: Callable):
    num_tokens, hidden = x.shape
    k = cfg.top_k
    fwd, bwd = expert_fns(cfg)
    accum = getattr(torch, cfg.accum_dtype)
    token_of_row = plan.order // k
    inverse = _inverse(plan.order)

    feeds = (
        SliceFeed(plan, exchange, group, x[token_of_row], x.dtype, cfg.comm_dtype),
        SliceFeed(plan, exchange, group, g_out.to(x.dtype)[token_of_row], x.dtype, cfg.comm_dtype),
        SliceFeed(plan, exchange, group, weights.reshape(-1)[plan.order].float()[:, None], torch.float32, None),
    )
    dx_rows = x.new_zeros((num_tokens * k, hidden))
    dweight_rows = torch.zeros((num_tokens * k, 1), dtype=torch.float32, device=x.device)
    dw_up = torch.zeros(w_up.shape, dtype=accum, device=x.device)
    dw_down = torch.zeros(w_down.shape, dtype=accum, device=x.device)

    for j, (xs, gs, ws) in _lookahead(plan, feeds):
        groups = plan.group_rows(j)
        y, saved = fwd(xs, w_up, w_down, groups)  # the slice's forward again: nothing per-slice was kept
        gs32 = gs.float()
        grads = bwd(xs, w_up, w_down, groups, saved, (ws * gs32).to(x.dtype))
        home = plan.combine_spec(j)
        exchange(grads.dx, dx_rows, home, group)
        exchange((gs32 * y.float()).sum(dim=-1, keepdim=True), dweight_rows, home, group)
        dw_up.add_(grads.dw_up)  # accumulates in `accum` whatever dtype the grouped GEMM returned
        dw_down.add_(grads.dw_down)

    dx = _sum_over_choices(dx_rows, inverse, num_tokens, k, None, x.dtype)
    d_weights = dweight_rows[inverse, 0].reshape(weights.shape).to(weights.dtype)
    return dx, d_weights, dw_up.to(w_up.dtype), dw_down.to(w_down.dtype)
