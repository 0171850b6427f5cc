"""The fused sm_100a expert kernels one at a time: `gmm`, `gmm_swiglu`, `gmm_dswiglu`, `tgmm`, and the per-slice
`expert_forward` / `expert_backward` built from them.

Same kernel-level surface as the reference's fused backend (src/chunked_moe/kernels/fused_expert.py:102-366): every
function takes an expert-major slice of at most S rows plus the rows per expert, runs ONE tcgen05 grouped-GEMM mode
of `csrc/gemm/grouped_gemm.cu` on it, and returns tensors the caller owns. Rows past `sum(group_sizes)` are padding:
they are never read into a weight gradient and their outputs are left as allocated (zeros here).

This is what `expert_compute="fused"` runs under a COLLECTIVE transport (`ragged_a2a`, `emulated` on a GPU): the
exchange delivers a slice, these kernels compute on it, and the residuals (`h`, `act`) of the forward are handed to
the backward, so nothing is recomputed. Inside the NVLink path the same modes run fused with the transport
(`ops/fused.py`). The kernel tests compare each function with `ops/expert.py`.
"""

from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch

from .. import _build
from ..config import B200_NUM_SMS
from .expert import ExpertGrads, ForwardResiduals

_runners: dict = {}


def _group_tensor(group_sizes, device) -> torch.Tensor:
    if isinstance(group_sizes, torch.Tensor):
        return group_sizes.to(device=device, dtype=torch.int32).contiguous()
    return torch.from_numpy(np.asarray(group_sizes, dtype=np.int32)).to(device, non_blocking=True)


def _runner(num_groups: int, rows: int, stripe: int, device: torch.device):
    """The cached launcher for slices of `rows` rows and `num_groups` experts (tile tables live in it)."""
    key = (num_groups, rows, stripe, device.index)
    runner = _runners.get(key)
    if runner is None:
        ext = _build.load()
        pairs = os.environ.get("CEM_CTA_PAIRS", "0") != "0"
        runner = ext.KernelRunner(num_groups, rows, stripe, int(os.environ.get("CEM_GEMM_GRID", B200_NUM_SMS)), pairs)
        _runners[key] = runner
    return runner


def _prepare(rows_tensor: torch.Tensor, num_groups: int, group_sizes, stripe: int):
    if rows_tensor.shape[0] % 8:
        raise ValueError(f"the fused kernels need a multiple of 8 rows per slice, got {rows_tensor.shape[0]}")
    runner = _runner(num_groups, rows_tensor.shape[0], stripe, rows_tensor.device)
    runner.set_groups(_group_tensor(group_sizes, rows_tensor.device))
    return runner


def gmm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes, *, transpose_rhs: bool = False,
        stripe: int = 64) -> torch.Tensor:
    """`out[rows_g] = lhs[rows_g] @ rhs[g]` (`rhs [L, K, N]`), or `@ rhs[g]^T` (`rhs [L, N, K]`) with `transpose_rhs`."""
    runner = _prepare(lhs, rhs.shape[0], group_sizes, stripe)
    out = lhs.new_zeros((lhs.shape[0], rhs.shape[1] if transpose_rhs else rhs.shape[2]))
    runner.gmm(lhs.contiguous(), rhs.contiguous(), out, transpose_rhs)
    return out


def gmm_swiglu(x: torch.Tensor, w_up: torch.Tensor, group_sizes, *, stripe: int,
               return_h: bool = False) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
    """`act = silu(x Wg) * (x Wu)` from the striped `w_up [L, D, 2F]`; with `return_h` also the rounded `h [S, 2F]`."""
    runner = _prepare(x, w_up.shape[0], group_sizes, stripe)
    act = x.new_zeros((x.shape[0], w_up.shape[2] // 2))
    h = x.new_zeros((x.shape[0], w_up.shape[2])) if return_h else None
    runner.gmm_swiglu(x.contiguous(), w_up.contiguous(), act, h)
    return act, h


def gmm_dswiglu(dy: torch.Tensor, w_down: torch.Tensor, h: torch.Tensor, group_sizes, *, stripe: int) -> torch.Tensor:
    """`dh = SwiGLU'(h) * (dy @ w_down[g]^T)`: the gradient of the striped pre-activation; `d_act` never leaves the SM."""
    runner = _prepare(dy, w_down.shape[0], group_sizes, stripe)
    dh = torch.zeros_like(h)
    runner.gmm_dswiglu(dy.contiguous(), w_down.contiguous(), h.contiguous(), dh)
    return dh


def tgmm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes, *, stripe: int = 64) -> torch.Tensor:
    """`out[g] = lhs[rows_g]^T @ rhs[rows_g]` -> `[L, lhs_cols, rhs_cols]` (bf16; fp32 accumulation over the rows)."""
    num_groups = len(group_sizes)
    runner = _prepare(lhs, num_groups, group_sizes, stripe)
    out = lhs.new_empty((num_groups, lhs.shape[1], rhs.shape[1]))
    runner.tgmm(lhs.contiguous(), rhs.contiguous(), out)
    return out


def expert_forward(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, group_sizes, *, stripe: int,
                   need_residuals: bool = True) -> tuple[torch.Tensor, Optional[ForwardResiduals]]:
    act, h = gmm_swiglu(x, w_up, group_sizes, stripe=stripe, return_h=need_residuals)
    y = gmm(act, w_down, group_sizes, stripe=stripe)
    return y, (ForwardResiduals(h=h, act=act) if need_residuals else None)


def expert_backward(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, group_sizes, res: ForwardResiduals,
                    dy: torch.Tensor, *, stripe: int) -> ExpertGrads:
    dh = gmm_dswiglu(dy, w_down, res.h, group_sizes, stripe=stripe)
    return ExpertGrads(dx=gmm(dh, w_up, group_sizes, transpose_rhs=True, stripe=stripe),
                       dw_up=tgmm(x, dh, group_sizes, stripe=stripe),
                       dw_down=tgmm(res.act, dy, group_sizes, stripe=stripe))


def check_status() -> None:
    """Synchronises and raises if a kernel launched through this module recorded an error."""
    for runner in _runners.values():
        runner.check_status()
