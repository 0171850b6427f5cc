"""Per-slice expert MLP on an expert-major slice: library (torch) implementation.

This is the `expert_compute="reference"` backend: grouped GEMMs through
`torch.nn.functional.grouped_mm` on CUDA (bf16/fp16) and through a per-group
loop everywhere else (CPU, fp32). It is the oracle for the fused sm_100a
kernels and the compute half of the NCCL baseline. Same contract as the
reference's `expert_forward` / `expert_backward`
(src/chunked_moe/expert.py:81-108): rows past `sum(group_sizes)` are padding
and are neither read for weight gradients nor given defined outputs.
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import numpy as np
import torch
import torch.nn.functional as F

from .striping import striped_swiglu, striped_swiglu_bwd


class ForwardResiduals(NamedTuple):
    h: torch.Tensor  # [S, 2F] striped pre-activation, stored in x.dtype
    act: torch.Tensor  # [S, F]


class ExpertGrads(NamedTuple):
    dx: torch.Tensor  # [S, D]
    dw_up: torch.Tensor  # [L, D, 2F] float32
    dw_down: torch.Tensor  # [L, F, D] float32


def _use_library_grouped_mm(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in (torch.bfloat16, torch.float16) and hasattr(F, "grouped_mm")


def _host_rows(group_sizes) -> np.ndarray:
    """Group sizes as a host array. The collective paths pass host values (their plan lives on the host), so nothing
    is read back from the device; a device tensor is accepted too and costs one synchronising copy."""
    if isinstance(group_sizes, torch.Tensor):
        return group_sizes.detach().cpu().numpy().astype(np.int64)
    return np.asarray(group_sizes, dtype=np.int64)


def _group_bounds(group_sizes) -> list[tuple[int, int]]:
    ends = np.cumsum(_host_rows(group_sizes))
    return [(int(e - n), int(e)) for e, n in zip(ends, _host_rows(group_sizes))]


def _group_ends(group_sizes, device: torch.device) -> torch.Tensor:
    """int32 end offset of every group, on `device` (what the library grouped GEMM takes)."""
    return torch.from_numpy(np.cumsum(_host_rows(group_sizes)).astype(np.int32)).to(device, non_blocking=True)


def gmm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes, out_dtype: torch.dtype,
        transpose_rhs: bool = False) -> torch.Tensor:
    """Grouped GEMM: rows of `lhs` in group g multiply `rhs[g]` (or `rhs[g]^T`), fp32 accumulate.

    Rows past `sum(group_sizes)` come back as zeros here; callers must treat
    them as undefined (the fused kernels never write them).
    """
    rhs_g = rhs.transpose(1, 2) if transpose_rhs else rhs
    if _use_library_grouped_mm(lhs):
        out = F.grouped_mm(lhs, rhs_g, offs=_group_ends(group_sizes, lhs.device))
        return out.to(out_dtype)
    out = lhs.new_zeros((lhs.shape[0], rhs_g.shape[2]), dtype=out_dtype)
    for g, (a, b) in enumerate(_group_bounds(group_sizes)):
        if b > a:
            out[a:b] = (lhs[a:b].float() @ rhs_g[g].float()).to(out_dtype)
    return out


def tgmm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes) -> torch.Tensor:
    """Per-group `lhs[rows_g]^T @ rhs[rows_g]` -> `[G, lhs_cols, rhs_cols]` (fp32 accumulate; fp32 out off the library path).

    Only rows inside a group are read, so NaN-poisoned padding rows cannot leak
    into a weight gradient (the reference masks with select for the same
    reason, src/chunked_moe/kernels/fused_expert.py:301-324).
    """
    num_groups = len(group_sizes)
    if _use_library_grouped_mm(lhs):
        # Ragged contraction dim: [cols_l, rows] x [rows, cols_r] with offsets over rows -> [G, cols_l, cols_r].
        return F.grouped_mm(lhs.t(), rhs, offs=_group_ends(group_sizes, lhs.device))  # library output dtype
    out = lhs.new_zeros((num_groups, lhs.shape[1], rhs.shape[1]), dtype=torch.float32)
    for g, (a, b) in enumerate(_group_bounds(group_sizes)):
        if b > a:
            out[g] = lhs[a:b].float().t() @ rhs[a:b].float()
    return out


def expert_forward(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, group_sizes, *,
                   stripe: int, need_residuals: bool = True) -> tuple[torch.Tensor, Optional[ForwardResiduals]]:
    """x: `[S, D]` expert-major slice -> y: `[S, D]` (+ residuals for the backward)."""
    h = gmm(x, w_up, group_sizes, x.dtype)
    act = striped_swiglu(h, stripe)
    y = gmm(act, w_down, group_sizes, x.dtype)
    return y, (ForwardResiduals(h, act) if need_residuals else None)


def expert_backward(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, group_sizes,
                    res: ForwardResiduals, dy: torch.Tensor, *, stripe: int) -> ExpertGrads:
    """Backward of `expert_forward` for one slice: dX rows and fp32 per-expert weight gradients."""
    # Chain towards the input: dy -> d_act -> dh -> dx; each weight gradient contracts the rows of its group between
    # the layer's input-side activation and output-side gradient (act^T dy, x^T dh).
    dh = striped_swiglu_bwd(res.h, gmm(dy, w_down, group_sizes, x.dtype, transpose_rhs=True), stripe)
    return ExpertGrads(dx=gmm(dh, w_up, group_sizes, x.dtype, transpose_rhs=True),
                       dw_up=tgmm(x, dh, group_sizes),
                       dw_down=tgmm(res.act, dy, group_sizes))
