"""Wire quantisation of token rows: e4m3 values with one fp32 scale per 1x128 block (plain torch).

The reference quantises with one absmax scale per row
(src/chunked_moe/moe.py:56-69); this build uses the tighter 1x128-block
format: each row is cut into blocks of 128 columns (one block spanning the
whole row when the width is not a multiple of 128) and every block carries
`scale = max(amax, 1e-12) / 448`. Rows are quantised once per pass, so the
forward and the backward's recomputed forward see identical values.
"""

from __future__ import annotations

from typing import Optional

import torch

BLOCK = 128
E4M3_MAX = 448.0


def comm_torch_dtype(comm_dtype: Optional[str]) -> Optional[torch.dtype]:
    if comm_dtype is None:
        return None
    if comm_dtype == "float8_e4m3fn":
        return torch.float8_e4m3fn
    raise ValueError(f"unsupported comm_dtype {comm_dtype!r}")


def block_width(hidden: int) -> int:
    return BLOCK if hidden % BLOCK == 0 else hidden


def quantize_rows(x: torch.Tensor, comm_dtype: Optional[str]) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
    """`[n, D]` -> (`[n, D]` e4m3 values, `[n, D/128]` fp32 scales); identity when `comm_dtype` is None."""
    dt = comm_torch_dtype(comm_dtype)
    if dt is None:
        return x, None
    n, hidden = x.shape
    blk = block_width(hidden)
    xf = x.float().reshape(n, hidden // blk, blk)
    amax = xf.abs().amax(dim=-1)
    scale = torch.clamp(amax, min=1e-12) / E4M3_MAX
    q = (xf / scale[..., None]).clamp_(-E4M3_MAX, E4M3_MAX).to(dt).reshape(n, hidden)
    return q, scale


def dequantize_rows(q: torch.Tensor, scale: Optional[torch.Tensor], dtype: torch.dtype) -> torch.Tensor:
    if scale is None:
        return q
    n, hidden = q.shape
    blk = hidden // scale.shape[1]
    return (q.float().reshape(n, scale.shape[1], blk) * scale[..., None]).reshape(n, hidden).to(dtype)
