"""Dense single-device MoE used as the numerical oracle.

Same definition as the reference oracle (src/chunked_moe/reference.py:9-15):
fp32 everywhere (nothing is rounded to the input dtype until the final cast),
so it bounds the error of every lower-precision path. Written per expert (loop over E with index_add) so it also
runs at sizes where gathering `w_up[ids]` would not fit in memory.
"""

from __future__ import annotations

import torch

from .striping import striped_swiglu


def reference_moe(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor,
                  w_down: torch.Tensor, *, stripe: int) -> torch.Tensor:
    """x: `[N, D]`, expert_ids / weights: `[N, K]`, w_up: `[E, D, 2F]` striped (global), w_down: `[E, F, D]`."""
    n, _ = x.shape
    num_experts = w_up.shape[0]
    xf = x.float()
    out = torch.zeros_like(xf)
    flat_ids = expert_ids.reshape(-1)
    flat_w = weights.reshape(-1).float()
    token = torch.arange(n, device=x.device).repeat_interleave(expert_ids.shape[1])
    for e in range(num_experts):
        sel = (flat_ids == e).nonzero(as_tuple=True)[0]
        if sel.numel() == 0:
            continue
        tok = token[sel]
        h = xf[tok] @ w_up[e].float()
        act = striped_swiglu(h, stripe)
        y = act @ w_down[e].float()
        out = out.index_add(0, tok, y * flat_w[sel][:, None])
    return out.to(x.dtype)
