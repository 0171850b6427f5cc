"""Striped gate/up weight layout and striped SwiGLU (plain torch).

`w_up` is `[L, D, 2F]` with gate and up columns interleaved in stripes of
`stripe` columns: `[gate 0:s | up 0:s | gate s:2s | up s:2s | ...]`, so one
contiguous N-tile of `2*s` columns holds a gate stripe next to its up stripe
and a GEMM epilogue can apply SwiGLU before anything reaches HBM. stripe=1 is
the per-column interleave. Mirrors the reference's layout helpers
(src/chunked_moe/expert.py:22-45, :65-78).
"""

from __future__ import annotations

import torch


def split_stripes(h: torch.Tensor, stripe: int) -> tuple[torch.Tensor, torch.Tensor]:
    """`[..., 2F]` striped -> (`[..., F]` gate, `[..., F]` up)."""
    two_f = h.shape[-1]
    if two_f % 2:
        raise ValueError(f"striped width {two_f} is odd")
    ffn = two_f // 2
    if ffn % stripe:
        raise ValueError(f"ffn dim {ffn} is not a multiple of stripe={stripe}")
    v = h.reshape(*h.shape[:-1], ffn // stripe, 2, stripe)
    return v[..., 0, :].reshape(*h.shape[:-1], ffn), v[..., 1, :].reshape(*h.shape[:-1], ffn)


def join_stripes(gate: torch.Tensor, up: torch.Tensor, stripe: int) -> torch.Tensor:
    """Inverse of `split_stripes`."""
    ffn = gate.shape[-1]
    if gate.shape != up.shape:
        raise ValueError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} differ")
    if ffn % stripe:
        raise ValueError(f"ffn dim {ffn} is not a multiple of stripe={stripe}")
    g = gate.reshape(*gate.shape[:-1], ffn // stripe, 1, stripe)
    u = up.reshape(*up.shape[:-1], ffn // stripe, 1, stripe)
    return torch.cat([g, u], dim=-2).reshape(*gate.shape[:-1], 2 * ffn)


def stripe_weights(w_gate: torch.Tensor, w_up: torch.Tensor, stripe: int) -> torch.Tensor:
    """`[L, D, F]` gate and `[L, D, F]` up -> `[L, D, 2F]` striped (contiguous)."""
    return join_stripes(w_gate, w_up, stripe).contiguous()


def unstripe_weights(w_striped: torch.Tensor, stripe: int) -> tuple[torch.Tensor, torch.Tensor]:
    """`[L, D, 2F]` striped -> (`[L, D, F]` gate, `[L, D, F]` up); checkpoint interchange format."""
    gate, up = split_stripes(w_striped, stripe)
    return gate.contiguous(), up.contiguous()


def striped_swiglu(h: torch.Tensor, stripe: int) -> torch.Tensor:
    """`act = silu(gate) * up`, evaluated in fp32 on the (already rounded) `h`, cast back to h.dtype."""
    gate, up = split_stripes(h.float(), stripe)
    return (torch.nn.functional.silu(gate) * up).to(h.dtype)


def striped_swiglu_bwd(h: torch.Tensor, d_act: torch.Tensor, stripe: int) -> torch.Tensor:
    """Gradient of `striped_swiglu` w.r.t. its striped input `h` (same striping as `h`), evaluated in fp32.

    With s = sigmoid(gate): d(silu)/d(gate) = s * (1 + gate * (1 - s)), so
    `d_gate = d_act * up * s * (1 + gate * (1 - s))` and `d_up = d_act * gate * s`.
    """
    gate, up = split_stripes(h.float(), stripe)
    s = torch.sigmoid(gate)
    scaled = d_act.float() * s
    return join_stripes(scaled * up * (1.0 + gate * (1.0 - s)), scaled * gate, stripe).to(h.dtype)
