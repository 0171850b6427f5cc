"""Fused CUDA ops of the decoder around the MoE layers: residual add + RMSNorm, rotary embedding straight out of the
qkv projection, the cross-entropy of bf16 logits, the sigmoid top-k router (everything after its logits GEMM) and the dense SwiGLU. Each is one kernel per direction (`csrc/model/`) instead of a
chain of framework elementwise kernels, which took a third of a trainer step's device time. On CPU tensors (and for
dtypes other than bf16) the same functions fall back to plain torch ops with identical semantics, so the model code
has one path. The reference ships no model code; these serve `models/deepseek_tiny.py`.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def _ext():
    from .. import _build

    return _build.load()


def _fusable(*tensors: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        d2 = delta.reshape(-1, shape[-1]).contiguous() if delta is not None else None
        s, y, rstd = _ext().add_rms_norm_fwd(x2, d2, weight.contiguous(), eps)
        ctx.save_for_backward(s, weight, rstd)
        ctx.has_delta = delta is not None
        ctx.shape = shape
        ctx.set_materialize_grads(False)
        return s.reshape(shape), y.reshape(shape)

    @staticmethod
    def backward(ctx, ds_in, dy):
        s, weight, rstd = ctx.saved_tensors
        cols = ctx.shape[-1]
        if dy is None:  # the normalised output was not used
            ds = ds_in
            dw = None
        else:
            ds_flat = ds_in.reshape(-1, cols).contiguous() if ds_in is not None else None
            ds, dw = _ext().add_rms_norm_bwd(dy.reshape(-1, cols).contiguous(), ds_flat, s, weight, rstd)
            ds = ds.reshape(ctx.shape)
            dw = dw.to(weight.dtype)
        return ds, (ds if ctx.has_delta else None), dw, None


def add_rms_norm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                 eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """`s = x + delta` (just `x` without a delta) and `RMSNorm(s) * weight`, statistics in fp32."""
    if _fusable(x, weight) and (delta is None or _fusable(delta)) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 2048:
        return _AddRMSNorm.apply(x, delta, weight, eps)
    s = x if delta is None else x + delta
    return s, F.rms_norm(s, (s.shape[-1],), weight, eps)


class _RopeQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin):
        q, k, v = _ext().rope_qkv_fwd(qkv.contiguous(), cos, sin)
        ctx.save_for_backward(cos, sin)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin = ctx.saved_tensors
        return _ext().rope_qkv_bwd(dq.contiguous(), dk.contiguous(), dv.contiguous(), cos, sin), None, None


def rope_qkv(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """`qkv [B, S, 3, H, hd]` -> `(q, k, v)` as `[B, H, S, hd]`, q and k rotated pairwise (even, odd) by the position's
    angles (`cos`, `sin`: `[S, hd/2]` fp32)."""
    if _fusable(qkv) and qkv.shape[-1] % 8 == 0:
        return _RopeQKV.apply(qkv, cos.contiguous(), sin.contiguous())
    q, k, v = qkv.permute(2, 0, 3, 1, 4)

    def rot(x):
        xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
        return torch.view_as_real(xc * torch.complex(cos, sin)).flatten(-2).to(x.dtype)

    return rot(q), rot(k), v


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        loss, lse = _ext().cross_entropy_fwd(logits, targets)
        ctx.save_for_backward(logits, targets, lse)
        return loss.mean()

    @staticmethod
    def backward(ctx, grad):
        logits, targets, lse = ctx.saved_tensors
        scale = (grad.float() / logits.shape[0]).reshape(1).contiguous()
        return _ext().cross_entropy_bwd(logits, targets, lse, scale), None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of `logits [N, V]` against `targets [N]`; softmax statistics in fp32 whatever the dtype."""
    if _fusable(logits) and logits.shape[-1] % 8 == 0:
        return _CrossEntropy.apply(logits.contiguous(), targets.contiguous().long())
    return F.cross_entropy(logits.float(), targets)


class _RouterSelect(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, top_k, scaling):
        ids, weights, counts, partial = _ext().router_fwd(logits, bias, top_k, scaling)
        ctx.save_for_backward(logits, ids)
        ctx.scaling = scaling
        ctx.mark_non_differentiable(ids, counts)
        return ids, weights, counts, partial.sum(0)

    @staticmethod
    def backward(ctx, _ids, d_weights, _counts, d_score_sums):
        logits, ids = ctx.saved_tensors
        if d_weights is None:
            d_weights = torch.zeros(ids.shape, dtype=torch.float32, device=logits.device)
        if d_score_sums is None:
            d_score_sums = torch.zeros(logits.shape[1], dtype=torch.float32, device=logits.device)
        d_logits = _ext().router_bwd(logits, ids, d_weights.contiguous().float(), d_score_sums.contiguous().float(),
                                     ctx.scaling)
        return d_logits, None, None, None


def router_select(logits: torch.Tensor, bias: torch.Tensor, top_k: int,
                  scaling: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sigmoid top-k routing from fp32 `logits [T, E]`: `(ids [T, K] int32, weights [T, K], counts [E], score_sums [E])`.

    Experts are chosen by `sigmoid(logits) + bias` (the bias takes part in the selection only), `weights` are the chosen
    sigmoid scores normalised over the chosen and multiplied by `scaling`, `counts` the tokens per expert, and
    `score_sums[e]` the sum over tokens of `score[t, e] / sum_e' score[t, e']` (its mean is the balance loss's P_e).
    `weights` and `score_sums` are differentiable w.r.t. `logits`.
    """
    num_experts = logits.shape[1]
    if (logits.is_cuda and logits.dtype == torch.float32 and num_experts % 32 == 0 and num_experts <= 256
            and top_k <= 32):
        return _RouterSelect.apply(logits.contiguous(), bias.float().contiguous(), top_k, float(scaling))
    scores = torch.sigmoid(logits.float())
    _, ids = torch.topk(scores + bias, top_k, dim=-1)
    chosen = torch.gather(scores, 1, ids)
    weights = chosen / chosen.sum(-1, keepdim=True).clamp_min(1e-20) * scaling
    counts = torch.bincount(ids.reshape(-1), minlength=num_experts)
    score_sums = (scores / scores.sum(-1, keepdim=True).clamp_min(1e-20)).sum(0)
    return ids.to(torch.int32), weights, counts, score_sums


class _DenseSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return _ext().dense_swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, d_act):
        (gate_up,) = ctx.saved_tensors
        return _ext().dense_swiglu_bwd(gate_up, d_act.contiguous())


def dense_swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up` for `gate_up = [..., gate | up]` (two halves of the last dimension), one kernel per direction."""
    ffn = gate_up.shape[-1] // 2
    if _fusable(gate_up) and ffn % 8 == 0 and gate_up.shape[-1] == 2 * ffn:
        flat = gate_up.reshape(-1, 2 * ffn).contiguous()
        return _DenseSwiGLU.apply(flat).reshape(*gate_up.shape[:-1], ffn)
    gate, up = gate_up.chunk(2, dim=-1)
    return F.silu(gate) * up
