"""DeepSeek-V3-style decoder with chunked expert-parallel MoE layers.

The reference ships only the MoE layer; the model around it lived in an external MaxText branch
(the reference's top-level design document, lines 230-263: router kept from the host framework — sigmoid scores, routed bias,
routed scaling, load-balance loss, bias-update counts — then `stripe_weights` + `chunked_moe`).
This module is that host model written for this framework so the layer can be trained end to end:

  RMSNorm -> RoPE multi-head attention -> RMSNorm -> FFN
  layer 0 (`first_dense`): dense SwiGLU FFN; later layers: routed experts (`chunked_moe` over the
  expert-parallel group) + one shared SwiGLU expert.

Expert weights are stored striped (`[L, D, 2F]`, `[L, F, D]`), rank-local (rank r owns experts
`r*L .. r*L+L-1`), so no per-step re-striping happens; `ops.striping.unstripe_weights` converts
for checkpoint interchange.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..api import chunked_moe
from ..config import ChunkedMoEConfig
from .fused_ops import add_rms_norm, cross_entropy, dense_swiglu, rope_qkv, router_select


@dataclasses.dataclass
class DeepSeekTinyConfig:
    vocab_size: int = 32000
    d_model: int = 1024
    n_layers: int = 5
    n_heads: int = 16
    head_dim: int = 64
    dense_ffn: int = 4096
    first_dense: int = 1  # leading layers that use the dense FFN
    num_experts: int = 64
    moe_ffn: int = 512
    top_k: int = 6
    shared_ffn: int = 512
    routed_scaling: float = 2.5
    aux_loss_coef: float = 0.001
    bias_update_rate: float = 0.001
    rope_theta: float = 10000.0
    norm_eps: float = 1e-6
    init_std: float = 0.02
    # MoE backend
    slice_size: int = 8192
    stripe_width: int = 64
    transport: str = "nvshmem"
    expert_compute: str = "fused"
    comm_dtype: Optional[str] = None

    def moe_config(self) -> ChunkedMoEConfig:
        return ChunkedMoEConfig(num_experts=self.num_experts, top_k=self.top_k, slice_size=self.slice_size,
                                transport=self.transport, expert_compute=self.expert_compute,
                                comm_dtype=self.comm_dtype, stripe_width=self.stripe_width)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x, delta=None):
        """Returns `(s, norm(s))` with `s = x + delta` (`s = x` without a delta): the residual add that precedes every
        norm in the decoder is folded into the norm's kernel (fp32 statistics, outputs in x's dtype)."""
        return add_rms_norm(x, delta, self.weight, self.eps)


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


class Attention(nn.Module):
    def __init__(self, cfg: DeepSeekTinyConfig):
        super().__init__()
        self.n_heads, self.head_dim = cfg.n_heads, cfg.head_dim
        inner = cfg.n_heads * cfg.head_dim
        self.qkv = nn.Linear(cfg.d_model, 3 * inner, bias=False)
        self.proj = nn.Linear(inner, cfg.d_model, bias=False)

    def forward(self, x, cos, sin):
        b, s, _ = x.shape
        # q and k are rotated (pairs (even, odd) of the head dimension, fp32 arithmetic) while they are brought from
        # the projection's [B, S, 3, H, hd] layout into the attention's [B, H, S, hd]: one kernel for the three tensors
        q, k, v = rope_qkv(self.qkv(x).view(b, s, 3, self.n_heads, self.head_dim), cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(o.transpose(1, 2).reshape(b, s, -1))


class DenseSwiGLU(nn.Module):
    def __init__(self, dim: int, ffn: int):
        super().__init__()
        self.gate_up = nn.Linear(dim, 2 * ffn, bias=False)
        self.down = nn.Linear(ffn, dim, bias=False)

    def forward(self, x):
        return self.down(dense_swiglu(self.gate_up(x)))


class Router(nn.Module):
    """Sigmoid router with a (non-trained) routed bias used for selection only, and routed scaling."""

    def __init__(self, cfg: DeepSeekTinyConfig):
        super().__init__()
        self.cfg = cfg
        self.weight = nn.Parameter(torch.empty(cfg.num_experts, cfg.d_model))
        self.register_buffer("routed_bias", torch.zeros(cfg.num_experts))
        self.register_buffer("load_counts", torch.zeros(cfg.num_experts))  # bias-update counts of the step

    def _apply(self, fn, *args, **kwargs):
        # `.to(dtype=bfloat16)` must not touch the balancing state: per-expert counts in the thousands and bias steps
        # of 1e-3 both vanish in bf16 rounding. Devices still follow the module.
        keep = {name: buf for name, buf in (("routed_bias", self.routed_bias), ("load_counts", self.load_counts))}
        super()._apply(fn, *args, **kwargs)
        for name, old in keep.items():
            new = getattr(self, name)
            if new.dtype != torch.float32:
                setattr(self, name, old.to(device=new.device, dtype=torch.float32))
        return self

    def forward(self, x):
        cfg = self.cfg
        logits = F.linear(x.float(), self.weight.float())  # [T, E] fp32
        ids, weights, counts, score_sums = router_select(logits, self.routed_bias, cfg.top_k, cfg.routed_scaling)
        with torch.no_grad():
            self.load_counts += counts
        # Load-balance loss: E * sum_i f_i * P_i with f_i the routed fraction and P_i the mean normalised score.
        frac = counts.float() / max(ids.numel(), 1)
        prob = score_sums / max(ids.shape[0], 1)
        aux = cfg.aux_loss_coef * cfg.num_experts * (frac * prob).sum()
        return ids, weights, aux

    @torch.no_grad()
    def update_bias(self, group=None):
        """Aux-loss-free balancing step: nudge the selection bias against this step's load (all ranks agree)."""
        counts = self.load_counts.clone()
        if group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            dist.all_reduce(counts, group=group)
        self.routed_bias += self.cfg.bias_update_rate * torch.sign(counts.mean() - counts)
        self.load_counts.zero_()


class MoEBlock(nn.Module):
    def __init__(self, cfg: DeepSeekTinyConfig, group=None):
        super().__init__()
        self.cfg, self.group = cfg, group
        world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        if cfg.num_experts % world:
            raise ValueError(f"num_experts={cfg.num_experts} is not divisible by the EP size {world}")
        self.local_experts = cfg.num_experts // world
        self.router = Router(cfg)
        self.w_up = nn.Parameter(torch.empty(self.local_experts, cfg.d_model, 2 * cfg.moe_ffn))  # striped
        self.w_down = nn.Parameter(torch.empty(self.local_experts, cfg.moe_ffn, cfg.d_model))
        self.shared = DenseSwiGLU(cfg.d_model, cfg.shared_ffn)
        self.moe_cfg = cfg.moe_config()

    def forward(self, x):
        b, s, d = x.shape
        flat = x.reshape(b * s, d)
        ids, weights, aux = self.router(flat)
        routed = chunked_moe(flat, ids, weights, self.w_up, self.w_down, self.moe_cfg, self.group)
        return (routed + self.shared(flat)).reshape(b, s, d), aux


class Block(nn.Module):
    def __init__(self, cfg: DeepSeekTinyConfig, dense: bool, group=None):
        super().__init__()
        self.norm1, self.norm2 = RMSNorm(cfg.d_model, cfg.norm_eps), RMSNorm(cfg.d_model, cfg.norm_eps)
        self.attn = Attention(cfg)
        self.ffn = DenseSwiGLU(cfg.d_model, cfg.dense_ffn) if dense else MoEBlock(cfg, group)
        self.dense = dense

    def forward(self, x, delta, cos, sin):
        """`x` is the residual stream BEFORE `delta` (the previous block's FFN output, None for the first block) has
        been added; returns the stream before this block's own FFN output is added, that output, and the aux loss."""
        x, normed = self.norm1(x, delta)
        x, normed = self.norm2(x, self.attn(normed, cos, sin))
        if self.dense:
            return x, self.ffn(normed), x.new_zeros((), dtype=torch.float32)
        y, aux = self.ffn(normed)
        return x, y, aux


class DeepSeekTiny(nn.Module):
    def __init__(self, cfg: DeepSeekTinyConfig, group=None):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg, i < cfg.first_dense, group) for i in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        self._rope = None

    @torch.no_grad()
    def init_weights(self, seed: int, rank: int = 0):
        """Dense parameters from `seed` (identical on every rank); expert shards from `seed + 1 + global expert id`."""
        cfg = self.cfg
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("w_up") or name.endswith("w_down"):
                continue
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.copy_(torch.randn(p.shape, generator=gen) * cfg.init_std)
        for li, blk in enumerate(self.blocks):
            if blk.dense:
                continue
            moe = blk.ffn
            for l in range(moe.local_experts):
                e = rank * moe.local_experts + l
                eg = torch.Generator(device="cpu").manual_seed(seed + 1 + li * 100003 + e)
                moe.w_up[l].copy_(torch.randn(moe.w_up[l].shape, generator=eg) * cfg.init_std)
                moe.w_down[l].copy_(torch.randn(moe.w_down[l].shape, generator=eg) * cfg.init_std)

    def expert_parameters(self):
        return [p for n, p in self.named_parameters() if n.endswith("w_up") or n.endswith("w_down")]

    def dense_parameters(self):
        return [p for n, p in self.named_parameters() if not (n.endswith("w_up") or n.endswith("w_down"))]

    def routers(self):
        return [blk.ffn.router for blk in self.blocks if not blk.dense]

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        b, s = tokens.shape
        if self._rope is None or self._rope[0].shape[0] < s or self._rope[0].device != tokens.device:
            self._rope = rope_tables(s, self.cfg.head_dim, self.cfg.rope_theta, tokens.device)
        cos, sin = self._rope[0][:s], self._rope[1][:s]
        x, delta = self.embed(tokens), None
        aux_total = x.new_zeros((), dtype=torch.float32)
        for blk in self.blocks:
            x, delta, aux = blk(x, delta, cos, sin)
            aux_total = aux_total + aux
        _, normed = self.norm(x, delta)
        logits = self.lm_head(normed)
        if targets is None:
            return logits, aux_total
        return cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1)), aux_total
