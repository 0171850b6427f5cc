"""Shared input builders for layer-vs-oracle tests."""

import math

import torch


def routing(gen, num_tokens, num_experts, top_k, skew, score="softmax"):
    """Top-k expert ids and combine weights; `skew` reproduces the reference's stress cases."""
    logits = torch.randn(num_tokens, num_experts, generator=gen)
    if skew == "all_one":  # every token's first choice is expert 0
        logits[:, 0] += 100.0
    elif skew == "rank0":  # every copy goes to the first quarter of the experts
        logits[:, : num_experts // 4] += 100.0
    if score == "softmax":
        weights, ids = torch.topk(torch.softmax(logits, dim=-1), top_k, dim=-1)
    elif score == "softmax_chosen":  # softmax over the chosen logits
        top, ids = torch.topk(logits, top_k, dim=-1)
        weights = torch.softmax(top, dim=-1)
    else:  # sigmoid scores normalised over the chosen k
        scores, ids = torch.topk(torch.sigmoid(logits), top_k, dim=-1)
        weights = scores / scores.sum(-1, keepdim=True)
    return ids.to(torch.int32), weights


def setup(ep, tokens_per_rank, num_experts, top_k, hidden, ffn, skew, seed=0, w_std=None, score="softmax"):
    gen = torch.Generator().manual_seed(seed)
    n = ep * tokens_per_rank
    x = torch.randn(n, hidden, generator=gen)
    ids, weights = routing(gen, n, num_experts, top_k, skew, score)
    if w_std is None:
        w_up = torch.randn(num_experts, hidden, 2 * ffn, generator=gen) / math.sqrt(hidden)
        w_down = torch.randn(num_experts, ffn, hidden, generator=gen) / math.sqrt(ffn)
    else:
        w_up = torch.randn(num_experts, hidden, 2 * ffn, generator=gen) * w_std
        w_down = torch.randn(num_experts, ffn, hidden, generator=gen) * w_std
    g = torch.randn(n, hidden, generator=gen)
    return x, ids, weights, w_up, w_down, g


def oracle(x, ids, weights, w_up, w_down, g, stripe):
    """Forward and the four gradients of sum(out * g) from the dense fp32 oracle."""
    from chunked_ep_moe_b200 import reference_moe

    xs, ws, us, ds = (t.clone().requires_grad_(True) for t in (x, weights, w_up, w_down))
    out = reference_moe(xs, ids, ws, us, ds, stripe=stripe)
    (out * g).sum().backward()
    return {"out": out.detach(), "dx": xs.grad, "dweights": ws.grad, "dw_up": us.grad, "dw_down": ds.grad}


def shard(t, rank, world):
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n].contiguous()
