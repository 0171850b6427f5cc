"""The decoder's fused CUDA ops (residual add + RMSNorm, rotary embedding out of qkv, cross-entropy of bf16 logits, router)
against plain PyTorch fp32 references of the same ops, forward and backward."""

import pytest
import torch
import torch.nn.functional as F

from chunked_ep_moe_b200.models import fused_ops

pytestmark = pytest.mark.gpu


def _close(got, want, name, tol):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    err = (got - want).abs().max() / want.abs().max().clamp_min(1e-6)
    assert err <= tol, f"{name}: max abs err {err:.5f} x max-abs (allowed {tol})"


@pytest.mark.parametrize("rows,cols,with_delta", [(300, 1024, True), (64, 2048, True), (129, 256, False)])
def test_add_rms_norm(rows, cols, with_delta):
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", generator=gen).bfloat16().requires_grad_(True)
    delta = torch.randn(rows, cols, device="cuda", generator=gen).bfloat16().requires_grad_(True) if with_delta else None
    w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=gen)).bfloat16().requires_grad_(True)
    gs = torch.randn(rows, cols, device="cuda", generator=gen).bfloat16()
    gy = torch.randn(rows, cols, device="cuda", generator=gen).bfloat16()
    s, y = fused_ops.add_rms_norm(x, delta, w, 1e-6)
    (s.float() * gs.float()).sum().add((y.float() * gy.float()).sum()).backward()
    xr = x.detach().float().requires_grad_(True)
    dr = delta.detach().float().requires_grad_(True) if with_delta else None
    wr = w.detach().float().requires_grad_(True)
    sr = xr
    if with_delta:  # the sum is stored rounded to bf16; gradients pass straight through the rounding
        sr = xr + dr + ((xr + dr).detach().bfloat16().float() - (xr + dr).detach())
    yr = sr * torch.rsqrt(sr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    (sr * gs.float()).sum().add((yr * gy.float()).sum()).backward()
    _close(s, sr.detach(), "s", 1e-2)
    _close(y, yr.detach(), "y", 1e-2)
    _close(x.grad, xr.grad, "dx", 2e-2)
    if with_delta:
        _close(delta.grad, dr.grad, "ddelta", 2e-2)
    _close(w.grad, wr.grad, "dweight", 2e-2)


def test_rope_qkv():
    B, S, H, hd = 2, 96, 4, 64
    gen = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn(B, S, 3, H, hd, device="cuda", generator=gen).bfloat16().requires_grad_(True)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(S, device="cuda", dtype=torch.float32), inv)
    cos, sin = ang.cos(), ang.sin()
    g = [torch.randn(B, H, S, hd, device="cuda", generator=gen).bfloat16() for _ in range(3)]
    q, k, v = fused_ops.rope_qkv(qkv, cos, sin)
    sum((t.float() * gi.float()).sum() for t, gi in zip((q, k, v), g)).backward()

    ref = qkv.detach().float().requires_grad_(True)
    rq, rk, rv = ref.permute(2, 0, 3, 1, 4)

    def rot(x):
        xc = torch.view_as_complex(x.reshape(*x.shape[:-1], -1, 2).contiguous())
        return torch.view_as_real(xc * torch.complex(cos, sin)).flatten(-2)

    outs = (rot(rq), rot(rk), rv)
    sum((t * gi.float()).sum() for t, gi in zip(outs, g)).backward()
    for name, a, b in zip("qkv", (q, k, v), outs):
        _close(a, b.detach(), name, 1e-2)
    _close(qkv.grad, ref.grad, "dqkv", 1e-2)


@pytest.mark.parametrize("rows,cols", [(257, 32000), (16, 1024)])
def test_cross_entropy(rows, cols):
    gen = torch.Generator(device="cuda").manual_seed(2)
    logits = (3 * torch.randn(rows, cols, device="cuda", generator=gen)).bfloat16().requires_grad_(True)
    targets = torch.randint(0, cols, (rows,), device="cuda", generator=gen)
    loss = fused_ops.cross_entropy(logits, targets)
    (loss * 1.7).backward()
    ref = logits.detach().float().requires_grad_(True)
    want = F.cross_entropy(ref, targets)
    (want * 1.7).backward()
    assert abs(float(loss) - float(want)) <= 1e-3 * max(1.0, abs(float(want)))
    _close(logits.grad, ref.grad, "dlogits", 1e-2)


@pytest.mark.parametrize("tokens,experts,top_k", [(1000, 64, 6), (8192, 256, 8), (7, 32, 1), (333, 96, 5)])
def test_router_select(tokens, experts, top_k):
    """Selection, weights, load counts, score sums and the gradient w.r.t. the logits against fp64 torch ops."""
    gen = torch.Generator(device="cuda").manual_seed(tokens + experts)
    logits = torch.randn(tokens, experts, generator=gen, device="cuda").requires_grad_(True)
    bias = 0.1 * torch.randn(experts, generator=gen, device="cuda")
    gw = torch.randn(tokens, top_k, generator=gen, device="cuda")
    gs = torch.randn(experts, generator=gen, device="cuda")
    scaling = 2.5
    ids, weights, counts, sums = fused_ops.router_select(logits, bias, top_k, scaling)
    ((weights * gw).sum() + (sums * gs).sum()).backward()
    assert ids.dtype == torch.int32 and tuple(ids.shape) == (tokens, top_k)

    ref_logits = logits.detach().double().requires_grad_(True)
    scores = torch.sigmoid(ref_logits)
    keys = (scores + bias.double()).detach()
    picked = torch.gather(keys, 1, ids.long())
    # a valid top-k: distinct experts, in descending order of score + bias, none of the others beats the last one
    assert (torch.sort(ids.long(), dim=1).values.diff(dim=1) > 0).all() or top_k == 1
    assert (picked.diff(dim=1) <= 1e-6).all()
    rest = keys.scatter(1, ids.long(), float("-inf"))
    assert (rest.max(dim=1).values <= picked[:, -1] + 1e-6).all()
    chosen = torch.gather(scores, 1, ids.long())
    ref_weights = chosen / chosen.sum(-1, keepdim=True).clamp_min(1e-20) * scaling
    ref_sums = (scores / scores.sum(-1, keepdim=True).clamp_min(1e-20)).sum(0)
    ((ref_weights * gw.double()).sum() + (ref_sums * gs.double()).sum()).backward()
    torch.testing.assert_close(weights.double(), ref_weights.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(counts.long(), torch.bincount(ids.long().reshape(-1), minlength=experts))
    torch.testing.assert_close(sums.double(), ref_sums.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(logits.grad.double(), ref_logits.grad, rtol=1e-4, atol=1e-6)


def test_router_select_is_deterministic():
    gen = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(4096, 64, generator=gen, device="cuda")
    bias = torch.zeros(64, device="cuda")
    a = fused_ops.router_select(logits, bias, 6, 1.0)
    b = fused_ops.router_select(logits, bias, 6, 1.0)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("rows,ffn", [(300, 512), (8192, 2048), (5, 8)])
def test_dense_swiglu(rows, ffn):
    gen = torch.Generator(device="cuda").manual_seed(rows)
    gu = torch.randn(rows, 2 * ffn, device="cuda", generator=gen).bfloat16().requires_grad_(True)
    go = torch.randn(rows, ffn, device="cuda", generator=gen).bfloat16()
    out = fused_ops.dense_swiglu(gu)
    out.backward(go)
    ref_in = gu.detach().float().requires_grad_(True)
    gate, up = ref_in.chunk(2, dim=-1)
    ref = F.silu(gate) * up
    ref.backward(go.float())
    _close(out, ref, "act", 1e-2)
    _close(gu.grad, ref_in.grad, "d_gate_up", 1e-2)
