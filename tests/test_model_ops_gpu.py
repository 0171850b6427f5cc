"""The decoder's fused CUDA ops (residual add + RMSNorm, rotary embedding out of qkv, cross-entropy of bf16 logits)
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
