"""Each fused sm_100a GEMM mode on its own against the plain torch implementation of the same op.

Follows the reference's kernel tests (tests/test_fused_kernels.py:18-67): forward intermediates `h`, `act`, `y` and
backward results `dx`, `dW_up`, `dW_down` one by one, bf16, tolerance 3e-2 of max-abs, group shapes with a partial
slice, an empty expert and a one-row expert; padding rows are poisoned with NaN and must not reach any result. Beyond
the reference's toy width the same checks run at real contraction depth (D=2048/F=1024, and D=7168/F=2048, the
DeepSeek-V3 expert), where a tile accumulates over 112 k-blocks.
"""

import math

import pytest
import torch

from chunked_ep_moe_b200.ops import expert as ref
from chunked_ep_moe_b200.ops import fused_expert as fx

pytestmark = pytest.mark.gpu

TOL = 3e-2

SHAPES = [
    # rows S, D, F, stripe, rows per expert
    (128, 256, 256, 128, [40, 0, 70]),      # partial slice (18 padding rows), empty expert
    (128, 256, 256, 64, [64, 1, 63]),       # full slice, one-row expert
    (512, 2048, 1024, 64, [130, 0, 255, 127]),
    (1024, 7168, 2048, 64, [300, 1, 270, 453]),
]


def _close(got, want, name, rows=None):
    got, want = got.float(), want.float()
    if rows is not None:
        got, want = got[:rows], want[:rows]
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    err = (got - want).abs().max() / want.abs().max().clamp_min(1e-6)
    assert err <= TOL, f"{name}: max abs err {err:.4f} x max-abs (allowed {TOL})"


def _inputs(S, D, F, groups, seed=0):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    L, rows = len(groups), sum(groups)
    bf = torch.bfloat16
    x = torch.randn(S, D, generator=gen, device="cuda").to(bf)
    dy = torch.randn(S, D, generator=gen, device="cuda").to(bf)
    x[rows:] = float("nan")  # padding rows: whatever they hold must never matter
    dy[rows:] = float("nan")
    w_up = (torch.randn(L, D, 2 * F, generator=gen, device="cuda") / math.sqrt(D)).to(bf)
    w_down = (torch.randn(L, F, D, generator=gen, device="cuda") / math.sqrt(F)).to(bf)
    return x, dy, w_up, w_down, rows


@pytest.mark.parametrize("pairs", ["0", "1"], ids=["single", "pairs"])
@pytest.mark.parametrize("S,D,F,stripe,groups", SHAPES, ids=lambda v: str(v) if not isinstance(v, list) else "g")
def test_every_mode_matches_torch(S, D, F, stripe, groups, pairs, monkeypatch):
    monkeypatch.setenv("CEM_CTA_PAIRS", pairs)
    fx._runners.clear()
    x, dy, w_up, w_down, rows = _inputs(S, D, F, groups)
    sizes = torch.tensor(groups)

    # forward: act and h from the up-projection kernel, y from the plain grouped GEMM
    act, h = fx.gmm_swiglu(x, w_up, groups, stripe=stripe, return_h=True)
    want_h = ref.gmm(x, w_up, sizes, x.dtype)
    want_act = ref.striped_swiglu(want_h, stripe)
    _close(h, want_h, "h", rows)
    _close(act, want_act, "act", rows)
    y = fx.gmm(want_act, w_down, groups, stripe=stripe)
    _close(y, ref.gmm(want_act, w_down, sizes, x.dtype), "y", rows)
    act_only, none = fx.gmm_swiglu(x, w_up, groups, stripe=stripe)
    assert none is None
    _close(act_only, want_act, "act (no h)", rows)

    # backward, every kernel fed with the torch intermediates so that one kernel's error cannot hide another's
    want_dh = ref.striped_swiglu_bwd(want_h, ref.gmm(dy, w_down, sizes, x.dtype, transpose_rhs=True), stripe)
    dh = fx.gmm_dswiglu(dy, w_down, want_h, groups, stripe=stripe)
    _close(dh, want_dh, "dh", rows)
    dx = fx.gmm(want_dh, w_up, groups, transpose_rhs=True, stripe=stripe)
    _close(dx, ref.gmm(want_dh, w_up, sizes, x.dtype, transpose_rhs=True), "dx", rows)
    poisoned_act = want_act.clone()
    poisoned_act[rows:] = float("nan")
    poisoned_dh = want_dh.clone()
    poisoned_dh[rows:] = float("nan")
    dw_down = fx.tgmm(poisoned_act, dy, groups, stripe=stripe)
    _close(dw_down, ref.tgmm(want_act[:rows], dy[:rows], sizes), "dW_down")
    dw_up = fx.tgmm(x, poisoned_dh, groups, stripe=stripe)
    _close(dw_up, ref.tgmm(x[:rows], want_dh[:rows], sizes), "dW_up")
    for l, n in enumerate(groups):
        if n == 0:
            assert float(dw_up[l].abs().max()) == 0.0 and float(dw_down[l].abs().max()) == 0.0
    fx.check_status()


@pytest.mark.parametrize("S,D,F,stripe,groups", SHAPES[:3], ids=lambda v: str(v) if not isinstance(v, list) else "g")
def test_expert_forward_backward_wrappers(S, D, F, stripe, groups):
    """`expert_forward` / `expert_backward` (residual-consuming, nothing recomputed) against the torch pair."""
    fx._runners.clear()
    x, dy, w_up, w_down, rows = _inputs(S, D, F, groups, seed=3)
    sizes = torch.tensor(groups)
    y, res = fx.expert_forward(x, w_up, w_down, groups, stripe=stripe)
    want_y, want_res = ref.expert_forward(x[:rows], w_up, w_down, sizes, stripe=stripe)
    _close(y, want_y, "y", rows)
    _close(res.h, want_res.h, "h", rows)
    _close(res.act, want_res.act, "act", rows)
    grads = fx.expert_backward(x, w_up, w_down, groups, res, dy, stripe=stripe)
    want = ref.expert_backward(x[:rows], w_up, w_down, sizes, want_res, dy[:rows], stripe=stripe)
    _close(grads.dx, want.dx, "dx", rows)
    _close(grads.dw_up, want.dw_up, "dW_up")
    _close(grads.dw_down, want.dw_down, "dW_down")
    y_only, none = fx.expert_forward(x, w_up, w_down, groups, stripe=stripe, need_residuals=False)
    assert none is None
    _close(y_only, want_y, "y (no residuals)", rows)
    fx.check_status()


def test_down_gemm_with_d_weight_epilogue():
    """The backward's recomputed down-projection: `dy = w * g` and the per-tile partial sums of `<g, act W_down>`."""
    from chunked_ep_moe_b200 import _build

    S, D, F, stripe, groups = 256, 1024, 512, 64, [100, 0, 90, 40]
    fx._runners.clear()
    x, g, w_up, w_down, rows = _inputs(S, D, F, groups, seed=5)
    sizes = torch.tensor(groups)
    act = ref.striped_swiglu(ref.gmm(x, w_up, sizes, x.dtype), stripe)
    act[rows:] = float("nan")
    w = torch.rand(S, device="cuda") + 0.1
    runner = fx._prepare(act, len(groups), groups, stripe)
    dy = torch.zeros_like(g)
    dwp = torch.zeros(S, D // 256, device="cuda")
    runner.gmm_down_dw(act, w_down, g, w, dy, dwp)
    torch.cuda.synchronize()
    y = ref.gmm(act[:rows], w_down, sizes, x.dtype)
    _close(dy, (w[:, None] * g.float()).to(g.dtype), "dy", rows)
    _close(dwp.sum(dim=1), (g[:rows].float() * y.float()).sum(dim=-1), "d_weight", rows)
    fx.check_status()
    del _build
