"""The sampled fp32 check (`utils/verify.py`) on CPU ranks: a correct step passes with tiny errors on 1 and on 4
ranks, and a damaged output row, weight gradient or router-weight gradient is caught."""

import torch

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe
from chunked_ep_moe_b200.utils.verify import sampled_check

import moe_cases
from dist_utils import run_ranks

DIMS = (24, 8, 2, 16, 24)  # tokens/rank, E, K, D, F
STRIPE = 4


def _step(rank, world, damage):
    tokens, experts, top_k, hidden, ffn = DIMS
    cfg = ChunkedMoEConfig(num_experts=experts, top_k=top_k, slice_size=16, transport="emulated", stripe_width=STRIPE)
    x, ids, weights, w_up, w_down, g = moe_cases.setup(world, tokens, experts, top_k, hidden, ffn, "uniform")
    sh = lambda t: moe_cases.shard(t, rank, world)
    xs, ws, us, ds = (sh(t).requires_grad_(True) for t in (x, weights, w_up, w_down))
    out = chunked_moe(xs, sh(ids), ws, us, ds, cfg, None)
    out.backward(sh(g))
    out, dx, dwt, dwu, dwd = out.detach().clone(), xs.grad.clone(), ws.grad.clone(), us.grad.clone(), ds.grad.clone()
    if damage == "out" and rank == world - 1:
        out[0] += 1.0  # token 0 is always among the sampled positions
    if damage == "dw_down" and rank == 0:
        dwd[0, 3, 5] += 10.0
    if damage == "d_weights" and rank == 0:
        dwt[0, 1] = -dwt[0, 1] + 5.0
    return sampled_check(xs.detach(), sh(ids), ws.detach(), sh(g), us.detach(), ds.detach(), out, dx, dwt, dwu, dwd,
                         stripe=STRIPE, group=None, sample=8, tol=1e-4)


def _all(rank, world):
    return {d: _step(rank, world, d) for d in (None, "out", "dw_down", "d_weights")}


def test_sampled_check_single_rank():
    res = _all(0, 1)
    assert res[None]["ok"] and res[None]["max_rel_err"] < 1e-5
    assert not res["out"]["ok"] and res["out"]["out"] > 1e-2 and res["out"]["dx"] < 1e-5
    assert not res["dw_down"]["ok"] and res["dw_down"]["dw_down"] > 1e-2
    assert not res["d_weights"]["ok"] and res["d_weights"]["d_weights"] > 1e-2


def test_sampled_check_four_ranks():
    for res in run_ranks(_all, 4):
        assert res[None]["ok"] and res[None]["max_rel_err"] < 1e-5, res[None]
        # every rank reports the maximum over ranks, wherever the damage was
        assert not res["out"]["ok"] and res["out"]["out"] > 1e-2
        assert not res["dw_down"]["ok"] and res["dw_down"]["dw_down"] > 1e-2
        assert not res["d_weights"]["ok"] and res["d_weights"]["d_weights"] > 1e-2
