"""Chunked EP MoE vs the dense oracle on CPU ranks over gloo.

Mirrors the reference's layer tests (tests/test_moe.py:49-100): forward and the
four gradients for skew x slice size x stripe width, the fp8 wire tolerance,
and the 8-rank oracle configuration (T=32/rank, D=64, F=96, E=16, K=4, S=8,
stripe=4, uniform and first-choice-expert-0 routing).
"""

import itertools

import pytest
import torch

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe

import moe_cases
from dist_utils import run_ranks

NAMES = ["out", "dx", "dweights", "dw_up", "dw_down"]


def _run_case(rank, world, dims, skew, slice_size, stripe, comm_dtype, transport, score, w_std):
    tokens, experts, top_k, hidden, ffn = dims
    cfg = ChunkedMoEConfig(num_experts=experts, top_k=top_k, slice_size=slice_size, transport=transport,
                           comm_dtype=comm_dtype, stripe_width=stripe)
    x, ids, weights, w_up, w_down, g = moe_cases.setup(world, tokens, experts, top_k, hidden, ffn, skew,
                                                       w_std=w_std, score=score)
    want = moe_cases.oracle(x, ids, weights, w_up, w_down, g, stripe)
    sh = lambda t: moe_cases.shard(t, rank, world)
    xs, ws, us, ds = (sh(t).requires_grad_(True) for t in (x, weights, w_up, w_down))
    out = chunked_moe(xs, sh(ids), ws, us, ds, cfg, None)
    (out * sh(g)).sum().backward()
    got = {"out": out.detach(), "dx": xs.grad, "dweights": ws.grad, "dw_up": us.grad, "dw_down": ds.grad}
    errs = {}
    for name in NAMES:
        a, b = got[name], sh(want[name])
        errs[name] = (float((a - b).abs().max()), float((a - b).norm() / b.norm().clamp_min(1e-30)),
                      bool(torch.allclose(a, b, rtol=1e-4, atol=1e-4)))
    return errs


def _all_cases(rank, world, cases):
    return {case: _run_case(rank, world, *case) for case in cases}


SMALL = (16, 8, 2, 8, 12)  # tokens/rank, E, K, D, F at EP=4 (the reference's test sizes)
GRID = [(SMALL, skew, s, stripe, None, "emulated", "softmax", None)
        for skew, s, stripe in itertools.product(["uniform", "rank0", "all_one"], [3, 8, 64], [1, 4])]
GRID += [(SMALL, "uniform", 8, 4, None, "ragged_a2a", "softmax", None),
         (SMALL, "all_one", 3, 1, None, "ragged_a2a", "softmax", None)]
FP8 = [(SMALL, skew, 8, 4, "float8_e4m3fn", "emulated", "softmax", None) for skew in ["uniform", "all_one"]]
ORACLE8 = [((32, 16, 4, 64, 96), skew, 8, 4, None, "emulated", "softmax_chosen", 0.02)
           for skew in ["uniform", "all_one"]]


@pytest.fixture(scope="module")
def ep4_results():
    return run_ranks(_all_cases, 4, GRID + FP8)


@pytest.fixture(scope="module")
def ep8_results():
    return run_ranks(_all_cases, 8, ORACLE8)


@pytest.mark.parametrize("case", GRID, ids=lambda c: f"{c[1]}-S{c[2]}-stripe{c[3]}-{c[5]}")
def test_forward_and_grads_match_reference(ep4_results, case):
    for rank, res in enumerate(ep4_results):
        for name in NAMES:
            max_abs, _, close = res[case][name]
            assert close, f"rank {rank} {name}: max abs err {max_abs:.3e}"


@pytest.mark.parametrize("case", FP8, ids=lambda c: c[1])
def test_fp8_wire_is_close(ep4_results, case):
    for rank, res in enumerate(ep4_results):
        for name in NAMES:
            assert res[case][name][1] < 0.08, f"rank {rank} {name}: relative error {res[case][name][1]:.4f}"


@pytest.mark.parametrize("case", ORACLE8, ids=lambda c: c[1])
def test_eight_rank_oracle_config(ep8_results, case):
    for rank, res in enumerate(ep8_results):
        for name in NAMES:
            max_abs, rel, close = res[case][name]
            assert close, f"rank {rank} {name}: max abs err {max_abs:.3e} rel {rel:.3e}"
