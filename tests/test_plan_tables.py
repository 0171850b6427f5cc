"""The extension's per-pass plan tables (the code the single-CTA plan kernel runs) vs the host planner."""

import numpy as np
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from chunked_ep_moe_b200 import _build
from chunked_ep_moe_b200.ops import plan as plan_lib


def _counts(P, L, tokens, top_k, skew, seed):
    gen = torch.Generator().manual_seed(seed)
    E = P * L
    logits = torch.randn(P * tokens, E, generator=gen)
    if skew == "all_one":
        logits[:, 0] += 100.0
    elif skew == "empty":  # some experts get nothing at all
        logits[:, 1::3] -= 100.0
    ids = torch.topk(logits, top_k, dim=1).indices.reshape(P, tokens, top_k)
    sc = [plan_lib.sort_and_count(ids[r], E) for r in range(P)]
    counts = torch.stack([c.reshape(P, L) for _, c in sc])
    return ids, [o for o, _ in sc], counts


@pytest.mark.parametrize("P,L,S", [(1, 4, 16), (2, 2, 4), (4, 2, 5), (8, 4, 24), (4, 8, 1000)])
@pytest.mark.parametrize("skew", ["uniform", "all_one", "empty"])
def test_tables_match_host_planner(P, L, S, skew):
    _check_tables(P, L, S, 16, 2, skew, seed=P * 100 + L)


@settings(max_examples=40, deadline=None)
@given(P=st.integers(1, 6), L=st.integers(1, 5), S=st.integers(1, 40), tokens=st.integers(1, 24),
       top_k=st.integers(1, 3), skew=st.sampled_from(["uniform", "all_one", "empty"]), seed=st.integers(0, 10**6))
def test_tables_match_host_planner_fuzzed(P, L, S, tokens, top_k, skew, seed):
    """Arbitrary small geometries: single rows, S = 1, slices longer than the whole stream, experts with nothing."""
    _check_tables(P, L, S, tokens, min(top_k, P * L), skew, seed)


def _check_tables(P, L, S, tokens, top_k, skew, seed):
    ext = _build.load()
    ids, orders, counts = _counts(P, L, tokens, top_k, skew, seed=seed)
    max_slices = P * tokens * top_k // S + 2
    lay = ext.plan_layout(P, L, S, max_slices)
    n = P * L
    for me in range(P):
        ref = plan_lib.RoutingPlan(orders[me], counts, S, me)
        tab = ext.plan_build_host(counts.to(torch.int32).contiguous(), S, max_slices, me).numpy()
        assert tab[0] == ref.num_slices
        assert tab[1] == int(ref.rows[me])
        assert tab[5] == tokens * top_k
        sl = lambda key, cnt: tab[lay[key]: lay[key] + cnt]
        np.testing.assert_array_equal(sl("send_start", n), ref.send_begin[me].reshape(-1))
        np.testing.assert_array_equal(sl("seg_start", n), ref.stream_begin[:, :, me].reshape(-1))
        np.testing.assert_array_equal(sl("seg_size", n), ref.counts[me].reshape(-1))
        np.testing.assert_array_equal(sl("in_start", n), ref.stream_begin[me].T.reshape(-1))
        np.testing.assert_array_equal(sl("in_size", n), ref.counts[:, me, :].reshape(-1))
        np.testing.assert_array_equal(sl("src_send_start", n), ref.send_begin[:, me, :].reshape(-1))
        np.testing.assert_array_equal(sl("expert_start", L), ref.expert_begin[me])
        np.testing.assert_array_equal(sl("expert_rows", L), ref.expert_rows[me])
        seen_final = np.zeros(L, dtype=np.int64)
        for j in range(max_slices):
            d = ref.dispatch_spec(j)
            groups = ref.group_rows(j)
            put = tab[lay["put"] + 4 * n * j: lay["put"] + 4 * n * (j + 1)].reshape(n, 4)
            if j < ref.num_slices:
                np.testing.assert_array_equal(put[:, 1], d.send_rows)
                live = put[:, 1] > 0
                np.testing.assert_array_equal(put[live, 0], d.src_offset[live])
                np.testing.assert_array_equal(put[live, 2], d.dst_offset[live])
                chunks = -(-put[:, 1] // lay["put_chunk_rows"])
                np.testing.assert_array_equal(put[:, 3], np.cumsum(chunks) - chunks)
                assert tab[lay["num_chunks"] + j] == chunks.sum()
            else:
                assert tab[lay["num_chunks"] + j] == 0
            # row tiles: cover each expert's rows of the slice exactly, in expert order, 128 rows at most
            num_m = tab[lay["num_mtiles"] + j]
            mt = tab[lay["mtiles"] + 4 * lay["max_mtiles"] * j:][: 4 * num_m].reshape(num_m, 4)
            starts = np.cumsum(groups) - groups
            covered = np.zeros(L, dtype=np.int64)
            for e, row0, nrows, _ in mt:
                assert 0 < nrows <= lay["tile_m"]
                assert row0 == starts[e] + covered[e]
                covered[e] += nrows
            np.testing.assert_array_equal(covered, groups if j < ref.num_slices else 0 * groups)
            # row-tile pairs (2-CTA GEMMs): same coverage in 256-row steps
            num_p = tab[lay["num_ptiles"] + j]
            pt = tab[lay["ptiles"] + 4 * lay["max_ptiles"] * j:][: 4 * num_p].reshape(num_p, 4)
            covered_p = np.zeros(L, dtype=np.int64)
            for e, row0, nrows, _ in pt:
                assert 0 < nrows <= 2 * lay["tile_m"]
                assert row0 == starts[e] + covered_p[e]
                covered_p[e] += nrows
            np.testing.assert_array_equal(covered_p, covered)
            # weight-gradient groups: one per expert present; first/final flags; empty experts once in slice 0
            num_g = tab[lay["num_gtiles"] + j]
            gt = tab[lay["gtiles"] + 4 * lay["max_gtiles"] * j:][: 4 * num_g].reshape(num_g, 4)
            for e, row0, nrows, flags in gt:
                es, er = int(ref.expert_begin[me][e]), int(ref.expert_rows[me][e])
                if nrows == 0:
                    assert j == 0 and er == 0 and flags == 3
                else:
                    assert nrows == groups[e] and row0 == starts[e]
                    assert bool(flags & 1) == (es >= j * S)
                    assert bool(flags & 2) == (es + er <= (j + 1) * S)
                seen_final[e] += bool(flags & 2)
            present = set(gt[:, 0].tolist())
            assert present >= {e for e in range(L) if groups[e] > 0}
        np.testing.assert_array_equal(seen_final, np.ones(L))  # every expert's gradient is finalised exactly once


def test_status_block_text():
    """The message `check_status` raises for a recorded kernel error (formatting runs without a GPU)."""
    from chunked_ep_moe_b200 import _build

    ext = _build.load()
    text = ext.format_status([5, 2, 0, 1, 5, 64, 67, 3], 2)
    assert "index check failed" in text and "detail 5" in text and "expected 64" in text and "rank 2" in text
    assert "pipeline barrier timed out" in ext.format_status([1, 1, 4, 17, 302, 0, 0, 9], 0)
    assert "expected 4294967295" in ext.format_status([2, 1, 0, 0, 0, -1, 0, 0], 0)  # counters are unsigned
    assert "malformed" in ext.format_status([1, 2], 0)


@pytest.mark.gpu
@pytest.mark.parametrize("P,L,S,tokens,top_k", [(1, 4, 16, 16, 2), (1, 256, 8192, 8192, 8), (4, 64, 8192, 8192, 8),
                                                (8, 32, 8192, 8192, 8), (8, 4, 24, 16, 2), (3, 5, 7, 33, 3),
                                                (2, 40, 100, 300, 4)])
@pytest.mark.parametrize("skew", ["uniform", "all_one", "empty"])
def test_plan_kernel_matches_host_tables(P, L, S, tokens, top_k, skew):
    """The plan kernel (shared-memory copy of the matrix, one warp per slice) writes the host restatement's tables."""
    ext = _build.load()
    _, _, counts = _counts(P, L, tokens, top_k, skew, seed=P * 1000 + L)
    counts = counts.to(torch.int32).contiguous()
    max_slices = P * tokens * top_k // S + 2
    lay = ext.plan_layout(P, L, S, max_slices)
    n = P * L
    for me in sorted({0, P - 1}):
        host = ext.plan_build_host(counts, S, max_slices, me).numpy()
        dev = ext.plan_build_device(counts.cuda(), S, max_slices, me).cpu().numpy()
        header_and_sums = lay["num_mtiles"]  # header + the per-segment and per-expert sums
        np.testing.assert_array_equal(dev[:header_and_sums], host[:header_and_sums])
        for key in ("num_mtiles", "num_gtiles", "num_chunks", "num_ptiles"):
            np.testing.assert_array_equal(dev[lay[key]: lay[key] + max_slices], host[lay[key]: lay[key] + max_slices])
        for j in range(max_slices):
            for key, cap, num in (("mtiles", lay["max_mtiles"], "num_mtiles"), ("gtiles", lay["max_gtiles"], "num_gtiles"),
                                  ("ptiles", lay["max_ptiles"], "num_ptiles")):
                used = 4 * host[lay[num] + j]
                at = lay[key] + 4 * cap * j
                np.testing.assert_array_equal(dev[at: at + used], host[at: at + used])
            if j < host[0]:
                at = lay["put"] + 4 * n * j
                np.testing.assert_array_equal(dev[at: at + 4 * n], host[at: at + 4 * n])
