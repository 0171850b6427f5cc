"""Properties of the slice plan, checked directly rather than through numerics.

Mirrors the reference's invariant list (tests/test_plan.py:49-69): same
iteration count everywhere, no padding on the wire, every slice <= S rows,
empty tails, full interior slices, group sizes consistent, every segment
delivered once and returned once, combine mirrors dispatch.
"""

import numpy as np
import pytest
import torch

from chunked_ep_moe_b200.ops import plan as plan_lib

EP, TOKENS, EXPERTS, TOP_K = 4, 32, 8, 2


def _ids(skew, seed=0):
    gen = torch.Generator().manual_seed(seed)
    logits = torch.randn(EP * TOKENS, EXPERTS, generator=gen)
    if skew:
        logits[:, 0] += 100.0
    return torch.topk(logits, TOP_K, dim=1).indices.to(torch.int32)


def _plans(ids, slice_size, ep=EP, experts=EXPERTS):
    per_rank = ids.reshape(ep, -1, ids.shape[1])
    sorted_counts = [plan_lib.sort_and_count(per_rank[r], experts) for r in range(ep)]
    counts = torch.stack([c.reshape(ep, experts // ep) for _, c in sorted_counts])  # what the all-gather yields
    return [plan_lib.RoutingPlan(sorted_counts[r][0], counts, slice_size, r) for r in range(ep)], counts


def test_worked_example():
    counts = torch.tensor([[[3, 1], [2, 2]], [[1, 0], [4, 3]]])
    plan = plan_lib.RoutingPlan(torch.zeros(8, dtype=torch.int64), counts, 4, 1)
    assert plan.send_begin.reshape(2, 4).tolist() == [[0, 3, 4, 6], [0, 1, 1, 5]]
    assert plan.expert_rows.tolist() == [[4, 1], [6, 5]]
    assert plan.expert_begin.tolist() == [[0, 4], [0, 6]]
    assert plan.stream_begin[0].tolist() == [[0, 3], [4, 5]]
    assert plan.stream_begin[1].tolist() == [[0, 2], [6, 8]]
    assert plan.num_slices == 3
    assert plan.group_rows(1).tolist() == [2, 2]
    d = plan.dispatch_spec(1)
    seg = 1 * 2 + 0  # (receiver 1, local expert 0) as seen by sender 1
    assert (int(d.src_offset[seg]), int(d.send_rows[seg]), int(d.dst_offset[seg])) == (3, 2, 0)
    assert (int(d.land_offset[seg]), int(d.recv_rows[seg])) == (0, 2)  # rank 1 receives its own rows there too


@pytest.mark.parametrize("skew", [False, True])
@pytest.mark.parametrize("slice_size", [1, 5, 16, 1000])
def test_slices_cover_streams_exactly(skew, slice_size):
    plans, counts = _plans(_ids(skew), slice_size)
    counts = counts.numpy()
    local = EXPERTS // EP
    max_slices = EP * TOKENS * TOP_K // slice_size + 2
    n = plans[0].num_slices
    assert all(p.num_slices == n for p in plans), "all ranks must loop the same number of times"
    stream_rows = plans[0].rows
    assert n == -(-int(stream_rows.max()) // slice_size)

    def table(method, field):
        return np.stack([np.stack([getattr(getattr(p, method)(j), field) for j in range(max_slices)])
                         for p in plans])

    send, recv = table("dispatch_spec", "send_rows"), table("dispatch_spec", "recv_rows")
    c_send, c_recv = table("combine_spec", "send_rows"), table("combine_spec", "recv_rows")
    groups = np.stack([np.stack([p.group_rows(j) for j in range(max_slices)]) for p in plans])
    # What a sender aims at is what the receiver's own copy of the plan expects, in both directions.
    for method in ("dispatch_spec", "combine_spec"):
        dst, land = table(method, "dst_offset"), table(method, "land_offset")
        sent, got = table(method, "send_rows"), table(method, "recv_rows")
        for a in range(EP):
            for b in range(EP):
                out_ab = slice(b * local, (b + 1) * local)  # a's segments for peer b
                in_ba = slice(a * local, (a + 1) * local)   # b's segments from peer a
                np.testing.assert_array_equal(sent[a][:, out_ab], got[b][:, in_ba])
                live = sent[a][:, out_ab] > 0
                np.testing.assert_array_equal(dst[a][:, out_ab][live], land[b][:, in_ba][live])

    for r in range(EP):
        assert recv[r].sum() == stream_rows[r] == counts[:, r, :].sum()  # no padding on the wire
        per_slice_rows = recv[r].sum(axis=1)
        assert (per_slice_rows <= slice_size).all()
        assert (per_slice_rows[n:] == 0).all()
        active = per_slice_rows[: -(-int(stream_rows[r]) // slice_size)]
        assert (active[:-1] == slice_size).all()
        np.testing.assert_array_equal(groups[r].sum(axis=1), per_slice_rows)
        np.testing.assert_array_equal(recv[r].sum(axis=0).reshape(EP, local), counts[:, r, :])
        np.testing.assert_array_equal(c_send[r].sum(axis=0).reshape(EP, local), counts[:, r, :])
    for s in range(EP):
        np.testing.assert_array_equal(send[s].sum(axis=0).reshape(EP, local), counts[s])
        np.testing.assert_array_equal(c_recv[s], send[s])  # results come back in the shape they left


@pytest.mark.parametrize("slice_size", [3, 16])
def test_offsets_address_the_right_rows(slice_size):
    """Following dispatch offsets must reproduce each receiver's expert-major stream exactly."""
    ids = _ids(False, seed=3)
    plans, _ = _plans(ids, slice_size)
    local = EXPERTS // EP
    per_rank_ids = ids.reshape(EP, TOKENS, TOP_K)
    for r in range(EP):
        stream = []
        for j in range(plans[r].num_slices):
            buf = np.full(slice_size, -1, dtype=np.int64)
            for s in range(EP):
                d = plans[s].dispatch_spec(j)
                flat_sorted = per_rank_ids[s].reshape(-1)[plans[s].order].numpy()
                for l in range(local):
                    i = r * local + l
                    a, n, o = int(d.src_offset[i]), int(d.send_rows[i]), int(d.dst_offset[i])
                    assert (buf[o:o + n] == -1).all(), "segments must not overlap"
                    buf[o:o + n] = flat_sorted[a:a + n]
            stream.append(buf)
        stream = np.concatenate(stream) if stream else np.zeros(0, dtype=np.int64)
        rows = int(plans[r].rows[r])
        got = stream[:rows]
        assert (got >= r * local).all() and (got < (r + 1) * local).all()
        assert (np.diff(got) >= 0).all(), "receive stream must be expert-major"
        assert (stream[rows:] == -1).all()
