"""A host-side model of the cross-rank protocol, run under random interleavings (no GPU, no processes).

The fused path's ranks only talk through a few words of each other's memory: traffic-matrix rows with epoch flags,
slice buffers double buffered by a global slice sequence number, cumulative arrival counters per (source, expert),
credits, a returned-row counter. This test replays that protocol with P ranks as state machines whose steps a seeded
scheduler interleaves at random, driven by the REAL per-pass tables (`plan_build_host`, the code the plan kernel
runs). It checks what the kernels rely on:

* nobody deadlocks, whatever the order of steps and however skewed the routing;
* a slice buffer row is never overwritten before the slice that owns it was consumed, and a consumer only ever reads
  rows of its own pass and slice (arrival targets are exact; counters never need a reset);
* every dispatched row comes back exactly once, at its send-order position, before the sender sums it;
* a rank never reads a traffic matrix that a faster rank has already overwritten with a later pass.

The reference argues its semaphore protocol in comments and leaves it unverified
(src/chunked_moe/transport/nvshmem.py:135-137, :168-169; README.md:118-120).
"""

import random

import numpy as np
import pytest
import torch

from chunked_ep_moe_b200 import _build
from chunked_ep_moe_b200.ops import plan as plan_lib


class Tables:
    """One rank's view of one plan (the arrays the kernels index)."""

    def __init__(self, ext, counts, S, max_slices, me):
        P, _, L = counts.shape
        self.P, self.L, self.S, self.me = P, L, S, me
        lay = ext.plan_layout(P, L, S, max_slices)
        tab = ext.plan_build_host(torch.from_numpy(counts).to(torch.int32).contiguous(), S, max_slices, me).numpy()
        n = P * L
        self.num_slices = int(tab[0])
        self.rows_sent = int(tab[5])
        take = lambda key, cnt: tab[lay[key]: lay[key] + cnt].copy()
        self.in_start, self.in_size = take("in_start", n), take("in_size", n)
        self.src_send_start = take("src_send_start", n)
        self.expert_start, self.expert_rows = take("expert_start", L), take("expert_rows", L)
        self.put = [tab[lay["put"] + 4 * n * j: lay["put"] + 4 * n * (j + 1)].reshape(n, 4).copy()
                    for j in range(self.num_slices)]


class Rank:
    def __init__(self, r, P, L, S):
        self.r, self.P, self.L, self.S = r, P, L, S
        self.arrive = np.zeros(P * L, dtype=np.int64)          # cumulative, written by senders
        self.expected_total = np.zeros(P * L, dtype=np.int64)  # local bookkeeping of pass_begin
        self.pass_base = np.zeros(P * L, dtype=np.int64)
        self.credit = np.zeros(P, dtype=np.int64)              # credit[peer]: slices `peer` has finished with
        self.buf = [[None] * S, [None] * S]                    # slice buffers: (source, send position, pass id)
        self.ret = {}                                          # send position -> pass id of the returned row
        self.ret_count = 0
        self.ret_target = 0
        self.traffic = [dict(), dict()]                        # parity -> {source: (epoch, row)}
        self.flags = [np.zeros(P, dtype=np.int64), np.zeros(P, dtype=np.int64)]
        self.consumed_seq = -1                                 # last slice sequence this rank released (slice_done)


def simulate(P, L, S, routings, seed, use_credits=True):
    """`routings`: one numpy [P, P, L] count matrix per forward pass; every forward is followed by its backward.

    `use_credits=False` removes the senders' wait for the receivers' credits (to show that the checks notice).
    """
    ext = _build.load()
    rng = random.Random(seed)
    ranks = [Rank(r, P, L, S) for r in range(P)]
    passes = []  # (pass id, plan index, needs_exchange)
    for k in range(len(routings)):
        passes += [(2 * k, k, True), (2 * k + 1, k, False)]
    max_slices = max(int(c.sum()) for c in routings) // S + 2

    # Each rank runs four cooperating threads (host order + the streams): main, comm (puts), compute, release.
    # A thread is a generator that yields a guard (callable -> bool) before every step that has to wait.
    seq_base = {}

    def main_thread(me):
        rk = ranks[me]
        seq = 0
        epoch = 0
        for pid, k, exchange in passes:
            if exchange:
                epoch += 1
                parity = epoch & 1
                # PLAN_SEND: my counts row and my epoch flag into every rank's matrix of this parity
                for peer in rng.sample(range(P), P):
                    yield lambda: True
                    ranks[peer].traffic[parity][me] = (epoch, routings[k][me].copy())
                    ranks[peer].flags[parity][me] = epoch
                # PLAN_READ: wait for every row of this epoch, then use the matrix
                yield lambda: all(rk.flags[parity][s] >= epoch for s in range(P))
                for s in range(P):
                    got_epoch, row = rk.traffic[parity][s]
                    assert got_epoch == epoch, f"rank {me} read rank {s}'s row of epoch {got_epoch} in epoch {epoch}"
                    assert np.array_equal(row, routings[k][s]), "traffic matrix row of another pass"
            tabs = Tables(ext, routings[k], S, max_slices, me)
            n = tabs.num_slices
            # every rank loops the same number of slices: the sequence numbers agree without communication
            assert seq_base.setdefault(pid, seq) == seq, "ranks disagree on the global slice sequence"
            # pass_begin: targets of this pass start where all earlier passes' rows end (no reset of the counters)
            yield lambda: True
            rk.pass_base = rk.expected_total.copy()
            rk.expected_total = rk.expected_total + tabs.in_size
            rk.ret_target += tabs.rows_sent
            rk.ret = {}
            state[me] = {"pid": pid, "tabs": tabs, "seq0": seq, "puts_done": 0, "consumes_done": 0, "released": 0}
            # combine_reduce: every row I sent has come back, exactly once
            yield lambda: state[me]["released"] == n and rk.ret_count >= rk.ret_target
            assert rk.ret_count == rk.ret_target
            assert sorted(rk.ret) == list(range(tabs.rows_sent)), "a row did not come back"
            assert all(v == pid for v in rk.ret.values())
            state[me] = None
            seq += n

    state = [None] * P

    def comm_thread(me):
        rk = ranks[me]
        for pid, k, _ in passes:
            yield lambda: state[me] is not None and state[me]["pid"] == pid
            st = state[me]
            tabs, seq0 = st["tabs"], st["seq0"]
            for j in range(tabs.num_slices):
                q = seq0 + j
                # host order: this rank's own release of slice q-2, then the kernel's credit wait on every receiver
                yield lambda: q < 2 or rk.consumed_seq >= q - 2
                yield lambda: q < 2 or not use_credits or all(rk.credit[r] >= q - 1 for r in range(P))
                segs = [i for i in range(P * L) if tabs.put[j][i][1] > 0]
                rng.shuffle(segs)
                for i in segs:
                    yield lambda: True
                    in_off, rows, out_off, _ = (int(v) for v in tabs.put[j][i])
                    dest, l = divmod(i, L)
                    target = ranks[dest]
                    assert target.consumed_seq >= q - 2, "overwrote a slice buffer its owner had not released"
                    for t in range(rows):
                        target.buf[q & 1][out_off + t] = (me, in_off + t, pid, q)
                    target.arrive[me * L + l] += rows
                st["puts_done"] = j + 1

    def compute_thread(me):
        rk = ranks[me]
        for pid, k, _ in passes:
            yield lambda: state[me] is not None and state[me]["pid"] == pid
            st = state[me]
            tabs, seq0 = st["tabs"], st["seq0"]
            for j in range(tabs.num_slices):
                q = seq0 + j
                yield lambda: st["puts_done"] > j           # same-GPU dependency: an event after my own put(j)
                yield lambda: st["released"] >= j - 1       # two slices in flight
                experts = list(range(L))
                rng.shuffle(experts)
                lo, hi = j * S, (j + 1) * S
                for l in experts:
                    first = max(int(tabs.expert_start[l]), lo)
                    last = min(int(tabs.expert_start[l] + tabs.expert_rows[l]), hi)
                    if last <= first:
                        continue
                    # the producer warp's wait: P counters of this expert reach base + rows due through slice j
                    def arrived(l=l):
                        for s in range(P):
                            i = s * L + l
                            through = min(max(hi - int(tabs.in_start[i]), 0), int(tabs.in_size[i]))
                            if rk.arrive[i] < rk.pass_base[i] + through:
                                return False
                        return True
                    yield arrived
                    for stream_row in range(first, last):
                        src = pos = None
                        for s in range(P):
                            i = s * L + l
                            st0, sz = int(tabs.in_start[i]), int(tabs.in_size[i])
                            if st0 <= stream_row < st0 + sz:
                                src, pos = s, int(tabs.src_send_start[i]) + stream_row - st0
                        assert src is not None, "a slice row belongs to no segment"
                        got = rk.buf[q & 1][stream_row - lo]
                        assert got == (src, pos, pid, q), f"rank {me} slice {q} row {stream_row - lo}: {got}"
                        home = ranks[src]
                        assert pos not in home.ret, "a row came back twice"
                        home.ret[pos] = pid
                        home.ret_count += 1
                st["consumes_done"] = j + 1

    def release_thread(me):
        rk = ranks[me]
        for pid, k, _ in passes:
            yield lambda: state[me] is not None and state[me]["pid"] == pid
            st = state[me]
            for j in range(st["tabs"].num_slices):
                yield lambda: st["consumes_done"] > j
                q = st["seq0"] + j
                rk.consumed_seq = q
                for s in rng.sample(range(P), P):
                    ranks[s].credit[me] = q + 1
                st["released"] = j + 1

    threads = []
    for me in range(P):
        for make in (main_thread, comm_thread, compute_thread, release_thread):
            gen = make(me)
            threads.append({"gen": gen, "guard": next(gen), "rank": me, "name": make.__name__})
    steps = 0
    while threads:
        ready = [t for t in threads if t["guard"]()]
        assert ready, "deadlock: " + ", ".join(f"{t['name']}@{t['rank']}" for t in threads)
        t = rng.choice(ready)
        try:
            t["guard"] = next(t["gen"])
        except StopIteration:
            threads.remove(t)
        steps += 1
        assert steps < 2_000_000
    return steps


def _routing(P, L, tokens, top_k, skew, seed):
    gen = torch.Generator().manual_seed(seed)
    E = P * L
    logits = torch.randn(P * tokens, E, generator=gen)
    if skew == "all_one":
        logits[:, 0] += 100.0
    elif skew == "one_rank_silent":  # rank 0's tokens all go to its own experts: it exchanges rows with nobody else
        logits[:tokens, L:] -= 100.0
        logits[tokens:, :L] -= 100.0
    ids = torch.topk(logits, top_k, dim=1).indices.reshape(P, tokens, top_k)
    counts = torch.stack([plan_lib.sort_and_count(ids[r], E)[1].reshape(P, L) for r in range(P)])
    return counts.numpy().astype(np.int64)


@pytest.mark.parametrize("P,L,S", [(2, 2, 4), (3, 2, 5), (4, 2, 8), (4, 3, 3)])
@pytest.mark.parametrize("skew", ["uniform", "all_one", "one_rank_silent"])
def test_protocol_under_random_interleavings(P, L, S, skew):
    top_k = 2 if P * L >= 2 else 1
    for seed in range(6):
        routings = [_routing(P, L, 6, top_k, skew, 100 * seed + k) for k in range(3)]
        simulate(P, L, S, routings, seed)


def test_the_model_notices_a_missing_credit_wait():
    """The checker has teeth: without the credit wait some schedule overwrites a slice buffer that is still in use."""
    P, L, S = 3, 2, 3
    routings = [_routing(P, L, 8, 2, "uniform", k) for k in range(2)]
    caught = None
    for seed in range(60):
        try:
            simulate(P, L, S, routings, seed, use_credits=False)
        except AssertionError as e:
            caught = str(e)
            break
    assert caught is not None and ("overwrote a slice buffer" in caught or "slice" in caught), caught
