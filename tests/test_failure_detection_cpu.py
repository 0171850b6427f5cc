"""Failure detection, exercised on the host only (CPU ranks over gloo; no GPU is faulted, trapped or hung).

* a rank that leaves between steps is named by the survivors' heartbeat check before their next launch;
* a rank that announces a failure is reported at once, without waiting for the deadline;
* a corrupted traffic matrix is caught before anything is dispatched;
* a collective whose peer never joins ends with an error after a short process-group timeout.
"""

import datetime
import time

import pytest
import torch
import torch.distributed as dist

from chunked_ep_moe_b200.ops import plan as plan_lib
from chunked_ep_moe_b200.utils.health import PeerFailure, PlanMismatch, RankHealth, verify_plan_agreement

from dist_utils import run_ranks


def _leaver(rank, world, quitter, announce_failure):
    store = dist.distributed_c10d._get_default_store()
    health = RankHealth(store, rank, world, timeout_s=3.0)
    log = []
    for step in range(4):
        if rank == quitter and step == 2:
            if announce_failure:
                health.mark_failed("synthetic host-side exception")
            return {"left_at": step, "log": log}
        t0 = time.monotonic()
        try:
            health.step_barrier(step)
        except PeerFailure as e:
            return {"failure": (e.step, e.missing), "waited": time.monotonic() - t0, "log": log}
        log.append(step)
    return {"log": log}


@pytest.mark.parametrize("announce_failure", [False, True])
def test_a_rank_leaving_between_steps_is_named_by_the_survivors(announce_failure):
    world, quitter = 4, 2
    results = run_ranks(_leaver, world, quitter, announce_failure, timeout=120)
    for rank, res in enumerate(results):
        if rank == quitter:
            assert res["left_at"] == 2 and res["log"] == [0, 1]
        else:
            step, missing = res["failure"]
            assert missing == [quitter], res
            if announce_failure:
                # the announcement may overtake a slower survivor that is still checking step 1
                assert step in (1, 2) and res["log"] == list(range(step))
                assert res["waited"] < 2.5, "an announced failure must not wait for the deadline"
            else:
                assert step == 2 and res["log"] == [0, 1]


def _corrupt(rank, world):
    gen = torch.Generator().manual_seed(rank)
    ids = torch.randint(0, 8, (16, 2), generator=gen, dtype=torch.int32)
    _, my_counts = plan_lib.sort_and_count(ids, 8)
    counts = plan_lib.gather_traffic_matrix(my_counts, world, None)
    verify_plan_agreement(counts, my_counts, rank)  # healthy: no exception
    outcome = {}
    bad = counts.clone()
    if rank == 1:
        bad[0, 0, 0] += 1  # one rank sees a different matrix
    try:
        verify_plan_agreement(bad, my_counts, rank)
        outcome["disagree"] = "missed"
    except PlanMismatch as e:
        outcome["disagree"] = str(e)
    stale = counts.clone()
    stale[rank] = 0  # my own row is not what I sent
    try:
        verify_plan_agreement(stale, my_counts, rank)
        outcome["stale"] = "missed"
    except PlanMismatch as e:
        outcome["stale"] = str(e)
    return outcome


def test_corrupted_traffic_matrix_is_caught_before_dispatch():
    for res in run_ranks(_corrupt, 4, timeout=120):
        assert "disagree on the traffic matrix" in res["disagree"]
        assert "own counts" in res["stale"]


def _absent_peer(rank, world):
    # A second, short-timeout group; rank 1 never calls the collective (it left between steps).
    group = dist.new_group(list(range(world)), timeout=datetime.timedelta(seconds=3), backend="gloo")
    if rank == 1:
        time.sleep(6.0)
        return "left"
    t0 = time.monotonic()
    try:
        dist.all_reduce(torch.ones(4), group=group)
        return "no error"
    except Exception as e:  # gloo raises a RuntimeError describing the timeout
        return ("error", time.monotonic() - t0, type(e).__name__)


def test_collective_with_an_absent_peer_errors_out_instead_of_hanging():
    results = run_ranks(_absent_peer, 2, timeout=120)
    assert results[1] == "left"
    kind, waited, _ = results[0]
    assert kind == "error" and waited < 30.0


class _DeadStore:
    """A store whose server has gone away: every call fails the way a closed TCP store does."""

    def set(self, key, value):
        raise RuntimeError("Connection was likely closed")

    def check(self, keys):
        raise RuntimeError("Connection was likely closed")

    def get(self, key):
        raise RuntimeError("Connection was likely closed")


def test_a_dead_store_names_the_rank_that_hosted_it():
    health = RankHealth(_DeadStore(), rank=3, world=4, timeout_s=1.0)
    with pytest.raises(PeerFailure) as info:
        health.check_peers(5)
    assert info.value.missing == [0] and info.value.step == 5
