"""Host-side model of the CTA-pair kernel's stage barriers in the weight-gradient mode (csrc/gemm/grouped_gemm_pair.cu).

The kernel's rule: every load of both CTAs credits the LEADER's full barrier of its stage (two arrivals per phase, one
`expect_tx` from each CTA's producer), except the peer's load of a tile's ragged last k-block. That one lands on the
peer's OWN full barrier; the peer's warp 1 waits for it, zero-fills the rows past the group and only then makes the
second arrival on the leader's barrier. The leader issues a stage's MMAs once its full barrier's phase has completed
(for a ragged tail: after zero-filling its own rows too) and commits to both CTAs' empty barriers.

The model runs the four actors (two producers, the leader's MMA warp, the peer's warp 1) as generators under a seeded
random scheduler, with mbarriers that count arrivals and transaction bytes per phase, and checks: no deadlock; the
leader never issues a k-block before both halves have landed and, for a ragged tail, both zero-fills are done; no stage
is reloaded before the MMAs that read it have been committed. Two broken variants must be caught.
"""

import random

import pytest

STAGES = 6
BYTES = 32 * 1024


class Barrier:
    """An mbarrier: a phase completes when `count` arrivals have been made and every expected byte has landed."""

    def __init__(self, count):
        self.count = count
        self.phase = 0
        self.arrivals = 0
        self.tx = 0

    def _maybe_complete(self):
        if self.arrivals == self.count and self.tx == 0:
            self.phase += 1
            self.arrivals = 0

    def arrive(self, expect=0):
        assert self.arrivals < self.count, "more arrivals than the barrier was initialised for"
        self.arrivals += 1
        self.tx += expect
        self._maybe_complete()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self._maybe_complete()

    def done(self, phase):
        return self.phase > phase


class Pair:
    def __init__(self, tiles, variant):
        self.tiles = tiles  # [(k_blocks, ragged)]
        self.variant = variant
        self.full = [[Barrier(2) for _ in range(STAGES)], [Barrier(1) for _ in range(STAGES)]]  # [cta][stage]
        self.empty = [[Barrier(1) for _ in range(STAGES)] for _ in range(2)]
        self.landed = [[None] * STAGES for _ in range(2)]   # [cta][stage] -> (tile, kb) whose data is in place
        self.zeroed = [[None] * STAGES for _ in range(2)]   # [cta][stage] -> (tile, kb) whose rows were cleaned
        self.in_flight = []                                  # loads issued and not landed: (cta, stage, key, barrier)
        self.issued = []

    # ---- actors: generators that yield a wait predicate (None = nothing to wait for) -----------------------------
    def producer(self, cta):
        it = 0
        for t, (k_blocks, ragged) in enumerate(self.tiles):
            for kb in range(k_blocks):
                s, use = it % STAGES, it // STAGES
                if use > 0:
                    yield lambda s=s, use=use: self.empty[cta][s].done(use - 1)
                assert not any(f[0] == cta and f[1] == s for f in self.in_flight), "stage reloaded while a load flies"
                own = cta == 1 and ragged and kb == k_blocks - 1 and self.variant != "tail_credits_leader"
                bar = self.full[1][s] if own else self.full[0][s]
                bar.arrive(expect=BYTES)
                self.landed[cta][s] = None
                self.in_flight.append((cta, s, (t, kb), bar))
                it += 1
                yield None

    def leader_mma(self):
        it = 0
        for t, (k_blocks, ragged) in enumerate(self.tiles):
            for kb in range(k_blocks):
                s, use = it % STAGES, it // STAGES
                yield lambda s=s, use=use: self.full[0][s].done(use)
                tail = ragged and kb == k_blocks - 1
                if tail:
                    self.zeroed[0][s] = (t, kb)
                assert self.landed[0][s] == (t, kb) and self.landed[1][s] == (t, kb), "MMA before both halves landed"
                if tail:
                    assert self.zeroed[1][s] == (t, kb), "MMA on a ragged k-block before the peer cleaned its rows"
                self.issued.append((t, kb))
                self.empty[0][s].arrive()  # tcgen05.commit to both CTAs' empty barriers
                self.empty[1][s].arrive()
                it += 1
                yield None

    def peer_warp1(self):
        it = 0
        own_uses = [0] * STAGES
        for t, (k_blocks, ragged) in enumerate(self.tiles):
            it += k_blocks - 1 if ragged else k_blocks  # keeps count of the stages only
            if not ragged:
                continue
            s = it % STAGES
            if self.variant != "tail_credits_leader":
                yield lambda s=s, use=own_uses[s]: self.full[1][s].done(use)
                own_uses[s] += 1
                assert self.landed[1][s] == (t, k_blocks - 1)
                self.zeroed[1][s] = (t, k_blocks - 1)
                if self.variant != "relay_forgets_to_arrive":
                    self.full[0][s].arrive()  # the arrival the peer's producer makes for every other k-block
            it += 1
            yield None

    # ---- the copy engine: a random in-flight load lands -----------------------------------------------------------
    def land_one(self, rng):
        cta, s, key, bar = self.in_flight.pop(rng.randrange(len(self.in_flight)))
        self.landed[cta][s] = key
        bar.complete_tx(BYTES)


def run(tiles, seed, variant="correct"):
    rng = random.Random(seed)
    pair = Pair(tiles, variant)
    actors = {"producer0": pair.producer(0), "producer1": pair.producer(1), "mma": pair.leader_mma(),
              "peer_warp1": pair.peer_warp1()}
    waiting = {name: None for name in actors}
    for _ in range(200000):
        ready = [n for n in actors if waiting[n] is None or waiting[n]()]
        choices = ready + (["land"] if pair.in_flight else [])
        if not choices:
            if not actors:
                return pair
            raise RuntimeError(f"deadlock with {sorted(actors)} waiting")
        pick = rng.choice(choices)
        if pick == "land":
            pair.land_one(rng)
            continue
        try:
            waiting[pick] = next(actors[pick])
        except StopIteration:
            del actors[pick]
            del waiting[pick]
    raise RuntimeError("did not finish")


def _tiles(rng, count):
    return [(rng.randint(1, 9), rng.random() < 0.5) for _ in range(count)]


@pytest.mark.parametrize("seed", range(12))
def test_every_k_block_is_issued_once_in_order(seed):
    rng = random.Random(1000 + seed)
    tiles = _tiles(rng, 14)
    pair = run(tiles, seed)
    assert pair.issued == [(t, kb) for t, (k, _) in enumerate(tiles) for kb in range(k)]
    assert not pair.in_flight


def test_ragged_tails_only_and_single_k_block_tiles():
    for seed in range(6):
        run([(1, True)] * 20, seed)
        run([(7, True), (1, False), (1, True), (6, False)] * 4, seed)


def test_a_peer_tail_that_credits_the_leader_directly_is_caught():
    """If the peer's ragged-tail load credited the leader like any other, the leader could issue before the peer's rows
    are clean: the model must see that under some schedule."""
    with pytest.raises(AssertionError, match="before the peer cleaned"):
        for seed in range(50):
            run([(3, True)] * 10, seed, variant="tail_credits_leader")


def test_a_forgotten_forwarded_arrival_deadlocks():
    with pytest.raises(RuntimeError, match="deadlock"):
        run([(3, True)] * 4, 0, variant="relay_forgets_to_arrive")
