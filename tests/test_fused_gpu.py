"""Fused sm_100a path on a real GPU vs plain-PyTorch fp32 references of the same ops.

Follows the reference's kernel-test strategy (tests/test_fused_kernels.py:18-67): partial slices,
an empty expert, a one-row expert, NaN-poisoned padding, bf16 tolerance 3e-2 x max-abs; plus the
layer grid of tests/test_moe.py run through the single-device lockstep harness for P > 1.
"""

import math

import pytest
import torch

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe, stripe_weights
from chunked_ep_moe_b200.ops import plan as plan_lib

import moe_cases

pytestmark = pytest.mark.gpu

TOL = 3e-2


def _close(got, want, name, tol=TOL):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    scale = want.abs().max().clamp_min(1e-6)
    err = (got - want).abs().max() / scale
    assert err <= tol, f"{name}: max abs err {err:.4f} x max-abs (allowed {tol})"


def _ids_with_groups(group_rows, top_k, num_experts, gen):
    """Token routing whose per-expert copy counts are exactly `group_rows` (K distinct experts per token not required)."""
    flat = torch.cat([torch.full((n,), e, dtype=torch.int32) for e, n in enumerate(group_rows)])
    flat = flat[torch.randperm(flat.numel(), generator=gen)]
    assert flat.numel() % top_k == 0
    return flat.reshape(-1, top_k)


def _oracle_dev(x, ids, weights, w_up, w_down, g, stripe):
    return moe_cases.oracle(x.float().cpu(), ids.cpu(), weights.float().cpu(), w_up.float().cpu(),
                            w_down.float().cpu(), g.float().cpu(), stripe)


def test_expert_sort_matches_stable_argsort():
    from chunked_ep_moe_b200 import _build
    from chunked_ep_moe_b200.parallel.lockstep import LockstepWorld

    gen = torch.Generator().manual_seed(0)
    cfg = ChunkedMoEConfig(num_experts=64, top_k=4, slice_size=256, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    world = LockstepWorld(cfg, 1, 256, 256, 1500)
    ids = torch.randint(0, 64, (1500, 4), generator=gen, dtype=torch.int32).cuda()
    order = torch.empty(6000, dtype=torch.int32, device="cuda")
    inv = torch.empty_like(order)
    counts = torch.zeros(64, dtype=torch.int32, device="cuda")
    world.ranks[0].sort_only(ids, order, inv, counts)
    ref_order, ref_counts = plan_lib.sort_and_count(ids.cpu(), 64)
    assert torch.equal(order.cpu().long(), ref_order)
    assert torch.equal(counts.cpu().long(), ref_counts)
    assert torch.equal(inv.cpu().long()[ref_order], torch.arange(6000))
    world.close()


CASES = [
    # (group rows per expert, slice size, stripe)
    ([40, 0, 70, 18], 128, 64),      # partial slice, empty expert
    ([64, 1, 63, 0], 128, 128),      # full slice, one-row expert, trailing empty expert
    ([300, 5, 0, 203], 200, 32),     # experts straddling several slices, S not a multiple of 128
    ([130, 126, 256, 0], 1024, 64),  # one slice larger than the whole stream
]


@pytest.mark.parametrize("group_rows,slice_size,stripe", CASES)
def test_single_rank_layer_matches_oracle(group_rows, slice_size, stripe):
    _check_single_rank_case(group_rows, slice_size, stripe)


@pytest.mark.parametrize("switch", ["CEM_RET_BLOCKED", "CEM_RET_LSU"])
def test_alternative_return_paths_match_oracle(monkeypatch, switch):
    """The two measurement variants of the combine epilogues must not change the layer's results. `CEM_RET_BLOCKED=1`:
    runs of rows stored into return buffers kept column tile by column tile, which `combine_reduce` then reads.
    `CEM_RET_LSU=1`: staged rows written out with coalesced vector stores instead of bulk stores."""
    from chunked_ep_moe_b200.ops import fused

    fused.release_workspaces()  # the switches are read when a workspace's executor is created
    monkeypatch.setenv(switch, "1")
    try:
        for group_rows, slice_size, stripe in CASES[:3]:
            _check_single_rank_case(group_rows, slice_size, stripe, hidden=768)  # three column tiles
    finally:
        fused.release_workspaces()


def _check_single_rank_case(group_rows, slice_size, stripe, hidden=256):
    gen = torch.Generator().manual_seed(1)
    E, K, D, F = len(group_rows), 2, hidden, 256
    ids = _ids_with_groups(group_rows, K, E, gen)
    T = ids.shape[0]
    x = torch.randn(T, D, generator=gen)
    weights = torch.rand(T, K, generator=gen) + 0.1
    w_gate = torch.randn(E, D, F, generator=gen) / math.sqrt(D)
    w_upp = torch.randn(E, D, F, generator=gen) / math.sqrt(D)
    w_down = torch.randn(E, F, D, generator=gen) / math.sqrt(F)
    g = torch.randn(T, D, generator=gen)
    w_up = stripe_weights(w_gate, w_upp, stripe)

    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=slice_size, transport="nvshmem",
                           expert_compute="fused", stripe_width=stripe)
    dev = lambda t: t.cuda().to(torch.bfloat16)
    xs, us, ds = dev(x).requires_grad_(True), dev(w_up).requires_grad_(True), dev(w_down).requires_grad_(True)
    ws = weights.cuda().requires_grad_(True)
    out = chunked_moe(xs, ids.cuda(), ws, us, ds, cfg, None)
    (out.float() * g.cuda()).sum().backward()
    torch.cuda.synchronize()

    want = _oracle_dev(xs.detach(), ids, ws.detach(), us.detach(), ds.detach(), dev(g), stripe)
    _close(out.detach().cpu(), want["out"], "out")
    _close(xs.grad.cpu(), want["dx"], "dx")
    _close(ws.grad.cpu(), want["dweights"], "dweights")
    _close(us.grad.cpu(), want["dw_up"], "dw_up")
    _close(ds.grad.cpu(), want["dw_down"], "dw_down")


def test_launch_count_matches_the_formula():
    """One forward+backward launches exactly `expected_launches(slices)` kernels (what bench.py reports)."""
    from chunked_ep_moe_b200.ops import fused

    torch.manual_seed(0)
    T, D, F, E, K, S = 192, 256, 256, 4, 2, 128
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True)
    ids = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).int()
    w = torch.rand(T, K, device="cuda").requires_grad_(True)
    w_up = (torch.randn(E, D, 2 * F, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    w_down = (torch.randn(E, F, D, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    chunked_moe(x, ids, w, w_up, w_down, cfg, None).sum().backward()  # builds the workspace
    before = fused.launches()
    chunked_moe(x, ids, w, w_up, w_down, cfg, None).sum().backward()
    torch.cuda.synchronize()
    slices = -(-T * K // S)
    assert fused.launches() - before == fused.expected_launches(slices)


def test_pipeline_counters_count_every_k_block():
    """The GEMM kernels' own counters: k-blocks issued = tiles x K/64 for the forward modes, and cycles were counted."""
    from chunked_ep_moe_b200.ops import fused

    torch.manual_seed(0)
    T, D, F, E, K, S = 256, 512, 256, 2, 1, 256
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    x = torch.randn(T, D, device="cuda").bfloat16()
    ids = (torch.arange(T, device="cuda") % E).int().reshape(T, K)  # 128 rows per expert: one full row tile each
    w = torch.ones(T, K, device="cuda")
    w_up = (torch.randn(E, D, 2 * F, device="cuda") * 0.05).bfloat16()
    w_down = (torch.randn(E, F, D, device="cuda") * 0.05).bfloat16()
    chunked_moe(x, ids, w, w_up, w_down, cfg, None)  # builds the workspace
    counters = fused.pipeline_counters(True)
    try:
        chunked_moe(x, ids, w, w_up, w_down, cfg, None)
        torch.cuda.synchronize()
    finally:
        fused.pipeline_counters(False)
    slot = {n: i for i, n in enumerate(fused.PIPELINE_COUNTER_SLOTS)}
    total = sum(t for t in counters).sum(1)  # [modes, slots]
    row_tiles = T * K // 128
    swiglu, down = fused.GEMM_MODE_NAMES.index("swiglu"), fused.GEMM_MODE_NAMES.index("down_fwd")
    assert int(total[swiglu, slot["tiles"]]) == row_tiles * (2 * F // 256)
    assert int(total[swiglu, slot["k_blocks"]]) == row_tiles * (2 * F // 256) * (D // 64)
    assert int(total[down, slot["k_blocks"]]) == row_tiles * (D // 256) * (F // 64)
    assert int(total[swiglu, slot["loop_cycles"]]) > 0 and int(total[swiglu, slot["loop_ns"]]) > 0
    assert int(total[fused.GEMM_MODE_NAMES.index("tgmm"), slot["k_blocks"]]) == 0  # no backward ran


def test_bad_send_order_entry_is_reported_not_dereferenced():
    """A send-order entry outside the token range: the put kernel records it and skips the row (no wild read)."""
    from chunked_ep_moe_b200.ops import fused

    torch.manual_seed(0)
    T, D, F, E, K, S = 64, 256, 256, 2, 2, 136  # a geometry no other test uses: the workspace is thrown away below
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    ws = fused.get_workspace(cfg, None, D, F, T * K)
    rank = ws.rank
    x = torch.randn(T, D, device="cuda").bfloat16()
    ids = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).int().contiguous()
    w_flat = torch.rand(T * K, device="cuda")
    plan = torch.empty(ws.plan_ints, dtype=torch.int32, device="cuda")
    order = torch.empty(T * K, dtype=torch.int32, device="cuda")
    inv_order = torch.empty_like(order)
    try:
        n = rank.begin_forward(ids, plan, order, inv_order, ws.dummy_counts, False)
        assert n == 1
        order[5] = T * K + 7  # token index T + 3: past the end of x
        rank.put(0, plan, order, x, None, w_flat)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="index check failed"):
            rank.check_status()
        rank.check_status()  # the block was cleared: a second check is clean
    finally:
        torch.cuda.synchronize()
        fused.release_workspaces()  # the pass was abandoned half way: do not reuse this workspace


def test_invalid_expert_id_is_reported_by_the_forward():
    """An expert id outside [0, E): the sort records it, every kernel launched on the guessed slice count returns at
    once, and the forward raises when it reads the pass's header (nothing is dereferenced, no wait runs out)."""
    from chunked_ep_moe_b200.ops import fused

    torch.manual_seed(0)
    T, D, F, E, K, S = 64, 256, 256, 2, 2, 152  # a geometry no other test uses: the workspace is thrown away below
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    x = torch.randn(T, D, device="cuda").bfloat16()
    ids = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).int().contiguous()
    w = torch.rand(T, K, device="cuda")
    w_up = (torch.randn(E, D, 2 * F, device="cuda") * 0.05).bfloat16()
    w_down = (torch.randn(E, F, D, device="cuda") * 0.05).bfloat16()
    try:
        chunked_moe(x, ids, w, w_up, w_down, cfg, None)  # a good pass first: the next one launches on its slice count
        bad = ids.clone()
        bad[7, 1] = E
        with pytest.raises(RuntimeError, match="index check failed"):
            chunked_moe(x, bad, w, w_up, w_down, cfg, None)
        torch.cuda.synchronize()
        fused.check_status()  # the block was cleared when the error was raised
    finally:
        torch.cuda.synchronize()
        fused.release_workspaces()  # the pass was abandoned half way: do not reuse this workspace


def test_slice_count_guess_is_corrected_in_both_directions():
    """The forward launches on the previous pass's slice count before it knows its own: passes that need more slices
    than the one before, and fewer, must both match the oracle (the same workspace throughout)."""
    gen = torch.Generator().manual_seed(9)
    E, K, D, F, stripe, S = 4, 2, 256, 256, 64, 128
    bf = lambda t: t.cuda().to(torch.bfloat16)
    w_up = bf(torch.randn(E, D, 2 * F, generator=gen) / math.sqrt(D))
    w_down = bf(torch.randn(E, F, D, generator=gen) / math.sqrt(F))
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=stripe)
    T = 192  # 384 copies: 3 slices when balanced ...
    for groups in ([96, 96, 96, 96], [100, 90, 102, 92], [96, 96, 96, 96]):
        tokens = T
        ids = _ids_with_groups(groups, K, E, gen)
        assert ids.shape[0] == tokens
        # ... and the second and third tensors below shrink the pass to 2 slices, then grow it back
        for keep in (tokens, 100, tokens):
            x, g = bf(torch.randn(keep, D, generator=gen)), bf(torch.randn(keep, D, generator=gen))
            weights = (torch.rand(keep, K, generator=gen) + 0.1).cuda()
            xs, ws = x.clone().requires_grad_(True), weights.clone().requires_grad_(True)
            us, ds = w_up.clone().requires_grad_(True), w_down.clone().requires_grad_(True)
            out = chunked_moe(xs, ids[:keep].cuda(), ws, us, ds, cfg, None)
            out.backward(g)
            torch.cuda.synchronize()
            want = _oracle_dev(x, ids[:keep], weights, w_up, w_down, g, stripe)
            _close(out.detach().cpu(), want["out"], f"out ({keep} tokens)")
            _close(xs.grad.cpu(), want["dx"], f"dx ({keep} tokens)")
            _close(us.grad.cpu(), want["dw_up"], f"dw_up ({keep} tokens)")
            _close(ds.grad.cpu(), want["dw_down"], f"dw_down ({keep} tokens)")


def test_gemm_whose_rows_never_arrive_gives_up_and_reports(monkeypatch):
    """The real swiglu kernel waiting for rows nobody sends: its bounded wait runs out, every warp unwinds promptly
    (the barrier waits watch the CTA's abort flag), later kernels of the pass return at once, the host raises."""
    import time

    from chunked_ep_moe_b200.ops import fused

    torch.manual_seed(0)
    T, D, F, E, K, S = 64, 256, 256, 2, 2, 144  # a geometry no other test uses: the workspace is thrown away below
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    monkeypatch.setenv("CEM_SPIN_LIMIT", "2000")  # ~1 ms of polling instead of seconds
    ws = fused.get_workspace(cfg, None, D, F, T * K)
    rank = ws.rank
    ids = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).int().contiguous()
    w_up = (torch.randn(E, D, 2 * F, device="cuda") * 0.05).bfloat16()
    w_down = (torch.randn(E, F, D, device="cuda") * 0.05).bfloat16()
    plan = torch.empty(ws.plan_ints, dtype=torch.int32, device="cuda")
    order = torch.empty(T * K, dtype=torch.int32, device="cuda")
    inv_order = torch.empty_like(order)
    try:
        assert rank.begin_forward(ids, plan, order, inv_order, ws.dummy_counts, False) == 1
        t0 = time.monotonic()
        rank.compute_forward(0, plan, w_up, w_down)  # no put was launched: the arrival counters never move
        torch.cuda.synchronize()
        assert time.monotonic() - t0 < 5.0, "unwinding must not wait for the barrier limits"
        with pytest.raises(RuntimeError, match="dispatched rows never arrived"):
            rank.check_status()
        rank.check_status()
    finally:
        torch.cuda.synchronize()
        fused.release_workspaces()


def test_fused_expert_compute_on_a_collective_transport():
    """`expert_compute="fused"` under `transport="ragged_a2a"`: the library exchange feeds the sm_100a kernels."""
    gen = torch.Generator().manual_seed(4)
    E, K, D, F, stripe, S = 4, 2, 256, 256, 64, 96
    ids = _ids_with_groups([50, 0, 77, 33], K, E, gen)
    T = ids.shape[0]
    bf = lambda t: t.cuda().to(torch.bfloat16)
    x, g = bf(torch.randn(T, D, generator=gen)), bf(torch.randn(T, D, generator=gen))
    weights = (torch.rand(T, K, generator=gen) + 0.1).cuda()
    w_up = bf(torch.randn(E, D, 2 * F, generator=gen) / math.sqrt(D))
    w_down = bf(torch.randn(E, F, D, generator=gen) / math.sqrt(F))
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="ragged_a2a", expert_compute="fused",
                           stripe_width=stripe)
    xs, ws = x.clone().requires_grad_(True), weights.clone().requires_grad_(True)
    us, ds = w_up.clone().requires_grad_(True), w_down.clone().requires_grad_(True)
    out = chunked_moe(xs, ids.cuda(), ws, us, ds, cfg, None)
    out.backward(g)
    torch.cuda.synchronize()
    want = _oracle_dev(x, ids, weights, w_up, w_down, g, stripe)
    _close(out.detach().cpu(), want["out"], "out")
    _close(xs.grad.cpu(), want["dx"], "dx")
    _close(ws.grad.cpu(), want["dweights"], "dweights")
    _close(us.grad.cpu(), want["dw_up"], "dw_up")
    _close(ds.grad.cpu(), want["dw_down"], "dw_down")


@pytest.mark.parametrize("cta_pairs", [True, False], ids=["pairs", "single"])
def test_nan_poisoned_padding_does_not_leak(cta_pairs):
    """Scratch and slice buffers full of NaN patterns: rows outside a group must never reach an output."""
    from chunked_ep_moe_b200 import _build
    from chunked_ep_moe_b200.parallel.lockstep import LockstepWorld

    ext = _build.load()
    gen = torch.Generator().manual_seed(2)
    E, K, D, F, S, stripe = 4, 2, 256, 256, 256, 64
    group_rows = [70, 0, 41, 9]
    ids = _ids_with_groups(group_rows, K, E, gen)
    T = ids.shape[0]
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=stripe)
    world = LockstepWorld(cfg, 1, D, F, T, cta_pairs=cta_pairs)
    lay = ext.arena_layout(1, E, S, D, T * K, False)
    ext.arena_fill(world.arenas.bases[0] + lay["xbuf"], lay["xq"] - lay["xbuf"], 0xFF)  # x, g, w slice buffers
    ext.arena_fill(world.arenas.bases[0] + lay["ret"], lay["arrive"] - lay["ret"], 0xFF)
    rk = world.ranks[0]
    for t in (rk.act(), rk.h(), rk.dh(), rk.dy()):
        t.fill_(float("nan"))
    bf = lambda t: t.cuda().to(torch.bfloat16)
    x, g = bf(torch.randn(T, D, generator=gen)), bf(torch.randn(T, D, generator=gen))
    weights = (torch.rand(T, K, generator=gen) + 0.1).cuda()
    w_up = bf(torch.randn(E, D, 2 * F, generator=gen) / math.sqrt(D))
    w_down = bf(torch.randn(E, F, D, generator=gen) / math.sqrt(F))
    outs, saved = world.forward([x], [ids.cuda()], [weights], [w_up], [w_down])
    dxs, dws, dw_ups, dw_downs = world.backward([x], [g], [w_up], [w_down], saved)
    torch.cuda.synchronize()
    want = _oracle_dev(x, ids, weights, w_up, w_down, g, stripe)
    _close(outs[0].cpu(), want["out"], "out")
    _close(dxs[0].cpu(), want["dx"], "dx")
    _close(dws[0].reshape(T, K).cpu(), want["dweights"], "dweights")
    _close(dw_ups[0].cpu(), want["dw_up"], "dw_up")
    _close(dw_downs[0].cpu(), want["dw_down"], "dw_down")
    world.close()


@pytest.mark.parametrize("cta_pairs", [True, False], ids=["pairs", "single"])
@pytest.mark.parametrize("world_size,skew,slice_size", [(2, "uniform", 128), (4, "uniform", 64), (4, "all_one", 64),
                                                        (4, "rank0", 256), (8, "uniform", 2048)])
def test_lockstep_multi_rank_matches_oracle(world_size, skew, slice_size, cta_pairs):
    from chunked_ep_moe_b200.parallel.lockstep import LockstepWorld

    T, E, K, D, F, stripe = 48, 16, 4, 256, 256, 64
    x, ids, weights, w_up, w_down, g = moe_cases.setup(world_size, T, E, K, D, F, skew, seed=3)
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=slice_size, transport="nvshmem",
                           expert_compute="fused", stripe_width=stripe)
    bf = lambda t: t.cuda().to(torch.bfloat16).contiguous()
    sh = lambda t, r: moe_cases.shard(t, r, world_size)
    xs = [bf(sh(x, r)) for r in range(world_size)]
    gs = [bf(sh(g, r)) for r in range(world_size)]
    idl = [sh(ids, r).cuda() for r in range(world_size)]
    wl = [sh(weights, r).cuda() for r in range(world_size)]
    ups = [bf(sh(w_up, r)) for r in range(world_size)]
    downs = [bf(sh(w_down, r)) for r in range(world_size)]
    world = LockstepWorld(cfg, world_size, D, F, T, cta_pairs=cta_pairs)
    outs, saved = world.forward(xs, idl, wl, ups, downs)
    dxs, dws, dw_ups, dw_downs = world.backward(xs, gs, ups, downs, saved)
    torch.cuda.synchronize()
    want = _oracle_dev(torch.cat(xs), ids, weights, torch.cat(ups), torch.cat(downs), torch.cat(gs), stripe)
    _close(torch.cat(outs).cpu(), want["out"], "out")
    _close(torch.cat(dxs).cpu(), want["dx"], "dx")
    _close(torch.cat(dws).reshape(-1, K).cpu(), want["dweights"], "dweights")
    _close(torch.cat(dw_ups).cpu(), want["dw_up"], "dw_up")
    _close(torch.cat(dw_downs).cpu(), want["dw_down"], "dw_down")
    # a second pass through the same workspace: counters, credits and double buffers carry over
    outs2, saved2 = world.forward(xs, idl, wl, ups, downs)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(outs, outs2)), "the forward must be bitwise reproducible"
    world.close()


@pytest.mark.parametrize("world_size,skew", [(1, "uniform"), (4, "uniform"), (4, "all_one")])
def test_fp8_wire_is_close(world_size, skew):
    """Rows travel as e4m3 with one fp32 scale per 1x128 block; outputs stay within e4m3 error of the oracle."""
    from chunked_ep_moe_b200.parallel.lockstep import LockstepWorld

    T, E, K, D, F, stripe, S = 64, 8, 2, 256, 256, 64, 128
    x, ids, weights, w_up, w_down, g = moe_cases.setup(world_size, T, E, K, D, F, skew, seed=5)
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=stripe, comm_dtype="float8_e4m3fn")
    bf = lambda t: t.cuda().to(torch.bfloat16).contiguous()
    sh = lambda t, r: moe_cases.shard(t, r, world_size)
    xs = [bf(sh(x, r)) for r in range(world_size)]
    gs = [bf(sh(g, r)) for r in range(world_size)]
    idl = [sh(ids, r).cuda() for r in range(world_size)]
    wl = [sh(weights, r).cuda() for r in range(world_size)]
    ups = [bf(sh(w_up, r)) for r in range(world_size)]
    downs = [bf(sh(w_down, r)) for r in range(world_size)]
    world = LockstepWorld(cfg, world_size, D, F, T)
    outs, saved = world.forward(xs, idl, wl, ups, downs)
    dxs, dws, dw_ups, dw_downs = world.backward(xs, gs, ups, downs, saved)
    torch.cuda.synchronize()
    want = _oracle_dev(torch.cat(xs), ids, weights, torch.cat(ups), torch.cat(downs), torch.cat(gs), stripe)
    got = {"out": torch.cat(outs), "dx": torch.cat(dxs), "dweights": torch.cat(dws).reshape(-1, K),
           "dw_up": torch.cat(dw_ups), "dw_down": torch.cat(dw_downs)}
    for name, val in got.items():
        a, b = val.float().cpu(), want[name].float()
        assert torch.isfinite(a).all(), name
        rel = float((a - b).norm() / b.norm())
        assert rel < 0.08, f"{name}: relative error {rel:.4f}"
    world.close()


def test_bounded_wait_reports_instead_of_hanging():
    """A wait on a counter nobody advances runs out after its limit and leaves an error status; the context survives."""
    from chunked_ep_moe_b200 import _build

    ext = _build.load()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    ext.wait_probe(flag, 5, 2000, status)
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    assert st[0] == 2 and st[1] == 5 and st[5] == 5 and st[6] == 0, st
    assert float(torch.ones(4, device="cuda").sum()) == 4.0  # the device still answers


@pytest.mark.parametrize("skew", ["uniform", "all_one", "rank0"])
def test_buffers_and_wire_rows_do_not_depend_on_the_routing(skew):
    """Whatever the routing, a rank holds the same bytes (every per-iteration buffer is S rows) and receives exactly
    the rows the traffic matrix says, no padding: the arrival counters of every (source, expert) segment end at that
    segment's row count."""
    from chunked_ep_moe_b200 import _build
    from chunked_ep_moe_b200.parallel.lockstep import LockstepWorld

    ext = _build.load()
    P, E, K, D, F, T, S = 4, 8, 2, 256, 256, 96, 64
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    x, ids, weights, w_up, w_down, _ = moe_cases.setup(P, T, E, K, D, F, skew, seed=2)
    bf = lambda t: t.cuda().to(torch.bfloat16)
    sh = lambda t, r: moe_cases.shard(t, r, P)
    world = LockstepWorld(cfg, P, D, F, T, cta_pairs=False)
    # geometry alone fixes what a rank holds; the routing is not an argument of either size
    assert world.arenas.nbytes == ext.arena_bytes(P, E // P, S, D, T * K, False)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    outs, saved = world.forward([bf(sh(x, r)) for r in range(P)], [sh(ids, r).cuda() for r in range(P)],
                                [sh(weights, r).cuda() for r in range(P)], [bf(sh(w_up, r)) for r in range(P)],
                                [bf(sh(w_down, r)) for r in range(P)])
    torch.cuda.synchronize()
    counts = torch.stack([torch.bincount(sh(ids, r).reshape(-1).long(), minlength=E) for r in range(P)])  # [s, e]
    lay = ext.arena_layout(P, E // P, S, D, T * K, False)
    L = E // P
    for r in range(P):
        arrived = ext.arena_read_i32(world.arenas.bases[r], lay["arrive"], P * L).reshape(P, L)
        assert torch.equal(arrived.long(), counts[:, r * L:(r + 1) * L]), f"rank {r}: rows received != rows routed"
    del outs, saved
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() <= before + (1 << 20), "a pass must not grow what the ranks hold"
    world.close()
