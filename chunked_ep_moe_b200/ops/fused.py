"""The fused NVLink path: `chunked_moe` on the sm_100a kernels (`transport="nvshmem"`, `expert_compute="fused"`).

Per pass the host launches, per slice, a put kernel on the comm stream and a handful of grouped
tcgen05 GEMMs on the compute streams; everything between ranks happens inside those kernels
(peer stores, arrival counters, credits). The host never waits for the device inside a pass: the
slice count of a forward is guessed from the previous pass and corrected once its real value has
reached the host. Compared with the reference's loop
(src/chunked_moe/moe.py:96-119, :148-206):

  * no `[T*K, D]` send buffer: the put kernel gathers rows straight from `x[token]`;
  * the router weight is applied in the down-projection epilogue, which stores every finished
    row into the source rank's return buffer; a local K-way fixed-order sum finishes the token;
  * the backward folds `y` into `d_weight = <g, y>` inside the recomputed down GEMM's epilogue
    and forms `dy = w * g` there, so `y` never reaches HBM;
  * weight gradients are written once per expert in bf16; only the (at most one) expert that
    straddles a slice boundary carries an fp32 partial to the next slice.

Only the inputs and the integer plan (tables, send order, its inverse) are kept for the backward.
"""

from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _build
from ..config import ChunkedMoEConfig
from ..parallel.symm import SymmetricArena

_DEFAULT_SPIN_LIMIT = 1 << 24  # polls (~0.3 us each) before a wait on another rank gives up
_PUT_BLOCKS = 128  # measured: 128 blocks finish a put soonest and disturb the GEMM beside it least

_workspaces: dict = {}
_retired: list = []  # workspaces replaced by `reserve()`; passes in flight may still hold them

#: Pass as `group` to run the fused kernels on this rank alone (a 1-rank expert-parallel world), whatever
#: process groups exist. Used by `ops.fused_expert` to serve `expert_compute="fused"` on collective transports.
SOLO = "solo"


def use_cta_pairs(tokens_times_k: int, local_experts: int) -> bool:
    """Which GEMM kernel family a workspace runs: CTA pairs (`cta_group::2`, 256-row tiles) or single CTAs.

    The pair kernels are faster per tile but round every expert's rows in a slice up to 256 instead of 128, so they
    win once an expert receives many rows per pass (measured cross-over: ~512 rows per expert is a draw, 1024 rows
    +5 %, 2048 rows +8 %). `CEM_CTA_PAIRS=0/1` overrides the choice.
    """
    env = os.environ.get("CEM_CTA_PAIRS")
    if env is not None:
        return env != "0"
    return tokens_times_k // max(local_experts, 1) >= 768


class FusedWorkspace:
    """Symmetric arena + per-rank executor for one (geometry, process group)."""

    def __init__(self, cfg: ChunkedMoEConfig, group, hidden: int, ffn: int, tk_cap: int):
        ext = _build.load()
        initialised = dist.is_available() and dist.is_initialized() and group is not SOLO
        self.world = dist.get_world_size(group) if initialised else 1
        self.rank_index = dist.get_rank(group) if initialised else 0
        self.local_experts = cfg.num_experts // self.world
        if group is SOLO:
            group = None
        if self.world > 1:  # the arena layout must be identical everywhere: agree on the capacity
            cap = torch.tensor([tk_cap], device="cuda", dtype=torch.int64)
            dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=group)
            tk_cap = int(cap.item())
        self.tk_cap = tk_cap
        self.fp8 = cfg.comm_dtype == "float8_e4m3fn"
        self.max_slices = max(1, math.ceil(self.world * tk_cap / cfg.slice_size)) + 1
        nbytes = ext.arena_bytes(self.world, self.local_experts, cfg.slice_size, hidden, tk_cap, self.fp8)
        self.arena = SymmetricArena(nbytes, group, solo=self.world == 1)
        self.rank = ext.FusedRank(
            P=self.world, L=self.local_experts, me=self.rank_index, S=cfg.slice_size, D=hidden, F=ffn, K=cfg.top_k,
            stripe=cfg.stripe_width, tk_cap=tk_cap, max_slices=self.max_slices,
            num_sms=int(os.environ.get("CEM_GEMM_GRID", cfg.num_sms)), fp8=self.fp8,
            arena=self.arena.local, peer_arenas=self.arena.peers, use_comm_stream=True,
            spin_limit=int(os.environ.get("CEM_SPIN_LIMIT", _DEFAULT_SPIN_LIMIT)), put_blocks=int(os.environ.get("CEM_PUT_BLOCKS", _PUT_BLOCKS)),
            cta_pairs=use_cta_pairs(tk_cap, self.local_experts),
            tgmm_pairs=os.environ.get("CEM_TGMM_PAIRS", "1") != "0")
        if "CEM_MBAR_LIMIT_US" in os.environ:
            self.rank.set_mbar_limit_us(int(os.environ["CEM_MBAR_LIMIT_US"]))
        self.plan_ints = self.rank.plan_ints()
        self.dummy_counts = torch.zeros(1, dtype=torch.int32, device="cuda")


def _workspace_key(cfg: ChunkedMoEConfig, group, hidden: int, ffn: int):
    # The process group OBJECT is part of the key (not its id): the dictionary keeps it alive, so a later group can
    # never be mistaken for it.
    return (group, cfg.num_experts, cfg.top_k, cfg.slice_size, cfg.stripe_width, cfg.comm_dtype, cfg.num_sms, hidden,
            ffn, torch.cuda.current_device())


def get_workspace(cfg: ChunkedMoEConfig, group, hidden: int, ffn: int, tokens_times_k: int) -> FusedWorkspace:
    """The cached workspace for this geometry and group; the first call creates it (collectively).

    A workspace never shrinks, moves or is freed behind a pass that still holds it: its capacity is fixed when it is
    created (the largest `T*K` over the ranks at that moment). A later call that needs more gets a new, larger one
    when this rank is alone; among several ranks it raises, because making room is a collective decision:
    `reserve()` is the way to do that.
    """
    key = _workspace_key(cfg, group, hidden, ffn)
    ws = _workspaces.get(key)
    if ws is None:
        ws = FusedWorkspace(cfg, group, hidden, ffn, tokens_times_k)
        _workspaces[key] = ws
    elif ws.tk_cap < tokens_times_k and ws.world == 1:
        ws = reserve(cfg, group, hidden, ffn, tokens_times_k)  # nobody to agree with: make room right away
    elif ws.tk_cap < tokens_times_k:
        raise RuntimeError(
            f"chunked_moe fused path: this call has {tokens_times_k} token copies but the workspace of this geometry "
            f"was created for {ws.tk_cap}. Capacity is agreed between the ranks when the workspace is created; call "
            f"ops.fused.reserve(cfg, group, hidden, ffn, tokens_times_k) on every rank first.")
    return ws


def reserve(cfg: ChunkedMoEConfig, group, hidden: int, ffn: int, tokens_times_k: int) -> FusedWorkspace:
    """Collective: makes sure the workspace of this geometry holds `tokens_times_k` token copies on every rank.

    A workspace that is too small is replaced, not freed: passes whose backward has not run yet keep using the arena
    they started with, and the old workspace is only released by `release_workspaces()`.
    """
    key = _workspace_key(cfg, group, hidden, ffn)
    ws = _workspaces.get(key)
    need = tokens_times_k
    if dist.is_available() and dist.is_initialized() and group is not SOLO and dist.get_world_size(group) > 1:
        t = torch.tensor([need, ws.tk_cap if ws is not None else 0], device="cuda", dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        need, have = int(t[0]), int(t[1])
    else:
        have = ws.tk_cap if ws is not None else 0
    if ws is None or have < need:  # every rank takes the same branch: both numbers are maxima over the ranks
        if ws is not None:
            _retired.append(ws)
        ws = FusedWorkspace(cfg, group, hidden, ffn, need)
        _workspaces[key] = ws
    return ws


def release_workspaces() -> None:
    """Frees every workspace, cached or replaced (collective when a process group is involved). A pass whose backward
    has not run yet must not be kept across this call: its backward raises."""
    for ws in list(_workspaces.values()) + _retired:
        ws.rank = None
        ws.arena.close()
    _workspaces.clear()
    _retired.clear()


def last_plan_stats(cfg: ChunkedMoEConfig) -> list:
    """Load statistics of the most recent pass of every cached workspace (rows, slices, padding, remote rows)."""
    from ..utils.stats import header_stats

    return [header_stats(list(ws.rank.plan_header()), cfg.slice_size) for ws in _workspaces.values()
            if ws.rank is not None]


def check_status() -> None:
    """Synchronises and raises if any kernel of a cached workspace recorded an error (a wait that ran out).

    The forward checks on its own (it has to read the slice count back anyway); the backward does not synchronise,
    so a training loop calls this once per step, before the optimizer consumes the gradients.
    """
    for ws in _workspaces.values():
        if ws.rank is not None:
            ws.rank.check_status()


def launches() -> int:
    """Kernels launched so far by every cached workspace of this process."""
    return sum(int(ws.rank.launches()) for ws in _workspaces.values() if ws.rank is not None)


def expected_launches(num_slices: int, fp8: bool = False) -> int:
    """Kernels one forward+backward of the fused layer launches on a rank that loops `num_slices` slices.

    Forward: sort (3) + plan build + pass begin + per slice (put, swiglu, down+combine, slice done) + combine reduce.
    Backward: pass begin + per slice (put, swiglu+h, down->d_weight/dy, dswiglu, dW_down, dx+combine, dW_up, slice
    done) + combine reduce. The fp8 wire adds one dequantisation kernel per slice and pass.
    """
    per_slice = 12 + (2 if fp8 else 0)
    return 8 + per_slice * num_slices


def memory_plan(world: int, experts: int, top_k: int, tokens_per_rank: int, hidden: int, ffn: int, slice_size: int,
                fp8: bool = False, tk_cap: int | None = None) -> dict:
    """Bytes one rank of the fused path holds, by purpose (no GPU needed: sizes come from the arena layout).

    `tk_cap` is the workspace capacity in token copies (default `tokens_per_rank * top_k`).
    """
    ext = _build.load()
    L = experts // world
    tk = tokens_per_rank * top_k if tk_cap is None else tk_cap
    S, D, F = slice_size, hidden, ffn
    arena = int(ext.arena_bytes(world, L, S, D, tk, fp8))
    scratch = 2 * (S * F * 2 + S * 2 * F * 2 + S * D * 2 + S * 2 * F * 2 + S * (D // 256) * 4)  # act, h, dy, dh, dwp x2
    carry = 2 * (D * 2 * F + F * D) * 4
    weights = L * (D * 2 * F + F * D) * 2
    max_slices = max(1, math.ceil(world * tk / S)) + 1
    plan = int(ext.plan_layout(world, L, S, max_slices)["total"]) * 4
    saved = tokens_per_rank * D * 2 + tk * 4 * 3 + plan  # x, router weights, order, inverse order, plan tables
    out = {
        "arena (slice buffers x2 for x and g, return rows, counters, traffic matrix)": arena,
        "scratch (act, h, dy, dh, d_weight partials; two slices in flight)": scratch,
        "weight-gradient carry tiles (fp32, two per matrix)": carry,
        "expert weights (bf16)": weights,
        "expert weight gradients (bf16)": weights,
        "saved for backward (x, router weights, sort order, plan)": saved,
    }
    out["total"] = sum(out.values())
    return out


PIPELINE_COUNTER_SLOTS = ("loop_cycles", "loop_ns", "producer_wait_free_stage", "mma_wait_filled_stage",
                          "mma_wait_accumulator", "k_blocks", "epilogue_wait_accumulator", "tiles")
GEMM_MODE_NAMES = ("swiglu", "down_fwd", "down_dw", "dswiglu", "dx", "tgmm")


def pipeline_counters(enable: bool = True) -> list:
    """Turns the GEMM kernels' in-kernel pipeline counters on (or off) for every cached workspace.

    Returns one zeroed int64 tensor `[6 modes, CTAs, 8 slots]` per workspace (slot names:
    `PIPELINE_COUNTER_SLOTS`); every later GEMM launch adds its CTAs' cycle counts to it. The counters say which
    side of the operand ring waits for the other (loads or MMAs) and, from cycles / nanoseconds, the SM clock the
    kernels really ran at. Diagnostics: counting costs a few clock reads per k-block.
    """
    out = []
    for ws in _workspaces.values():
        if ws.rank is None:
            continue
        if not enable:
            ws.rank.set_pipeline_counters(None)
            continue
        t = torch.zeros(6, max(148, torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count),
                        len(PIPELINE_COUNTER_SLOTS), dtype=torch.int64, device="cuda")
        ws.rank.set_pipeline_counters(t)
        out.append(t)
    return out


def nvtx(name: str):
    from ..utils.nvtx import nvtx_range

    return nvtx_range(name)


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError("chunked_moe fused path: " + msg)


class _ChunkedMoEFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, expert_ids, weights, w_up, w_down, cfg, group):
        tokens, hidden = x.shape
        ffn = w_down.shape[1]
        ws = get_workspace(cfg, group, hidden, ffn, tokens * cfg.top_k)
        rank = ws.rank
        dev = x.device
        plan = torch.empty(ws.plan_ints, dtype=torch.int32, device=dev)
        order = torch.zeros(tokens * cfg.top_k, dtype=torch.int32, device=dev)  # no stray indices if an id is invalid
        inv_order = torch.zeros_like(order)
        ids32 = expert_ids.to(torch.int32).contiguous()
        w_flat = weights.detach().float().reshape(-1).contiguous()
        xc, w_up_c, w_down_c = x.detach().contiguous(), w_up.detach().contiguous(), w_down.detach().contiguous()
        def run_slices(lo: int, hi: int) -> None:
            if hi <= lo:
                return
            rank.put(lo, plan, order, xc, None, w_flat)
            for j in range(lo, hi):
                with nvtx(f"chunked_moe/fwd slice {j}"):
                    if j + 1 < hi:
                        rank.put(j + 1, plan, order, xc, None, w_flat)  # slice j+1 is in flight while slice j computes
                    rank.compute_forward(j, plan, w_up_c, w_down_c)

        # The slice count is a device value (it depends on the routing). The host does not wait for it: it launches
        # as many slices as the previous pass of this workspace needed, THEN reads the real count (by then long on
        # the host) and launches what is missing. Too many is harmless: a slice past the real count finds empty
        # tables on every rank. Every rank guesses and learns the same numbers, so all ranks loop alike.
        with nvtx("chunked_moe/plan"):
            guess = max(0, rank.begin_forward_async(ids32, plan, order, inv_order, ws.dummy_counts, False))
        out = torch.empty_like(xc)
        run_slices(0, guess)
        n = rank.resolve_slices()  # raises here if an earlier kernel recorded an error (bad expert id, timed-out wait)
        run_slices(guess, n)
        rank.set_pass_slices(max(guess, n))
        with nvtx("chunked_moe/combine"):
            rank.finish_forward(inv_order, out)
        ctx.save_for_backward(xc, weights, w_up_c, w_down_c, plan, order, inv_order)
        ctx.cfg, ctx.group, ctx.ws, ctx.num_slices = cfg, group, ws, int(n)
        ctx.mark_non_differentiable(expert_ids)
        return out

    @staticmethod
    def backward(ctx, g_out):
        x, weights, w_up, w_down, plan, order, inv_order = ctx.saved_tensors
        rank = ctx.ws.rank
        if rank is None or ctx.ws.arena.local == 0:
            raise RuntimeError("chunked_moe fused path: the workspace of this pass was released before its backward")
        g = g_out.to(x.dtype).contiguous()
        w_flat = weights.detach().float().reshape(-1).contiguous()
        # The slice count is the forward's: nothing is read back, the host never waits for the device here.
        n = rank.begin_backward(plan, ctx.num_slices, order.numel())
        dw_up, dw_down = torch.empty_like(w_up), torch.empty_like(w_down)
        if n > 0:
            rank.put(0, plan, order, x, g, w_flat)
        else:
            dw_up.zero_()
            dw_down.zero_()
        for j in range(n):
            with nvtx(f"chunked_moe/bwd slice {j}"):
                if j + 1 < n:
                    rank.put(j + 1, plan, order, x, g, w_flat)
                rank.compute_backward(j, plan, w_up, w_down, dw_up, dw_down)
        dx = torch.empty_like(x)
        d_weights = torch.empty(weights.numel(), dtype=torch.float32, device=x.device)
        rank.finish_backward(inv_order, dx, d_weights)
        return dx, None, d_weights.reshape(weights.shape).to(weights.dtype), dw_up, dw_down, None, None


def unsupported_reason(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                       cfg: ChunkedMoEConfig) -> Optional[str]:
    """Why these tensors cannot run on the fused kernels (shape or dtype), or None. The caller may then fall back to
    a collective transport, as the reference's put kernel does for rows it cannot move
    (src/chunked_moe/transport/nvshmem.py:115-118)."""
    if x.dtype != torch.bfloat16 or w_up.dtype != torch.bfloat16 or w_down.dtype != torch.bfloat16:
        return "x, w_up and w_down must be bfloat16"
    if x.shape[1] % 256 or w_down.shape[1] % 256:
        return f"D={x.shape[1]} and F={w_down.shape[1]} must be multiples of 256"
    if cfg.stripe_width not in (32, 64, 128):
        return f"stripe_width={cfg.stripe_width} must be 32, 64 or 128"
    if cfg.slice_size % 8:
        return f"slice_size={cfg.slice_size} must be a multiple of 8"
    if cfg.accum_dtype != "float32":
        return f"accum_dtype={cfg.accum_dtype!r}: the kernels accumulate weight gradients in float32"
    return None


def chunked_moe_fused(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor,
                      w_down: torch.Tensor, cfg: ChunkedMoEConfig,
                      group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    _require(cfg.expert_compute == "fused", 'transport="nvshmem" requires expert_compute="fused"')
    _require(x.is_cuda, "inputs must be CUDA tensors (the sm_100a extension has no CPU path)")
    _require(x.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16,
             "x, w_up and w_down must be bfloat16")
    _require(x.shape[1] % 256 == 0 and w_down.shape[1] % 256 == 0, "needs D % 256 == 0 and F % 256 == 0")
    _require(cfg.stripe_width in (32, 64, 128), "needs stripe_width in {32, 64, 128}")
    _require(cfg.slice_size % 8 == 0, "needs slice_size % 8 == 0")
    _require(cfg.accum_dtype == "float32", "weight gradients are accumulated in float32 (accum_dtype)")
    return _ChunkedMoEFused.apply(x, expert_ids, weights, w_up, w_down, cfg, group)
