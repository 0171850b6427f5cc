"""Sampled correctness check of one layer step against an fp32 oracle, at any size and any number of ranks.

A dense oracle of the whole layer is out of reach at benchmark sizes (DeepSeek-V3: 256 experts x 88 MB of weights,
65,536 token copies per rank), and a rank does not even hold the weights of most of the experts its tokens visit.
What this check does instead, all ranks together:

  * tokens: every rank picks the same `sample` token positions and all-gathers those tokens' inputs (x, the output
    gradient, expert ids, router weights): a few MB. Every rank then evaluates, in fp32 and with ITS OWN experts'
    weights, every (sampled token, choice) pair routed to one of its experts: the contribution to the token's output,
    to its dX, and the d(router weight) of that choice. One all-reduce adds the partial sums up, and each rank
    compares its own sampled rows with what the layer returned.
  * weight gradients: for two experts per rank (its first and its last) all ranks send the rows they routed to that
    expert to everybody (variable-length all-gather); the owner recomputes that expert's dW_up and dW_down in fp32
    from all of its rows and compares the full matrices.

Errors are max-abs differences relative to the oracle's max-abs, the measure the kernel tests use
(reference tolerance for bf16 kernels: 3e-2, tests/test_fused_kernels.py:41-46).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.striping import striped_swiglu, striped_swiglu_bwd


def _world(group) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _all_gather_rows(t: torch.Tensor, group, world: int) -> torch.Tensor:
    """Concatenates equally shaped tensors of all ranks along dim 0."""
    if world == 1:
        return t
    out = torch.empty((world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def _all_gather_ragged(t: torch.Tensor, group, world: int) -> torch.Tensor:
    """Concatenates tensors whose dim 0 differs between ranks (padded to the longest for the collective)."""
    if world == 1:
        return t
    n = torch.tensor([t.shape[0]], device=t.device, dtype=torch.int64)
    sizes = torch.empty(world, device=t.device, dtype=torch.int64)
    dist.all_gather_into_tensor(sizes, n, group=group)
    sizes = sizes.tolist()
    padded = t.new_zeros((max(max(sizes), 1),) + tuple(t.shape[1:]))
    padded[: t.shape[0]] = t
    everyone = _all_gather_rows(padded, group, world).reshape((world, padded.shape[0]) + tuple(t.shape[1:]))
    return torch.cat([everyone[r, : sizes[r]] for r in range(world)], dim=0)


def _rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.float(), want.float()
    if not torch.isfinite(got).all():
        return float("inf")
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-12))


def _expert_rows_fp32(x, g, w, w_up_e, w_down_e, stripe):
    """fp32 forward and backward of one expert on rows `x` with output gradient `g` and router weight `w` per row.

    Returns (weighted output rows, dX rows, d(router weight) per row, dW_up, dW_down).
    """
    wu, wd = w_up_e.float(), w_down_e.float()
    h = x @ wu
    act = striped_swiglu(h, stripe)
    y = act @ wd
    dy = w[:, None] * g
    dh = striped_swiglu_bwd(h, dy @ wd.t(), stripe)
    return w[:, None] * y, dh @ wu.t(), (g * y).sum(dim=-1), x.t() @ dh, act.t() @ dy


def sampled_check(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, g_out: torch.Tensor,
                  w_up: torch.Tensor, w_down: torch.Tensor, out: torch.Tensor, dx: torch.Tensor,
                  d_weights: torch.Tensor, dw_up: torch.Tensor, dw_down: torch.Tensor, *, stripe: int,
                  group: Optional[dist.ProcessGroup] = None, sample: int = 64, tol: float = 3e-2) -> dict:
    """Compares one step's results with the sampled fp32 oracle. Collective: every rank of `group` must call it.

    All tensors are this rank's: inputs `x [T, D]`, `expert_ids [T, K]`, `weights [T, K]`, `g_out [T, D]`, local
    weights `w_up [L, D, 2F]`, `w_down [L, F, D]`, and the step's results `out`, `dx`, `d_weights [T, K]`, `dw_up`,
    `dw_down`. Returns the five relative errors (maximum over ranks), their maximum, `tol`, and `ok`.
    """
    world, rank = _world(group)
    num_tokens, hidden = x.shape
    top_k = expert_ids.shape[1]
    local = w_up.shape[0]
    dev = x.device
    sample = min(sample, num_tokens)
    picks = torch.linspace(0, num_tokens - 1, sample, device=dev).round().long()

    # ---- sampled tokens: every rank evaluates the (token, choice) pairs that visit its experts -------------------
    xs = _all_gather_rows(x[picks].float(), group, world)
    gs = _all_gather_rows(g_out[picks].float(), group, world)
    ids = _all_gather_rows(expert_ids[picks].to(torch.int64), group, world)
    ws = _all_gather_rows(weights[picks].float(), group, world)
    out_ref = torch.zeros_like(xs)
    dx_ref = torch.zeros_like(xs)
    dwt_ref = torch.zeros_like(ws)
    for l in range(local):
        tok, choice = (ids == rank * local + l).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        y, dxr, dwt, _, _ = _expert_rows_fp32(xs[tok], gs[tok], ws[tok, choice], w_up[l], w_down[l], stripe)
        out_ref.index_add_(0, tok, y)
        dx_ref.index_add_(0, tok, dxr)
        dwt_ref[tok, choice] = dwt
    if world > 1:
        for t in (out_ref, dx_ref, dwt_ref):
            dist.all_reduce(t, group=group)
    mine = slice(rank * sample, (rank + 1) * sample)
    errs = {
        "out": _rel_err(out[picks], out_ref[mine]),
        "dx": _rel_err(dx[picks], dx_ref[mine]),
        "d_weights": _rel_err(d_weights[picks], dwt_ref[mine]),
        "dw_up": 0.0,
        "dw_down": 0.0,
    }

    # ---- weight gradients of each rank's first and last expert, from ALL ranks' rows ------------------------------
    flat_ids = expert_ids.reshape(-1).to(torch.int64)
    for owner in range(world):
        for l in sorted({0, local - 1}):
            sel = (flat_ids == owner * local + l).nonzero(as_tuple=True)[0]
            tok = sel // top_k
            rows_x = _all_gather_ragged(x[tok], group, world)
            rows_g = _all_gather_ragged(g_out[tok], group, world)
            rows_w = _all_gather_ragged(weights.reshape(-1)[sel].float(), group, world)
            if owner != rank:
                continue
            if rows_x.shape[0] == 0:
                want_up, want_down = torch.zeros_like(dw_up[l], dtype=torch.float32), torch.zeros_like(
                    dw_down[l], dtype=torch.float32)
            else:
                _, _, _, want_up, want_down = _expert_rows_fp32(rows_x.float(), rows_g.float(), rows_w, w_up[l],
                                                                w_down[l], stripe)
            errs["dw_up"] = max(errs["dw_up"], _rel_err(dw_up[l], want_up))
            errs["dw_down"] = max(errs["dw_down"], _rel_err(dw_down[l], want_down))

    vals = torch.tensor([errs[k] for k in ("out", "dx", "d_weights", "dw_up", "dw_down")], device=dev,
                        dtype=torch.float64)
    vals = torch.nan_to_num(vals, nan=float("inf"), posinf=1e30)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX, group=group)
    names = ("out", "dx", "d_weights", "dw_up", "dw_down")
    result = {name: float(v) for name, v in zip(names, vals.tolist())}
    worst = max(result.values())
    return {"max_rel_err": worst, "tol": tol, "ok": bool(worst <= tol), "sampled_tokens_per_rank": sample,
            "experts_checked_per_rank": len({0, local - 1}), **result}
