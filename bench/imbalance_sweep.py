"""Routing-imbalance stress of the DeepSeek-V3-size layer: Zipf(1.2) expert popularity and "every token's first
choice is expert 0", each at slice sizes 2048 and 8192, fused path and NCCL baseline, in ONE launch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench/imbalance_sweep.py

Per cell rank 0 prints one JSON line: ms per step (CUDA events, max over ranks) of both implementations, the plan's
load statistics (longest receive stream, slices every rank loops, padding rows of the busiest rank, rows that leave
each GPU), and the bytes the fused path holds per rank, which depend on (ranks, experts, S, D, T*K) only: whatever
the routing, every per-iteration buffer is S rows.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe  # noqa: E402
from chunked_ep_moe_b200.ops import fused  # noqa: E402
from chunked_ep_moe_b200.ops.plan import make_plan  # noqa: E402


def routing(gen, tokens, experts, top_k, skew, device):
    logits = torch.randn(tokens, experts, generator=gen, device=device)
    if skew == "zipf":  # Zipf(s=1.2) popularity over experts, sampled without replacement per token
        pop = 1.0 / torch.arange(1, experts + 1, device=device, dtype=torch.float32) ** 1.2
        ids = torch.multinomial(pop.expand(tokens, experts), top_k, replacement=False, generator=gen)
        scores = torch.sigmoid(torch.gather(logits, 1, ids))
    else:
        if skew == "expert0":
            logits[:, 0] += 100.0
        scores, ids = torch.topk(torch.sigmoid(logits), top_k, dim=-1)
    return ids.to(torch.int32), (scores / scores.sum(-1, keepdim=True)).float()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--baseline-steps", type=int, default=1)
    ap.add_argument("--skews", default="zipf,expert0")
    ap.add_argument("--slice-sizes", default="2048,8192")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    T, D, F, E, K = args.tokens, args.hidden, args.ffn, args.experts, args.top_k
    L = E // world
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    w_up = torch.empty(L, D, 2 * F, device=dev, dtype=torch.bfloat16)
    w_down = torch.empty(L, F, D, device=dev, dtype=torch.bfloat16)
    for l in range(L):
        w_up[l] = (torch.randn(D, 2 * F, generator=gen, device=dev) * 0.006).to(torch.bfloat16)
        w_down[l] = (torch.randn(F, D, generator=gen, device=dev) * 0.006).to(torch.bfloat16)
    w_up.requires_grad_(True)
    w_down.requires_grad_(True)
    x = torch.randn(T, D, generator=gen, device=dev).to(torch.bfloat16)
    g = torch.randn(T, D, generator=gen, device=dev).to(torch.bfloat16)

    def timed(cfg, ids, weights, warmup, steps):
        def step():
            xs, ws = x.detach().requires_grad_(True), weights.detach().requires_grad_(True)
            w_up.grad = None
            w_down.grad = None
            chunked_moe(xs, ids, ws, w_up, w_down, cfg, group).backward(g)

        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        w_up.grad = None
        w_down.grad = None
        return float(ms)

    for skew in args.skews.split(","):
        ids, weights = routing(gen, T, E, K, skew, dev)
        for S in (int(v) for v in args.slice_sizes.split(",")):
            fused_cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, stripe_width=64, transport="nvshmem",
                                         expert_compute="fused")
            base_cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, stripe_width=64,
                                        transport="ragged_a2a", expert_compute="reference")
            stats = make_plan(ids, E, S, group).stats()
            fused_ms = timed(fused_cfg, ids, weights, 2, args.steps)
            fused.check_status()
            mem = fused.memory_plan(world, E, K, T, D, F, S)
            fused.release_workspaces()
            torch.cuda.empty_cache()
            try:
                base_ms = timed(base_cfg, ids, weights, 1, args.baseline_steps)
            except Exception as exc:  # noqa: BLE001 - e.g. out of memory in the library path
                base_ms, stats["baseline_error"] = None, f"{type(exc).__name__}: {exc}"[:160]
            torch.cuda.empty_cache()
            if rank == 0:
                rows = stats["stream_rows"]
                print(json.dumps({
                    "skew": skew, "slice_size": S, "n_gpus": world, "fused_ms_per_step": fused_ms,
                    "baseline_ms_per_step": base_ms, "speedup": (base_ms / fused_ms) if base_ms else None,
                    "tokens_per_s_per_gpu": T / (fused_ms / 1e3), "slices": stats["num_slices"],
                    "max_stream_rows": max(rows), "min_stream_rows": min(rows),
                    "padding_rows_busiest_rank": -(-max(rows) // S) * S - max(rows),
                    "rows_sent_remote_rank0": stats["rows_sent_remote"],
                    "remote_bytes_rank0_fwd": stats["rows_sent_remote"] * (D * 2 + 4),
                    "arena_bytes_per_rank": mem["arena (slice buffers x2 for x and g, return rows, counters, "
                                                "traffic matrix)"],
                    "scratch_bytes_per_rank": mem["scratch (act, h, dy, dh, d_weight partials; two slices in "
                                                  "flight)"],
                }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
