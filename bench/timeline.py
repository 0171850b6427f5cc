"""Device timeline of ONE forward+backward step of the fused layer on one GPU (no profiler replay).

Uses torch.profiler's CUDA activity records: start, end and duration of every kernel of the step, in launch
order, plus per-kernel means. Useful for seeing overlap (put beside GEMM, weight-gradient GEMMs on the auxiliary
stream) and gaps that a serialising profiler hides.

    python bench/timeline.py                 # DeepSeek-V3-size layer, 256 experts on this GPU
    python bench/timeline.py --experts 32    # the per-GPU share of an 8-GPU run (32 experts, same tokens)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench/timeline.py
                                             # rank 0's timeline inside a real 8-GPU run
"""

import argparse
import collections
import os
import re
import sys

import torch
from torch.profiler import ProfilerActivity, profile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--slice-size", type=int, default=8192)
    ap.add_argument("--comm-dtype", default=None)
    ap.add_argument("--quiet", action="store_true", help="only the per-kernel summary")
    ap.add_argument("--steps", type=int, default=1,
                    help="steps recorded back to back without a host synchronisation between them (per-kernel means "
                         "then include how kernels of consecutive steps wait for other ranks)")
    args = ap.parse_args()
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    T, D, F, E, K = args.tokens, args.hidden, args.ffn, args.experts, args.top_k
    L = E // world
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=args.slice_size, transport="nvshmem",
                           expert_compute="fused", stripe_width=64, comm_dtype=args.comm_dtype)
    gen = torch.Generator(device=dev).manual_seed(rank)
    w_up = torch.empty(L, D, 2 * F, device=dev, dtype=torch.bfloat16)
    w_down = torch.empty(L, F, D, device=dev, dtype=torch.bfloat16)
    for l in range(L):
        w_up[l] = (torch.randn(D, 2 * F, generator=gen, device=dev) * 0.006).to(torch.bfloat16)
        w_down[l] = (torch.randn(F, D, generator=gen, device=dev) * 0.006).to(torch.bfloat16)
    w_up.requires_grad_(True)
    w_down.requires_grad_(True)
    x = torch.randn(T, D, generator=gen, device=dev).to(torch.bfloat16)
    g = torch.randn(T, D, generator=gen, device=dev).to(torch.bfloat16)
    scores, ids = torch.topk(torch.sigmoid(torch.randn(T, E, generator=gen, device=dev)), K, dim=-1)
    w = scores / scores.sum(-1, keepdim=True)

    def step():
        xs, ws = x.detach().requires_grad_(True), w.detach().requires_grad_(True)
        w_up.grad = None
        w_down.grad = None
        chunked_moe(xs, ids.int(), ws, w_up, w_down, cfg, None).backward(g)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        from chunked_ep_moe_b200.ops import fused

        if rank != 0:
            fused.release_workspaces()
            dist.destroy_process_group()
            return
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    t0 = events[0].time_range.start
    summary = collections.OrderedDict()
    for e in events:
        start, end = e.time_range.start - t0, e.time_range.end - t0
        m = re.search(r"(grouped_gemm\w*<\d>|dispatch_put|combine_reduce|plan_build|sort_\w+|slice_done|pass_begin|"
                      r"dequant_slice|Memcpy \w+)", e.name)
        key = m.group(1) if m else e.name[:40]
        acc = summary.setdefault(key, [0, 0.0])
        acc[0] += 1
        acc[1] += (end - start) / 1000.0
        if not args.quiet:
            print(f"{start / 1000:9.3f} {end / 1000:9.3f}  {(end - start) / 1000:8.3f} ms  {e.name[:80]}")
    span = (max(e.time_range.end for e in events) - t0) / 1000.0
    print("\nkernel                          launches   total ms    mean ms")
    for key, (n, total) in summary.items():
        print(f"{key:32s} {n:6d} {total:10.3f} {total / n:10.3f}")
    flops = 24.0 * D * F * T * K
    span /= args.steps
    print(f"\nstep span {span:.3f} ms   {T / (span / 1e3):.0f} tokens/s   {flops / (span / 1e3) / 1e12:.0f} TFLOP/s"
          + (f"   (mean of {args.steps} steps back to back)" if args.steps > 1 else ""))
    if world > 1:
        from chunked_ep_moe_b200.ops import fused

        fused.release_workspaces()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
