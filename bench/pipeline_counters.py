"""In-kernel pipeline counters of the grouped GEMM modes over a few forward+backward steps (one GPU, no profiler).

For every mode: SM cycles per k-block (512 is the tensor pipe's floor for a 128x256x64 bf16 block), the SM clock the
kernels really ran at (cycles / global-timer nanoseconds) and the share of the MMA warp's loop spent waiting for a
filled stage (loads late), for an accumulator (epilogue late), and of the producer's time waiting for a free stage
(MMAs late).

    python bench/pipeline_counters.py                 # DeepSeek-V3-size layer, 256 experts on this GPU
    python bench/pipeline_counters.py --experts 32    # the per-GPU share of an 8-GPU run, every row local
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe  # noqa: E402
from chunked_ep_moe_b200.ops import fused  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--slice-size", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T, D, F, E, K = args.tokens, args.hidden, args.ffn, args.experts, args.top_k
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=args.slice_size, transport="nvshmem",
                           expert_compute="fused", stripe_width=64)
    gen = torch.Generator(device=dev).manual_seed(0)
    w_up = torch.empty(E, D, 2 * F, device=dev, dtype=torch.bfloat16)
    w_down = torch.empty(E, F, D, device=dev, dtype=torch.bfloat16)
    for l in range(E):
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
    counters = fused.pipeline_counters(True)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    fused.pipeline_counters(False)
    print(f"{args.steps} steps with counters on: {start.elapsed_time(stop) / args.steps:.2f} ms per step; "
          f"CEM_CTA_PAIRS={os.environ.get('CEM_CTA_PAIRS', '0')}")
    c = sum(t.double() for t in counters).cpu()  # [6, CTAs, 8]
    s = {n: i for i, n in enumerate(fused.PIPELINE_COUNTER_SLOTS)}
    print("mode       k-blocks  cycles/k-block  SM GHz  mma wait loads %  mma wait epilogue %  producer wait mma %  "
          "epilogue idle %")
    for m, name in enumerate(fused.GEMM_MODE_NAMES):
        tot = c[m].sum(0)
        kb = tot[s["k_blocks"]].item()
        if kb == 0:
            continue
        loop = tot[s["loop_cycles"]].item()
        # producer counters come from every CTA, the MMA warp's from the CTAs that issue (all, or the pair leaders)
        issuing = (c[m][:, s["k_blocks"]] > 0).sum().item()
        loading = (c[m][:, s["producer_wait_free_stage"]] > 0).sum().item()
        scale = issuing / max(loading, 1)
        print(f"{name:9s} {kb:9.0f}  {loop / kb:14.1f}  {loop / max(tot[s['loop_ns']].item(), 1):6.3f}  "
              f"{100 * tot[s['mma_wait_filled_stage']].item() / loop:16.1f}  "
              f"{100 * tot[s['mma_wait_accumulator']].item() / loop:19.1f}  "
              f"{100 * scale * tot[s['producer_wait_free_stage']].item() / loop:19.1f}  "
              f"{100 * tot[s['epilogue_wait_accumulator']].item() / loop:15.1f}")


if __name__ == "__main__":
    main()
