"""Small single-GPU case for kernel profiling: two forward+backward passes of the fused layer.

Default: 16 experts, D=2048, F=1024, 16384 token copies. `--experts 16 --tokens 512 --top-k 8 --hidden 7168
--ffn 2048` gives the weight-gradient shape of the 256-experts-per-GPU layout (256 rows per expert, 1.4 GB of
weights) in one slice.

Sized so that a full-section profiler capture of a few launches ends in about a minute: 16 experts,
D=2048, F=1024 (201 MB of bf16 expert weights, larger than the 126 MB L2), 16384 token copies in
two 8192-row slices. Launch order of one pass: forward = sort x3, plan, pass_begin, put, put,
[swiglu, down+combine, done] x2, combine_reduce; backward = pass_begin, put, put,
[swiglu, down(d_weight), dswiglu, tgmm(dW_down), dx+combine, tgmm(dW_up), done] x2, combine_reduce.

    python bench/profile_case.py            # prints per-pass device times
"""

import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1024)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--slice-size", type=int, default=8192)
    args = ap.parse_args()
    torch.manual_seed(0)
    dev = torch.device("cuda:0")
    E, K, D, F, T, S = args.experts, args.top_k, args.hidden, args.ffn, args.tokens, args.slice_size
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, transport="nvshmem", expert_compute="fused",
                           stripe_width=64)
    x = torch.randn(T, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    scores, ids = torch.topk(torch.sigmoid(torch.randn(T, E, device=dev)), K, dim=-1)
    weights = (scores / scores.sum(-1, keepdim=True)).requires_grad_(True)
    w_up = (torch.randn(E, D, 2 * F, device=dev) / math.sqrt(D)).to(torch.bfloat16).requires_grad_(True)
    w_down = (torch.randn(E, F, D, device=dev) / math.sqrt(F)).to(torch.bfloat16).requires_grad_(True)
    for it in range(2):
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        w_up.grad = w_down.grad = x.grad = weights.grad = None
        e0.record()
        out = chunked_moe(x, ids.int(), weights, w_up, w_down, cfg, None)
        e1.record()
        out.backward(g)
        e2.record()
        torch.cuda.synchronize()
        print(f"pass {it}: forward {e0.elapsed_time(e1):.3f} ms, backward {e1.elapsed_time(e2):.3f} ms")


if __name__ == "__main__":
    main()
