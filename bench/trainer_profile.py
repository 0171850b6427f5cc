"""Where one training step of the DeepSeek-V3-style decoder spends its device time (one GPU, no profiler replay).

Runs the trainer's step (`chunked_ep_moe_b200.train` defaults: 5 layers, D=1024, 64 experts of F=512, top-6, 4096-token
sequences) for one rank's share of the 8-GPU job (4 sequences = 2 micro-batches of 2), records the CUDA activity of
one step with torch.profiler and prints device time per kernel name, grouped into the fused MoE kernels, library GEMMs
and attention, and PyTorch elementwise/reduction glue.

    python bench/trainer_profile.py
    python bench/trainer_profile.py --slice-size 8192
"""

import argparse
import collections
import os
import sys

import torch
from torch.profiler import ProfilerActivity, profile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from chunked_ep_moe_b200 import train as trainer  # noqa: E402
from chunked_ep_moe_b200.models.deepseek_tiny import DeepSeekTiny  # noqa: E402


def group_of(name: str) -> str:
    if "cem::" in name:
        return "fused MoE kernels"
    if "nvjet" in name or "cutlass" in name or "sgemm" in name or "gemm" in name.lower():
        return "library GEMMs"
    if "sdpa" in name or "flash" in name or "fmha" in name:
        return "attention"
    if "multi_tensor_apply" in name:
        return "optimizer"
    if "Memcpy" in name or "Memset" in name:
        return "copies"
    return "elementwise / reductions / softmax"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slice-size", type=int, default=None)
    ap.add_argument("--top", type=int, default=25)
    opts = ap.parse_args()
    argv = ["--global-batch", "4", "--micro-batch", "2", "--steps", "1"]
    if opts.slice_size:
        argv += ["--slice-size", str(opts.slice_size)]
    args = trainer.build_parser().parse_args(argv)
    torch.cuda.set_device(0)
    trainer.use_tf32_for_fp32_matmuls()
    cfg = trainer.model_config(args)
    model = DeepSeekTiny(cfg, None).to(device="cuda", dtype=torch.bfloat16)
    model.init_weights(0, 0)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True)

    def step(i):
        opt.zero_grad(set_to_none=True)
        for mb in range(2):
            tok, tgt = trainer.synthetic_batch(i * 2 + mb, 0, 2, args.seq_len, cfg.vocab_size, 0, "cuda")
            ce, aux = model(tok, tgt)
            ((ce + aux) / 2).backward()
        opt.step()
        for router in model.routers():
            router.update_bias(None)

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    step(3)
    e1.record()
    torch.cuda.synchronize()
    print(f"step without the profiler: {e0.elapsed_time(e1):.1f} ms (slice size {cfg.slice_size})")
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step(4)
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and not e.name.startswith("Optimizer")]
    per_kernel = collections.defaultdict(lambda: [0, 0.0])
    per_group = collections.defaultdict(lambda: [0, 0.0])
    for e in events:
        for table, key in ((per_kernel, e.name[:100]), (per_group, group_of(e.name))):
            table[key][0] += 1
            table[key][1] += e.device_time
    total = sum(v[1] for v in per_group.values())
    span = max(e.time_range.end for e in events) - min(e.time_range.start for e in events)
    print(f"{len(events)} kernels, {total / 1e3:.1f} ms of kernel time over a {span / 1e3:.1f} ms span")
    for key, (count, us) in sorted(per_group.items(), key=lambda kv: -kv[1][1]):
        print(f"  {us / 1e3:8.2f} ms {100 * us / total:5.1f} %  {count:5d} launches  {key}")
    print(f"top {opts.top} kernels")
    for key, (count, us) in sorted(per_kernel.items(), key=lambda kv: -kv[1][1])[:opts.top]:
        print(f"  {us:9.0f} us {count:5d}x  {key}")


if __name__ == "__main__":
    main()
