"""End-to-end trainer for the DeepSeek-V3-style decoder (bf16 weights + AdamW, expert parallel).

    python -m chunked_ep_moe_b200.train --steps 8                                      # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m chunked_ep_moe_b200.train --steps 8

Every rank holds the dense parameters (replicated) and its own `E / N` experts. The global batch is
split over ranks (data parallel); inside a MoE layer the ranks are expert parallel. After the
backward, dense gradients are all-reduced (mean) over the group; expert gradients need no
reduction (each rank's dW already sums every rank's tokens routed to it) and are only divided by
the world size so they are gradients of the same global-mean loss. Token ids are uniform-random
from the seed; weights are random-init (no datasets or checkpoints are needed).
"""

from __future__ import annotations

import argparse
import json
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from .models.deepseek_tiny import DeepSeekTiny, DeepSeekTinyConfig
from .utils import checkpoint as ckpt
from .utils.timing import DeviceTimer


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--global-batch", type=int, default=32, help="sequences per optimizer step, over all ranks")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=2, help="sequences per forward/backward on one rank")
    ap.add_argument("--impl", default="fused", choices=["fused", "baseline"])
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--layers", type=int, default=5)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--moe-ffn", type=int, default=512)
    ap.add_argument("--dense-ffn", type=int, default=4096)
    ap.add_argument("--top-k", type=int, default=6)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--slice-size", type=int, default=16384,
                    help="rows per slice; with these small experts (D=1024, F=512) larger slices mean fewer, fuller "
                         "launches (measured on one GPU: 58 ms per step at 8192, 42 ms at 16384, 41 ms at 49152)")
    ap.add_argument("--comm-dtype", default=None, choices=[None, "float8_e4m3fn"])
    ap.add_argument("--save", default=None, help="directory to write a checkpoint to after the last step")
    ap.add_argument("--resume", default=None, help="directory to resume from")
    ap.add_argument("--health-timeout", type=float, default=0.0,
                    help="seconds to wait for every rank's heartbeat before each step (0 = no heartbeat)")
    ap.add_argument("--json", action="store_true", help="print one JSON summary line at the end (rank 0)")
    return ap


def model_config(args) -> DeepSeekTinyConfig:
    fused = args.impl == "fused"
    return DeepSeekTinyConfig(
        vocab_size=args.vocab, d_model=args.d_model, n_layers=args.layers, n_heads=args.d_model // 64, head_dim=64,
        dense_ffn=args.dense_ffn, num_experts=args.experts, moe_ffn=args.moe_ffn, top_k=args.top_k,
        shared_ffn=args.moe_ffn, slice_size=args.slice_size, transport="nvshmem" if fused else "ragged_a2a",
        expert_compute="fused" if fused else "reference", comm_dtype=args.comm_dtype)


def synthetic_batch(step: int, rank: int, seqs: int, seq_len: int, vocab: int, seed: int, device):
    """Uniform-random token ids, a function of (seed, step, rank) only, so runs are reproducible and resumable."""
    gen = torch.Generator(device="cpu").manual_seed(seed * 1_000_003 + step * 1009 + rank)
    tokens = torch.randint(0, vocab, (seqs, seq_len + 1), generator=gen)
    return tokens[:, :-1].to(device, non_blocking=True), tokens[:, 1:].to(device, non_blocking=True)


def reduce_gradients(model: DeepSeekTiny, world: int, group=None) -> None:
    if world == 1:
        return
    dense = [p.grad for p in model.dense_parameters() if p.grad is not None]
    flat = torch.cat([g.reshape(-1).float() for g in dense])
    dist.all_reduce(flat, group=group)
    flat /= world
    off = 0
    for g in dense:
        g.copy_(flat[off:off + g.numel()].reshape(g.shape))
        off += g.numel()
    for p in model.expert_parameters():
        if p.grad is not None:
            p.grad /= world


def use_tf32_for_fp32_matmuls() -> None:
    """The model's only fp32 matmuls are the router's logits and their backward. In the forward both operands are bf16
    values widened to fp32, which TF32 holds exactly, so the tensor-core TF32 GEMM forms the same products as the SIMT
    fp32 GEMM (accumulation stays fp32) in a fraction of its time."""
    torch.backends.cuda.matmul.allow_tf32 = True


def train(args, group=None) -> dict:
    use_tf32_for_fp32_matmuls()
    distributed = dist.is_available() and dist.is_initialized()
    world = dist.get_world_size(group) if distributed else 1
    rank = dist.get_rank(group) if distributed else 0
    device = torch.device("cuda", torch.cuda.current_device())
    if args.global_batch % world:
        raise ValueError(f"global batch {args.global_batch} is not divisible by {world} ranks")
    per_rank = args.global_batch // world
    micro = min(args.micro_batch, per_rank)
    if per_rank % micro:
        raise ValueError(f"per-rank batch {per_rank} is not divisible by the micro batch {micro}")
    accum = per_rank // micro

    cfg = model_config(args)
    model = DeepSeekTiny(cfg, group).to(device=device, dtype=torch.bfloat16)
    model.init_weights(args.seed, rank)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=args.weight_decay, betas=(0.9, 0.95),
                            fused=True)
    start_step = 0
    if args.resume:
        start_step = ckpt.load_checkpoint(args.resume, model, opt, rank)

    health = None
    if distributed and world > 1 and args.health_timeout > 0:
        from .utils.health import RankHealth

        health = RankHealth(dist.distributed_c10d._get_default_store(), rank, world, timeout_s=args.health_timeout)

    losses, step_ms = [], []
    timer = DeviceTimer()
    for step in range(start_step, start_step + args.steps):
        if health is not None:
            health.step_barrier(step)  # a missing peer is reported here, on the host, with nothing in flight
        timer.start()
        opt.zero_grad(set_to_none=True)
        loss_sum = torch.zeros((), device=device)
        for mb in range(accum):
            tokens, targets = synthetic_batch(step * accum + mb, rank, micro, args.seq_len, cfg.vocab_size, args.seed,
                                              device)
            ce, aux = model(tokens, targets)
            ((ce + aux) / accum).backward()
            loss_sum += ce.detach() / accum
        if args.impl == "fused":
            from .ops import fused

            fused.check_status()  # the fused backward does not synchronise: surface a recorded kernel error here
        reduce_gradients(model, world, group)
        opt.step()
        for router in model.routers():
            router.update_bias(group)
        if world > 1:
            dist.all_reduce(loss_sum, group=group)
            loss_sum /= world
        ms = timer.stop(world, group)
        losses.append(float(loss_sum))
        step_ms.append(ms)
        if rank == 0 and not args.json:
            toks = args.global_batch * args.seq_len
            print(f"step {step:4d}  loss {losses[-1]:.4f}  {ms:9.1f} ms  {toks / (ms / 1e3):12.0f} tokens/s", flush=True)
    if args.save:
        ckpt.save_checkpoint(args.save, model, opt, start_step + args.steps, rank)
    timed = step_ms[1:] if len(step_ms) > 1 else step_ms
    summary = {
        "impl": args.impl, "n_gpus": world, "losses": losses, "ms_per_step": sum(timed) / max(len(timed), 1),
        "tokens_per_s": args.global_batch * args.seq_len / (sum(timed) / max(len(timed), 1) / 1e3),
        "global_batch": args.global_batch, "seq_len": args.seq_len, "micro_batch": micro,
    }
    if rank == 0 and args.json:
        print(json.dumps(summary), flush=True)
    return summary


def main(argv: Optional[list] = None):
    args = build_parser().parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        train(args)
    finally:
        if world > 1:
            from .ops import fused

            torch.cuda.synchronize()
            dist.barrier()
            fused.release_workspaces()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
