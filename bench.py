"""Headline benchmark: DeepSeek-V3-size chunked expert-parallel MoE layer, forward + backward.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 5 --warmup 3

Config (per rank): T=8192 tokens (seq 4096 x micro-batch 2), D=7168, F=2048, 256 routed experts
(256/N per GPU), top-8 of sigmoid(logits ~ N(0,1)) normalised over the chosen 8, S=8192, stripe 64,
bf16, weights ~ N(0, 0.006), synthetic seeded inputs. Weak scaling: per-GPU tokens are fixed.

One step = one forward + one backward of the layer through `chunked_moe` (gradients for x, router
weights, w_up, w_down). Rank 0 prints ONE JSON line. `value` is tokens/s summed over all GPUs from
the device-timed loop (CUDA events, max over ranks); `e2e` is the same step driven through the
public API with the step's inputs copied from pinned host memory and the loss read back every
step. `--impl baseline` runs the in-repo NCCL all_to_all + library grouped-GEMM layer;
`--impl reference` is the reference's own JAX build, which cannot be installed offline here.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

CONFIGS = {
    # name: tokens/rank, D, F, E, K, S, stripe, weight std
    "dsv3": dict(tokens=8192, hidden=7168, ffn=2048, experts=256, top_k=8, slice_size=8192, stripe=64, std=0.006),
    "tiny": dict(tokens=16384, hidden=1024, ffn=512, experts=64, top_k=6, slice_size=8192, stripe=64, std=0.02),
    "smoke": dict(tokens=1024, hidden=512, ffn=256, experts=16, top_k=4, slice_size=1024, stripe=64, std=0.02),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fused", choices=["fused", "baseline", "reference"])
    ap.add_argument("--config", default="dsv3", choices=sorted(CONFIGS))
    ap.add_argument("--comm-dtype", default=None, choices=[None, "float8_e4m3fn"])
    ap.add_argument("--slice-size", type=int, default=None)
    ap.add_argument("--skew", default="none", choices=["none", "zipf", "expert0"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the sampled fp32 check of one step")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip timing the NCCL + library grouped-GEMM layer on the same tensors (fills vs_baseline)")
    ap.add_argument("--baseline-steps", type=int, default=2)
    ap.add_argument("--per-step", action="store_true",
                    help="also print every timed step's device time on rank 0 (stderr), from events between the steps")
    return ap.parse_args()


def reference_unavailable():
    if int(os.environ.get("RANK", "0")) != 0:  # one line per job, also when launched once per GPU
        return
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a JAX package (hatchling build backend, jax>=0.11.1); neither hatchling nor "
                       "jax is in the image or the offline wheelhouse, so it can be neither installed nor imported",
    }))


def bind_near_gpu(index: int) -> str:
    """Best effort: run this process (and allocate its pinned buffers) on the CPUs next to GPU `index`.

    Only this process's own CPU affinity changes, nothing of the GPU's. Returns a note for the log; any failure
    (no NVML, a cpuset that excludes those CPUs) leaves the affinity as it was.
    """
    try:
        import pynvml

        import torch

        pynvml.nvmlInit()
        uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)  # CUDA and NVML may number GPUs differently
        handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        both = near & allowed
        if not both or both == allowed:
            return "cpu affinity unchanged"
        os.sched_setaffinity(0, both)
        return f"bound to {len(both)} CPUs near GPU {index}"
    except Exception as exc:  # noqa: BLE001 - purely advisory
        return f"cpu affinity unchanged ({type(exc).__name__})"


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while the timed loops run (read-only NVML queries).

    A thread of this process asks NVML every 50 ms (two cheap queries); only rank 0 samples. (One `nvidia-smi -lms` process per rank,
    started right before the timed loop, cost the first timed step ~9 ms on 4 GPUs while the tools attached to every
    GPU of the box, and an occasional step later.) Without NVML in the process the `nvidia-smi` loop is the fallback,
    started before the warm-up so that its start-up is over when the timing begins.
    """

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.samples = []  # (monotonic time, sm MHz, reasons bitmask)
        self.smax = None
        self.thread = None
        self.proc = None
        self.path = None
        self.window = [None, None]

    def _nvml_loop(self, nvml, handle):
        import threading  # noqa: F401

        while not self._stop:
            try:
                mhz = nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
                try:
                    mask = nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except AttributeError:
                    mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((time.monotonic(), float(mhz), int(mask)))
            except Exception:  # noqa: BLE001 - a failed query is a missing sample
                pass
            time.sleep(0.05)

    def start(self):
        try:
            import threading

            import pynvml

            import torch

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + str(torch.cuda.get_device_properties(self.gpu_index).uuid))
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._stop = False
            self.thread = threading.Thread(target=self._nvml_loop, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001 - fall back to the command-line tool
            self.thread = None
        try:
            self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.window[0] = time.monotonic()

    def mark_end(self):
        self.window[1] = time.monotonic()

    def stop(self) -> dict:
        if self.thread is not None:
            time.sleep(0.25)
            self._stop = True
            self.thread.join(timeout=2)
            lo, hi = self.window[0] or 0.0, self.window[1] or float("inf")
            inside = [(mhz, mask) for t, mhz, mask in self.samples if lo <= t <= hi] or \
                     [(mhz, mask) for _, mhz, mask in self.samples]
            sm = sorted(m for m, _ in inside)
            seen = 0
            for _, mask in inside:
                seen |= mask
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.smax,
                    "reasons": sorted(name for bit, name in self.REASONS.items() if seen & bit),
                    "samples": len(sm), "source": "nvml, sampled during the timed loops"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML and no nvidia-smi"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax = float(parts[2])
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi -lms 200 (whole run)"}


class NvlinkCounter:
    """NVLink payload bytes this GPU sent and received, from NVML's per-device throughput counters (read-only).

    Used to set the bytes the fused kernels really put on the wire against the algorithmic bytes of the layer. Any
    failure (no NVML, counters not exposed: on this pool's B200 boxes the query answers "not supported") yields None:
    the number is evidence, never a dependency.
    """

    TX, RX = 138, 139  # NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX / _RX, KiB since the driver was loaded

    def __init__(self, index: int):
        self.handle = None
        try:
            import pynvml

            import torch

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + str(torch.cuda.get_device_properties(index).uuid))
        except Exception:  # noqa: BLE001
            self.handle = None
        if self.read() is None:  # counters not exposed on this system: later reads cost nothing
            self.handle = None

    def read(self):
        if self.handle is None:
            return None
        try:
            vals = self.nvml.nvmlDeviceGetFieldValues(self.handle, [(self.TX, 0xFFFFFFFF), (self.RX, 0xFFFFFFFF)])
            out = []
            for v in vals:
                if v.nvmlReturn != 0:
                    return None
                out.append(int(v.value.ullVal) * 1024)
            return tuple(out)
        except Exception:  # noqa: BLE001
            return None


def make_routing(gen, tokens, experts, top_k, skew, device):
    import torch

    logits = torch.randn(tokens, experts, generator=gen, device=device)
    if skew == "zipf":  # Zipf(s=1.2) popularity over experts, sampled without replacement per token
        pop = 1.0 / torch.arange(1, experts + 1, device=device, dtype=torch.float32) ** 1.2
        ids = torch.multinomial(pop.expand(tokens, experts), top_k, replacement=False, generator=gen)
        scores = torch.sigmoid(torch.gather(logits, 1, ids))
    else:
        if skew == "expert0":  # adversarial: every token's first choice is expert 0
            logits[:, 0] += 100.0
        scores, ids = torch.topk(torch.sigmoid(logits), top_k, dim=-1)
    weights = scores / scores.sum(-1, keepdim=True)
    return ids.to(torch.int32), weights.float()


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_unavailable()
        return

    import torch
    import torch.distributed as dist

    from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    affinity_note = bind_near_gpu(local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    c = dict(CONFIGS[args.config])
    if args.slice_size:
        c["slice_size"] = args.slice_size
    T, D, F, E, K, S = c["tokens"], c["hidden"], c["ffn"], c["experts"], c["top_k"], c["slice_size"]
    L = E // world
    fused = args.impl == "fused"
    cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, stripe_width=c["stripe"],
                           transport="nvshmem" if fused else "ragged_a2a",
                           expert_compute="fused" if fused else "reference", comm_dtype=args.comm_dtype)

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    w_up = torch.empty(L, D, 2 * F, device=dev, dtype=torch.bfloat16)
    w_down = torch.empty(L, F, D, device=dev, dtype=torch.bfloat16)
    for l in range(L):  # per expert: no 30 GB fp32 temporary at L=256
        w_up[l] = (torch.randn(D, 2 * F, generator=gen, device=dev) * c["std"]).to(torch.bfloat16)
        w_down[l] = (torch.randn(F, D, generator=gen, device=dev) * c["std"]).to(torch.bfloat16)
    w_up.requires_grad_(True)
    w_down.requires_grad_(True)

    # Host-side step inputs in pinned memory (the end-to-end loop copies them in every step).
    ids_d, weights_d = make_routing(gen, T, E, K, args.skew, dev)
    x_h = torch.randn(T, D, generator=torch.Generator().manual_seed(99 + rank)).to(torch.bfloat16).pin_memory()
    g_d = torch.randn(T, D, generator=gen, device=dev).to(torch.bfloat16)
    ids_h, weights_h = ids_d.cpu().pin_memory(), weights_d.cpu().pin_memory()
    loss_h = torch.zeros(1, dtype=torch.float32).pin_memory()
    x_d = x_h.to(dev)

    def step(x, ids, weights):
        x = x.requires_grad_(True)
        weights = weights.requires_grad_(True)
        w_up.grad = None
        w_down.grad = None
        out = chunked_moe(x, ids, weights, w_up, w_down, cfg, group)
        out.backward(g_d)
        return out, x.grad, weights.grad

    # End-to-end step: this step's inputs come from pinned host memory (copied on a side stream into one of two
    # preallocated device slots while the previous step computes) and the step's scalar result is read back to the
    # host before the step ends.
    copy_stream = torch.cuda.Stream(device=dev)
    slots = [(torch.empty_like(x_d), torch.empty_like(ids_d), torch.empty_like(weights_d)) for _ in range(2)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [None, None]
    staged = [False, False]
    e2e_count = [0]

    def stage_inputs(slot):
        with torch.cuda.stream(copy_stream):
            if consumed[slot] is not None:
                copy_stream.wait_event(consumed[slot])  # the step that last read this slot has finished
            slots[slot][0].copy_(x_h, non_blocking=True)
            slots[slot][1].copy_(ids_h, non_blocking=True)
            slots[slot][2].copy_(weights_h, non_blocking=True)
            ready[slot].record(copy_stream)
        staged[slot] = True

    def step_e2e():
        slot = e2e_count[0] & 1
        if not staged[slot]:
            stage_inputs(slot)
        cur = torch.cuda.current_stream()
        cur.wait_event(ready[slot])
        staged[slot] = False
        stage_inputs(slot ^ 1)  # the next step's copy overlaps this step's compute
        x, ids, weights = slots[slot]
        out, dx, dw = step(x.detach(), ids, weights.detach())
        # fp32 accumulation inside the reduction kernels: no fp32 copies of the two [T, D] tensors
        loss_h.copy_((out.mean(dtype=torch.float32) + dx.mean(dtype=torch.float32)).reshape(1), non_blocking=True)
        consumed[slot] = torch.cuda.Event()
        consumed[slot].record(cur)
        cur.synchronize()  # the host owns the step's result before the next step starts
        e2e_count[0] += 1
        return float(loss_h[0])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)
            torch.cuda.synchronize()

    def launches():
        if not fused:
            return 0
        from chunked_ep_moe_b200.ops import fused as fused_mod

        return fused_mod.launches()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()  # well before the timed region: whatever its start-up costs is over by then
    nvlink = NvlinkCounter(local_rank)
    for _ in range(max(args.warmup, 3)):
        step(x_d.clone(), ids_d, weights_d.clone())
    sync_all()

    # One step at the benchmarked size against a sampled fp32 oracle (outside every timed region): 64 tokens per rank
    # (output, dX, router-weight gradients) and both weight gradients of each rank's first and last expert.
    check = None
    if not args.no_check:
        from chunked_ep_moe_b200.utils.verify import sampled_check

        out_c, dx_c, dwt_c = step(x_d.clone(), ids_d, weights_d.clone())
        check = sampled_check(x_d, ids_d, weights_d, g_d, w_up.detach(), w_down.detach(), out_c.detach(), dx_c, dwt_c,
                              w_up.grad, w_down.grad, stripe=c["stripe"], group=group,
                              tol=8e-2 if args.comm_dtype else 3e-2)
        del out_c, dx_c, dwt_c
        sync_all()

    # The check above keeps the GPU idle for seconds and its clocks fall; the first step after an idle spell measured
    # 9-12 ms longer than the following ones on 4 GPUs. Two more untimed steps bring the device back to the state the
    # warm-up left it in; only the barrier and the synchronisation sit between them and the timed loop.
    for _ in range(2):
        step(x_d.clone(), ids_d, weights_d.clone())
    l0 = launches()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    if sampler:
        sampler.mark_begin()
    link0 = nvlink.read()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)] if args.per_step else None
    start.record()
    for i in range(args.steps):
        if marks:
            marks[i].record()
        step(x_d.detach(), ids_d, weights_d.detach())
    stop.record()
    if marks:
        marks[-1].record()
    sync_all()
    if marks and rank == 0:
        print("per-step ms (device-timed loop):",
              " ".join(f"{marks[i].elapsed_time(marks[i + 1]):.2f}" for i in range(args.steps)), file=sys.stderr)
    link1 = nvlink.read()
    ms = start.elapsed_time(stop) / args.steps
    total_launches = launches() - l0
    n_launch = total_launches // max(args.steps, 1)

    e2e = None
    if not args.no_e2e:
        step_e2e()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step_e2e()
        e1.record()
        sync_all()
        e2e_ms = e0.elapsed_time(e1) / args.steps
    if sampler:
        sampler.mark_end()
    clocks = sampler.stop() if sampler else None

    # Exposed all-to-all: the same per-GPU work (same L experts, same rows per expert in expectation) with every
    # row local, i.e. this rank alone as a 1-rank expert-parallel group, timed the same way.
    local_ms = None
    if world > 1 and fused:
        solo = None
        for r in range(world):  # every rank must take part in creating every subgroup
            g_r = dist.new_group([r])
            if r == rank:
                solo = g_r
        cfg_local = ChunkedMoEConfig(num_experts=L, top_k=K, slice_size=S, stripe_width=c["stripe"],
                                     transport="nvshmem", expert_compute="fused", comm_dtype=args.comm_dtype)
        ids_l, weights_l = make_routing(gen, T, L, K, "none", dev)

        def step_local():
            x = x_d.detach().requires_grad_(True)
            w = weights_l.detach().requires_grad_(True)
            w_up.grad = None
            w_down.grad = None
            chunked_moe(x, ids_l, w, w_up, w_down, cfg_local, solo).backward(g_d)

        for _ in range(3):
            step_local()
        sync_all()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            step_local()
        s1.record()
        sync_all()
        local_ms = s0.elapsed_time(s1) / args.steps

    # Comparison arm in the same process, on the same tensors: the same layer on NCCL `all_to_all_single` + the
    # library grouped GEMM (`transport="ragged_a2a"`, `expert_compute="reference"`), timed the same way.
    base_ms, base_note = None, None
    if fused and not args.no_baseline:
        cfg_base = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, stripe_width=c["stripe"],
                                    transport="ragged_a2a", expert_compute="reference", comm_dtype=args.comm_dtype)

        def step_base():
            x = x_d.detach().requires_grad_(True)
            w = weights_d.detach().requires_grad_(True)
            w_up.grad = None
            w_down.grad = None
            chunked_moe(x, ids_d, w, w_up, w_down, cfg_base, group).backward(g_d)

        try:
            w_up.grad = None
            w_down.grad = None
            torch.cuda.empty_cache()
            step_base()
            sync_all()
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            for _ in range(args.baseline_steps):
                step_base()
            b1.record()
            sync_all()
            base_ms = b0.elapsed_time(b1) / args.baseline_steps
        except Exception as exc:  # noqa: BLE001 - the headline number must survive a failing comparison arm
            base_note = f"{type(exc).__name__}: {exc}"[:200]
            base_ms = None
        w_up.grad = None
        w_down.grad = None

    failed = torch.tensor([1.0 if base_ms is None else 0.0], device=dev, dtype=torch.float64)
    t = torch.tensor([ms, e2e_ms if not args.no_e2e else 0.0, local_ms or 0.0, base_ms or 0.0], device=dev,
                     dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        dist.all_reduce(failed, op=dist.ReduceOp.MAX, group=group)
    ms, e2e_ms, local_ms = float(t[0]), float(t[1]), (float(t[2]) if local_ms is not None else None)
    base_ms = float(t[3]) if float(failed[0]) == 0.0 else None
    if not args.no_e2e:
        h2d = x_h.numel() * 2 + ids_h.numel() * 4 + weights_h.numel() * 4
        e2e = {"value": world * T / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4}

    if rank == 0:
        flops = 24.0 * D * F * T * K  # per rank, fwd + bwd with full remat
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(REPO, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = peaks.get("bf16_tflops_sustained", 1400.0)
        result = {
            "metric": "moe_layer_fwd_bwd_tokens_per_s",
            "value": world * T / (ms / 1e3),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms,
            "higher_is_better": True,
            "scaling": "weak",
            # No published number exists for this metric (the reference was never run on a GPU), so the ratio is
            # against the in-repo NCCL + library grouped-GEMM layer timed in this same process (`baseline` below).
            "vs_baseline": (base_ms / ms) if base_ms else None,
            "dtype": "bf16",
            "data": "synthetic (seeded N(0,1) tokens, random-init N(0,%g) weights, top-%d of sigmoid logits)" % (c["std"], K),
            "impl": args.impl,
            "tokens_per_s_per_gpu": T / (ms / 1e3),
            "tflops_per_gpu": flops / (ms / 1e3) / 1e12,
            "frac_of_measured_sustained_bf16_peak": flops / (ms / 1e3) / 1e12 / peak,
            "config": {"model": "DeepSeek-V3-size MoE layer" if args.config == "dsv3" else args.config,
                       "tokens_per_rank": T, "global_batch": world * T, "seq_len": 4096, "hidden": D, "ffn": F,
                       "experts": E, "experts_per_gpu": L, "top_k": K, "slice_size": S, "stripe_width": c["stripe"],
                       "comm_dtype": args.comm_dtype or "bf16", "skew": args.skew,
                       "parallelism": f"ep{world}",
                       "l2": "inputs larger than L2: %.1f GB of expert weights stream through every step"
                             % ((w_up.numel() + w_down.numel()) * 2 / 1e9)},
            "clocks": clocks,
            "check": check,
            "baseline": ({"impl": "same layer on NCCL all_to_all_single + torch grouped_mm, same process and tensors",
                          "ms_per_step": base_ms, "steps": args.baseline_steps, "warmup": 1,
                          "value": world * T / (base_ms / 1e3)} if base_ms else
                         ({"unavailable": base_note or "not run"} if fused else None)),
            "e2e": e2e,
            # rank 0's NVLink payload per step from NVML's counters, next to what the layer has to move: five row
            # streams (x; x, g; y; dx) of T*K rows of D bf16 values (the dispatch streams at the wire dtype), of which
            # (N-1)/N leave the GPU with uniform routing
            "nvlink": ({"tx_bytes_per_step": (link1[0] - link0[0]) / args.steps,
                        "rx_bytes_per_step": (link1[1] - link0[1]) / args.steps,
                        "algorithmic_bytes_per_step_each_way":
                            T * K * D * (2 * 2 + 3 * (1 if args.comm_dtype else 2)) * (world - 1) / world}
                       if (link0 and link1 and world > 1) else None),
            "gpu_launches": int(total_launches),  # this repo's kernels launched inside the timed region (all steps)
            "gpu_launches_per_step": int(n_launch),
            "host": affinity_note,
            "local_only_ms_per_step": local_ms,
            "exposed_a2a_ms_per_step": (ms - local_ms) if local_ms is not None else (0.0 if world == 1 else None),
        }
        print(json.dumps(result))
    if world > 1:
        dist.barrier(group=group)
        from chunked_ep_moe_b200.ops import fused as fused_mod

        fused_mod.release_workspaces()
        dist.destroy_process_group()
    if check is not None and not check["ok"]:
        raise SystemExit(f"sampled fp32 check failed: {check}")


if __name__ == "__main__":
    main()
