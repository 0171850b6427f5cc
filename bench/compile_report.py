"""Compile-only report for the fused layer: needs nvcc, no GPU.

What the reference's deviceless compile script (scripts/compile_gpu_aot.py:27-105) answers for its XLA program, answered
for this build's kernels: does everything compile for sm_100a, what does each kernel cost in registers, spills and
shared memory (`ptxas -v`), how many kernels does one forward+backward launch, what does one rank hold in memory, how
much work and NVLink traffic is a step. Defaults are the DeepSeek-V3-size layer on 8 ranks.

    python bench/compile_report.py
    python bench/compile_report.py --world 1 --tokens 8192 --slice-size 8192 --skip-ptxas
"""

import argparse
import math
import os
import re
import shutil
import subprocess
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from chunked_ep_moe_b200 import _build  # noqa: E402
from chunked_ep_moe_b200.ops import fused  # noqa: E402

_ENTRY = re.compile(r"Compiling entry function '([^']+)'")
_SPILL = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
_USED = re.compile(r"Used (\d+) registers(?:, used (\d+) barriers)?(?:, (\d+) bytes smem)?")


def parse_ptxas(text: str) -> list:
    """[(mangled kernel name, registers, spill bytes, static shared bytes)] from `nvcc -Xptxas -v` output."""
    out, name, spill = [], None, 0
    for line in text.splitlines():
        m = _ENTRY.search(line)
        if m:
            name, spill = m.group(1), 0
            continue
        m = _SPILL.search(line)
        if m and name:
            spill = int(m.group(2)) + int(m.group(3))
            continue
        m = _USED.search(line)
        if m and name:
            out.append((name, int(m.group(1)), spill, int(m.group(3) or 0)))
            name = None
    return out


def demangle(names: list) -> list:
    tool = shutil.which("cu++filt") or shutil.which("c++filt")
    if not tool or not names:
        return names
    res = subprocess.run([tool] + names, capture_output=True, text=True)
    lines = res.stdout.strip().splitlines()
    return lines if res.returncode == 0 and len(lines) == len(names) else names


def short(name: str) -> str:
    name = name.replace("cem::", "").replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
    name = name.replace("void ", "").replace("(GemmMode)", "mode ").replace("(int)", "")
    cut = name.find(">(")
    name = name[:cut + 1] if cut >= 0 else re.sub(r"\(.*", "", name)  # drop the parameter list
    return name.strip()


def ptxas_report() -> list:
    """Cross-compiles every .cu of the extension with `-Xptxas -v` and returns its kernels' resource use."""
    rows = []
    with tempfile.TemporaryDirectory() as tmp:
        for src in _build._sources():
            if not src.endswith(".cu"):
                continue
            cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
                   "-lineinfo", "-I", _build._CSRC, "-Xptxas", "-v", "-c", src, "-o",
                   os.path.join(tmp, os.path.basename(src) + ".o")]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{res.stderr[-2000:]}")
            parsed = parse_ptxas(res.stderr + res.stdout)
            for (_, regs, spill, smem), nice in zip(parsed, demangle([p[0] for p in parsed])):
                rows.append((os.path.relpath(src, _build._CSRC), short(nice), regs, spill, smem))
    return rows


def work_report(world, experts, top_k, tokens, hidden, ffn, slice_size, fp8) -> dict:
    rows = tokens * top_k                      # token copies a rank sends = copies it receives under uniform routing
    slices = math.ceil(rows / slice_size)
    flops = 18 * rows * hidden * ffn + 6 * rows * hidden * ffn  # fwd 6, remat 6, dgrad 6, wgrad 6 (x D x F per row)
    wire_elem = 1 + 4 / 128 if fp8 else 2      # e4m3 + one fp32 scale per 128, or bf16
    remote = rows * (world - 1) / world
    dispatch = remote * hidden * wire_elem * 3  # x (fwd), x and g (bwd)
    combine = remote * hidden * 2 * 2           # y (fwd), dx (bwd): bf16
    return {
        "rows per rank per pass": rows,
        "slices per pass (uniform routing)": slices,
        "kernel launches per step": fused.expected_launches(slices, fp8),
        "GEMM TFLOP per rank per step": flops / 1e12,
        "NVLink GB out per rank per step": (dispatch + combine) / 1e9,
    }


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per rank")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--slice-size", type=int, default=8192)
    ap.add_argument("--comm-dtype", default=None, choices=[None, "float8_e4m3fn"])
    ap.add_argument("--skip-ptxas", action="store_true", help="only the memory and work sections")
    args = ap.parse_args()
    fp8 = args.comm_dtype is not None

    _build.build()
    print("extension: built for sm_100a at", os.path.relpath(_build._so_path()))
    if not args.skip_ptxas:
        print(f"\nkernel resources (ptxas -v; dynamic shared memory of the GEMM kernels: "
              f"{_build.load().gemm_smem_bytes} B per CTA)")
        print(f"{'file':28s} {'kernel':60s} {'regs':>5s} {'spill B':>8s} {'static smem B':>14s}")
        for src, name, regs, spill, smem in ptxas_report():
            print(f"{src:28s} {name[:60]:60s} {regs:5d} {spill:8d} {smem:14d}")

    print(f"\nmemory held by one rank (world {args.world}, {args.experts // args.world} experts per rank)")
    plan = fused.memory_plan(args.world, args.experts, args.top_k, args.tokens, args.hidden, args.ffn, args.slice_size,
                             fp8)
    for k, v in plan.items():
        print(f"  {v / 2**30:9.3f} GiB  {k}")
    print(f"  {plan['total'] / (180 * 1e9) * 100:8.1f} %    of 180 GB")

    print("\nwork per step (forward + backward, one rank)")
    for k, v in work_report(args.world, args.experts, args.top_k, args.tokens, args.hidden, args.ffn, args.slice_size,
                            fp8).items():
        print(f"  {v:12.3f}  {k}" if isinstance(v, float) else f"  {v:12d}  {k}")


if __name__ == "__main__":
    main()
