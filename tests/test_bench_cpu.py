"""bench.py pieces that run without a GPU: routing generators, the clock-sample parser, the reference arm's line."""

import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, timeout=120)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_routing_generators():
    gen = torch.Generator().manual_seed(0)
    for skew in ("none", "zipf", "expert0"):
        ids, w = bench.make_routing(gen, 512, 64, 8, skew, "cpu")
        assert ids.shape == (512, 8) and ids.dtype == torch.int32 and w.shape == (512, 8)
        assert int(ids.min()) >= 0 and int(ids.max()) < 64
        assert torch.allclose(w.sum(-1), torch.ones(512), atol=1e-5)
        assert all(len(set(row.tolist())) == 8 for row in ids[:32]), "experts of one token must be distinct"
        if skew == "expert0":
            assert (ids[:, 0] == 0).all()
    ids, _ = bench.make_routing(gen, 4096, 64, 8, "zipf", "cpu")
    counts = torch.bincount(ids.reshape(-1).long(), minlength=64)
    assert counts[0] > 4 * counts[32:].float().mean(), "Zipf routing must be visibly skewed"


def test_clock_sample_parser(tmp_path):
    sampler = bench.ClockSampler(0)
    sampler.proc = type("P", (), {"terminate": lambda s: None, "wait": lambda s, timeout=None: 0,
                                   "kill": lambda s: None})()
    sampler.path = str(tmp_path / "clocks.csv")
    with open(sampler.path, "w") as f:
        f.write("0, 1320, 1965, 998.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1340, 1965, 1001.7, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1965, 1965, 300.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n")
        f.write("garbage line\n")
    got = sampler.stop()
    assert got["sm_mhz"] == 1340.0 and got["sm_max_mhz"] == 1965.0
    assert got["reasons"] == ["sw_power_cap"] and got["samples"] == 3


def test_clock_samples_from_nvml_are_cut_to_the_timed_window():
    """The in-process sampler: only samples between the two marks count; reasons are decoded from NVML's bit mask."""
    sampler = bench.ClockSampler(0)
    sampler.thread = type("T", (), {"join": lambda s, timeout=None: None})()
    sampler._stop = False
    sampler.smax = 1965.0
    sampler.samples = [(1.0, 1965.0, 0x0), (2.0, 1300.0, 0x4), (2.2, 1320.0, 0x4), (2.4, 1310.0, 0x4 | 0x20),
                       (9.0, 1965.0, 0x0)]
    sampler.window = [1.5, 3.0]
    got = sampler.stop()
    assert got["sm_mhz"] == 1310.0 and got["sm_max_mhz"] == 1965.0 and got["samples"] == 3
    assert got["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]


def test_compile_report_pieces():
    """The compile-only report's parser, launch formula and memory plan (no nvcc run, no GPU)."""
    sys.path.insert(0, os.path.join(ROOT, "bench"))
    import compile_report
    from chunked_ep_moe_b200.ops import fused

    text = """ptxas info    : Compiling entry function '_Zk1' for 'sm_100a'
ptxas info    : Function properties for _Zk1
    0 bytes stack frame, 8 bytes spill stores, 4 bytes spill loads
ptxas info    : Used 112 registers, used 1 barriers, 16 bytes smem
ptxas info    : Compiling entry function '_Zk2' for 'sm_100a'
ptxas info    : Function properties for _Zk2
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 32 registers"""
    assert compile_report.parse_ptxas(text) == [("_Zk1", 112, 12, 16), ("_Zk2", 32, 0, 0)]
    assert compile_report.short("void cem::<unnamed>::grouped_gemm_kernel<(cem::GemmMode)3>(cem::GemmParams)") == \
        "grouped_gemm_kernel<mode 3>"

    # 8 slices: the 1-GPU bench layout launches 104 kernels per step, 9 slices (8 GPUs, random routing) 116
    assert fused.expected_launches(8) == 104 and fused.expected_launches(9) == 116
    assert fused.expected_launches(8, fp8=True) == 104 + 16

    plan = fused.memory_plan(world=8, experts=256, top_k=8, tokens_per_rank=8192, hidden=7168, ffn=2048,
                             slice_size=8192)
    assert plan["expert weights (bf16)"] == 32 * (7168 * 4096 + 2048 * 7168) * 2
    assert plan["total"] == sum(v for k, v in plan.items() if k != "total")
    assert plan["total"] < 16 * 2**30, "the DeepSeek-V3-size layer on 8 ranks fits in a fraction of 180 GB"
    work = compile_report.work_report(8, 256, 8, 8192, 7168, 2048, 8192, False)
    assert abs(work["GEMM TFLOP per rank per step"] - 23.09) < 0.01
    assert work["kernel launches per step"] == 104


def test_host_side_helpers_degrade_quietly():
    """CPU affinity binding without NVML, and the trainer profile's kernel grouping."""
    assert bench.bind_near_gpu(0).startswith("cpu affinity unchanged")
    sys.path.insert(0, os.path.join(ROOT, "bench"))
    import trainer_profile

    assert trainer_profile.group_of("void cem::(anonymous namespace)::grouped_gemm_kernel<0>(...)") == "fused MoE kernels"
    assert trainer_profile.group_of("nvjet_tst_256x256_64x4_2x2_2cta_v_bz_NNT") == "library GEMMs"
    assert trainer_profile.group_of("cudnn_generated_fort_native_sdpa_sm100_flash_fprop_f16") == "attention"
    glue = trainer_profile.group_of("void at::native::vectorized_elementwise_kernel<8, ...>")
    assert glue == "elementwise / reductions / softmax"
