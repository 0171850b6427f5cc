"""End-to-end training on one GPU: the fused layer and the NCCL/library baseline must give the same loss curve.

Mirrors the reference's external check (losses equal to the default MoE within bf16 rounding, a few steps).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(impl, **kw):
    from chunked_ep_moe_b200.train import build_parser

    argv = ["--steps", "4", "--global-batch", "4", "--seq-len", "256", "--micro-batch", "2", "--layers", "3",
            "--d-model", "256", "--experts", "8", "--moe-ffn", "256", "--dense-ffn", "512", "--top-k", "2",
            "--vocab", "512", "--slice-size", "512", "--impl", impl, "--json"]
    for k, v in kw.items():
        argv += [f"--{k.replace('_', '-')}", str(v)]
    return build_parser().parse_args(argv)


def test_fused_and_baseline_loss_curves_agree():
    from chunked_ep_moe_b200.train import train

    torch.cuda.set_device(0)
    fused = train(_args("fused"))
    base = train(_args("baseline"))
    assert all(l == l and l < 20 for l in fused["losses"]), fused["losses"]
    for a, b in zip(fused["losses"], base["losses"]):
        assert abs(a - b) <= 2e-2 * max(1.0, abs(b)), (fused["losses"], base["losses"])


def test_checkpoint_resume_continues_the_same_run(tmp_path):
    from chunked_ep_moe_b200.train import train

    torch.cuda.set_device(0)
    full = train(_args("fused", steps=4))
    first = train(_args("fused", steps=2, save=str(tmp_path)))
    second = train(_args("fused", steps=2, resume=str(tmp_path)))
    got = first["losses"] + second["losses"]
    for a, b in zip(got, full["losses"]):
        assert abs(a - b) <= 1e-2 * max(1.0, abs(b)), (got, full["losses"])
