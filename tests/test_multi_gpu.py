"""The fused NVLink path on real peers: one process per GPU over NCCL + CUDA IPC (needs >= 2 GPUs).

Checks the fused layer and the NCCL baseline against the dense oracle, twice in a row through the
same workspace (counters, credits and double buffers carry over), for balanced and skewed routing.
NVLS is switched off for these short-lived ranks.
"""

import os
import socket
import tempfile
import traceback

import pytest
import torch

import moe_cases

pytestmark = pytest.mark.gpu

TOL = 3e-2


def _free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, cases):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    result = {"ok": True, "errors": {}}
    try:
        from chunked_ep_moe_b200 import ChunkedMoEConfig, chunked_moe
        from chunked_ep_moe_b200.ops import fused

        for case in cases:
            skew, S, comm = case
            T, E, K, D, F, stripe = 96, 8, 2, 256, 256, 64
            x, ids, weights, w_up, w_down, g = moe_cases.setup(world, T, E, K, D, F, skew, seed=11)
            bf = lambda t: t.to(torch.bfloat16)
            want = moe_cases.oracle(bf(x).float(), ids, weights, bf(w_up).float(), bf(w_down).float(), bf(g).float(),
                                    stripe)
            sh = lambda t: moe_cases.shard(t, rank, world).cuda()
            for impl in ("fused", "baseline"):
                if impl == "baseline" and comm is not None:
                    continue
                cfg = ChunkedMoEConfig(num_experts=E, top_k=K, slice_size=S, stripe_width=stripe, comm_dtype=comm,
                                       transport="nvshmem" if impl == "fused" else "ragged_a2a",
                                       expert_compute="fused" if impl == "fused" else "reference")
                for rep in range(2):
                    xs = bf(sh(x)).requires_grad_(True)
                    ws = sh(weights).requires_grad_(True)
                    us, ds = bf(sh(w_up)).requires_grad_(True), bf(sh(w_down)).requires_grad_(True)
                    out = chunked_moe(xs, sh(ids), ws, us, ds, cfg, None)
                    out.backward(bf(sh(g)))
                    torch.cuda.synchronize()
                    got = {"out": out.detach(), "dx": xs.grad, "dweights": ws.grad, "dw_up": us.grad,
                           "dw_down": ds.grad}
                    for name, val in got.items():
                        a, b = val.float().cpu(), moe_cases.shard(want[name], rank, world).float()
                        if comm is None:
                            err = float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
                        else:
                            err = float((a - b).norm() / b.norm().clamp_min(1e-6))
                        result["errors"][(case, impl, rep, name)] = (err, bool(torch.isfinite(a).all()))
        dist.barrier()
        fused.release_workspaces()
    except Exception:
        result = {"ok": False, "trace": traceback.format_exc()}
    torch.save(result, os.path.join(out_dir, f"{rank}.pt"))
    dist.destroy_process_group()


def _run(world, cases):
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as out_dir:
        mp.spawn(_worker, args=(world, _free_port(), out_dir, cases), nprocs=world, join=True)
        return [torch.load(os.path.join(out_dir, f"{r}.pt"), weights_only=False) for r in range(world)]


CASES = [("uniform", 128, None), ("all_one", 64, None), ("rank0", 256, None), ("uniform", 128, "float8_e4m3fn")]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_layer_on_real_peers(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    for rank, res in enumerate(_run(world, CASES)):
        assert res["ok"], f"rank {rank} failed:\n{res.get('trace')}"
        for key, (err, finite) in res["errors"].items():
            limit = 0.08 if key[0][2] is not None else TOL
            assert finite and err <= limit, f"rank {rank} {key}: err {err:.4f}"
