"""Spawn helpers for multi-process CPU tests (gloo ranks on 127.0.0.1)."""

import os
import socket
import tempfile
import time
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        result = fn(rank, world, *args)
        torch.save({"ok": True, "result": result}, os.path.join(out_dir, f"{rank}.pt"))
    except Exception:  # the parent re-raises with the traceback text
        torch.save({"ok": False, "error": traceback.format_exc()}, os.path.join(out_dir, f"{rank}.pt"))
        raise
    finally:
        # Rank 0 hosts the c10d store: it must be the last to leave, or a slower rank's store call fails with a
        # connection error that has nothing to do with what the test checks.
        try:
            store = dist.distributed_c10d._get_default_store()
            store.add("cem/test/exited", 1)
            if rank == 0:
                deadline = time.monotonic() + 60.0
                while int(store.add("cem/test/exited", 0)) < world and time.monotonic() < deadline:
                    time.sleep(0.05)
        except Exception:  # noqa: BLE001 - a dead store must not mask the test's own outcome
            pass
        dist.destroy_process_group()


def run_ranks(fn, world, *args, timeout=600):
    """Runs `fn(rank, world, *args)` on `world` gloo ranks; returns the list of per-rank results."""
    with tempfile.TemporaryDirectory() as out_dir:
        ctx = mp.spawn(_worker, args=(world, _free_port(), fn, args, out_dir), nprocs=world, join=False)
        try:
            deadline = time.monotonic() + timeout
            while not ctx.join(5.0):  # join() returns once any rank exits; loop until all have
                if time.monotonic() > deadline:
                    for p in ctx.processes:
                        if p.is_alive():
                            p.terminate()
                    raise TimeoutError(f"ranks did not finish within {timeout}s")
        except Exception:
            for r in range(world):
                path = os.path.join(out_dir, f"{r}.pt")
                if os.path.exists(path):
                    rec = torch.load(path, weights_only=False)
                    if not rec["ok"]:
                        raise AssertionError(f"rank {r} failed:\n{rec['error']}")
            raise
        return [torch.load(os.path.join(out_dir, f"{r}.pt"), weights_only=False)["result"] for r in range(world)]
