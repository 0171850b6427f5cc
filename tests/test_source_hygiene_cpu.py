"""Source rules that keep the tree runnable on shared multi-GPU hosts, checked mechanically.

* no batched-memcpy runtime/driver entry point is named anywhere (those calls faulted GPUs on the target driver);
* cluster-wide delivery is only ever used by `tcgen05.commit` (an mbarrier arrive in both CTAs of a pair): no TMA or
  bulk load is shared across a cluster, so no load can ever be pointed at another GPU's memory through one;
* `wgmma` (sm_90a only) does not appear.
"""

import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXTS = (".py", ".cu", ".cuh", ".cpp", ".h")
SKIP = ("_work", "gpurun_out", "baseline", ".git", "_ext", "__pycache__", ".hypothesis", ".pytest_cache")


def _sources():
    for root, dirs, files in os.walk(ROOT):
        dirs[:] = [d for d in dirs if d not in SKIP]
        for f in files:
            if f.endswith(EXTS):
                path = os.path.join(root, f)
                with open(path, errors="replace") as fh:
                    yield os.path.relpath(path, ROOT), fh.read()


def test_no_closed_calls_and_no_cluster_shared_loads():
    closed = [a + "Memcpy" + b + "Batch" + "Async" for a in ("cuda", "cu") for b in ("", "3D")]
    shared = "multi" + "cast"
    for rel, text in _sources():
        for name in closed:
            assert name not in text, f"{rel} names {name}"
        for n, line in enumerate(text.splitlines(), 1):
            if shared in line.lower():
                assert "tcgen05.commit" in line, f"{rel}:{n} uses cluster-wide delivery outside tcgen05.commit"
        if rel.endswith((".cu", ".cuh")):
            assert not re.search(r"\bwgmma\b", text), f"{rel} uses wgmma"


def test_hot_kernels_are_written_with_tcgen05_and_tma():
    text = dict(_sources())
    umma = text[os.path.join("chunked_ep_moe_b200", "csrc", "common", "umma.cuh")]
    for needle in ("tcgen05.mma.cta_group::1.kind::f16", "tcgen05.mma.cta_group::2.kind::f16", "tcgen05.ld.sync.aligned",
                   "tcgen05.alloc", "cp.async.bulk.tensor.2d", "cp.async.bulk.tensor.3d", "red.release.sys",
                   "ld.acquire.sys"):
        assert needle in umma, needle
