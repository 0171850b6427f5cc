"""Builds and loads the in-tree sm_100a extension (`chunked_ep_moe_b200/_C*.so`).

The extension is compiled for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`) with ninja
through `torch.utils.cpp_extension`, into `chunked_ep_moe_b200/_ext/`, and the resulting shared
object is imported from there. nvcc cross-compiles without a GPU, so `build()` works on a CPU-only
machine; loading the module needs no GPU either (the CPU plan builder lives in it).
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, "csrc")
_BUILD_DIR = os.path.join(_PKG_DIR, "_ext")
_NAME = "chunked_ep_moe_b200_C"
_SOURCES = [
    "bindings.cpp",
    "runtime/tensor_map.cpp",
    "runtime/fused_rank.cpp",
    "runtime/kernel_runner.cpp",
    "gemm/grouped_gemm.cu",
    "gemm/grouped_gemm_pair.cu",
    "comm/comm_kernels.cu",
    "plan/plan_kernel.cu",
    "plan/expert_sort_noalloc.cu",
    "model/model_kernels.cu",
    "model/router_kernels.cu",
    "model/model_ops.cpp",
]
_lock = threading.Lock()
_module = None


def _sources() -> list[str]:
    out = []
    for rel in _SOURCES:
        path = os.path.join(_CSRC, rel)
        if os.path.exists(path) and os.path.splitext(path)[1] in (".cpp", ".cu"):
            out.append(path)
    return out


def _so_path() -> str:
    return os.path.join(_BUILD_DIR, _NAME + ".so")


def _source_digest() -> str:
    """Content hash of every file under csrc/ (what the built object depends on)."""
    h = hashlib.sha256()
    for root, dirs, files in os.walk(_CSRC):
        dirs.sort()
        for f in sorted(files):
            path = os.path.join(root, f)
            h.update(os.path.relpath(path, _CSRC).encode())
            with open(path, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _digest_path() -> str:
    return os.path.join(_BUILD_DIR, _NAME + ".sha256")


def _is_stale() -> bool:
    """True when there is no built object or it was built from different sources (file times play no role:
    a copied tree keeps its object usable)."""
    if not os.path.exists(_so_path()) or not os.path.exists(_digest_path()):
        return True
    with open(_digest_path()) as f:
        return f.read().strip() != _source_digest()


def build(verbose: bool = False, force: bool = False):
    """Compiles the extension if its sources are newer than the built object; returns the module."""
    global _module
    with _lock:
        if _module is not None and not force:
            return _module
        if force or _is_stale():
            if os.environ.get("CEM_NO_BUILD") == "1":
                raise RuntimeError("the sm_100a extension is missing or stale and CEM_NO_BUILD=1 forbids building it")
            from torch.utils.cpp_extension import load

            os.makedirs(_BUILD_DIR, exist_ok=True)
            os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
            load(
                name=_NAME,
                sources=_sources(),
                extra_cflags=["-O3", "-std=c++17"],
                extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
                                   "--expt-relaxed-constexpr"],
                extra_include_paths=[_CSRC],
                build_directory=_BUILD_DIR,
                verbose=verbose,
                is_python_module=False,
            )
            with open(_digest_path(), "w") as f:
                f.write(_source_digest())
        spec = importlib.util.spec_from_file_location(_NAME, _so_path())
        module = importlib.util.module_from_spec(spec)
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        spec.loader.exec_module(module)
        sys.modules[_NAME] = module
        _module = module
        return module


def load():
    """Returns the extension, building it first when needed. Raises if it cannot be had."""
    return build()


def is_built() -> bool:
    return os.path.exists(_so_path())
