"""Checkpoint / resume for the trainer, and the striped <-> separate gate/up interchange format.

The reference has no checkpointing; its only persistent-layout code is `stripe_weights` /
`unstripe_weights` (src/chunked_moe/expert.py:39-45), with "store weights striped and convert
checkpoints" left as future work. Here parameters live striped; a checkpoint is one file per rank
(expert shards are rank-local, dense parameters are replicated so every rank's file has them) with
model, AdamW state, the step and the RNG state. `export_unstriped` / `import_unstriped` convert a
model state dict to and from separate `w_gate` / `w_up_proj` tensors for other frameworks.
"""

from __future__ import annotations

import os

import torch

from ..ops.striping import stripe_weights, unstripe_weights


def _path(directory: str, rank: int) -> str:
    return os.path.join(directory, f"rank{rank:03d}.pt")


def save_checkpoint(directory: str, model, optimizer, step: int, rank: int) -> str:
    os.makedirs(directory, exist_ok=True)
    path = _path(directory, rank)
    tmp = path + ".tmp"
    torch.save({
        "step": step,
        "model": model.state_dict(),
        "optimizer": optimizer.state_dict(),
        "rng_cpu": torch.get_rng_state(),
        "rng_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
    }, tmp)
    os.replace(tmp, path)  # a killed save never leaves a truncated checkpoint behind
    return path


def load_checkpoint(directory: str, model, optimizer, rank: int) -> int:
    state = torch.load(_path(directory, rank), map_location="cpu", weights_only=False)
    model.load_state_dict(state["model"])
    optimizer.load_state_dict(state["optimizer"])
    torch.set_rng_state(state["rng_cpu"])
    if state.get("rng_cuda") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["rng_cuda"])
    return int(state["step"])


def export_unstriped(state_dict: dict, stripe: int) -> dict:
    """Replaces every striped `...w_up` `[L, D, 2F]` entry by `...w_gate` and `...w_up_proj` `[L, D, F]`."""
    out = {}
    for name, t in state_dict.items():
        if name.endswith("w_up") and t.dim() == 3:
            gate, up = unstripe_weights(t, stripe)
            out[name[:-4] + "w_gate"] = gate
            out[name[:-4] + "w_up_proj"] = up
        else:
            out[name] = t
    return out


def import_unstriped(state_dict: dict, stripe: int) -> dict:
    """Inverse of `export_unstriped`."""
    out = {}
    for name, t in state_dict.items():
        if name.endswith("w_gate"):
            out[name[:-6] + "w_up"] = stripe_weights(t, state_dict[name[:-6] + "w_up_proj"], stripe)
        elif name.endswith("w_up_proj"):
            continue
        else:
            out[name] = t
    return out
