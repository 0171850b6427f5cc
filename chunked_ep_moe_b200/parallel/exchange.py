"""Slice exchange transports that run on torch.distributed collectives.

Both functions implement the ragged exchange contract the layer loops are
written against (reference: src/chunked_moe/transport/ragged.py:14-53):

    output = exchange(operand, output, SliceArgs, group)

`SliceArgs` holds `P*L` segments per call, laid out `[peer * L + l]`. Segment i
is `operand[input_offsets[i] : +send_sizes[i]]`; it lands on peer `i // L` at
the *sender-chosen* row `output_offsets[i]` of that peer's `output`. Several
segments per peer is what lets a sender write straight into the expert-major
positions of a receiver's slice buffer.

  ragged_exchange    variable-split `all_to_all_single` (NCCL on GPU, gloo on
                     CPU) + one fixed-size exchange of the destination
                     offsets. This is the baseline transport.
  emulated_exchange  padded dense windows, equal-split all-to-all of windows
                     and of the sender-chosen offsets, masked writes. Only
                     affordable at test sizes; it exists so the algorithm can
                     be checked on any backend.

The product transport (one-sided NVLink stores fused into the GEMM kernels)
does not go through this interface; see `parallel/symm.py` and `ops/fused.py`.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.plan import SliceArgs


def _world(group: Optional[dist.ProcessGroup]) -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group)
    return 1


def _segment_rows(offsets: torch.Tensor, sizes: torch.Tensor) -> torch.Tensor:
    """Row indices of the concatenation of segments `[offsets[i], offsets[i]+sizes[i])`, in segment order."""
    total = int(sizes.sum())
    if total == 0:
        return offsets.new_zeros((0,))
    seg = torch.repeat_interleave(torch.arange(sizes.numel(), device=sizes.device), sizes)
    starts = torch.cumsum(sizes, 0) - sizes
    within = torch.arange(total, device=sizes.device) - starts[seg]
    return offsets[seg] + within


def ragged_exchange(operand: torch.Tensor, output: torch.Tensor, args: SliceArgs,
                    group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Ragged all-to-all built on `all_to_all_single` with per-peer split sizes."""
    num_ranks = _world(group)
    num_segments = args.send_sizes.numel()
    per_peer = num_segments // num_ranks
    send_sizes = args.send_sizes.to(torch.int64)
    recv_sizes = args.recv_sizes.to(torch.int64)
    send_rows = _segment_rows(args.input_offsets.to(torch.int64), send_sizes)
    packed = operand.index_select(0, send_rows)

    if num_ranks == 1:
        received, dest_offsets = packed, args.output_offsets.to(torch.int64)
    else:
        in_splits = send_sizes.reshape(num_ranks, per_peer).sum(1).tolist()
        out_splits = recv_sizes.reshape(num_ranks, per_peer).sum(1).tolist()
        received = operand.new_empty((sum(out_splits),) + tuple(operand.shape[1:]))
        dist.all_to_all_single(received, packed.contiguous(), out_splits, in_splits, group=group)
        dest_offsets = torch.empty_like(args.output_offsets)
        dist.all_to_all_single(dest_offsets, args.output_offsets.contiguous(), group=group)
        dest_offsets = dest_offsets.to(torch.int64)

    dest_rows = _segment_rows(dest_offsets, recv_sizes)
    if dest_rows.numel():
        output.index_copy_(0, dest_rows, received)
    return output


def emulated_exchange(operand: torch.Tensor, output: torch.Tensor, args: SliceArgs,
                      group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Same semantics as `ragged_exchange` with padded `[cap]`-row windows and equal-split all-to-alls."""
    num_ranks = _world(group)
    num_segments = args.send_sizes.numel()
    cap = max(1, min(output.shape[0], operand.shape[0]))  # no segment is longer than either buffer
    rows = torch.arange(cap, device=operand.device)
    src = (args.input_offsets.to(torch.int64)[:, None] + rows[None, :]).clamp_(0, max(operand.shape[0] - 1, 0))
    if operand.shape[0] == 0:
        windows = operand.new_zeros((num_segments, cap) + tuple(operand.shape[1:]))
    else:
        windows = operand[src.reshape(-1)].reshape((num_segments, cap) + tuple(operand.shape[1:]))
    keep = rows[None, :] < args.send_sizes.to(torch.int64)[:, None]
    windows = torch.where(keep.reshape((num_segments, cap) + (1,) * (operand.dim() - 1)), windows,
                          torch.zeros_like(windows))

    offsets = args.output_offsets.contiguous()
    if num_ranks == 1:
        received, dest_offsets = windows, offsets
    else:
        received = torch.empty_like(windows)
        dist.all_to_all_single(received, windows.contiguous(), group=group)
        dest_offsets = torch.empty_like(offsets)
        dist.all_to_all_single(dest_offsets, offsets, group=group)

    recv_sizes = args.recv_sizes.to(torch.int64)
    for i in range(num_segments):
        n = int(recv_sizes[i])
        if n:
            start = int(dest_offsets[i])
            output[start:start + n] = received[i, :n]
    return output


def exchange_fn(transport: str):
    """Maps a config transport string to a collective exchange function."""
    if transport == "ragged_a2a":
        return ragged_exchange
    if transport == "emulated":
        return emulated_exchange
    raise ValueError(f"transport {transport!r} has no collective exchange function")
