"""Slice exchange transports that run on torch.distributed collectives.

Both functions implement the ragged exchange contract the layer loops are
written against (reference: src/chunked_moe/transport/ragged.py:14-53):

    output = exchange(operand, output, ExchangeSpec, group)

An `ExchangeSpec` (ops/plan.py) holds `P*L` segments per call, laid out
`[peer * L + l]`, as HOST arrays. Segment i is
`operand[src_offset[i] : +send_rows[i]]`; it lands on peer `i // L` at the
*sender-chosen* row `dst_offset[i]` of that peer's `output`. Several segments
per peer is what lets a sender write straight into the expert-major positions
of a receiver's slice buffer.

  ragged_exchange    one variable-split `all_to_all_single` (NCCL on GPU, gloo
                     on CPU); receivers place rows with their own copy of the
                     plan. This is the baseline transport.
  emulated_exchange  padded dense windows, equal-split all-to-all of windows
                     and of the sender-chosen offsets (checked against the
                     receiver's plan). Only affordable at test sizes; it
                     exists so the algorithm can be checked on any backend.

The product transport (one-sided NVLink stores fused into the GEMM kernels)
does not go through this interface; see `parallel/symm.py` and `ops/fused.py`.
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops.plan import ExchangeSpec


def _world(group: Optional[dist.ProcessGroup]) -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group)
    return 1


def _segment_rows(offsets: np.ndarray, sizes: np.ndarray, device: torch.device) -> torch.Tensor:
    """Row indices of the concatenation of segments `[offsets[i], offsets[i]+sizes[i])`, in segment order.

    Offsets and sizes are host arrays, so the total is known without asking the device: the two small arrays go up
    in one copy and the index is expanded there.
    """
    total = int(sizes.sum())
    if total == 0:
        return torch.zeros((0,), dtype=torch.int64, device=device)
    starts = np.cumsum(sizes) - sizes
    table = torch.from_numpy(np.stack([offsets - starts, sizes])).to(device, non_blocking=True)  # [2, n]
    seg = torch.repeat_interleave(torch.arange(sizes.size, device=device), table[1], output_size=total)
    return torch.arange(total, device=device) + table[0][seg]


def ragged_exchange(operand: torch.Tensor, output: torch.Tensor, spec: ExchangeSpec,
                    group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Ragged all-to-all: ONE variable-split `all_to_all_single` per exchange.

    Senders pack their segments peer by peer; receivers place what arrives at the rows the plan gives them
    (`land_offset`). Split sizes and offsets are host values from the plan, so nothing is read back from the device
    and no second collective carries offsets.
    """
    num_ranks = _world(group)
    dev = operand.device
    packed = operand.index_select(0, _segment_rows(spec.src_offset, spec.send_rows, dev))
    if num_ranks == 1:
        received = packed
    else:
        received = operand.new_empty((int(spec.recv_rows.sum()),) + tuple(operand.shape[1:]))
        dist.all_to_all_single(received, packed.contiguous(), spec.recv_splits, spec.send_splits, group=group)
    rows = _segment_rows(spec.land_offset, spec.recv_rows, dev)
    if rows.numel():
        output.index_copy_(0, rows, received)
    return output


def emulated_exchange(operand: torch.Tensor, output: torch.Tensor, spec: ExchangeSpec,
                      group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Same contract with equal-split collectives only: every segment travels as a padded `[cap]`-row window.

    For backends (or tests) without a variable-split all-to-all. `cap` bounds any segment: it can be longer neither
    than the operand nor than the output. The sender-chosen destination offsets travel too and are checked against
    the receiver's own view of the plan, which makes this path a consistency test of the planner. Only affordable at
    test sizes.
    """
    num_ranks = _world(group)
    dev = operand.device
    n = spec.send_rows.size
    cap = max(1, min(output.shape[0], operand.shape[0]))
    windows = operand.new_zeros((n, cap) + tuple(operand.shape[1:]))
    for i in np.flatnonzero(spec.send_rows):
        a, k = int(spec.src_offset[i]), int(spec.send_rows[i])
        windows[i, :k] = operand[a:a + k]
    aimed = torch.from_numpy(np.stack([spec.dst_offset, spec.send_rows])).t().contiguous().to(dev)  # [n, 2]
    if num_ranks > 1:
        got, got_aimed = torch.empty_like(windows), torch.empty_like(aimed)
        dist.all_to_all_single(got, windows, group=group)
        dist.all_to_all_single(got_aimed, aimed, group=group)
        windows, aimed = got, got_aimed
    aimed = aimed.cpu().numpy()
    for i in np.flatnonzero(spec.recv_rows):
        a, k = int(spec.land_offset[i]), int(spec.recv_rows[i])
        if (int(aimed[i, 0]), int(aimed[i, 1])) != (a, k):
            raise RuntimeError(f"segment {i}: the sender aims {int(aimed[i, 1])} rows at row {int(aimed[i, 0])}, "
                               f"this rank's plan expects {k} rows at row {a}")
        output[a:a + k] = windows[i, :k]
    return output


def exchange_fn(transport: str):
    """Maps a config transport string to a collective exchange function."""
    if transport == "ragged_a2a":
        return ragged_exchange
    if transport == "emulated":
        return emulated_exchange
    raise ValueError(f"transport {transport!r} has no collective exchange function")
