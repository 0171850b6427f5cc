"""Per-step observability that falls out of the plan for free.

The reference has no counters or logging (only prints in its compile script). These helpers turn a
plan (the host `RoutingPlan`'s own `stats()` or the fused path's plan header) into the numbers one wants
on a dashboard: rows per rank, slices, padding, imbalance, bytes on the wire, and the roofline of
the layer for the measured peaks.
"""

from __future__ import annotations

import json
import os
from typing import Optional


def wire_bytes(rows_remote: int, hidden: int, comm_dtype: Optional[str], backward: bool) -> dict:
    """Bytes this rank puts on NVLink in one pass (dispatch) and receives back (combine)."""
    elem = 1 if comm_dtype == "float8_e4m3fn" else 2
    scale = (hidden // 128) * 4 if comm_dtype == "float8_e4m3fn" else 0
    streams = 2 if backward else 1  # x (+ g)
    dispatch = rows_remote * (streams * (hidden * elem + scale) + 4)  # + fp32 router weight per row
    combine = rows_remote * (hidden * 2 + (4 if backward else 0))  # y or dx rows come back in bf16 (+ d_weight)
    return {"dispatch_bytes": dispatch, "combine_bytes": combine}


def layer_flops(rows: int, hidden: int, ffn: int, backward: bool) -> float:
    """FLOPs of the expert MLP on `rows` token copies: forward 6*D*F per row, backward (with remat) 18*D*F."""
    return float(rows) * hidden * ffn * (18.0 if backward else 6.0)


def load_measured_peaks(path: Optional[str] = None) -> dict:
    """Measured copy bandwidth and bf16 GEMM throughput of this pool's B200s, with documented fallbacks."""
    fallback = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            peaks = json.load(f)
        peaks["source"] = "measured"
        return peaks
    except (OSError, ValueError):
        return fallback


def roofline_ms(flops: float, nvlink_bytes: float, peaks: dict, sustained: bool = True,
                link_gbs: float = 770.0) -> dict:
    """Target time of a fused compute+collective pass: the slower of its math at peak and its bytes over NVLink."""
    tf = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    compute = flops / (tf * 1e12) * 1e3
    wire = nvlink_bytes / (link_gbs * 1e9) * 1e3
    return {"compute_ms": compute, "wire_ms": wire, "roofline_ms": max(compute, wire)}


def header_stats(header: list, slice_size: int) -> dict:
    """Decodes the fused path's plan header (`FusedRank.plan_header()`)."""
    num_slices, my_rows, max_rows, remote = header[0], header[1], header[2], header[3]
    active = -(-my_rows // slice_size)
    return {
        "num_slices": num_slices,
        "my_stream_rows": my_rows,
        "max_stream_rows": max_rows,
        "my_active_slices": active,
        "my_padding_rows": active * slice_size - my_rows,
        "rows_sent_remote": remote,
        "token_copies": header[5],
    }
