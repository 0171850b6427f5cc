"""Static configuration of the chunked expert-parallel MoE layer.

Field-for-field the same surface as the reference's `ChunkedMoEConfig`
(src/chunked_moe/config.py:10-50): the dataclass is frozen and hashable so it
can key caches (workspaces, compiled plans).

Backends selected by string:

  transport      "emulated"   dense gloo/CPU exchange that honours the ragged
                              contract (sender-chosen destination offsets)
                 "ragged_a2a" NCCL `all_to_all_single` exchange (the baseline)
                 "nvshmem"    one-sided NVLink peer stores with arrival flags,
                              fused into the sm_100a GEMM kernels (the product)
  expert_compute "reference"  torch grouped GEMM (library)
                 "fused"      hand-written tcgen05/TMEM kernels
"""

from __future__ import annotations

import dataclasses
from typing import Literal, Optional

Transport = Literal["ragged_a2a", "nvshmem", "emulated"]
ExpertCompute = Literal["reference", "fused"]

_TRANSPORTS = ("ragged_a2a", "nvshmem", "emulated")
_EXPERT_COMPUTE = ("reference", "fused")
_COMM_DTYPES = (None, "float8_e4m3fn")

#: SM count of one B200 (2 dies x 74). The reference defaulted to 132 (H100).
B200_NUM_SMS = 148


@dataclasses.dataclass(frozen=True)
class ChunkedMoEConfig:
    """Hyper-parameters fixed for the lifetime of a layer.

    Attributes:
      num_experts: global number of routed experts E (E % EP size == 0).
      top_k: experts per token K.
      slice_size: rows S of one dispatch slice. Every receiver's packed,
        expert-major stream is cut into S-row slices; all per-iteration
        buffers are S rows whatever the routing imbalance.
      transport / expert_compute: see module docstring.
      comm_dtype: None (rows travel in the compute dtype) or "float8_e4m3fn"
        (rows are quantised on put with one fp32 scale per 1x128 block and
        dequantised on the receiver; GEMMs stay bf16).
      accum_dtype: dtype of the weight-gradient accumulation across slices.
      num_sms: persistent-grid size of the fused kernels.
      stripe_width: columns per gate/up stripe of the striped `w_up` layout.
    """

    num_experts: int
    top_k: int
    slice_size: int = 1024
    transport: Transport = "ragged_a2a"
    expert_compute: ExpertCompute = "reference"
    comm_dtype: Optional[str] = None
    accum_dtype: str = "float32"
    num_sms: int = B200_NUM_SMS
    stripe_width: int = 128

    def __post_init__(self):
        if self.slice_size <= 0:
            raise ValueError(f"slice_size must be positive, got {self.slice_size}")
        if self.top_k <= 0 or self.top_k > self.num_experts:
            raise ValueError(f"top_k={self.top_k} must be in [1, num_experts={self.num_experts}]")
        if self.transport not in _TRANSPORTS:
            raise ValueError(f"unknown transport {self.transport!r}; expected one of {_TRANSPORTS}")
        if self.expert_compute not in _EXPERT_COMPUTE:
            raise ValueError(f"unknown expert_compute {self.expert_compute!r}; expected one of {_EXPERT_COMPUTE}")
        if self.comm_dtype not in _COMM_DTYPES:
            raise ValueError(f"unsupported comm_dtype {self.comm_dtype!r}; expected one of {_COMM_DTYPES}")
        if self.stripe_width <= 0:
            raise ValueError(f"stripe_width must be positive, got {self.stripe_width}")
        if self.num_sms <= 0:
            raise ValueError(f"num_sms must be positive, got {self.num_sms}")

    @property
    def is_product_path(self) -> bool:
        """True when both the transport and the expert compute are the fused sm_100a kernels."""
        return self.transport == "nvshmem" and self.expert_compute == "fused"
