"""Dropless chunked expert-parallel MoE for B200 (sm_100a).

Public names match the reference package (src/chunked_moe/__init__.py:3-8).
"""

from .api import chunked_moe
from .config import ChunkedMoEConfig
from .ops.reference import reference_moe
from .ops.striping import stripe_weights, unstripe_weights

__all__ = ["ChunkedMoEConfig", "chunked_moe", "reference_moe", "stripe_weights", "unstripe_weights"]
__version__ = "0.1.0"
