"""The e4m3 + 1x128-block-scale wire format (plain torch; the put kernel and `dequant_slice` implement the same)."""

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from chunked_ep_moe_b200.ops import quant


def test_identity_without_a_comm_dtype():
    x = torch.randn(3, 256)
    q, scale = quant.quantize_rows(x, None)
    assert q is x and scale is None
    assert quant.dequantize_rows(q, scale, torch.float32) is x
    with pytest.raises(ValueError):
        quant.quantize_rows(x, "int4")


@settings(max_examples=30, deadline=None)
@given(rows=st.integers(1, 9), blocks=st.integers(1, 4), seed=st.integers(0, 10**6),
       magnitude=st.sampled_from([1e-6, 1.0, 3e4]))
def test_round_trip_error_is_bounded_per_block(rows, blocks, seed, magnitude):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, 128 * blocks, generator=gen) * magnitude
    x[0, :128] = 0.0  # an all-zero block must survive (scale floor, no division by zero)
    q, scale = quant.quantize_rows(x, "float8_e4m3fn")
    assert q.dtype == torch.float8_e4m3fn and q.shape == x.shape
    assert scale.shape == (rows, blocks) and scale.dtype == torch.float32 and (scale > 0).all()
    back = quant.dequantize_rows(q, scale, torch.float32)
    assert torch.isfinite(back).all() and (back[0, :128] == 0).all()
    amax = x.reshape(rows, blocks, 128).abs().amax(-1, keepdim=True)
    err = (back - x).reshape(rows, blocks, 128).abs()
    # e4m3 keeps 3 mantissa bits: half an ulp is 1/16 of the value, and nothing in a block exceeds its amax
    assert (err <= amax / 16 + 1e-30).all()
    # the largest element of every block maps to +-448 exactly, so it comes back exactly (up to the scale's rounding)
    top = x.reshape(rows, blocks, 128).abs().argmax(-1, keepdim=True)
    got = back.reshape(rows, blocks, 128).abs().gather(-1, top)
    assert torch.allclose(got, amax, rtol=1e-6, atol=0)


def test_rows_narrower_than_a_block_use_one_scale_per_row():
    x = torch.randn(5, 96)
    q, scale = quant.quantize_rows(x, "float8_e4m3fn")
    assert scale.shape == (5, 1)
    back = quant.dequantize_rows(q, scale, torch.bfloat16)
    assert back.dtype == torch.bfloat16 and back.shape == x.shape


def test_quantisation_is_deterministic():
    """Forward and the backward's recomputed forward must see identical rows."""
    x = torch.randn(7, 384, generator=torch.Generator().manual_seed(1)).bfloat16()
    a = quant.quantize_rows(x, "float8_e4m3fn")
    b = quant.quantize_rows(x.clone(), "float8_e4m3fn")
    assert torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8)) and torch.equal(a[1], b[1])
