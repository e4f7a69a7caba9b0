"""Scalar rounding rules of the quantize path, restated with integer bit arithmetic.

TEST INFRASTRUCTURE ONLY (see the package docstring).  Every function here works on
float32 CPU tensors and is written against the bit pattern, so that it is an
independent statement of what ``tensor.to(torch.bfloat16)``,
``tensor.to(torch.float8_e4m3fn)`` and compressed-tensors' ``cast_to_fp4`` do.
"""
from __future__ import annotations

import torch


def _bits(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF


def _from_bits(b: torch.Tensor) -> torch.Tensor:
    b = b & 0xFFFFFFFF
    b = torch.where(b >= 2**31, b - 2**32, b)
    return b.to(torch.int32).view(torch.float32)


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """float32 -> nearest bfloat16 (ties to even), returned as float32.

    Same result as ``x.to(torch.bfloat16).float()`` for finite inputs."""
    x = x.to(torch.float32)
    b = _bits(x)
    lsb = (b >> 16) & 1
    r = (b + 0x7FFF + lsb) & 0xFFFF0000
    out = _from_bits(r)
    return torch.where(torch.isfinite(x), out, x)


def cast_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Round float32 values (already clamped to +-448) to the FP8 E4M3 (fn) grid,
    ties to even, subnormals with step 2^-9; returned as float32.

    This is the rounding of ``tensor.to(torch.float8_e4m3fn)`` that
    ``round_to_quantized_type_args`` uses for 8-bit floats
    (CT/quantization/quant_args.py:462-464)."""
    x = x.to(torch.float32)
    a = x.abs()
    # exponent of the value, floored at the smallest normal exponent (-6)
    e = torch.floor(torch.log2(torch.clamp(a, min=2.0**-20)))
    e = torch.clamp(e, min=-6.0)
    step = torch.pow(torch.tensor(2.0), e - 3.0)  # 3 mantissa bits
    q = torch.round(a / step) * step  # torch.round is half-to-even; a/step is exact
    q = torch.clamp(q, max=448.0)
    return torch.copysign(q, x)


_E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def cast_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Round to the FP4 E2M1 value set {0,.5,1,1.5,2,3,4,6} with ties to the value
    whose mantissa bit is even, sign re-applied by multiplication so that a negative
    input that rounds to zero becomes -0.0 and +-0.0 inputs become +0.0
    (CT/quantization/quant_args.py:53-66)."""
    x = x.to(torch.float32)
    a = x.abs()
    out = torch.full_like(a, 6.0)
    out = torch.where(a <= 5.0, torch.full_like(a, 4.0), out)
    out = torch.where(a < 3.5, torch.full_like(a, 3.0), out)
    out = torch.where(a <= 2.5, torch.full_like(a, 2.0), out)
    out = torch.where(a < 1.75, torch.full_like(a, 1.5), out)
    out = torch.where(a <= 1.25, torch.full_like(a, 1.0), out)
    out = torch.where(a < 0.75, torch.full_like(a, 0.5), out)
    out = torch.where(a <= 0.25, torch.zeros_like(a), out)
    out = torch.where(torch.isnan(a), a, out)
    sign = torch.where(x > 0, 1.0, torch.where(x < 0, -1.0, 0.0)).to(torch.float32)
    return out * sign


def round_to_power_2(x: torch.Tensor) -> torch.Tensor:
    """Keep sign+exponent of ``x`` after adding a quarter of the exponent step, so
    that a mantissa of 1.75 or more carries into the next exponent
    (CT/quantization/utils/mxfp_utils.py:68-107).  Works for bfloat16 and float32
    inputs and returns the input dtype."""
    if x.dtype == torch.bfloat16:
        b = x.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        add, mask = 1 << (7 - 1 - 1), 0x1FF << 7
        r = (b + add) & mask
        r = torch.where(r >= 2**15, r - 2**16, r).to(torch.int16)
        return r.view(torch.bfloat16)
    assert x.dtype == torch.float32
    b = _bits(x)
    add, mask = 1 << (23 - 1 - 1), 0x1FF << 23
    return _from_bits((b + add) & mask)


def e8m0_from_amax(amax: torch.Tensor, num_bits: int) -> torch.Tensor:
    """Biased E8M0 exponent of the MX block scale for a block whose largest
    magnitude is ``amax``: 127 + floor(log2(round_to_power_2(amax))) - offset with
    offset 2 for FP4 (floor(log2 6)) and 8 for FP8 (floor(log2 448))
    (CT/quantization/utils/mxfp_utils.py:28-33,110-128).  Returned in the input
    dtype, like the reference (which keeps float arithmetic here)."""
    offset = {4: 2, 8: 8}[num_bits]
    p2 = round_to_power_2(amax)
    return 127 + torch.floor(torch.log2(p2)) - offset
