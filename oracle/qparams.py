"""Scale / zero-point / global-scale rules (test infrastructure only).

Restates ``calculate_qparams`` (CT/quantization/utils/helpers.py:50-137),
``calculate_range`` (:199-227), ``generate_gparam`` (:309-338) and
``_get_dtype_eps`` (:364-372).  Arithmetic is done in the dtype of the incoming
statistics, as the reference does: bf16 weights give bf16 min/max and therefore bf16
scales, except where a float32 ``global_scale`` promotes the product to float32.
"""
from __future__ import annotations

import torch

from .rounding import cast_e4m3, e8m0_from_amax


def qrange(args):
    """(q_min, q_max) of the code range (CT/quantization/utils/helpers.py:199-227)."""
    if args.type == "int":
        half = 2.0 ** args.num_bits / 2
        return -half, half - 1
    if args.type == "float":
        if args.num_bits == 8:
            return -448.0, 448.0
        if args.num_bits == 4:
            return -6.0, 6.0
        raise NotImplementedError("float range only for 4 and 8 bits")
    raise ValueError(f"invalid quantization type {args.type}")


def is_mx(args) -> bool:
    """MX formats: float codes, groups of 32, uint8 (E8M0) scales
    (CT/quantization/utils/mxfp_utils.py:36-43)."""
    return (
        args.num_bits in (4, 8)
        and args.type == "float"
        and args.group_size == 32
        and args.scale_dtype == torch.uint8
    )


def _dtype_eps(dtype) -> float:
    if dtype == torch.float8_e4m3fn:
        return 0.125
    if dtype.is_floating_point:
        return torch.finfo(dtype).eps
    return 1


def _round_to_dtype(t: torch.Tensor, dtype, back: bool = True) -> torch.Tensor:
    """``round_to_quantized_type_dtype`` (CT/quantization/quant_args.py:411-436)."""
    orig = t.dtype
    if dtype.is_floating_point:
        fi = torch.finfo(dtype)
        c = torch.clamp(t, fi.min, fi.max)
        if dtype == torch.float8_e4m3fn:
            r = cast_e4m3(c.float())
            return r.to(orig) if back else r.to(dtype)
        r = c.to(dtype)
    else:
        ii = torch.iinfo(dtype)
        r = torch.round(torch.clamp(t, ii.min, ii.max)).to(dtype)
    return r.to(orig) if back else r


def calculate_qparams(min_vals, max_vals, args, global_scale=None):
    """Scale and zero point from per-group statistics.

    Steps follow CT/quantization/utils/helpers.py:69-137 in order: force the range to
    contain zero; symmetric scale = absmax / (range/2) (or the E8M0 exponent for MX);
    asymmetric scale = (max-min)/range with zp = clamp(qmin - min/scale); multiply by the
    global scale; round to ``scale_dtype``; turn an MX exponent back into 2^(e-127);
    replace zero scales by eps; round the zero point to ``zp_dtype``."""
    min_vals = torch.min(min_vals, torch.zeros_like(min_vals))
    max_vals = torch.max(max_vals, torch.zeros_like(max_vals))
    qmin, qmax = qrange(args)
    bit_range = qmax - qmin
    if args.symmetric:
        amax = torch.max(min_vals.abs(), max_vals.abs())
        if is_mx(args):
            scales = e8m0_from_amax(amax, args.num_bits)
        else:
            scales = amax / (float(bit_range) / 2)
        zps = torch.zeros(scales.shape, dtype=min_vals.dtype)
    else:
        if args.num_bits == 4 and args.type == "float":
            raise NotImplementedError("asymmetric FP4 is not supported")
        scales = (max_vals - min_vals) / float(bit_range)
        zps = qmin - (min_vals / scales)
        zps = torch.clamp(zps, qmin, qmax)
    if global_scale is not None:
        scales = global_scale * scales
    if args.scale_dtype is not None:
        scales = _round_to_dtype(scales, args.scale_dtype)
    if is_mx(args):
        orig = scales.dtype
        e = scales.to(torch.int32) - 127
        scales = (2.0 ** e.to(torch.float32)).to(orig)
    eps = _dtype_eps(args.scale_dtype if args.scale_dtype is not None else scales.dtype)
    scales = torch.where(scales == 0, torch.tensor(eps, dtype=scales.dtype), scales)
    zps = _round_to_dtype(zps, args.zp_dtype, back=False)
    if scales.ndim == 0:
        scales = scales.reshape(1)
        zps = zps.reshape(1)
    return scales, zps


def generate_gparam(min_val, max_val):
    """NVFP4 tensor-wide scale 448*6 / absmax in the statistics' dtype, NaN/Inf -> 1,
    cast to float32 [1] (CT/quantization/utils/helpers.py:309-338)."""
    min_vals = torch.min(min_val, torch.zeros_like(min_val))
    max_vals = torch.max(max_val, torch.zeros_like(max_val))
    amax = torch.max(min_vals.abs(), max_vals.abs())
    amax = torch.clamp(amax, min=torch.finfo(amax.dtype).tiny)
    g = 448.0 * 6.0 / amax
    g = torch.nan_to_num(g, nan=1.0, posinf=1.0, neginf=1.0)
    return g.to(torch.float32).reshape([1])
