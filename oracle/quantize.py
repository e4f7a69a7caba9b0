"""fake-quantize / quantize / dequantize of a weight matrix (test infrastructure only).

Restates ``_quantize_dequantize`` / ``_quantize`` / ``_dequantize``
(CT/quantization/lifecycle/forward_helpers.py:176-268), the group / block / channel
broadcasting of ``_process_quantization`` (CT/quantization/lifecycle/forward.py:185-241,
forward_helpers.py:57-172) and ``round_to_quantized_type_args``
(CT/quantization/quant_args.py:439-475) for 2-D weights.

The dtype of each step is left to torch type promotion on purpose, because the
reference's results depend on it: with bf16 weights and bf16 scales the division
``x / scale`` is rounded to bf16 at pack time, while inside GPTQ ``x`` is float32 and
only the dequantised value ``q.to(scale.dtype) * scale`` is rounded to bf16.
"""
from __future__ import annotations

import torch

from .qparams import qrange
from .rounding import cast_e2m1, cast_e4m3


def _round_codes(v: torch.Tensor, args) -> torch.Tensor:
    """Clamp to the code range, then round; result keeps v's dtype."""
    qmin, qmax = qrange(args)
    orig = v.dtype
    v = torch.clamp(v, qmin, qmax)
    if args.type == "float":
        if args.num_bits == 8:
            r = cast_e4m3(v.float())
        elif args.num_bits == 4:
            r = cast_e2m1(v.float())
        else:
            raise NotImplementedError
    else:
        r = torch.round(v)
    return r.to(orig)


def _expand(p: torch.Tensor, shape, args, g_idx):
    """Broadcast a per-group / per-channel / per-tensor / per-block parameter to the
    weight's shape [N, K]."""
    N, K = shape
    if p is None:
        return None
    s = args.strategy
    if s == "tensor":
        return p.reshape(1, 1).expand(N, K)
    if s == "channel":
        return p.reshape(N, 1).expand(N, K)
    if s in ("group", "tensor_group"):
        g = args.group_size
        if p.ndim < 2:
            p = p.reshape(-1, 1)
        if g_idx is not None and not bool((g_idx == -1).any()):
            # column c uses group g_idx[c] (CT forward_helpers.py:142-170: the reference
            # sorts columns by g_idx, groups consecutively, then unsorts)
            order = torch.argsort(g_idx)
            col_group = torch.empty(K, dtype=torch.long)
            col_group[order] = torch.arange(K) // g
            return p[:, col_group]
        return p.repeat_interleave(g, dim=1)[:, :K]
    if s == "block":
        bh, bw = args.block_structure
        return p.repeat_interleave(bh, dim=0)[:N].repeat_interleave(bw, dim=1)[:, :K]
    raise ValueError(f"unsupported strategy {s}")


def _eff_scale(scale, global_scale):
    return scale / global_scale if global_scale is not None else scale


def fake_quantize(x, scale, zero_point, args, g_idx=None, global_scale=None):
    """Quantize then dequantize ``x`` [N,K]; returns a tensor of x's dtype for grouped
    strategies (the reference casts back, forward_helpers.py:164) and of the promoted
    dtype otherwise."""
    s = _expand(_eff_scale(scale, global_scale), x.shape, args, g_idx)
    zp = _expand(zero_point, x.shape, args, g_idx)
    v = x / s
    if zp is not None:
        v = v + zp.to(x.dtype)
    q = _round_codes(v, args)
    d = q.to(s.dtype)
    if zp is not None:
        d = d - zp.to(s.dtype)
    out = d * s
    if args.strategy in ("group", "tensor_group"):
        out = out.to(x.dtype)
    return out


def quantize_codes(x, scale, zero_point, args, dtype=None, g_idx=None, global_scale=None):
    """Codes of ``x`` (integer-valued or FP8/FP4-valued floats unless ``dtype`` asks for
    a storage type)."""
    s = _expand(_eff_scale(scale, global_scale), x.shape, args, g_idx)
    zp = _expand(zero_point, x.shape, args, g_idx)
    v = x / s
    if zp is not None:
        v = v + zp.to(x.dtype)
    q = _round_codes(v, args)
    if dtype is not None:
        q = q.to(dtype)
    elif args.strategy in ("group", "tensor_group"):
        q = q.to(x.dtype)
    return q


def dequantize_codes(q, scale, zero_point, args, dtype=None, g_idx=None, global_scale=None):
    s = _expand(_eff_scale(scale, global_scale), q.shape, args, g_idx)
    zp = _expand(zero_point, q.shape, args, g_idx)
    d = q.to(s.dtype)
    if zp is not None:
        d = d - zp.to(s.dtype)
    d = d * s
    return d.to(dtype) if dtype is not None else d
