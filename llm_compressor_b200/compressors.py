"""Per-module compression to the compressed-tensors checkpoint layout.

Mirrors ``compress_module`` / the ``compress`` classmethods of the pack-quantized, nvfp4,
mxfp4, mxfp8 and naive compressors and the format priority of compressed-tensors
(compressors/base.py:145-168, pack_quantized/base.py:36-77, nvfp4/base.py:40-72,
mxfp4/base.py:21-60, mxfp8/base.py:48-68, naive_quantized/base.py:34-82, format.py:18-27).
A state dict with the local names ``weight``, ``weight_scale``, ``weight_zero_point``,
``weight_global_scale``, ``weight_g_idx`` goes in; the tensors a compressed checkpoint
stores for that module come out.
"""
from __future__ import annotations

import torch

from . import ops
from .quant_args import QuantizationArgs, QuantizationScheme

__all__ = ["infer_module_format", "compress_state_dict", "pack_to_int32", "pack_fp4_to_uint8",
           "compress_mx_scale", "COMPRESSION_FORMAT_PRIORITY"]

COMPRESSION_FORMAT_PRIORITY = [
    "mxfp4-pack-quantized", "mxfp8-quantized", "nvfp4-pack-quantized", "pack-quantized",
    "int-quantized", "float-quantized", "naive-quantized", "dense",
]


def _can_compress(fmt: str, w: QuantizationArgs, has_act: bool) -> bool:
    fp = w.type == "float"
    if fmt == "mxfp4-pack-quantized":
        return w.num_bits == 4 and fp and w.group_size == 32
    if fmt == "mxfp8-quantized":
        return w.num_bits == 8 and fp and w.group_size == 32 and w.scale_dtype == torch.uint8
    if fmt == "nvfp4-pack-quantized":
        return w.num_bits == 4 and fp and w.group_size == 16
    if fmt == "pack-quantized":
        return (not has_act) and w.num_bits in (4, 8) and not fp
    if fmt == "int-quantized":
        return has_act and not fp
    if fmt == "float-quantized":
        return has_act and fp
    return fmt == "naive-quantized"


def infer_module_format(scheme) -> str:
    """Compression format of an nn.Linear with this scheme (first match in priority order)."""
    if isinstance(scheme, QuantizationScheme):
        w, has_act = scheme.weights, scheme.input_activations is not None
    else:
        w, has_act = QuantizationArgs.of(scheme), False
    if w is None:
        return "dense"
    for fmt in COMPRESSION_FORMAT_PRIORITY:
        if _can_compress(fmt, w, has_act):
            return fmt
    return "dense"


def pack_to_int32(value: torch.Tensor, num_bits: int, packed_dim: int = 1) -> torch.Tensor:
    """int8 codes -> int32 words (pack_quantized/helpers.py:20-89)."""
    if value.dtype is not torch.int8:
        raise ValueError("Tensor must be quantized to torch.int8 before packing")
    if num_bits not in (4, 8) or packed_dim != 0:
        raise NotImplementedError("use quantize_pack for weights; this packs zero points (dim 0)")
    return ops.pack_zero_points(value, num_bits)


def compress_mx_scale(scale: torch.Tensor) -> torch.Tensor:
    return ops.compress_scale(scale, "e8m0")


def pack_fp4_to_uint8(x: torch.Tensor) -> torch.Tensor:
    """E2M1-valued floats [..., K] -> uint8 [..., K/2]: 3-bit magnitude index with the sign bit on
    top (-0.0 packs as 0x8), element 2i in the low nibble (nvfp4/helpers.py:34-74).  A stand-alone
    helper in tensor operations for callers that already hold E2M1 values; the save path never
    calls it, its kernels emit packed codes directly."""
    if x.shape[-1] % 2:
        raise ValueError("tensor must have an even number of columns for nibble packing")
    mag = x.abs().to(torch.float32)
    steps = torch.tensor([0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=x.device)
    nibble = (mag.unsqueeze(-1) >= steps).sum(-1).to(torch.uint8) | (torch.signbit(x).to(torch.uint8) << 3)
    return nibble[..., 0::2] | (nibble[..., 1::2] << 4)


def compress_state_dict(state_dict: dict, scheme, fmt: str | None = None) -> dict:
    """``Compressor.compress(state_dict, scheme)`` for one module."""
    if isinstance(scheme, QuantizationScheme):
        args = scheme.weights
    else:
        args = QuantizationArgs.of(scheme)
    fmt = fmt or infer_module_format(scheme)
    sd = dict(state_dict)
    w = sd.pop("weight")
    scale = sd.get("weight_scale")
    zp = sd.get("weight_zero_point")
    g_idx = sd.get("weight_g_idx")
    gs = sd.get("weight_global_scale")
    if fmt == "pack-quantized":
        sd["weight_packed"] = ops.quantize_pack(w, scale, zp, args, g_idx=g_idx, pack_int8=True)
        sd["weight_shape"] = torch.tensor(list(w.shape), device=w.device)
        if not args.symmetric and args.strategy in ("group", "channel"):
            assert zp is not None, "Asymmetric quant requires zero-point values"
            sd["weight_zero_point"] = ops.pack_zero_points(zp, args.num_bits)
    elif fmt in ("nvfp4-pack-quantized", "mxfp4-pack-quantized"):
        sd["weight_packed"] = ops.quantize_pack(w, scale, zp, args, global_scale=gs)
        sd["weight_scale"] = ops.compress_scale(scale, "fp8" if fmt.startswith("nvfp4") else "e8m0")
    elif fmt in ("naive-quantized", "int-quantized", "float-quantized", "mxfp8-quantized"):
        sd["weight"] = ops.quantize_pack(w, scale, zp, args, g_idx=g_idx)
        if fmt == "mxfp8-quantized":
            sd["weight_scale"] = ops.compress_scale(scale, "e8m0")
    else:
        raise ValueError(f"unsupported compression format {fmt}")
    if args.symmetric:
        sd.pop("weight_zero_point", None)
    return sd
