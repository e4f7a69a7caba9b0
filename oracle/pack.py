"""Bit packing and per-format compression of one module (test infrastructure only).

Restates ``pack_to_int32`` (CT/compressors/pack_quantized/helpers.py:20-89),
``pack_fp4_to_uint8`` (CT/compressors/nvfp4/helpers.py:34-74), ``compress_mx_scale``
(CT/compressors/mx_utils.py:18-30), the format priority
(CT/compressors/format.py:18-27,75-96) and the ``compress`` classmethods of the
pack-quantized, nvfp4, mxfp4, mxfp8 and naive compressors
(CT/compressors/{pack_quantized,nvfp4,mxfp4,mxfp8,naive_quantized}/base.py).
"""
from __future__ import annotations

import numpy as np
import torch

from .quantize import quantize_codes


def pack_int32(codes: torch.Tensor, num_bits: int, packed_dim: int = 1) -> torch.Tensor:
    """int8 codes -> int32 words: code j of each run of 32/num_bits consecutive values
    (after adding 2^(bits-1)) occupies bits [j*bits, (j+1)*bits); rows are zero padded
    to a whole number of words."""
    assert codes.dtype == torch.int8
    v = (codes.to(torch.int16) + (1 << (num_bits - 1))).numpy().astype(np.uint8)
    if packed_dim == 0:
        v = v.T
    pf = 32 // num_bits
    rows, cols = v.shape
    pad = (-cols) % pf
    if pad:
        v = np.pad(v, ((0, 0), (0, pad)))
    v = v.reshape(rows, -1, pf).astype(np.uint32)
    out = np.zeros(v.shape[:2], dtype=np.uint32)
    for j in range(pf):
        out |= v[:, :, j] << np.uint32(j * num_bits)
    out = out.view(np.int32)
    if packed_dim == 0:
        out = np.ascontiguousarray(out.T)
    return torch.from_numpy(out.copy())


def unpack_int32(packed: torch.Tensor, num_bits: int, shape, packed_dim: int = 1) -> torch.Tensor:
    p = packed.numpy().view(np.uint32)
    if packed_dim == 0:
        p = p.T
    pf = 32 // num_bits
    mask = np.uint32((1 << num_bits) - 1)
    cols = [(p >> np.uint32(j * num_bits)) & mask for j in range(pf)]
    v = np.stack(cols, axis=-1).reshape(p.shape[0], -1).astype(np.int16)
    v = (v - (1 << (num_bits - 1))).astype(np.int8)
    if packed_dim == 0:
        v = v.T[: shape[0], : shape[1]]
    else:
        v = v[: shape[0], : shape[1]]
    return torch.from_numpy(np.ascontiguousarray(v))


_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def pack_fp4(x: torch.Tensor) -> torch.Tensor:
    """E2M1-valued floats -> nibbles: index of the nearest table entry (first on ties),
    bit 3 = sign bit (so -0.0 gives 0x8); element 2i in the low nibble."""
    m, n = x.shape
    assert n % 2 == 0, "even number of columns required"
    xf = x.float().numpy()
    idx = np.abs(np.abs(xf)[..., None] - _E2M1).argmin(-1).astype(np.uint8)
    idx |= (np.signbit(xf).astype(np.uint8) << 3)
    idx = idx.reshape(-1, 2)
    return torch.from_numpy((idx[:, 0] | (idx[:, 1] << 4)).astype(np.uint8).reshape(m, n // 2))


def compress_mx_scale(scale: torch.Tensor) -> torch.Tensor:
    """Power-of-two float scale -> biased exponent 127 + floor(log2 scale) as uint8."""
    return (127 + torch.floor(torch.log2(scale)).to(torch.int32)).to(torch.uint8)


def infer_format(args, has_input_activations: bool = False) -> str:
    """Compression format for an nn.Linear whose weights use ``args``
    (priority list of CT/compressors/format.py:18-27)."""
    fp = args.type == "float"
    if args.num_bits == 4 and fp and args.group_size == 32:
        return "mxfp4-pack-quantized"
    if args.num_bits == 8 and fp and args.group_size == 32 and args.scale_dtype == torch.uint8:
        return "mxfp8-quantized"
    if args.num_bits == 4 and fp and args.group_size == 16:
        return "nvfp4-pack-quantized"
    if not has_input_activations and args.num_bits in (4, 8) and not fp:
        return "pack-quantized"
    if has_input_activations and not fp:
        return "int-quantized"
    if has_input_activations and fp:
        return "float-quantized"
    return "naive-quantized"


def compress_weight(state: dict, args, fmt: str | None = None) -> dict:
    """Per-module ``compress``: local names weight / weight_scale / weight_zero_point /
    weight_global_scale / weight_g_idx in, compressed tensor set out."""
    fmt = fmt or infer_format(args)
    sd = dict(state)
    w = sd.pop("weight")
    scale = sd.get("weight_scale")
    zp = sd.get("weight_zero_point")
    g_idx = sd.get("weight_g_idx")
    if fmt == "pack-quantized":
        q = quantize_codes(w, scale, zp, args, dtype=torch.int8, g_idx=g_idx)
        sd["weight_packed"] = pack_int32(q, args.num_bits)
        sd["weight_shape"] = torch.tensor(w.shape)
        if not args.symmetric and args.strategy in ("group", "channel"):
            sd["weight_zero_point"] = pack_int32(zp, args.num_bits, packed_dim=0).contiguous()
    elif fmt in ("nvfp4-pack-quantized", "mxfp4-pack-quantized"):
        gs = sd.get("weight_global_scale")
        q = quantize_codes(w, scale, zp, args, global_scale=gs)
        sd["weight_packed"] = pack_fp4(q)
        if fmt == "nvfp4-pack-quantized":
            sd["weight_scale"] = scale.to(args.scale_dtype or torch.float8_e4m3fn)
        else:
            sd["weight_scale"] = compress_mx_scale(scale)
    elif fmt in ("naive-quantized", "int-quantized", "float-quantized", "mxfp8-quantized"):
        st = torch.float8_e4m3fn if args.type == "float" else torch.int8
        sd["weight"] = quantize_codes(w, scale, zp, args, dtype=st, g_idx=g_idx)
        if fmt == "mxfp8-quantized":
            sd["weight_scale"] = compress_mx_scale(scale)
    else:
        raise ValueError(fmt)
    if args.symmetric:
        sd.pop("weight_zero_point", None)
    return sd
