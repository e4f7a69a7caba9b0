"""Quantization-argument record used by the oracle (test infrastructure only).

Field names and value spellings mirror ``QuantizationArgs`` of compressed-tensors
(CT/quantization/quant_args.py:157-330) so that an instance of either class can be
handed to any oracle function: ``type`` is "int" | "float", ``strategy`` is "tensor" |
"channel" | "group" | "tensor_group" | "block", ``actorder`` is None | "group" |
"weight" ("static" is an alias of "weight", CT/quantization/quant_args.py:126-155).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional

import torch


@dataclass
class QSpec:
    num_bits: int = 8
    type: str = "int"
    symmetric: bool = True
    strategy: str = "tensor"
    group_size: Optional[int] = None
    block_structure: Optional[list] = None
    scale_dtype: Optional[torch.dtype] = None
    zp_dtype: Optional[torch.dtype] = None
    actorder: Optional[str] = None
    observer: str = "memoryless_minmax"
    observer_kwargs: dict = field(default_factory=dict)
    dynamic: bool = False

    def __post_init__(self):
        for f in ("scale_dtype", "zp_dtype"):
            v = getattr(self, f)
            if isinstance(v, str):
                setattr(self, f, getattr(torch, v.replace("torch.", "")))
        for f in ("type", "strategy", "actorder"):
            v = getattr(self, f)
            if v is not None and hasattr(v, "value"):
                setattr(self, f, v.value)
        if self.actorder == "static":
            self.actorder = "weight"
        if self.actorder == "dynamic" or self.actorder is True:
            self.actorder = "group"
        if self.zp_dtype is None:
            # CT/quantization/quant_args.py:396-420: symmetric -> int8 ("pytorch_dtype");
            # float types use the float dtype itself.
            if self.type == "float":
                self.zp_dtype = torch.float8_e4m3fn if self.num_bits == 8 else torch.float8_e4m3fn
            else:
                self.zp_dtype = torch.int8 if self.num_bits <= 8 else torch.int16

    def model_copy(self, update=None):
        return replace(self, **(update or {}))


def preset(name: str, **over) -> QSpec:
    """Weight-side arguments of the compressed-tensors preset schemes
    (CT/quantization/quant_scheme.py:145-428)."""
    name = name.upper()
    table = {
        "W4A16": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128),
        "W4A16_ASYM": dict(num_bits=4, type="int", symmetric=False, strategy="group", group_size=128),
        "W8A16": dict(num_bits=8, type="int", symmetric=True, strategy="channel"),
        "W8A8": dict(num_bits=8, type="int", symmetric=True, strategy="channel"),
        "FP8": dict(num_bits=8, type="float", symmetric=True, strategy="tensor"),
        "FP8_DYNAMIC": dict(num_bits=8, type="float", symmetric=True, strategy="channel"),
        "NVFP4A16": dict(num_bits=4, type="float", symmetric=True, strategy="tensor_group",
                         group_size=16, scale_dtype=torch.float8_e4m3fn,
                         zp_dtype=torch.float8_e4m3fn),
        "MXFP4A16": dict(num_bits=4, type="float", symmetric=True, strategy="group",
                         group_size=32, scale_dtype=torch.uint8, zp_dtype=torch.uint8),
        "MXFP8A16": dict(num_bits=8, type="float", symmetric=True, strategy="group",
                         group_size=32, scale_dtype=torch.uint8, zp_dtype=torch.uint8),
    }
    table["NVFP4"] = table["NVFP4A16"]
    table["MXFP4"] = table["MXFP4A16"]
    table["MXFP8"] = table["MXFP8A16"]
    d = dict(table[name])
    d.update(over)
    return QSpec(**d)
