"""Quantization arguments and preset schemes for the weight path.

Field names and value spellings follow ``QuantizationArgs`` / ``QuantizationScheme`` of
compressed-tensors (quantization/quant_args.py:157-410, quant_scheme.py:145-428) so that
recipes written for llm-compressor read the same here; an instance of the
compressed-tensors class is accepted wherever one of these is (``QuantizationArgs.of``).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Optional

import torch

from . import _lib

__all__ = ["QuantizationArgs", "QuantizationScheme", "preset_name_to_scheme", "PRESET_SCHEMES"]

_STRATEGY = {"tensor": _lib.TENSOR, "channel": _lib.CHANNEL, "group": _lib.GROUP,
             "tensor_group": _lib.TENSOR_GROUP, "block": _lib.BLOCK}


def _plain(v):
    return v.value if hasattr(v, "value") else v


@dataclass
class QuantizationArgs:
    num_bits: int = 8
    type: str = "int"
    symmetric: bool = True
    group_size: Optional[int] = None
    strategy: Optional[str] = None
    block_structure: Optional[list] = None
    dynamic: Any = False
    actorder: Optional[str] = None
    scale_dtype: Optional[torch.dtype] = None
    zp_dtype: Optional[torch.dtype] = None
    observer: Optional[str] = None
    observer_kwargs: dict = field(default_factory=dict)

    def __post_init__(self):
        self.type = _plain(self.type)
        self.strategy = _plain(self.strategy)
        self.actorder = _plain(self.actorder)
        for f in ("scale_dtype", "zp_dtype"):
            v = getattr(self, f)
            if isinstance(v, str):
                setattr(self, f, getattr(torch, v.replace("torch.", "")))
        # activation-ordering aliases (quant_args.py:126-155,264-271)
        if self.actorder is True or self.actorder == "dynamic":
            self.actorder = "group"
        elif self.actorder == "static":
            self.actorder = "weight"
        elif self.actorder is False:
            self.actorder = None
        # strategy inference (quant_args.py:285-300)
        if self.strategy is None:
            if self.group_size is None or self.group_size == -1:
                self.strategy = "tensor" if self.group_size is None else "channel"
            elif self.group_size > 0:
                self.strategy = "group"
            else:
                raise ValueError(f"invalid group_size {self.group_size}")
        if self.strategy in ("group", "tensor_group") and not (self.group_size and self.group_size > 0):
            raise ValueError(f"strategy {self.strategy} requires group_size to be set to a positive value")
        if self.strategy == "block" and not self.block_structure:
            raise ValueError("Block strategy requires block structure")
        if self.actorder is not None and self.strategy not in ("group", "tensor_group"):
            raise ValueError("Must use group or tensor_group quantization strategy in order to "
                             "apply activation ordering")
        if self.observer is None and self.dynamic is not True:
            self.observer = "memoryless_minmax"
        if self.zp_dtype is None:
            if self.type == "float":
                self.zp_dtype = torch.float8_e4m3fn
            else:
                self.zp_dtype = torch.int8 if self.num_bits <= 8 else torch.int16
        self.observer_kwargs = dict(self.observer_kwargs or {})

    @classmethod
    def of(cls, obj) -> "QuantizationArgs":
        """Accept this class, a compressed-tensors QuantizationArgs, or a dict."""
        if isinstance(obj, cls):
            return obj
        if isinstance(obj, dict):
            return cls(**obj)
        names = ("num_bits", "type", "symmetric", "group_size", "strategy", "block_structure",
                 "dynamic", "actorder", "scale_dtype", "zp_dtype", "observer", "observer_kwargs")
        return cls(**{n: getattr(obj, n) for n in names if hasattr(obj, n)})

    def model_copy(self, update=None) -> "QuantizationArgs":
        return replace(self, **(update or {}))

    def pytorch_dtype(self) -> torch.dtype:
        if self.type == "float":
            if self.num_bits == 8:
                return torch.float8_e4m3fn
            raise NotImplementedError("Only num_bits in (8) are supported")
        return torch.int8 if self.num_bits <= 8 else torch.int16

    # ---- kernel-side view -----------------------------------------------------------------
    @property
    def is_mx(self) -> bool:
        return (self.num_bits in (4, 8) and self.type == "float" and self.group_size == 32
                and self.scale_dtype == torch.uint8)

    def c_struct(self) -> _lib.QArgs:
        if self.scale_dtype is None:
            sk = _lib.SCALE_PLAIN
        elif self.scale_dtype == torch.float8_e4m3fn:
            sk = _lib.SCALE_FP8
        elif self.scale_dtype == torch.uint8 and self.is_mx:
            sk = _lib.SCALE_E8M0
        else:
            raise ValueError(f"unsupported scale_dtype {self.scale_dtype}")
        zk = {torch.int8: _lib.ZP_INT8, torch.float8_e4m3fn: _lib.ZP_FP8,
              torch.uint8: _lib.ZP_UINT8}.get(self.zp_dtype)
        if zk is None:
            raise ValueError(f"unsupported zp_dtype {self.zp_dtype}")
        bs = self.block_structure or [0, 0]
        return _lib.QArgs(self.num_bits, _lib.QFLOAT if self.type == "float" else _lib.QINT,
                          int(bool(self.symmetric)), _STRATEGY[self.strategy],
                          int(self.group_size or 0), int(bs[0]), int(bs[1]), sk, zk)

    def qparam_shape(self, N: int, K: int):
        s = self.strategy
        if s == "tensor":
            return (1,)
        if s == "channel":
            return (N, 1)
        if s in ("group", "tensor_group"):
            return (N, -(-K // self.group_size))
        bh, bw = self.block_structure
        return (-(-N // bh), -(-K // bw))


@dataclass
class QuantizationScheme:
    targets: list
    weights: Optional[QuantizationArgs] = None
    input_activations: Optional[QuantizationArgs] = None
    output_activations: Optional[QuantizationArgs] = None
    format: Optional[str] = None


def _w(**kw):
    return dict(kw)


# weight side of the presets and, where a preset also quantises input activations, that side:
# "dynamic" ones (per token / per group at run time) need no calibration and only decide the
# checkpoint format; FP8 calibrates a static per-tensor scale, NVFP4 a static global scale
# (CT/quantization/quant_scheme.py:145-428)
def _act(**kw):
    return dict(kw)


_TOKEN8 = _act(num_bits=8, type="int", symmetric=True, strategy="token", dynamic=True)
PRESET_SCHEMES = {
    "W4A16": (_w(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128), None),
    "W4A16_ASYM": (_w(num_bits=4, type="int", symmetric=False, strategy="group", group_size=128), None),
    "W8A16": (_w(num_bits=8, type="int", symmetric=True, strategy="channel"), None),
    "W8A8": (_w(num_bits=8, type="int", symmetric=True, strategy="channel"), _TOKEN8),
    "INT8": (_w(num_bits=8, type="int", symmetric=True, strategy="channel"), _TOKEN8),
    "W4A8": (_w(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128), _TOKEN8),
    "FP8": (_w(num_bits=8, type="float", symmetric=True, strategy="tensor"),
            _act(num_bits=8, type="float", symmetric=True, strategy="tensor", dynamic=False, observer="minmax")),
    "FP8_DYNAMIC": (_w(num_bits=8, type="float", symmetric=True, strategy="channel"),
                    _act(num_bits=8, type="float", symmetric=True, strategy="token", dynamic=True)),
    "FP8_BLOCK": (_w(num_bits=8, type="float", symmetric=True, strategy="block", block_structure=[128, 128]),
                  _act(num_bits=8, type="float", symmetric=True, strategy="group", group_size=128, dynamic=True)),
    "NVFP4A16": (_w(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16,
                    scale_dtype=torch.float8_e4m3fn, zp_dtype=torch.float8_e4m3fn), None),
    "NVFP4": (_w(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16,
                 scale_dtype=torch.float8_e4m3fn, zp_dtype=torch.float8_e4m3fn),
              _act(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16, dynamic="local",
                   observer="static_minmax", scale_dtype=torch.float8_e4m3fn, zp_dtype=torch.float8_e4m3fn)),
    "MXFP4A16": (_w(num_bits=4, type="float", symmetric=True, strategy="group", group_size=32,
                    scale_dtype=torch.uint8, zp_dtype=torch.uint8), None),
    "MXFP4": (_w(num_bits=4, type="float", symmetric=True, strategy="group", group_size=32,
                 scale_dtype=torch.uint8, zp_dtype=torch.uint8),
              _act(num_bits=4, type="float", symmetric=True, strategy="group", group_size=32, dynamic=True,
                   scale_dtype=torch.uint8, zp_dtype=torch.uint8)),
    "MXFP8A16": (_w(num_bits=8, type="float", symmetric=True, strategy="group", group_size=32,
                    scale_dtype=torch.uint8, zp_dtype=torch.uint8), None),
    "MXFP8": (_w(num_bits=8, type="float", symmetric=True, strategy="group", group_size=32,
                 scale_dtype=torch.uint8, zp_dtype=torch.uint8),
              _act(num_bits=8, type="float", symmetric=True, strategy="group", group_size=32, dynamic=True,
                   scale_dtype=torch.uint8, zp_dtype=torch.uint8)),
}


def preset_name_to_scheme(name: str, targets: list) -> QuantizationScheme:
    """Scheme of a preset name (CT/quantization/quant_scheme.py:116-142)."""
    key = name.upper()
    if key not in PRESET_SCHEMES:
        raise KeyError(f"Unknown preset scheme name {name}, available names: {list(PRESET_SCHEMES)}")
    w, act = PRESET_SCHEMES[key]
    scheme = QuantizationScheme(targets=list(targets), weights=QuantizationArgs(**w))
    if act is not None:
        scheme.input_activations = QuantizationArgs(**act)
    return scheme
