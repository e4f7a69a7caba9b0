"""Weight observers backed by the b200q kernels.

Mirrors ``Observer`` and its registered subclasses of llm-compressor for the weight
path (src/llmcompressor/observers/base.py:29-213, min_max.py:10-19, mse.py:12-131) and the
fusion of q/k/v and gate/up global scales (helpers.py:162-215, fusion.py:17-105):
``observer(weight)`` records statistics, ``get_qparams()`` turns them into
scale / zero point / global scale and drops them.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .quant_args import QuantizationArgs

__all__ = ["Observer", "MemorylessMinMaxObserver", "MemorylessMSEObserver", "NVFP4ExpandedMSEObserver",
           "StaticMinMaxObserver", "MinMaxObserver", "fuse_weight_observers", "FUSED_LAYER_NAMES"]

_REGISTRY: dict = {}

# weight observers are memoryless: the moving-average / static kinds named in a recipe map
# onto them (src/llmcompressor/modifiers/quantization/calibration.py:64-78)
_WEIGHT_ALIASES = {"minmax": "memoryless_minmax", "static_minmax": "memoryless_minmax",
                   "mse": "memoryless_mse"}


class Observer:
    """Base class: statistics -> qparams."""

    # statistic attribute -> how ranks combine it when activation statistics are synchronised
    # ("min" / "max" / "avg"; src/llmcompressor/observers/base.py:147-162)
    _act_sync_dict: dict = {}

    def __init__(self, base_name: str, args, **observer_kwargs):
        self.base_name = base_name
        self.args = QuantizationArgs.of(args)
        self.args.observer_kwargs = dict(self.args.observer_kwargs or {})
        self.args.observer_kwargs.update(observer_kwargs)
        self.min_vals: Optional[torch.Tensor] = None
        self.max_vals: Optional[torch.Tensor] = None
        self._fused: list = []        # partner observers (excluding self)
        self._fused_weights: list = []  # callables returning the partner's weight
        self._own_weight = None
        self._deletion_called = False

    # ---- registry (RegistryMixin-like) -------------------------------------------------
    @classmethod
    def register(cls, name):
        def deco(klass):
            if name in _REGISTRY and _REGISTRY[name] is not klass:
                raise ValueError(f"observer name {name} is already registered")
            _REGISTRY[name] = klass
            return klass
        return deco

    @classmethod
    def load_from_registry(cls, name: str, base_name: str = "weight", args=None, **kw):
        if base_name == "weight":
            name = _WEIGHT_ALIASES.get(name, name)
        if name not in _REGISTRY:
            raise KeyError(f"Unknown observer {name}; registered: {sorted(_REGISTRY)}")
        return _REGISTRY[name](base_name=base_name, args=args, **kw)

    # ---- statistics --------------------------------------------------------------------
    @property
    def has_statistics(self) -> bool:
        return self.min_vals is not None and self.max_vals is not None

    @property
    def is_weight_obs(self) -> bool:
        return self.base_name == "weight"

    def update_statistics_from_weight(self, weight: torch.Tensor) -> None:
        raise NotImplementedError

    def update_statistics_from_activation(self, value: torch.Tensor) -> None:
        raise NotImplementedError(f"{type(self).__name__} observes weights only")

    @torch.no_grad()
    def __call__(self, observed: torch.Tensor) -> "Observer":
        if observed.numel() == 0:
            return self
        if not self.is_weight_obs:
            self.update_statistics_from_activation(observed)
            return self
        if self.has_statistics:
            return self
        self.update_statistics_from_weight(observed)
        self._observe_partners()
        return self

    def sync_activation_stats(self) -> list:
        """All-reduce the accumulated activation statistics across ranks (weights are identical on
        every rank, only the calibration data differs).  Returns async work handles."""
        import torch.distributed as dist
        work = []
        for attr, how in self._act_sync_dict.items():
            val = getattr(self, attr, None)
            if val is None:
                continue
            if how == "avg":   # (gloo has no AVG)
                val.div_(dist.get_world_size())
                work.append(dist.all_reduce(val, op=dist.ReduceOp.SUM, async_op=True))
            else:
                op = dist.ReduceOp.MIN if how == "min" else dist.ReduceOp.MAX
                work.append(dist.all_reduce(val, op=op, async_op=True))
        return work

    forward = __call__

    def get_statistics(self):
        return {"min_vals": self.min_vals, "max_vals": self.max_vals}

    def delete_statistics(self, check_fused: bool = True) -> None:
        if check_fused and self._fused:
            # cooperative deletion: statistics go once every member of the fused group has
            # asked for its qparams (fusion.py:79-101)
            self._deletion_called = True
            if all(o._deletion_called for o in self._fused):
                for o in [self] + self._fused:
                    o._deletion_called = False
                    o.min_vals = o.max_vals = None
            return
        self.min_vals = self.max_vals = None

    # ---- fusion ------------------------------------------------------------------------
    def _observe_partners(self):
        for obs, getw in zip(self._fused, self._fused_weights):
            if not obs.has_statistics:
                w = getw()
                assert w is not None, "Fused module has been garbage collected before its weight was observed"
                obs.update_statistics_from_weight(w)

    def get_global_scale(self) -> Optional[torch.Tensor]:
        if self.args.strategy != "tensor_group":
            return None
        self._observe_partners()
        members = [self] + self._fused
        absmax = torch.zeros(1, dtype=torch.float32, device=self.min_vals.device)
        for m in members:
            ops.absmax_accumulate(m.min_vals, m.max_vals, absmax)
        return ops.global_scale_from_absmax(absmax, self.min_vals.dtype)

    @torch.no_grad()
    def get_qparams(self):
        assert self.has_statistics, "No statistics available. Call observer(value) first."
        global_scale = self.get_global_scale()
        scale, zero_point = ops.qparams(self.min_vals, self.max_vals, self.args, global_scale)
        self.delete_statistics()
        return {"scale": scale, "zero_point": zero_point, "global_scale": global_scale}


@Observer.register("memoryless_minmax")
class MemorylessMinMaxObserver(Observer):
    def update_statistics_from_weight(self, weight):
        self.min_vals, self.max_vals = ops.observe_minmax(weight, self.args)


@Observer.register("memoryless_mse")
class MemorylessMSEObserver(Observer):
    _defaults = dict(maxshrink=0.20, patience=5, grid=100.0, norm=2.4, expand=1.0)

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        ok = self.args.observer_kwargs
        for k, v in self._defaults.items():
            setattr(self, k, ok.get(k, v))
        if self.expand < 1.0:
            raise ValueError(f"expand value must be at least 1.0, got {self.expand}")

    def update_statistics_from_weight(self, weight):
        self.min_vals, self.max_vals = ops.observe_mse(
            weight, self.args, maxshrink=self.maxshrink, patience=self.patience, grid=self.grid,
            norm=self.norm, expand=self.expand)


@Observer.register("nvfp4_expanded_mse")
class NVFP4ExpandedMSEObserver(MemorylessMSEObserver):
    _defaults = dict(maxshrink=1 - 0.8 / 1.8, patience=1000, grid=200.0, norm=2.4, expand=1.8)


def _activation_minmax(value: torch.Tensor, args: QuantizationArgs):
    """Statistics of an activation [..., hidden] for a static scheme: one (min, max) over
    everything (TENSOR, and TENSOR_GROUP whose only calibrated quantity is the global scale)."""
    if args.strategy not in ("tensor", "tensor_group"):
        raise NotImplementedError(f"static activation quantisation with strategy {args.strategy}")
    x = value.reshape(-1, value.shape[-1])
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.to(torch.float32)
    if x.stride(1) != 1:
        x = x.contiguous()
    targs = QuantizationArgs(num_bits=args.num_bits, type=args.type, symmetric=args.symmetric, strategy="tensor")
    return ops.observe_minmax(x, targs)


@Observer.register("static_minmax")
class StaticMinMaxObserver(Observer):
    """Min / max over every batch seen (src/llmcompressor/observers/min_max.py:22-40).  Weight
    observers of this name are memoryless (see ``load_from_registry``)."""
    _act_sync_dict = {"min_vals": "min", "max_vals": "max"}

    def update_statistics_from_weight(self, weight):
        self.min_vals, self.max_vals = ops.observe_minmax(weight, self.args)

    def update_statistics_from_activation(self, value):
        mn, mx = _activation_minmax(value, self.args)
        if self.has_statistics:
            mn, mx = torch.minimum(mn, self.min_vals), torch.maximum(mx, self.max_vals)
        self.min_vals, self.max_vals = mn, mx


@Observer.register("minmax")
class MinMaxObserver(Observer):
    """Moving average of the per-batch min / max with ``averaging_constant`` (default 0.01;
    min_max.py:43-67)."""
    _act_sync_dict = {"min_vals": "avg", "max_vals": "avg"}

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.avg_constant = self.args.observer_kwargs.get("averaging_constant", 0.01)

    def update_statistics_from_weight(self, weight):
        self.min_vals, self.max_vals = ops.observe_minmax(weight, self.args)

    def update_statistics_from_activation(self, value):
        mn, mx = _activation_minmax(value, self.args)
        if self.has_statistics and self.avg_constant != 1.0:
            mn = torch.lerp(self.min_vals, mn, self.avg_constant)
            mx = torch.lerp(self.max_vals, mx, self.avg_constant)
        self.min_vals, self.max_vals = mn, mx


# layer names whose NVFP4 global scale is shared (helpers.py:162-171)
FUSED_LAYER_NAMES = [
    ("gate_proj", "up_proj"),
    ("q_proj", "k_proj", "v_proj"),
    ("q_a_proj", "kv_a_proj_with_mqa"),
    ("w1", "w3"),
]


def fuse_observers(observers_and_modules) -> None:
    pairs = list(observers_and_modules)
    for obs, _ in pairs:
        obs._fused = [o for o, _ in pairs if o is not obs]
        obs._fused_weights = [(lambda m=m: m.weight) for o, m in pairs if o is not obs]


def fuse_weight_observers(model: torch.nn.Module) -> None:
    """Link the weight observers of sibling q/k/v and gate/up projections that use
    TENSOR_GROUP quantisation so that they share one global scale."""
    for sub in model.modules():
        for names in FUSED_LAYER_NAMES:
            if not all(hasattr(sub, n) for n in names):
                continue
            pairs, only_obs, only_tg = [], True, True
            for n in names:
                layer = getattr(sub, n)
                if layer is None:
                    continue
                obs = getattr(layer, "weight_observer", None)
                if obs is None:
                    only_obs = False
                    continue
                if obs.args.strategy != "tensor_group":
                    only_tg = False
                    continue
                pairs.append((obs, layer))
            if not pairs:
                continue
            start = f"Some layers in fused group: {names} have"
            end = ", need all fused layers to have same quantization"
            assert only_obs, f"{start} no weight observer{end}"
            assert only_tg, f"{start} non-TENSOR_GROUP quantization{end}"
            if pairs:
                fuse_observers(pairs)
