"""Weight observers: min/max statistics and the MSE shrink-grid search
(test infrastructure only).

Restates ``flatten_for_calibration`` for weights
(src/llmcompressor/observers/helpers.py:28-102), ``_get_min_max``
(src/llmcompressor/observers/min_max.py:70-74), ``_grid_search_mse`` /
``_grid_search_eager`` / ``_calculate_error``
(src/llmcompressor/observers/mse_quant.py:19-141,255-284) and the statistics ->
qparams step of ``Observer.get_qparams`` / ``get_global_scale``
(src/llmcompressor/observers/base.py:78-123).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .qparams import calculate_qparams, generate_gparam, qrange
from .quantize import _round_codes


def flatten_weight(value: torch.Tensor, args) -> torch.Tensor:
    """[N,K] -> (1, *qparam_shape, elements_per_group)."""
    s = args.strategy
    if s == "tensor":
        return value.reshape(1, 1, -1)
    if s == "channel":
        return value.unsqueeze(-2).unsqueeze(0)
    if s in ("group", "tensor_group"):
        return value.unflatten(-1, (-1, args.group_size)).unsqueeze(0)
    if s == "block":
        bh, bw = args.block_structure
        N, K = value.shape
        value = F.pad(value, (0, (-K) % bw, 0, (-N) % bh))
        r, c = value.shape
        return (
            value.reshape(r // bh, bh, c // bw, bw).transpose(1, 2).flatten(-2, -1).unsqueeze(0)
        )
    raise ValueError(f"unsupported weight strategy {s}")


def observe_minmax(value: torch.Tensor, args):
    obs = flatten_weight(value, args)
    return torch.amin(obs, dim=(0, -1)), torch.amax(obs, dim=(0, -1))


def _mse_error(obs, args, mn, mx, norm):
    """Sum over each group of |fake_quant(x) - x|^norm for the candidate range
    (mse_quant.py:255-284).  The candidate qparams are computed without a global scale
    and the fake-quantisation is element-wise against [..., 1] parameters."""
    scale, zp = calculate_qparams(mn, mx, args, global_scale=None)
    s = scale.unsqueeze(-1)
    z = zp.unsqueeze(-1)
    v = obs / s
    v = v + z.to(obs.dtype)
    q = _round_codes(v, args)
    d = q.to(s.dtype) - z.to(s.dtype)
    fq = (d * s).to(obs.dtype)
    return torch.sum((fq - obs).abs().pow(norm), dim=(0, -1))


def observe_mse(value, args, maxshrink=0.20, patience=5, grid=100.0, norm=2.4, expand=1.0):
    """Shrink-grid search: candidate p = 1 - i/grid for i < int(maxshrink*grid); a group
    keeps the candidate with the strictly smallest error; the search stops once
    ``patience`` consecutive candidates improved no group at all
    (mse_quant.py:52-65,99-141)."""
    if args.strategy == "tensor_group" and args.scale_dtype is not None:
        args = args.model_copy(update={"scale_dtype": None})
    obs = flatten_weight(value, args)
    mn = torch.amin(obs, dim=(0, -1)) * expand
    mx = torch.amax(obs, dim=(0, -1)) * expand
    best_err = torch.full_like(mn, torch.finfo(mn.dtype).max)
    best_mn, best_mx = mn.clone(), mx.clone()
    stale = 0
    for i in range(int(maxshrink * grid)):
        p = 1 - i / grid
        smn, smx = mn * p, mx * p
        err = _mse_error(obs, args, smn, smx, norm)
        better = err < best_err
        if bool(better.any()):
            best_err[better] = err[better]
            best_mn[better] = smn[better]
            best_mx[better] = smx[better]
            stale = 0
        else:
            stale += 1
            if stale >= patience:
                break
    return best_mn, best_mx


class WeightObserver:
    """Statistics holder with the reference's memoryless weight-observer behaviour:
    a second observation while statistics exist is ignored
    (src/llmcompressor/observers/base.py:137-138); ``get_qparams`` consumes the
    statistics (:123).  ``fused`` lists partner observers that share one NVFP4 global
    scale (src/llmcompressor/observers/base.py:90-96, fusion.py:58-77)."""

    def __init__(self, args, kind: str | None = None, **kwargs):
        self.args = args
        kind = kind or getattr(args, "observer", None) or "memoryless_minmax"
        kind = {"minmax": "memoryless_minmax", "static_minmax": "memoryless_minmax",
                "mse": "memoryless_mse"}.get(kind, kind)
        self.kind = kind
        self.kwargs = dict(getattr(args, "observer_kwargs", None) or {})
        self.kwargs.update(kwargs)
        self.min_vals = self.max_vals = None
        self.fused = []

    @property
    def has_statistics(self):
        return self.min_vals is not None

    def __call__(self, value):
        if value.numel() == 0 or self.has_statistics:
            return self
        if self.kind == "memoryless_minmax":
            self.min_vals, self.max_vals = observe_minmax(value, self.args)
        elif self.kind in ("memoryless_mse", "nvfp4_expanded_mse"):
            kw = dict(self.kwargs)
            if self.kind == "nvfp4_expanded_mse":
                kw.setdefault("expand", 1.8)
                kw.setdefault("maxshrink", 1 - 0.8 / 1.8)
                kw.setdefault("grid", 200.0)
                kw.setdefault("patience", 1000)
            kw = {k: v for k, v in kw.items()
                  if k in ("maxshrink", "patience", "grid", "norm", "expand")}
            self.min_vals, self.max_vals = observe_mse(value, self.args, **kw)
        else:
            raise ValueError(f"unknown observer {self.kind}")
        return self

    def delete_statistics(self):
        self.min_vals = self.max_vals = None

    def get_global_scale(self):
        if self.args.strategy != "tensor_group":
            return None
        members = [self] + list(self.fused)
        amax = members[0].max_vals.max()
        for m in members:
            amax = torch.max(amax, -m.min_vals.min())
            amax = torch.max(amax, m.max_vals.max())
        return generate_gparam(-amax.reshape(1), amax.reshape(1))

    def get_qparams(self):
        assert self.has_statistics, "No statistics available. Call observer(value) first."
        gs = self.get_global_scale()
        scale, zp = calculate_qparams(self.min_vals, self.max_vals, self.args, global_scale=gs)
        self.delete_statistics()
        return {"scale": scale, "zero_point": zp, "global_scale": gs}
