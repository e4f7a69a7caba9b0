"""``AWQModifier``: activation-aware weight scaling ahead of weight quantisation.

Mirrors src/llmcompressor/modifiers/transform/awq/base.py:55-1057 and mappings.py:12-60 for
dense decoder models.  The modifier quantises nothing itself: for every mapping (a layer whose
output feeds a set of "balance" Linear layers) it searches a per-input-channel scale s that
minimises the output error of the parent module when the balance weights are quantised as
Q(W * s) / s, then folds s into the weights (balance layers times s, the smoothed layer divided
by s).  The quantisation inside the search is this package's observer -> qparams ->
fake-quantise kernels on the scheme that a QuantizationModifier / GPTQModifier in the same recipe
has attached; the forwards of the parent module are the model's own.

Not covered: ``activation_hook_target`` (parallel transformer blocks), loss masks, offloading of
the cached parent arguments (they stay in device memory).
"""
from __future__ import annotations

import inspect
import re
import warnings
from dataclasses import dataclass
from typing import Optional

import torch

from . import dist as bdist
from . import ops
from .modifiers import HooksMixin, _ObservingCache
from .observers import Observer, fuse_weight_observers

__all__ = ["AWQModifier", "AWQMapping", "default_mappings"]


@dataclass
class AWQMapping:
    """``smooth_layer``: name or ``re:`` pattern of the layer whose output is smoothed;
    ``balance_layers``: patterns of the layers that consume it (mappings.py:12-38)."""
    smooth_layer: str
    balance_layers: list
    activation_hook_target: Optional[str] = None


default_mappings = [
    AWQMapping("re:.*input_layernorm$", ["re:.*q_proj$", "re:.*k_proj$", "re:.*v_proj$"]),
    AWQMapping("re:.*v_proj$", ["re:.*o_proj$"]),
    AWQMapping("re:.*post_attention_layernorm$", ["re:.*gate_proj$", "re:.*up_proj$"]),
    AWQMapping("re:.*up_proj$", ["re:.*down_proj$"]),
]


@dataclass
class ResolvedMapping:
    smooth_name: str
    smooth_layer: torch.nn.Module
    balance_layers: list
    balance_names: list
    parent: torch.nn.Module
    parent_name: str


def _matches(name: str, pattern: str) -> bool:
    return re.match(pattern[3:], name) is not None if pattern.startswith("re:") else name == pattern


def _shared_depth(a: str, b: str) -> int:
    n = 0
    for x, y in zip(a.split("."), b.split(".")):
        if x != y:
            break
        n += 1
    return n


def _lowest_common_ancestor(names, model):
    """Name and module of the deepest module that contains all of ``names`` (a single name is
    its own ancestor); ModuleLists are skipped upwards, their forward is never called
    (base.py:1016-1038)."""
    parts = [n.split(".") for n in names]
    common = parts[0]
    for p in parts[1:]:
        k = 0
        while k < min(len(common), len(p)) and common[k] == p[k]:
            k += 1
        common = common[:k]
    name = ".".join(common)
    while True:
        if name == "":
            return "", model
        mod = model.get_submodule(name)
        if not isinstance(mod, torch.nn.ModuleList):
            return name, mod
        name = ".".join(name.split(".")[:-1])


def _layers_are_compatible(smooth_layer, smooth_name, balance_layers, balance_names) -> bool:
    """v_proj -> o_proj needs equal widths (grouped-query attention breaks it; base.py:984-1013)."""
    for layer, name in zip(balance_layers, balance_names):
        if (isinstance(smooth_layer, torch.nn.Linear) and isinstance(layer, torch.nn.Linear)
                and name.endswith(".o_proj")
                and ((smooth_name.endswith(".v_proj") and smooth_layer.out_features != layer.in_features)
                     or (smooth_name.endswith(".qkv_proj") and smooth_layer.out_features != 3 * layer.in_features))):
            return False
    return True


def compute_layer_means(layers) -> torch.Tensor:
    """Per input channel, the mean over the rows of all ``layers`` of |w| normalised by the largest
    |w| of its quantisation group / row / block / tensor (base.py:907-973)."""
    total, count = 0, 0
    for layer in layers:
        q_args = getattr(getattr(layer, "quantization_scheme", None), "weights", None)
        if not hasattr(layer, "weight") or q_args is None:
            continue
        weight = layer.weight.detach().clone()
        shape = weight.shape
        inter = None
        if q_args.strategy == "tensor":
            chunk = weight.numel()
        elif q_args.strategy == "channel":
            chunk = weight.size(1)
        elif q_args.strategy in ("group", "tensor_group"):
            chunk = q_args.group_size
        elif q_args.strategy == "block":
            bh, bw = q_args.block_structure
            weight = weight.unflatten(0, (-1, bh)).unflatten(-1, (-1, bw)).transpose(1, 2)
            inter = weight.shape
            chunk = bh * bw
        else:
            raise ValueError(f"unsupported strategy {q_args.strategy}")
        weight = weight.reshape(-1, chunk)
        weight.abs_()
        weight.div_(weight.amax(dim=1, keepdim=True) + 1e-6)
        if inter is not None:
            weight = weight.view(inter).transpose(1, 2)
        weight = weight.reshape(shape)
        count += weight.size(0)
        total = total + weight.sum(0, dtype=torch.float64)   # the reference's high precision (utils/dev.py:175-181)
    return total / count


def grid_search_params(duo_scaling, n_grid: int):
    """[(ratio, use_duo_scaling)] of the search (base.py:802-836)."""
    if duo_scaling == "both":
        n = int(n_grid / 2)
        return [(i / (n - 1), duo) for i in range(n) for duo in (False, True)]
    if duo_scaling is False:
        return [(i / (n_grid - 1), False) for i in range(n_grid)]
    if duo_scaling is True:
        return [(0.0, False)] + [(i / (n_grid - 2), True) for i in range(n_grid - 1)]
    raise ValueError(f"Found unexpected duo_scaling configuration {duo_scaling}")


def candidate_scales(x_mean: torch.Tensor, w_mean: Optional[torch.Tensor], ratio: float, duo: bool) -> torch.Tensor:
    """The per-channel scale of one grid point, normalised by sqrt(max * min) (base.py:668-679)."""
    if duo:
        scales = (x_mean.pow(ratio) / (w_mean.pow(1 - ratio) + 1e-4)).clamp(min=1e-4)
    else:
        scales = x_mean.pow(ratio).clamp(min=1e-4).view(-1)
    scales = scales / (scales.max() * scales.min()).sqrt()
    scales[torch.isinf(scales)] = 1
    scales[torch.isnan(scales)] = 1
    return scales


def scaled_fake_quantize(weights, scales: torch.Tensor, layers, parent=None) -> list:
    """Q(W * s) / s for every balance layer, in the weight's dtype: the scaled weight is rounded to
    the weight's dtype, observed with a memoryless min-max observer of the layer's scheme,
    fake-quantised, divided by s in float32 and rounded again (base.py:647-709).  Under
    TENSOR_GROUP the q/k/v or gate/up siblings inside ``parent`` share their global scale, as
    ``fuse_weight_observers(parent)`` arranges in the reference."""
    view = scales.view(1, -1)
    scaled = [(w * view).to(w.dtype) for w in weights]
    saved = [(getattr(layer, "weight_observer", None), layer.weight.data) for layer in layers]
    observers = []
    for layer, ws in zip(layers, scaled):
        obs = Observer.load_from_registry("memoryless_minmax", base_name="weight",
                                          args=layer.quantization_scheme.weights)
        observers.append(obs)
        layer.weight_observer = obs
        layer.weight.data = ws      # fused siblings are observed through their module's weight
    try:
        if parent is not None:
            fuse_weight_observers(parent)
        for obs, ws in zip(observers, scaled):
            obs(ws)
        params = [obs.get_qparams() for obs in observers]
    finally:
        for layer, (old, w) in zip(layers, saved):
            layer.weight.data = w
            if old is None:
                del layer.weight_observer
            else:
                layer.weight_observer = old
    out = []
    for ws, qp, layer, w in zip(scaled, params, layers, weights):
        fq = ops.fake_quantize(ws, qp["scale"], qp["zero_point"], layer.quantization_scheme.weights,
                               global_scale=qp["global_scale"])
        out.append((fq / view).to(w.dtype))
    return out


class AWQModifier(HooksMixin):
    """See the module docstring.  ``mappings``: list of ``AWQMapping`` (or dicts with the same
    fields); default: the Llama-style mappings.  ``duo_scaling``: True, False or "both";
    ``n_grid``: number of grid points."""

    requires_calibration_data = True

    def __init__(self, mappings=None, duo_scaling=True, n_grid: int = 20, offload_device=None):
        HooksMixin.__init__(self)
        if duo_scaling not in (True, False, "both"):
            raise ValueError(f"duo_scaling must be True, False or 'both', got {duo_scaling!r}")
        self.mappings = None if mappings is None else [m if isinstance(m, AWQMapping) else AWQMapping(**m)
                                                       for m in mappings]
        self.duo_scaling = duo_scaling
        self.n_grid = n_grid
        self.offload_device = offload_device
        self._resolved: list = []
        self._parent_args_cache: dict = {}
        self._smooth_activation_stats: dict = {}
        self.error_metrics: list = []

    def recipe_args(self) -> dict:
        maps = None if self.mappings is None else [
            {"smooth_layer": m.smooth_layer, "balance_layers": list(m.balance_layers)} for m in self.mappings]
        return dict(mappings=maps, duo_scaling=self.duo_scaling, n_grid=self.n_grid)

    # ---- life cycle ---------------------------------------------------------------------------
    def on_initialize(self, model, **_):
        if self.mappings is None:
            self.mappings = list(default_mappings)
        for m in self.mappings:
            if m.activation_hook_target:
                raise NotImplementedError("activation_hook_target is not supported")
        return True

    def on_calibration_start(self, model, **_):
        self._set_resolved_mappings(model)
        if self.duo_scaling is not False:
            for mapping in self._resolved:
                for name, layer in zip(mapping.balance_names, mapping.balance_layers):
                    w = getattr(getattr(layer, "quantization_scheme", None), "weights", None)
                    if w is not None and w.strategy == "tensor":
                        raise ValueError(
                            "duo_scaling is only supported with per-channel quantization strategies (group or "
                            f"channel), but found TENSOR strategy on layer {name}. Please set duo_scaling=False "
                            "or use a per-channel quantization strategy.")
        self._setup_activation_cache_hooks()

    def on_sequential_epoch_end(self, model, modules=None, **_):
        self._apply_smoothing(model)

    def on_calibration_end(self, model, **_):
        self._assert_all_activations_consumed()
        self.remove_hooks()

    def on_finalize(self, model, **_):
        self._parent_args_cache.clear()
        self._smooth_activation_stats.clear()
        self._resolved = []
        return True

    # ---- mappings -----------------------------------------------------------------------------
    def _set_resolved_mappings(self, model) -> None:
        """One ResolvedMapping per match of a mapping's smooth layer: its balance layers are the
        matches of the balance patterns that sit closest to it in the module tree (the same
        decoder layer; all experts of that layer for a mixture of experts) (base.py:281-387)."""
        named = dict(model.named_modules())
        resolved, incompatible = [], 0
        for mapping in self.mappings:
            smooth = [n for n in named if n and _matches(n, mapping.smooth_layer)]
            for smooth_name in smooth:
                balance_names = []
                for pattern in mapping.balance_layers:
                    cands = [n for n in named if n and _matches(n, pattern)]
                    if not cands:
                        continue
                    best = max(_shared_depth(smooth_name, n) for n in cands)
                    balance_names += [n for n in cands if _shared_depth(smooth_name, n) == best]
                smooth_layer = named[smooth_name]
                balance_layers = [named[n] for n in balance_names]
                targeted = hasattr(smooth_layer, "quantization_scheme") or any(
                    hasattr(layer, "quantization_scheme") for layer in balance_layers)
                if not _layers_are_compatible(smooth_layer, smooth_name, balance_layers, balance_names):
                    incompatible += 1
                    continue
                if not targeted or not balance_layers:
                    why = "no balance layers were found." if not balance_layers \
                        else "no layers are targeted for quantization."
                    warnings.warn(f"Skipping {smooth_name} for mapping {mapping} because {why}")
                    continue
                parent_name, parent = _lowest_common_ancestor(balance_names, model)
                resolved.append(ResolvedMapping(smooth_name, smooth_layer, balance_layers, balance_names,
                                                parent, parent_name))
        if incompatible:
            warnings.warn(f"{incompatible} mappings were skipped due to incompatible shapes.")
        self._resolved = resolved

    def _setup_activation_cache_hooks(self) -> None:
        """Record, per calibration batch, the arguments of every parent module (to replay its
        forward during the search) and the running sum of |x| per input channel of the first
        balance layer of every mapping (base.py:389-481)."""
        def cache_parent_kwargs(module, args, kwargs):
            bound = inspect.signature(module.forward).bind(*args, **kwargs).arguments
            bound = dict(bound)
            bound.update(bound.pop("kwargs", {}))
            for k, v in bound.items():
                if isinstance(v, _ObservingCache):
                    bound[k] = None
            self._parent_args_cache[module].append(bound)

        def make_stats_hook(smooth_name):
            def hook(_module, args, _output):
                act = args[0].abs().detach().flatten(0, -2)
                new_sum = act.float().sum(dim=0)
                stats = self._smooth_activation_stats.get(smooth_name)
                if stats is None:
                    self._smooth_activation_stats[smooth_name] = [new_sum, act.size(0)]
                else:
                    stats[0] += new_sum
                    stats[1] += act.size(0)
            return hook

        for mapping in self._resolved:
            if mapping.parent not in self._parent_args_cache:
                self._parent_args_cache[mapping.parent] = []
                self.register_hook(mapping.parent, cache_parent_kwargs, "forward_pre", with_kwargs=True)
            self.register_hook(mapping.balance_layers[0], make_stats_hook(mapping.smooth_name), "forward")

    # ---- smoothing ----------------------------------------------------------------------------
    @torch.no_grad()
    def _run_samples(self, module) -> list:
        outs = [module(**batch) for batch in self._parent_args_cache[module]]
        return [o[0] if isinstance(o, tuple) else o for o in outs]

    @torch.no_grad()
    def _apply_smoothing(self, model) -> None:
        todo = [m for m in self._resolved if m.smooth_name in self._smooth_activation_stats]
        for mapping in todo:
            with HooksMixin.disable_hooks():
                fp16_outputs = self._run_samples(mapping.parent)
                if not fp16_outputs or all(f.numel() == 0 for f in fp16_outputs):
                    del self._smooth_activation_stats[mapping.smooth_name]
                    continue
                if not all(bool(f.isfinite().all()) for f in fp16_outputs):
                    warnings.warn(f"Skipping smooth_layer {mapping.smooth_name}, NaN or inf outputs found during "
                                  f"forward pass of the parent module {mapping.parent_name}.")
                    del self._smooth_activation_stats[mapping.smooth_name]
                    continue
                originals = {layer: layer.weight.data.clone() for layer in mapping.balance_layers}
                best = self._compute_best_scale(mapping, fp16_outputs, originals)
                for layer in mapping.balance_layers:
                    layer.weight.data.copy_(originals[layer] * best.view(1, -1))
                smooth = mapping.smooth_layer
                if smooth.weight.ndim == 1:
                    smooth.weight.data.div_(best)
                else:
                    # the last rows, as wide as the scales, are the ones that feed the balance layers
                    # (a fused qkv projection smoothing o_proj; base.py:570-578)
                    smooth.weight.data[-best.size(0):].div_(best.view(-1, 1))
                if getattr(smooth, "bias", None) is not None:
                    smooth.bias.data.div_(best)
                del self._smooth_activation_stats[mapping.smooth_name]
            # the parent's cached arguments go once its last mapping has been smoothed
            if not any(m.parent is mapping.parent and m.smooth_name in self._smooth_activation_stats
                       for m in self._resolved):
                self._parent_args_cache.pop(mapping.parent, None)
        self._assert_all_activations_consumed()

    def _compute_loss(self, fp16_outputs, int_w_outputs) -> float:
        loss = torch.zeros((), device=fp16_outputs[0].device)
        n = 0
        for a, b in zip(fp16_outputs, int_w_outputs):
            loss += torch.nn.functional.mse_loss(a, b, reduction="sum")
            n += a.numel()
        if bdist.is_distributed():
            import torch.distributed as dist
            pack = torch.stack([loss, torch.tensor(float(n), device=loss.device)])
            dist.all_reduce(pack)
            return float(pack[0] / pack[1])
        return float(loss / n)

    def _compute_best_scale(self, mapping, fp16_outputs, originals) -> torch.Tensor:
        """Grid search over the smoothing ratio for one mapping (base.py:607-763)."""
        device = fp16_outputs[0].device
        x_sum, count = self._smooth_activation_stats[mapping.smooth_name]
        if bdist.is_distributed():
            import torch.distributed as dist
            pack = torch.cat([x_sum, torch.tensor([float(count)], device=x_sum.device)])
            dist.all_reduce(pack)
            x_sum, count = pack[:-1], float(pack[-1])
        x_mean = (x_sum / count).to(device)
        w_mean = compute_layer_means(mapping.balance_layers).to(device) if self.duo_scaling else None
        layers = [layer for layer in mapping.balance_layers
                  if getattr(getattr(layer, "quantization_scheme", None), "weights", None) is not None]
        weights = [originals[layer] for layer in layers]
        best_error, best_ratio, best_scales, initial, history = float("inf"), -1, None, None, []
        for ratio, duo in grid_search_params(self.duo_scaling, self.n_grid):
            scales = candidate_scales(x_mean, w_mean, ratio, duo)
            for layer, wq in zip(layers, scaled_fake_quantize(weights, scales, layers, mapping.parent)):
                layer.weight.data = wq
            loss = self._compute_loss(fp16_outputs, self._run_samples(mapping.parent))
            if initial is None:
                initial = loss
            history.append({"ratio": ratio, "duo_scaling": duo, "error": loss})
            if loss < best_error:
                best_error, best_ratio, best_scales = loss, ratio, scales.clone()
        for layer in layers:
            layer.weight.data = originals[layer]
        if best_ratio == -1:
            raise Exception("No finite loss was found in best scalesgrid search. This typically means NaN values "
                            "are appearing in the forward pass of the parent module.")
        self.error_metrics.append({"layer_name": mapping.smooth_name, "parent_name": mapping.parent_name,
                                   "initial_error": initial, "best_error": best_error, "best_ratio": best_ratio,
                                   "reduction": best_error / initial if initial > 0 else 1.0,
                                   "history": history})
        assert int(torch.isnan(best_scales).sum()) == 0, f"Nan found in scales: {best_scales}"
        return best_scales

    def _assert_all_activations_consumed(self):
        if self._smooth_activation_stats:
            raise RuntimeError("Some cached activations were not used")
