"""``GPTQModifier`` and ``QuantizationModifier`` with the reference's fields, lifecycle hooks
and error behaviour, running on the b200q kernels.

Mirrors src/llmcompressor/modifiers/gptq/base.py:47-400,
src/llmcompressor/modifiers/quantization/quantization/{base.py:24-110,mixin.py:56-440},
src/llmcompressor/modifiers/quantization/calibration.py:36-162 and the hook helper
src/llmcompressor/modifiers/utils/hooks.py:19-110.  Only weight quantisation is on this
package's path: schemes that also name input activations keep that information for the
checkpoint format, nothing is calibrated for it.
"""
from __future__ import annotations

import collections
import contextlib
import re
import time
import warnings
from typing import Any, Iterable, Optional

import torch

from . import dist as bdist
from . import gptq
from ._lib import B200QError
from .observers import Observer, fuse_weight_observers
from .streams import run_concurrent
from .quant_args import (PRESET_SCHEMES, QuantizationArgs, QuantizationScheme,
                         preset_name_to_scheme)

__all__ = ["GPTQModifier", "QuantizationModifier", "match_named_modules", "HooksMixin"]

_STATIC = "static"
_UNSET = object()


# ------------------------------------------------------------------------------------------
# module matching (compressed-tensors utils/match.py:34-70,344-456)
def _match_one(name: str, module: torch.nn.Module, target: str) -> bool:
    if target.startswith("re:"):
        return re.match(target[3:], name) is not None
    if name == target:
        return True
    return any(cls.__name__ == target for cls in type(module).__mro__)


def match_named_modules(model: torch.nn.Module, targets: Iterable[str], ignore: Iterable[str] = ()):
    """(name, module) pairs selected by ``targets`` and not by ``ignore``, in
    ``model.named_modules()`` order.  A target selects a module if it equals its name, if a
    ``re:`` target matches the name from its start, or if it names a class in the module's MRO."""
    targets, ignore = list(targets or []), list(ignore or [])
    out = []
    for name, module in model.named_modules():
        if not any(_match_one(name, module, t) for t in targets):
            continue
        if any(_match_one(name, module, t) for t in ignore):
            continue
        out.append((name, module))
    return out


# ------------------------------------------------------------------------------------------
class HooksMixin:
    """Forward hooks that can be switched off globally (hooks.py:54-66)."""

    _HOOKS_DISABLED = False

    def __init__(self):
        self._hooks: list = []

    @classmethod
    @contextlib.contextmanager
    def disable_hooks(cls):
        prev = HooksMixin._HOOKS_DISABLED
        HooksMixin._HOOKS_DISABLED = True
        try:
            yield
        finally:
            HooksMixin._HOOKS_DISABLED = prev

    def register_hook(self, module: torch.nn.Module, fn, kind: str = "forward", with_kwargs: bool = False):
        def wrapped(*a, **k):
            if HooksMixin._HOOKS_DISABLED:
                return None
            return fn(*a, **k)
        register = getattr(module, f"register_{kind}_hook")
        handle = register(wrapped, with_kwargs=True) if with_kwargs else register(wrapped)
        self._hooks.append(handle)
        return handle

    def remove_hooks(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []


# ------------------------------------------------------------------------------------------
class QuantizationMixin(HooksMixin):
    """Scheme resolution, qparam attachment and observer life cycle (mixin.py:56-440)."""

    def __init__(self, config_groups=None, targets="Linear", ignore=None, scheme=None,
                 kv_cache_scheme=None, weight_observer=None, input_observer=None,
                 output_observer=None, observer=None, bypass_divisibility_checks=False):
        HooksMixin.__init__(self)
        self.config_groups = config_groups
        self.targets = [targets] if isinstance(targets, str) else list(targets)
        self.ignore = list(ignore or [])
        self.scheme = scheme
        self.kv_cache_scheme = None if kv_cache_scheme is None else QuantizationArgs.of(kv_cache_scheme)
        self.weight_observer = weight_observer
        self.input_observer = input_observer
        self.output_observer = output_observer
        self.observer = observer
        self.bypass_divisibility_checks = bypass_divisibility_checks
        if self.kv_cache_scheme is not None:
            kv = self.kv_cache_scheme
            if kv.strategy != "tensor" or kv.dynamic is not False:
                raise NotImplementedError("kv-cache scales are calibrated per tensor and statically "
                                          f"(got strategy {kv.strategy!r}, dynamic {kv.dynamic!r})")
        self._resolved: Optional[dict] = None
        self._module_names: dict = {}
        self._attention_names: dict = {}   # attention modules that carry kv-cache scales

    def recipe_args(self) -> dict:
        """Constructor arguments for ``recipe.yaml`` (unset ones are left out by the writer)."""
        args = dict(config_groups=self.config_groups, targets=self.targets, ignore=self.ignore, scheme=self.scheme,
                    kv_cache_scheme=None if self.kv_cache_scheme is None else _plain_args(self.kv_cache_scheme),
                    weight_observer=self.weight_observer,
                    input_observer=self.input_observer, output_observer=self.output_observer,
                    observer=self.observer,
                    bypass_divisibility_checks=self.bypass_divisibility_checks or None)
        if isinstance(args["config_groups"], dict):
            args["config_groups"] = {k: (_plain_scheme(v)) for k, v in args["config_groups"].items()}
        return args

    # ---- scheme resolution ---------------------------------------------------------------
    def _apply_observer_overrides(self, scheme: QuantizationScheme) -> QuantizationScheme:
        has_individual = any(o is not None for o in (self.weight_observer, self.input_observer,
                                                     self.output_observer))
        if has_individual and self.observer is not None:
            raise ValueError(
                "Cannot specify both individual observer parameters (weight_observer, "
                "input_observer, output_observer) and observer dict. "
                "Please use either individual parameters or the observer dict.")
        weight_obs = self.weight_observer
        if self.observer is not None:
            weight_obs = self.observer.get("weights", weight_obs)
        if weight_obs is not None and scheme.weights is not None:
            scheme.weights = scheme.weights.model_copy(update={"observer": weight_obs})
        return scheme

    def resolve_quantization_config(self) -> dict:
        """``{"group_i": QuantizationScheme}`` (mixin.py:335-386)."""
        scheme, config_groups = self.scheme, self.config_groups
        if scheme is not None and config_groups is not None:
            raise ValueError("Please specify either `scheme` or `config_groups`")
        groups = {}
        if scheme is not None:
            if isinstance(scheme, str):
                scheme = {scheme: self.targets}
            for idx, (key, tg) in enumerate(scheme.items()):
                if key.upper() not in PRESET_SCHEMES:
                    raise ValueError(f"Unknown preset scheme {key}")
                tg = [tg] if isinstance(tg, str) else list(tg)
                groups[f"group_{idx}"] = self._apply_observer_overrides(preset_name_to_scheme(key, tg))
        elif config_groups:
            for name, g in config_groups.items():
                if isinstance(g, dict):
                    w = g.get("weights")
                    g = QuantizationScheme(targets=list(g.get("targets", self.targets)),
                                           weights=None if w is None else QuantizationArgs.of(w),
                                           input_activations=g.get("input_activations"))
                elif not isinstance(g, QuantizationScheme):
                    g = QuantizationScheme(targets=list(g.targets),
                                           weights=None if g.weights is None else QuantizationArgs.of(g.weights),
                                           input_activations=getattr(g, "input_activations", None))
                groups[name] = self._apply_observer_overrides(g)
        else:
            groups["group_0"] = self._apply_observer_overrides(
                QuantizationScheme(targets=list(self.targets), weights=QuantizationArgs(num_bits=8)))
        return groups

    # ---- attach / detach -------------------------------------------------------------------
    def initialize_quantization(self, model: torch.nn.Module) -> None:
        """Attach ``quantization_scheme`` and empty scale / zero-point (/ global scale / g_idx)
        parameters to every targeted module (CT lifecycle/initialize.py:132-254)."""
        groups = self.resolve_quantization_config()
        self._resolved = groups
        bad = []
        for scheme in groups.values():
            for name, module in match_named_modules(model, scheme.targets, self.ignore):
                if not hasattr(module, "weight") or module.weight is None or module.weight.ndim != 2:
                    continue
                if isinstance(module, torch.nn.Embedding):
                    continue
                w = scheme.weights
                if w is None:
                    continue
                N, K = module.weight.shape
                if (w.strategy in ("group", "tensor_group") and K >= w.group_size and K % w.group_size
                        and not self.bypass_divisibility_checks):
                    bad.append((name, K, w.group_size))
                    continue
                module.quantization_scheme = scheme
                module.quantization_status = "initialized"   # "frozen" once its qparams are written
                self._module_names[module] = name
                dev, dt = module.weight.device, module.weight.dtype
                shape = w.qparam_shape(N, K)

                def reg(pname, t):
                    module.register_parameter(pname, torch.nn.Parameter(t, requires_grad=False))
                if w.strategy == "tensor_group":
                    reg("weight_global_scale", torch.empty(1, dtype=torch.float32, device=dev))
                reg("weight_scale", torch.empty(shape, dtype=dt if dt.is_floating_point else torch.float16,
                                                device=dev))
                reg("weight_zero_point", torch.zeros(shape, dtype=w.zp_dtype, device=dev))
                if w.actorder == "group":
                    reg("weight_g_idx", torch.full((K,), -1, dtype=torch.int32, device=dev))
                a = scheme.input_activations
                if a is not None and a.dynamic is not True:
                    # statically calibrated input activations (CT lifecycle/initialize.py:164-254):
                    # a per-tensor scale / zero point, or (dynamic "local") only the global scale
                    if a.strategy == "tensor_group":
                        reg("input_global_scale", torch.empty(1, dtype=torch.float32, device=dev))
                    if a.dynamic is False:
                        if a.strategy != "tensor":
                            raise NotImplementedError("static input activations are supported per tensor")
                        reg("input_scale", torch.empty(1, dtype=dt if dt.is_floating_point else torch.float16,
                                                       device=dev))
                        reg("input_zero_point", torch.zeros(1, dtype=a.zp_dtype, device=dev))
        if self.kv_cache_scheme is not None:
            # attention modules get k_scale / v_scale (CT lifecycle/initialize.py:255-310); the scheme
            # sits on the module as its input_activations, as the reference's config resolution puts it
            kv = self.kv_cache_scheme
            attn = match_named_modules(model, KV_CACHE_TARGETS, self.ignore)
            if not attn:
                raise ValueError(f"kv_cache_scheme given but no module matches {KV_CACHE_TARGETS}")
            for name, module in attn:
                first = next(module.parameters(), None)
                if first is None:
                    raise ValueError(f"attention module {name} has no parameters to take device and dtype from")
                module.quantization_scheme = QuantizationScheme(targets=list(KV_CACHE_TARGETS), weights=None,
                                                                input_activations=kv)
                module.quantization_status = "initialized"
                self._attention_names[module] = name
                dt = first.dtype if first.dtype.is_floating_point else torch.float16
                for base in ("k", "v"):
                    module.register_parameter(f"{base}_scale", torch.nn.Parameter(
                        torch.empty(1, dtype=dt, device=first.device), requires_grad=False))
                    if not kv.symmetric:
                        module.register_parameter(f"{base}_zero_point", torch.nn.Parameter(
                            torch.zeros(1, dtype=kv.zp_dtype, device=first.device), requires_grad=False))
        if bad:
            lines = "\n".join(f"  {n}: columns {k} not divisible by group_size {g}" for n, k, g in bad)
            raise ValueError(
                "The following layers have weight column counts that are not divisible by the "
                f"quantization group size:\n{lines}\nAdd them to `ignore` or set "
                "bypass_divisibility_checks=True")

    def quantized_modules(self, model: torch.nn.Module):
        return [(n, m) for n, m in model.named_modules() if hasattr(m, "quantization_scheme")
                and m in self._module_names]

    def start_calibration(self, model: torch.nn.Module) -> None:
        for _, module in self.quantized_modules(model):
            w = module.quantization_scheme.weights
            module.weight_observer = Observer.load_from_registry(
                w.observer or "memoryless_minmax", base_name="weight", args=w)
            a = module.quantization_scheme.input_activations
            if a is not None and a.dynamic is not True:
                name = a.observer if a.observer not in (None, "memoryless_minmax") else "minmax"
                module.input_observer = Observer.load_from_registry(name, base_name="input", args=a)
                self.register_hook(module, _calibrate_input_hook, "forward_pre")
        for module in self._attention_names:
            a = module.quantization_scheme.input_activations
            name = a.observer if a.observer not in (None, "memoryless_minmax") else "minmax"
            module.k_observer = Observer.load_from_registry(name, base_name="k", args=a)
            module.v_observer = Observer.load_from_registry(name, base_name="v", args=a)
            self.register_hook(module, _observing_cache_hook, "forward_pre", with_kwargs=True)
        fuse_weight_observers(model)

    @property
    def calibrates_activations(self) -> bool:
        """True when some resolved scheme has statically calibrated input activations."""
        groups = self._resolved if self._resolved is not None else self.resolve_quantization_config()
        return self.kv_cache_scheme is not None or any(
            s.input_activations is not None and s.input_activations.dynamic is not True for s in groups.values())

    def update_activation_qparams(self, modules) -> None:
        """Epoch end for activation observers: combine the ranks' statistics, then write
        ``input_scale`` / ``input_zero_point`` / ``input_global_scale``
        (quantization/base.py:83-108, calibration.py:109-162)."""
        modules = list(modules)
        pending = []
        seen = []
        for base in ("input", "k", "v"):
            mods = [m for m in modules if getattr(m, f"{base}_observer", None) is not None
                    and getattr(m, f"{base}_observer").has_statistics]
            if mods and bdist.is_distributed():
                for m in mods:
                    pending.extend(getattr(m, f"{base}_observer").sync_activation_stats())
            seen.append((base, mods))
        bdist.wait_for_comms(pending)
        for base, mods in seen:
            update_qparams(mods, base)
            if base == "v":
                for m in mods:
                    m.quantization_status = "frozen"

    def end_calibration(self, model: torch.nn.Module) -> None:
        self.remove_hooks()
        for module in [m for _, m in self.quantized_modules(model)] + list(self._attention_names):
            for name in ("weight_observer", "input_observer", "k_observer", "v_observer"):
                if hasattr(module, name):
                    delattr(module, name)


KV_CACHE_TARGETS = ("re:.*self_attn$",)   # the reference's match for attention modules (mixin.py:216-218)


class _ObservingCache:
    """Stands in for ``past_key_values`` during a calibration forward of an attention module: the
    attention calls ``update(key_states, value_states, layer_idx, ...)`` with the post-rotary keys
    and the values, [batch, kv_heads, tokens, head_dim], which are what a cache would store.  They
    go to the module's k / v observers and on to the cache that was passed in, if any
    (compressed-tensors modeling/kvcache.py:29-84, calibration.py:187-196)."""

    def __init__(self, module, inner):
        self.module, self.inner = module, inner

    def update(self, key_states, value_states, *args, **kwargs):
        self.module.k_observer(key_states)
        self.module.v_observer(value_states)
        if self.inner is not None:
            return self.inner.update(key_states, value_states, *args, **kwargs)
        return key_states, value_states

    def __getattr__(self, name):   # anything else an attention implementation asks of a cache
        inner = self.__dict__.get("inner")
        if inner is None:
            raise AttributeError(name)
        return getattr(inner, name)


def _observing_cache_hook(module, args, kwargs):
    import inspect
    name = "past_key_values" if "past_key_values" in inspect.signature(module.forward).parameters \
        else "past_key_value"
    kwargs[name] = _ObservingCache(module, kwargs.get(name))
    return args, kwargs


def _calibrate_input_hook(module, args):
    """calibration.py:165-170: the input observer sees every calibration batch."""
    module.input_observer(args[0] if isinstance(args, tuple) else args)


def observe(modules: Iterable[torch.nn.Module], base_name: str = "weight") -> None:
    for m in modules:
        obs = getattr(m, f"{base_name}_observer", None)
        if obs is not None:
            obs(m.weight.data)


def update_qparams(modules: Iterable[torch.nn.Module], base_name: str = "weight") -> None:
    """Copy the observer's scale / zero point / global scale into the module's parameters
    (calibration.py:109-162)."""
    for m in modules:
        obs = getattr(m, f"{base_name}_observer", None)
        if obs is None:
            continue
        if not obs.has_statistics:
            warnings.warn(f"Observer of {type(m).__name__} has no statistics; qparams not updated")
            continue
        qp = obs.get_qparams()
        if hasattr(m, f"{base_name}_scale"):    # absent for locally dynamic activations (global scale only)
            getattr(m, f"{base_name}_scale").data.copy_(qp["scale"].reshape(getattr(m, f"{base_name}_scale").shape))
            if hasattr(m, f"{base_name}_zero_point"):   # symmetric kv-cache scales carry none
                getattr(m, f"{base_name}_zero_point").data.copy_(qp["zero_point"].reshape(
                    getattr(m, f"{base_name}_zero_point").shape))
        if qp["global_scale"] is not None and hasattr(m, f"{base_name}_global_scale"):
            getattr(m, f"{base_name}_global_scale").data.copy_(qp["global_scale"])
        if base_name == "weight":
            m.quantization_status = "frozen"


# ------------------------------------------------------------------------------------------
class QuantizationModifier(QuantizationMixin):
    """Round-to-nearest weight quantisation: observe weights, write qparams; the weight is
    left as is until it is packed at save time (quantization/base.py:24-110)."""

    @property
    def requires_calibration_data(self) -> bool:
        return self.calibrates_activations

    def on_initialize(self, model, **_):
        self.initialize_quantization(model)
        return True

    def on_calibration_start(self, model, **_):
        self.start_calibration(model)

    def on_sequential_epoch_end(self, model, modules: Iterable[torch.nn.Module], **_):
        modules = list(modules)
        self.update_activation_qparams(modules)
        modules = [m for m in modules if hasattr(m, "weight_observer")
                   and getattr(m, "quantization_status", None) != "frozen"]
        if bdist.is_distributed():
            # owners by weight size; each rank observes its share, scales are broadcast
            items, rank_to, to_rank = bdist.greedy_bin_packing(
                list(modules), bdist.world_size(), item_weight_fn=lambda m: m.weight.numel())
            mine = rank_to[bdist.rank()]
            observe(mine)
            update_qparams(mine)
            bdist.broadcast_module_params(items, to_rank,
                                          ("weight_scale", "weight_zero_point", "weight_global_scale"))
            for m in items:
                m.quantization_status = "frozen"
        else:
            observe(modules)
            update_qparams(modules)

    def pending_modules(self):
        """Targeted modules whose parameters have not been written yet (modules behind the
        sequential blocks)."""
        return [m for m in self._module_names if hasattr(m, "weight_observer")
                and getattr(m, "quantization_status", None) != "frozen"]

    def on_calibration_end(self, model, **_):
        self.end_calibration(model)

    def on_finalize(self, model, **_):
        return True


class GPTQModifier(QuantizationMixin):
    """GPTQ weight quantisation (gptq/base.py:47-400).

    Forward hooks accumulate H += 2 X^T X per calibration batch; at the end of each sequential
    epoch the modules of that epoch are observed and quantised column block by column block.
    Modules that receive the very same input tensor (q/k/v, gate/up, experts under all-expert
    calibration) share one Hessian accumulation and one factorisation; set
    ``share_hessians=False`` to keep one per module like the reference.  The solves of different
    Hessians run concurrently on up to ``parallel_streams`` CUDA streams (1: one after another
    on the current stream, like the reference).  Calibration batches smaller than
    ``hessian_stage_tokens`` tokens are gathered and added to the Hessian together (0: one kernel
    call per batch).  When an epoch holds ``batch_small_hessians`` or more Hessians of one width of
    at most ``small_hessian_columns`` columns (the experts of a mixture-of-experts layer), their
    factorisations and sweeps run as batched launches, one thread block per problem, instead of
    dozens of launches per module (0 switches this off).
    """

    requires_calibration_data = True

    def __init__(self, block_size: int = 128, dampening_frac: Optional[float] = 0.01,
                 actorder: Any = _UNSET, offload_hessians: bool = False, share_hessians: bool = True,
                 parallel_streams: int = 4, hessian_stage_tokens: int = 32768,
                 batch_small_hessians: int = 16, small_hessian_columns: int = 2048, **quant_kwargs):
        kw = dict(quant_kwargs)
        kw.setdefault("targets", "Linear")
        super().__init__(**kw)
        self.block_size = block_size
        self.dampening_frac = dampening_frac
        self.actorder = actorder
        self.offload_hessians = offload_hessians
        self.share_hessians = share_hessians
        self.parallel_streams = parallel_streams
        self.hessian_stage_tokens = hessian_stage_tokens
        self.batch_small_hessians = batch_small_hessians
        self.small_hessian_columns = small_hessian_columns
        self._groups: dict = {}        # module -> _HessianGroup
        self._num_samples: dict = {}   # module -> None (membership: modules awaiting compression)
        self.trace = None              # optional callback(event: str, module | None) for instrumentation
        self._hooked: list = []        # every module that got a calibration hook
        self._done: set = set()        # modules whose quantised weight has been written
        self.losses: dict = {}

    def recipe_args(self) -> dict:
        args = super().recipe_args()
        args.update(block_size=self.block_size, dampening_frac=self.dampening_frac,
                    offload_hessians=self.offload_hessians or None)
        if self.actorder is not _UNSET:
            args["actorder"] = self.actorder   # None is dropped by the writer, as the reference drops it
        return args

    # ---- config ------------------------------------------------------------------------------
    def resolve_quantization_config(self) -> dict:
        groups = super().resolve_quantization_config()

        def resolve(existing):
            if self.actorder is _UNSET:  # sentinel default only fills an unset scheme value
                return "weight" if existing is None else existing
            mine = QuantizationArgs(num_bits=4, group_size=128, actorder=self.actorder).actorder \
                if self.actorder not in (None, False) else None
            if existing is None or mine == existing:
                return mine
            raise ValueError(
                "Cannot resolve activation ordering when both `GPTQModifier.actorder` and "
                f"`QuantizationScheme.actorder` are provided and differ ({self.actorder}, {existing}). "
                "Either unset `GPTQModifier.actorder` or remove `actorder` from config groups.")

        for scheme in groups.values():
            w = scheme.weights
            if w is None:
                continue
            # the modifier-level setting is applied to every strategy, as the reference does by
            # assigning past the argument validation (base.py:176-192): "weight"/"static" then
            # permutes the sweep of channel / tensor / block schemes too
            a = resolve(w.actorder)
            if a == "group" and w.strategy not in ("group", "tensor_group"):
                warnings.warn(f"ActivationOrdering.GROUP is not compatible with strategy={w.strategy}; "
                              "falling back to actorder=None for this scheme.")
                a = None
            scheme.weights = _with_actorder(w, a)
        return groups

    # ---- lifecycle -----------------------------------------------------------------------------
    def on_initialize(self, model, **_):
        self.initialize_quantization(model)
        return True

    def on_calibration_start(self, model, **_):
        self.start_calibration(model)
        self._hooked, self._done = [], set()   # a fresh calibration
        added = False
        for _, module in self.quantized_modules(model):
            if isinstance(module, torch.nn.Embedding):
                continue
            if getattr(module, "quantization_scheme", None) is None or module.quantization_scheme.weights is None:
                continue
            self.register_hook(module, self.calibrate_module, "forward")
            self._hooked.append(module)
            added = True
        if not added:
            raise ValueError(
                "GPTQModifier requires a weight quantization config be specified by this modifier or a "
                "modifier preceding it")

    def pending_modules(self):
        """Hooked modules that have not been compressed yet."""
        return [m for m in self._hooked if m not in self._done]

    def calibrate_module(self, module, args, _output):
        if module in self._done:
            return
        inp = args[0]
        group = self._groups.get(module)
        if group is None:
            group = self._find_shared(inp) if self.share_hessians else None
            if group is None:
                group = _HessianGroup(module, offload=self.offload_hessians, stage_tokens=self.hessian_stage_tokens)
            else:
                group.members.append(module)
            self._groups[module] = group
            self._num_samples[module] = None
        elif module is not group.members[0] and not group.same_input(inp):
            # membership was decided on the first batch; the first member adds every batch and
            # the others must keep receiving that very tensor
            raise RuntimeError(
                f"{self._module_names.get(module, type(module).__name__)} shared a Hessian with "
                f"{self._module_names.get(group.members[0], type(group.members[0]).__name__)} because both received "
                "the same input on the first calibration batch, but its input differs on a later batch; "
                "set GPTQModifier(share_hessians=False)")
        group.accumulate(inp)

    def _find_shared(self, inp):
        for g in {id(g): g for g in self._groups.values()}.values():
            if g.same_input(inp):
                return g
        return None

    def on_sequential_epoch_end(self, model, modules: Iterable[torch.nn.Module], **_):
        modules = list(modules)
        self.update_activation_qparams(modules)
        mods = [m for m in modules if m in self._num_samples]
        # the weight observers are called by the solves themselves (gptq._sweep_input), on the rank
        # and stream that quantises the module, next to the rest of its work
        self.compress_modules(mods)

    def _trace(self, event, module=None):
        if self.trace is not None:
            self.trace(event, module)

    def compress_modules(self, modules=None):
        modules = list(self._num_samples.keys()) if modules is None else list(modules)
        if not bdist.is_distributed():
            self._trace("solve")
            self.compress_module_list(modules)
            self._trace("done")
            return
        # owners by Hessian width over the distinct Hessians (base.py:306-318).  A Hessian shared by
        # many modules (the gate / up projections of every expert under all-expert calibration)
        # would make its owner sweep all of them alone: such a Hessian is summed onto every rank
        # instead, every rank factors it, and its modules are dealt out round robin.
        world = bdist.world_size()
        groups = list({id(self._groups[m]): self._groups[m] for m in modules}.values())
        members = {id(g): [m for m in modules if self._groups[m] is g] for g in groups}
        spread = [g for g in groups if len(members[id(g)]) >= 2 * world]
        owned = [g for g in groups if len(members[id(g)]) < 2 * world]
        items, rank_to, to_rank = bdist.greedy_bin_packing(owned, world, item_weight_fn=lambda g: g.H.shape[0])
        for g in spread:
            to_rank[g] = None
        items = items + spread
        for g in items:
            g.flush()   # staged calibration tokens
        self._trace("reduce")
        bdist.reduce_hessians(items, to_rank)
        mod_rank = {}    # before the solve drops the groups
        for g in items:
            for i, m in enumerate(members[id(g)]):
                mod_rank[m] = to_rank[g] if to_rank[g] is not None else i % world
        mine = [m for m in modules if mod_rank[m] == bdist.rank()]
        self._trace("solve")
        self.compress_module_list(mine)
        self._trace("broadcast")
        bdist.broadcast_module_params(modules, mod_rank, ("weight", "weight_scale", "weight_zero_point",
                                                          "weight_g_idx", "weight_global_scale"))
        for m in modules:
            self._num_samples.pop(m, None)
            self._groups.pop(m, None)
            m.quantization_status = "frozen"
            self._done.add(m)
        self._trace("done")

    def compress_module_list(self, module_list):
        """Quantise the modules; the modules of one Hessian form a job (one factorisation per
        act-order setting, then their sweeps) and jobs run concurrently on side streams."""
        by_group: dict = {}
        for module in module_list:
            by_group.setdefault(id(self._groups[module]), []).append(module)
        jobs = sorted(by_group.values(), key=lambda mods: -mods[0].weight.shape[1])
        if not jobs:
            return
        device = jobs[0][0].weight.device
        if self.batch_small_hessians and self.block_size == 128:
            # small problems that come in numbers: many Hessians of one width, or one Hessian
            # shared by many modules (the gate / up projections under all-expert calibration)
            width = collections.Counter()
            for mods in jobs:
                width[mods[0].weight.shape[1]] += len(mods)
            small = [mods for mods in jobs if mods[0].weight.shape[1] <= self.small_hessian_columns
                     and width[mods[0].weight.shape[1]] >= self.batch_small_hessians]
            if small:
                taken = {id(mods) for mods in small}
                jobs = [mods for mods in jobs if id(mods) not in taken]
                self._compress_small_jobs(small)
        if jobs:
            run_concurrent([lambda mods=mods: self._compress_group(mods) for mods in jobs], device,
                           max_streams=self.parallel_streams)

    def _queue_factors(self, module_list, make_factor):
        """Take the modules of one Hessian out of the pending tables and give each the factor of its
        act-order setting, made by ``make_factor(H, actorder)`` once per distinct setting.
        Returns ([(module, qargs, factor)], the Hessian's device status word or None)."""
        factors = {}
        left = {module.quantization_scheme.weights.actorder for module in module_list}
        taken, status = [], None
        for module in module_list:
            group = self._groups.pop(module)
            status = group.status
            self._num_samples.pop(module, None)
            qargs = module.quantization_scheme.weights
            if qargs.actorder not in factors:
                left.discard(qargs.actorder)
                H = group.finalized(keep=bool(left))  # the factorisation consumes its argument
                factors[qargs.actorder] = make_factor(H, qargs.actorder)
                self._trace("job_factored", module)
            taken.append((module, qargs, factors[qargs.actorder]))
        return taken, status

    @staticmethod
    def _check_status_words(words):
        words = [w for w in words if w is not None]
        if words and int(torch.cat([w.reshape(-1)[:1] for w in words]).abs().amax().item()) != 0:
            raise B200QError("a bounded wait inside the Hessian or GEMM kernels of this job expired; "
                             "its results are incomplete")

    def _finish_queued(self, queued, t0):
        """``queued``: [(module, qargs, factor, loss, out)] of deferred solves whose factors have been
        resolved.  Redo the modules whose Hessian was not positive definite with the identity, as
        the reference falls back (gptq_quantize.py:157-164), then write every result to its module."""
        redo = [q for q in queued if not q[2].ok]
        # the deferred call consumed the observers' statistics: observe again before the
        # round-to-nearest redo (act-order "group" re-observes the permuted weight itself)
        for module, qargs, *_ in redo:
            if qargs.actorder != "group":
                module.weight_observer.delete_statistics(check_fused=False)
        for module, qargs, *_ in redo:
            if qargs.actorder != "group":
                module.weight_observer(module.weight.data)
        results = []
        for module, qargs, factor, loss, out in queued:
            if not factor.ok:
                with torch.no_grad():
                    loss, out = gptq.quantize_weight(module, qargs, None, blocksize=self.block_size,
                                                     percdamp=self.dampening_frac, factor=factor)
            results.append((module, loss, out))
        # one read for all the losses that are still on the device
        on_device = [i for i, (_, loss, _) in enumerate(results) if isinstance(loss, torch.Tensor)]
        if on_device:
            values = torch.stack([results[i][1].reshape(()) for i in on_device]).tolist()
            for i, v in zip(on_device, values):
                results[i] = (results[i][0], v, results[i][2])
        # the weights go back in one multi-tensor copy
        if results:
            torch._foreach_copy_([module.weight.data for module, _, _ in results],
                                 [out["weight"] for _, _, out in results])
        for module, loss, out in results:
            loss = float(loss)
            name = self._module_names.get(module, type(module).__name__)
            self.losses[name] = loss
            self._log_metric(name, time.perf_counter() - t0, loss)
            for attr, val in out.items():
                if attr == "weight":
                    continue
                elif hasattr(module, attr):
                    p = getattr(module, attr)
                    val = val.reshape(p.shape)
                    if val.dtype == p.dtype and val.device == p.device and val.is_contiguous():
                        p.data = val        # a fresh tensor of the solve: no copy into the placeholder
                    else:
                        p.data.copy_(val)
                else:
                    module.register_parameter(attr, torch.nn.Parameter(val, requires_grad=False))
            module.quantization_status = "frozen"
            self._done.add(module)

    def _compress_group(self, module_list):
        """Everything is queued on the current stream without waiting for the device; the
        factorisation status and the losses are read once at the end."""
        t0 = time.perf_counter()
        self._trace("job_start", module_list[0])
        taken, hess_status = self._queue_factors(
            module_list, lambda H, actorder: gptq.factor_hessian(H, self.dampening_frac, actorder, defer=True))
        queued = []
        for module, qargs, factor in taken:
            with torch.no_grad():
                loss, out = gptq.quantize_weight(module, qargs, None, blocksize=self.block_size,
                                                 percdamp=self.dampening_frac, factor=factor, defer=True)
            queued.append((module, qargs, factor, loss, out))
        self._trace("job_swept", module_list[0])
        # one read for every device status word of the job (the first wait for the device)
        self._check_status_words([out.pop("_status", None) for *_, out in queued] + [hess_status])
        gptq.resolve_factors([q[2] for q in queued])
        self._finish_queued(queued, t0)

    def _compress_small_jobs(self, jobs):
        """Many Hessians of few columns: the same steps as ``_compress_group`` for every job, but the
        factorisations of one width and the sweeps of one weight shape and scheme are gathered
        into batched launches (one thread block per problem) on the current stream."""
        t0 = time.perf_counter()
        self._trace("job_start", jobs[0][0])
        requests = []   # (H, actorder, holder): the holder receives the factor once it exists

        def ask(H, actorder):
            holder = []
            requests.append((H, actorder, holder))
            return holder

        taken, words = [], []
        for mods in jobs:
            part, status = self._queue_factors(mods, ask)
            taken += part
            words.append(status)
        by_kind: dict = {}
        for H, actorder, holder in requests:
            by_kind.setdefault((H.shape[0], H.stride(0), actorder), []).append((H, holder))
        for (_, _, actorder), items in by_kind.items():
            if len(items) >= self.batch_small_hessians:
                factors = gptq.factor_hessians_batched([H for H, _ in items], self.dampening_frac, actorder)
            else:   # a few matrices: the tensor-core factorisation, one after another
                factors = [gptq.factor_hessian(H, self.dampening_frac, actorder, defer=True) for H, _ in items]
            for (_, holder), factor in zip(items, factors):
                holder.append(factor)
        del requests, by_kind
        by_shape: dict = {}
        for module, qargs, holder in taken:
            key = (tuple(module.weight.shape), module.weight.dtype, repr(qargs))
            by_shape.setdefault(key, []).append((module, qargs, holder[0]))
        queued = []
        # the class with the most device work first: its sweep runs while the host prepares the others
        classes = sorted(by_shape.values(), key=lambda it: -len(it) * it[0][0].weight.shape[0]
                         * it[0][0].weight.shape[1] ** 2)
        for items in classes:
            with torch.no_grad():
                if len(items) >= 4:
                    done = gptq.quantize_weights_batched([m for m, _, _ in items], items[0][1],
                                                         [f for _, _, f in items], blocksize=self.block_size,
                                                         percdamp=self.dampening_frac)
                else:
                    done = [gptq.quantize_weight(m, q, None, blocksize=self.block_size, percdamp=self.dampening_frac,
                                                 factor=f, defer=True) for m, q, f in items]
                    words += [out.pop("_status", None) for _, out in done]
            queued += [(m, q, f, loss, out) for (m, q, f), (loss, out) in zip(items, done)]
        self._trace("job_swept", jobs[0][0])
        self._check_status_words(words)
        gptq.resolve_factors([q[2] for q in queued])
        self._finish_queued(queued, t0)

    @staticmethod
    def _log_metric(name, seconds, loss):
        # shape of the reference's METRIC lines (src/llmcompressor/utils/metric_logging.py:42-65)
        import logging
        logging.getLogger("llm_compressor_b200").info("METRIC - %s time %.2fs error %.2f", name, seconds, loss)

    def on_calibration_end(self, model, **_):
        self.end_calibration(model)

    def on_finalize(self, model, **_):
        if len(self._num_samples) > 0:
            raise ValueError(f"Failed to compress {len(self._num_samples)} modules")
        missed = self.pending_modules()
        if missed:
            names = ", ".join(self._module_names.get(m, type(m).__name__) for m in missed[:8])
            raise ValueError(f"{len(missed)} targeted modules never received calibration data and were not "
                             f"compressed: {names}{' ...' if len(missed) > 8 else ''}")
        self._groups, self._num_samples, self._hooked = {}, {}, []
        return True


def _plain_args(a: QuantizationArgs) -> dict:
    """QuantizationArgs as plain recipe / config values."""
    out = {}
    for k, v in vars(a).items():
        if v is None or (k == "observer_kwargs" and not v):
            continue
        out[k] = str(v).replace("torch.", "") if isinstance(v, torch.dtype) else v
    return out


def _plain_scheme(g):
    """A config group as plain data for the recipe file."""
    if isinstance(g, dict):
        return {k: (_plain_scheme(v) if isinstance(v, (dict, QuantizationArgs, QuantizationScheme)) else v)
                for k, v in g.items()}
    out = {}
    for k, v in vars(g).items():
        if v is None or v == {} or v is False:
            continue
        if isinstance(v, (QuantizationArgs, QuantizationScheme)):
            v = _plain_scheme(v)
        elif isinstance(v, torch.dtype):
            v = str(v)
        out[k] = v
    return out


def _with_actorder(qargs: QuantizationArgs, actorder):
    a = qargs.model_copy()
    object.__setattr__(a, "actorder", actorder)
    return a


class _HessianGroup:
    """One Hessian shared by the modules that see the same input.

    Small calibration batches are gathered in a bf16 staging buffer and added with one kernel
    call per ``stage_tokens`` tokens: the symmetric rank-k update re-reads and re-writes the lower
    triangle of H on every call and fills the machine in whole waves of 256x256 tiles, so a call
    over 2048 tokens runs at about half the rate of a call over 32768 (K = 4096)."""

    def __init__(self, module, offload=False, stage_tokens: int = 0):
        self.members = [module]
        K = module.weight.shape[1]
        self.device = module.weight.device
        self.H = torch.zeros((K, K), dtype=torch.float32, device=self.device)
        self.n = 0
        self._last = None  # (tensor kept alive, version) of the batch accumulated last
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)   # bounded-wait expiry of any update
        self.offload = offload
        self._final = None
        self.stage_tokens = int(stage_tokens)
        self._stage = None   # [stage_tokens, K] bf16, allocated on first use
        self._fill = 0

    def same_input(self, inp: torch.Tensor) -> bool:
        if self._last is None:
            return False
        t, ver = self._last
        return (t.data_ptr() == inp.data_ptr() and t.shape == inp.shape and t.stride() == inp.stride()
                and t.dtype == inp.dtype and ver == inp._version)

    def _syrk(self, x: torch.Tensor) -> None:
        if self.offload and self.H.device != self.device:
            self.H = self.H.to(self.device)
        gptq.ops.hessian_syrk(x, self.H, alpha=2.0, status=self.status)
        if self.offload:
            self.H = self.H.to("cpu")

    def flush(self) -> None:
        if self._fill:
            self._syrk(self._stage[: self._fill])
            self._fill = 0

    def accumulate(self, inp: torch.Tensor) -> None:
        if self.same_input(inp):
            return  # another member already added this batch
        x, added = gptq._tokens_2d(inp, self.device)
        t = x.shape[0]
        if self.stage_tokens <= 0 or t >= self.stage_tokens:
            self.flush()
            self._syrk(x)
        else:
            if self._stage is None:
                self._stage = torch.empty((self.stage_tokens, x.shape[1]), dtype=torch.bfloat16, device=self.device)
            if self._fill + t > self.stage_tokens:
                self.flush()
            self._stage[self._fill: self._fill + t].copy_(x)
            self._fill += t
        self.n += added
        self._last = (inp, inp._version)

    def finalized(self, keep: bool = False) -> torch.Tensor:
        """Full symmetric H / n.  The caller's factorisation consumes the matrix it gets;
        ``keep`` asks for a copy because another act-order setting still needs H."""
        self._last = None
        if self._final is None:
            self.flush()
            self._stage = None
            H = self.H.to(self.device)
            self.H = None
            self._final = gptq.finalize_hessian(H, self.n)
        out = self._final.clone() if keep else self._final
        if not keep:
            self._final = None
        return out
