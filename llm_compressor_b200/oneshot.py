"""``oneshot`` entry point and the two calibration drivers it needs.

Signature and behaviour follow src/llmcompressor/entrypoints/oneshot.py:316-479.  The
drivers are this package's own, not the reference's fx tracer: the sequential driver walks the
model's decoder layers (the modules named by ``sequential_targets``, default the model's
``_no_split_modules``) in the order of src/llmcompressor/pipelines/sequential/pipeline.py:136-178
(calibration pass with hooks, epoch end, propagation pass without hooks); the data-free driver is
src/llmcompressor/pipelines/data_free/pipeline.py:18-38.  Activations stay in HBM between layers.
"""
from __future__ import annotations

import json
import os
import re
from typing import Optional

import torch

from . import dist as bdist
from .compressors import compress_state_dict, infer_module_format
from .modifiers import HooksMixin

__all__ = ["oneshot", "save_compressed_model"]


class _StopForward(Exception):
    pass


def _as_batches(dataset, num_calibration_samples, max_seq_length, batch_size, device):
    """Normalise the calibration data to a list of keyword dicts on ``device``."""
    if dataset is None:
        return []
    if isinstance(dataset, torch.Tensor):
        rows = [dataset[i] for i in range(dataset.shape[0])]
    else:
        rows = list(dataset)
    samples = []
    for item in rows:
        if isinstance(item, dict):
            d = {k: torch.as_tensor(v) for k, v in item.items()}
        else:
            d = {"input_ids": torch.as_tensor(item)}
        d = {k: (v.unsqueeze(0) if v.ndim == 1 else v) for k, v in d.items()}
        if max_seq_length:
            d = {k: v[..., :max_seq_length] for k, v in d.items()}
        samples.append(d)
    if num_calibration_samples:
        samples = samples[:num_calibration_samples]
    if bdist.is_distributed():
        keep = bdist.partition_samples(len(samples), bdist.rank(), bdist.world_size())
        samples = [samples[i] for i in keep]
    batches = []
    for i in range(0, len(samples), max(1, batch_size)):
        chunk = samples[i:i + batch_size]
        batches.append({k: torch.cat([c[k] for c in chunk], 0).to(device) for k in chunk[0]})
    return batches


def _sequential_layers(model, sequential_targets):
    names = sequential_targets
    if names is None:
        names = list(getattr(model, "_no_split_modules", None) or [])
    if isinstance(names, str):
        names = [names]
    if not names:
        # no hint from the model: take the class of the longest ModuleList of same-class blocks
        # (the decoder stack of the usual architectures)
        best = None
        for _, m in model.named_modules():
            if isinstance(m, torch.nn.ModuleList) and len(m) > 0 and len({type(c) for c in m}) == 1:
                if best is None or len(m) > len(best):
                    best = m
        if best is not None:
            names = [type(best[0]).__name__]
    layers = [(n, m) for n, m in model.named_modules() if type(m).__name__ in names]
    # keep outermost matches only
    out = []
    for n, m in layers:
        if not any(n.startswith(p + ".") for p, _ in out):
            out.append((n, m))
    if not out:
        raise ValueError(f"no module of class {names} found for the sequential pipeline")
    return out


class _PhaseClock:
    """Wall seconds per phase, with a device synchronisation at every boundary (only when asked for)."""

    def __init__(self, sink):
        self.sink = sink
        self.t = None
        if sink is not None and torch.cuda.is_available():
            torch.cuda.synchronize()
        import time
        self._now = time.perf_counter
        self.t = self._now()

    def mark(self, name):
        if self.sink is None:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        now = self._now()
        self.sink[name] = self.sink.get(name, 0.0) + (now - self.t)
        self.t = now


def _tree_map(fn, obj):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, tuple):
        return tuple(_tree_map(fn, o) for o in obj)
    if isinstance(obj, list):
        return [_tree_map(fn, o) for o in obj]
    if isinstance(obj, dict):
        return {k: _tree_map(fn, v) for k, v in obj.items()}
    return obj


class _ActivationStore:
    """The inputs of the current sequential block, one ``(args, kwargs)`` per calibration batch.

    By default everything stays in device memory (a whole calibration set of hidden states is a few
    GB against 180 GB of HBM).  With ``offload`` (a device, e.g. "cpu") tensors of at least 1 MiB
    are parked there between uses - in pinned memory when it is the host - and brought back per
    batch; with ``prefetch`` the next batch is fetched on a copy stream while the current one runs
    (src/llmcompressor/pipelines/cache.py:244-375, pipelines/sequential/pipeline.py:28-47)."""

    _MIN_BYTES = 1 << 20

    def __init__(self, device, offload=None, prefetch: bool = False):
        self.device = torch.device(device)
        self.offload = None if offload is None else torch.device(offload)
        if self.offload is not None and self.offload == self.device:
            self.offload = None
        self.prefetch = bool(prefetch) and self.offload is not None and self.device.type == "cuda"
        self.items: list = []
        self._copy_stream = torch.cuda.Stream(device=self.device) if self.prefetch else None

    def __len__(self):
        return len(self.items)

    def _park(self, t: torch.Tensor) -> torch.Tensor:
        if self.offload is None or t.device != self.device or t.numel() * t.element_size() < self._MIN_BYTES:
            return t
        if self.offload.type == "cpu" and t.is_cuda:
            out = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            out.copy_(t, non_blocking=True)
            return out
        return t.to(self.offload)

    def append(self, value) -> None:
        self.items.append(_tree_map(self._park, value))

    def settle(self) -> None:
        """Wait for the copies of ``append`` (the parked host buffers are read only after this)."""
        if self.offload is not None and self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    def _fetch(self, i: int):
        return _tree_map(lambda t: t.to(self.device, non_blocking=True) if t.device != self.device else t,
                         self.items[i])

    def batches(self, release: bool = False):
        """Yield every batch on the device, in order; ``release`` drops a batch once it has been
        handed out (its block is done with it)."""
        n = len(self.items)
        if not self.prefetch:
            for i in range(n):
                value = self._fetch(i)
                if release:
                    self.items[i] = None
                yield value
            return
        current = torch.cuda.current_stream(self.device)

        def start(i):
            self._copy_stream.wait_stream(current)
            with torch.cuda.stream(self._copy_stream):
                value = self._fetch(i)
            done = torch.cuda.Event()
            done.record(self._copy_stream)
            return value, done

        nxt = start(0) if n else None
        for i in range(n):
            value, done = nxt
            nxt = start(i + 1) if i + 1 < n else None
            current.wait_event(done)
            _tree_map(lambda t: t.record_stream(current) if t.is_cuda else None, value)
            if release:
                self.items[i] = None
            yield value


def _run_sequential(model, modifiers, batches, sequential_targets, phase_times=None, offload_device=None,
                    prefetch: bool = False, propagate_error: bool = True):
    clock = _PhaseClock(phase_times)
    layers = _sequential_layers(model, sequential_targets)
    first = layers[0][1]
    device = next(model.parameters()).device
    store = _ActivationStore(device, offload_device, prefetch)

    def grab(_m, args, kwargs):
        store.append((args, kwargs))
        raise _StopForward()

    handle = first.register_forward_pre_hook(grab, with_kwargs=True)
    use_cache = getattr(getattr(model, "config", None), "use_cache", None)
    if use_cache is not None:
        model.config.use_cache = False
    try:
        with torch.no_grad(), HooksMixin.disable_hooks():
            for b in batches:
                try:
                    model(**b)
                except _StopForward:
                    pass
    finally:
        handle.remove()
        if use_cache is not None:
            model.config.use_cache = use_cache
    store.settle()
    for m in modifiers:
        m.on_calibration_start(model)
    clock.mark("capture")
    for _name, layer in layers:
        nxt = _ActivationStore(device, offload_device, prefetch)
        with torch.no_grad():
            # calibration pass: hooks fire.  Without error propagation its outputs (those of the
            # block before it is quantised) are the next block's inputs and there is no second pass
            for args, kwargs in store.batches(release=not propagate_error):
                out = layer(*args, **kwargs)
                if not propagate_error:
                    nxt.append(_with_hidden(args, kwargs, out[0] if isinstance(out, (tuple, list)) else out))
                del out
        clock.mark("calibrate")
        members = list(layer.modules())
        for m in modifiers:
            m.on_sequential_epoch_end(model, members)
        clock.mark("compress")
        if propagate_error:
            with torch.no_grad(), HooksMixin.disable_hooks():
                # propagation pass with the quantised weights; a batch is released once consumed
                for args, kwargs in store.batches(release=True):
                    out = layer(*args, **kwargs)
                    hidden = out[0] if isinstance(out, (tuple, list)) else out
                    nxt.append(_with_hidden(args, kwargs, hidden))
        nxt.settle()
        store = nxt
        clock.mark("propagate")
    del store
    # targeted modules outside the blocks (an lm_head that is not ignored, a head or adapter behind
    # the stack): one more pass over the whole model, whose blocks now carry their quantised
    # weights, calibrates them; modules that are already done ignore their hooks
    rest = [mod for m in modifiers for mod in getattr(m, "pending_modules", lambda: [])()]
    if rest:
        with torch.no_grad():
            for b in batches:
                model(**b)
        for m in modifiers:
            m.on_sequential_epoch_end(model, rest)
        clock.mark("remainder")
    for m in modifiers:
        m.on_calibration_end(model)


def _with_hidden(args, kwargs, hidden):
    """The next block's call: the previous block's output in place of its hidden states, which
    may have been passed positionally or as the ``hidden_states`` keyword."""
    if args:
        return (hidden,) + tuple(args[1:]), kwargs
    if "hidden_states" in kwargs:
        return (), dict(kwargs, hidden_states=hidden)
    raise ValueError("cannot tell which argument of the sequential block carries the hidden states")


def _run_data_free(model, modifiers):
    for m in modifiers:
        m.on_calibration_start(model)
    members = list(model.modules())
    for m in modifiers:
        m.on_sequential_epoch_end(model, members)
    for m in modifiers:
        m.on_calibration_end(model)


def oneshot(model, recipe=None, dataset=None, num_calibration_samples: int = 512,
            max_seq_length: Optional[int] = None, batch_size: int = 1, pipeline: str = "independent",
            sequential_targets=None, moe_calibrate_all_experts: bool = True,
            output_dir: Optional[str] = None, save_compressed: bool = True, phase_times: Optional[dict] = None,
            sequential_offload_device=None, sequential_prefetch: bool = False, propagate_error: bool = True,
            **_ignored):
    """Apply the recipe's modifiers to ``model`` in one calibration pass and return it.

    ``recipe`` is a modifier or a list of modifiers (GPTQModifier / QuantizationModifier);
    ``dataset`` is a DataLoader, a list of ``{"input_ids": ...}`` dicts / id tensors, or a
    [samples, length] tensor of token ids; it may be None for data-free recipes.  ``phase_times``
    (a dict) asks for wall seconds per phase of the sequential driver (capture, calibrate, compress,
    propagate), at the price of a device synchronisation at every phase boundary.
    ``sequential_offload_device`` (default None: activations stay in device memory; the reference
    defaults to "cpu"), ``sequential_prefetch`` and ``propagate_error`` are the reference's dataset
    arguments of the same names (src/llmcompressor/args/dataset_arguments.py:244-300)."""
    if isinstance(model, str):
        raise NotImplementedError("pass an instantiated model; loading checkpoints is outside this package")
    if recipe is None:
        raise ValueError("oneshot needs a recipe")
    modifiers = list(recipe) if isinstance(recipe, (list, tuple)) else [recipe]
    if pipeline not in ("independent", "sequential", "datafree", "basic"):
        raise ValueError(f"unknown pipeline {pipeline}")
    device = next(model.parameters()).device
    model.eval()
    for m in modifiers:
        m.on_initialize(model)
    # "independent": each modifier runs alone with the driver it needs (pipelines/independent)
    for m in modifiers:
        needs_data = getattr(m, "requires_calibration_data", False) and pipeline != "datafree"
        if needs_data:
            batches = _as_batches(dataset, num_calibration_samples, max_seq_length, batch_size, device)
            if not batches:
                raise ValueError(f"{type(m).__name__} needs calibration data but no dataset was given")
            _run_sequential(model, [m], batches, sequential_targets, phase_times,
                            offload_device=sequential_offload_device, prefetch=sequential_prefetch,
                            propagate_error=propagate_error)
        else:
            _run_data_free(model, [m])
    for m in modifiers:
        m.on_finalize(model)
    if output_dir is not None:
        save_compressed_model(model, output_dir, compress=save_compressed, recipe=modifiers)
    return model


def compressed_state_dict(model, compress: bool = True):
    """``(state, quantization_config)`` of ``model`` in the compressed-tensors layout:
    ``<module>.weight_packed`` / ``weight_scale`` / ``weight_shape`` / ... per quantised module,
    everything else as it is, tensors on the CPU (CT model_compressor.py:177-213)."""
    state, formats, groups, ignore = {}, set(), {}, []
    quantised = {n: m for n, m in model.named_modules() if hasattr(m, "quantization_scheme")}
    skip = set()
    kv_cache_scheme = None
    for name, mod in quantised.items():
        scheme = mod.quantization_scheme
        if scheme.weights is None and hasattr(mod, "k_scale"):
            # an attention module that only carries kv-cache scales: no config group of its own, its
            # k_scale / v_scale are saved as they are (CT quant_config.py:184-208)
            if getattr(mod, "quantization_status", "frozen") != "frozen":
                raise ValueError(f"{name} has a kv-cache scheme but its k / v scales were never calibrated")
            kv_cache_scheme = scheme.input_activations
            continue
        if scheme.weights is not None and getattr(mod, "quantization_status", "frozen") != "frozen":
            raise ValueError(f"{name} has a weight quantisation scheme but was never calibrated: its scale is "
                             "uninitialised (was it outside the calibrated blocks, or never reached by a forward pass?)")
        local = {k: getattr(mod, k).data for k in ("weight", "weight_scale", "weight_zero_point",
                                                   "weight_global_scale", "weight_g_idx") if hasattr(mod, k)}
        if "weight_g_idx" in local and bool((local["weight_g_idx"] < 0).any()):
            local.pop("weight_g_idx")
        fmt = infer_module_format(scheme)
        formats.add(fmt)
        out = compress_state_dict(local, scheme, fmt) if compress else local
        for k, v in out.items():
            state[f"{name}.{k}"] = v.detach().contiguous().cpu()
        for k in ("weight", "weight_scale", "weight_zero_point", "weight_global_scale", "weight_g_idx"):
            skip.add(f"{name}.{k}")
        gname = next((g for g, s in groups.items() if s is scheme), None)
        if gname is None:
            groups[f"group_{len(groups)}"] = scheme
    for k, v in model.state_dict().items():
        if k not in skip and k not in state:
            state[k] = v.detach().contiguous().cpu()
    for n, m in model.named_modules():
        if (isinstance(m, torch.nn.Linear) or type(m).__name__ == "Linear") and n not in quantised:
            ignore.append(n)

    def args_dict(a):
        if a is None:
            return None
        return {"num_bits": a.num_bits, "type": a.type, "symmetric": a.symmetric, "group_size": a.group_size,
                "strategy": a.strategy, "block_structure": a.block_structure, "dynamic": a.dynamic,
                "actorder": a.actorder, "scale_dtype": None if a.scale_dtype is None else str(a.scale_dtype),
                "zp_dtype": None if a.zp_dtype is None else str(a.zp_dtype), "observer": a.observer,
                "observer_kwargs": a.observer_kwargs}

    fmt = "dense" if not formats else (formats.pop() if len(formats) == 1 else "mixed-precision")
    qconfig = {
        "quant_method": "compressed-tensors", "format": fmt,
        "quantization_status": "compressed" if compress else "frozen",
        "config_groups": {g: {"targets": s.targets, "weights": args_dict(s.weights),
                              "input_activations": args_dict(s.input_activations),
                              "output_activations": None, "format": infer_module_format(s)}
                          for g, s in groups.items()},
        "ignore": ignore, "kv_cache_scheme": args_dict(kv_cache_scheme), "sparsity_config": {}, "transform_config": {},
        "global_compression_ratio": None,
    }
    return state, qconfig


FORMAT_VERSION = "0.15.0.1"   # compressed-tensors layout this writer produces


def _ct_version() -> str:
    try:
        import compressed_tensors
        return str(compressed_tensors.__version__)
    except Exception:  # noqa: BLE001 - the package is optional here
        return FORMAT_VERSION


def _parse_size(v) -> int:
    if isinstance(v, (int, float)):
        return int(v)
    m = re.fullmatch(r"\s*([0-9.]+)\s*([KMGT]?)i?B?\s*", str(v), re.IGNORECASE)
    if not m:
        raise ValueError(f"cannot read max_shard_size {v!r}")
    return int(float(m.group(1)) * {"": 1, "K": 10**3, "M": 10**6, "G": 10**9, "T": 10**12}[m.group(2).upper()])


def recipe_dict(modifiers, stage: str = "default") -> dict:
    """``{stage_stage: {stage_modifiers: {ModifierClass: args}}}``, the layout of the reference's
    recipe.yaml (src/llmcompressor/recipe/utils.py:56-96)."""
    group = {}
    for m in modifiers:
        args = m.recipe_args() if hasattr(m, "recipe_args") else {}
        group[type(m).__name__] = {k: v for k, v in args.items() if v is not None}
    return {f"{stage}_stage": {f"{stage}_modifiers": group}}


def _drop_retied_output_embedding(model, state: dict, cfg: dict) -> None:
    """An output embedding that holds exactly the input embedding's tensors is one table: write it
    once and mark the config tied (compressed_tensors_utils.py:37-80)."""
    get_in, get_out = getattr(model, "get_input_embeddings", None), getattr(model, "get_output_embeddings", None)
    if not callable(get_in) or not callable(get_out):
        return
    try:
        inp, out = get_in(), get_out()
    except Exception:  # noqa: BLE001 - models without embeddings
        return
    if inp is None or out is None or inp is out:
        return
    names = {id(m): n for n, m in model.named_modules()}
    ni, no = names.get(id(inp)), names.get(id(out))
    if ni is None or no is None:
        return
    ti = {k[len(ni) + 1:]: v for k, v in state.items() if k.startswith(ni + ".")}
    to = {k[len(no) + 1:]: v for k, v in state.items() if k.startswith(no + ".")}
    if not ti or ti.keys() != to.keys():
        return
    if not all(ti[k].shape == to[k].shape and ti[k].dtype == to[k].dtype and
               torch.equal(ti[k].view(torch.uint8) if ti[k].dtype.itemsize == 1 else ti[k],
                           to[k].view(torch.uint8) if to[k].dtype.itemsize == 1 else to[k]) for k in ti):
        return
    for k in to:
        del state[f"{no}.{k}"]
    cfg["tie_word_embeddings"] = True


def save_compressed_model(model, output_dir: str, compress: bool = True, recipe=None,
                          max_shard_size="20GB") -> dict:
    """Write the compressed-tensors checkpoint layout: safetensors with
    ``<module>.weight_packed`` / ``weight_scale`` / ``weight_shape`` / ... per quantised module
    (one ``model.safetensors``, or ``model-0000i-of-0000n.safetensors`` plus
    ``model.safetensors.index.json`` once the tensors exceed ``max_shard_size``), ``config.json``
    carrying ``quantization_config`` with its ``version`` (CT model_compressor.py:177-213) and, when
    ``recipe`` (a list of modifiers) is given, ``recipe.yaml``
    (src/llmcompressor/transformers/compression/compressed_tensors_utils.py:106-176,231-246).
    Only rank 0 packs and writes.  Returns the state dict that was written (empty on other ranks)."""
    from safetensors.torch import save_file

    state = {}
    if bdist.rank() == 0:
        state, qconfig = compressed_state_dict(model, compress)
        os.makedirs(output_dir, exist_ok=True)
        cfg = model.config.to_dict() if hasattr(model, "config") and hasattr(model.config, "to_dict") else {}
        _drop_retied_output_embedding(model, state, cfg)
        # tied tensors that remain share storage; safetensors wants distinct buffers
        seen = {}
        for k in list(state):
            p = state[k].data_ptr()
            if p in seen and state[k].numel():
                state[k] = state[k].clone()
            seen[p] = k
        limit = _parse_size(max_shard_size)
        shards, cur, cur_bytes = [], {}, 0
        for k, v in state.items():
            nb = v.numel() * v.element_size()
            if cur and cur_bytes + nb > limit:
                shards.append(cur)
                cur, cur_bytes = {}, 0
            cur[k] = v
            cur_bytes += nb
        shards.append(cur)
        if len(shards) == 1:
            save_file(shards[0], os.path.join(output_dir, "model.safetensors"), metadata={"format": "pt"})
        else:
            weight_map = {}
            for i, sh in enumerate(shards):
                fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
                save_file(sh, os.path.join(output_dir, fname), metadata={"format": "pt"})
                weight_map.update({k: fname for k in sh})
            total = sum(v.numel() * v.element_size() for v in state.values())
            with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
        cfg["quantization_config"] = {"version": _ct_version(), **qconfig}
        with open(os.path.join(output_dir, "config.json"), "w") as f:
            json.dump(cfg, f, indent=2, sort_keys=True, default=str)
        if recipe:
            import yaml
            mods = list(recipe) if isinstance(recipe, (list, tuple)) else [recipe]
            with open(os.path.join(output_dir, "recipe.yaml"), "w") as f:
                yaml.dump(recipe_dict(mods), f, allow_unicode=True, sort_keys=False, default_flow_style=None, width=88)
    if bdist.is_distributed():
        torch.distributed.barrier()
    return state
