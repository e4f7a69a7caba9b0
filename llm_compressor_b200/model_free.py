"""``model_free_ptq``: data-free weight quantisation straight from safetensors shards, no model
definition (src/llmcompressor/entrypoints/model_free/__init__.py:45-135, process.py:89-304,
validate.py:22-80, microscale.py).

Every shard is one job: its tensors are loaded onto a GPU, 3-D fused MoE expert tensors are
split into per-expert 2-D weights, the 2-D ``*.weight`` tensors selected by the scheme's
targets become parameter-less "Linear" modules of a throw-away module tree, and the
``QuantizationModifier`` life cycle (observers -> qparams) plus the pack kernels produce the
compressed-tensors entries that replace the weight in the output shard.  Jobs are dealt round
robin over the given devices and run on a thread pool.

NVFP4 (TENSOR_GROUP) keeps one global scale per fused q/k/v and gate/up set.  When the members of
a set sit in different shards, the job of every shard that owns a member also reads the other
members (a partial read of just those tensors) so that the observers can be fused; unlike the
reference, which re-saves the partners in the first owner's shard, each tensor stays in the
shard it came from.
"""
from __future__ import annotations

import json
import os
import shutil
from collections import defaultdict
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Dict, Iterable, List, Optional

import torch

from .modifiers import QuantizationModifier
from .observers import FUSED_LAYER_NAMES
from .quant_args import PRESET_SCHEMES, QuantizationScheme, preset_name_to_scheme

__all__ = ["model_free_ptq", "split_fused_moe_experts", "fused_sets", "build_module_tree"]

INDEX_NAME = "model.safetensors.index.json"


class Linear(torch.nn.Module):
    """A weight without a model definition.  The class name is what ``targets=["Linear"]``
    matches (compressed-tensors matches class names along the MRO)."""

    def __init__(self, weight: torch.Tensor):
        super().__init__()
        self.weight = torch.nn.Parameter(weight, requires_grad=False)

    @property
    def in_features(self):
        return self.weight.shape[1]

    @property
    def out_features(self):
        return self.weight.shape[0]


def validate_scheme(scheme) -> QuantizationScheme:
    """validate.py:22-80: a preset name or a scheme; weights are required, activations must be
    dynamic, empty targets mean "Linear"."""
    if isinstance(scheme, str):
        if scheme.upper() not in PRESET_SCHEMES:
            raise ValueError(f"Unknown preset scheme {scheme}")
        scheme = preset_name_to_scheme(scheme, [])
    if scheme.weights is None:
        raise ValueError("Must provide a weights quantization scheme to perform weights-only PTQ")
    act = scheme.input_activations
    if act is not None and getattr(act, "dynamic", True) is not True:
        raise ValueError("Model Free PTQ cannot calibrate activations. Please use `oneshot` instead.")
    if not scheme.targets:
        scheme.targets = ["Linear"]
    return scheme


def _group_scheme(g) -> QuantizationScheme:
    """One entry of a config's ``config_groups``: a scheme object, a dict in the scheme's field
    names, or a preset name with targets (``{"scheme": "W4A16", "targets": [...]}``)."""
    from .quant_args import QuantizationArgs
    if isinstance(g, QuantizationScheme):
        return validate_scheme(g)
    if isinstance(g, dict) and "scheme" in g:
        s = validate_scheme(g["scheme"])
        s.targets = list(g.get("targets") or s.targets)
        return s
    get = g.get if isinstance(g, dict) else (lambda k, d=None: getattr(g, k, d))
    w, a = get("weights"), get("input_activations")
    return validate_scheme(QuantizationScheme(targets=list(get("targets") or []),
                                              weights=None if w is None else QuantizationArgs.of(w),
                                              input_activations=None if a is None else QuantizationArgs.of(a)))


def split_fused_moe_experts(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """3-D ``...gate_up_proj`` [E, 2I, H] and ``...down_proj`` [E, H, I] tensors become 2-D
    ``...{e}.gate_proj.weight`` / ``{e}.up_proj.weight`` / ``{e}.down_proj.weight`` views
    (process.py:244-304)."""
    parts = {"gate_up_proj": ["gate_proj", "up_proj"], "down_proj": ["down_proj"]}
    out = {}
    for name, t in tensors.items():
        keys = [k for k in parts if k in name]
        if len(keys) >= 2:
            raise ValueError(f"Found multiple keys matching {name}: {keys}")
        if len(keys) == 1 and t.ndim == 3:
            names = parts[keys[0]]
            if t.shape[1] % len(names) != 0:
                raise ValueError(f"{keys[0]} expects a second dimension divisible by {len(names)} "
                                 f"but got shape: {tuple(t.shape)}")
            inter = t.shape[1] // len(names)
            for e in range(t.shape[0]):
                for sub, layer in zip(names, t[e].split(inter, dim=0)):
                    key = name.replace(keys[0], f"{e}.{sub}")
                    if not key.endswith(".weight"):
                        key = f"{key}.weight"
                    out[key] = layer
        else:
            out[name] = t
    return out


def fused_sets(names: Iterable[str]) -> List[List[str]]:
    """Weight names that must share one NVFP4 global scale: siblings q/k/v and gate/up of one
    parent module (src/llmcompressor/observers/helpers.py:162-171)."""
    by_parent = defaultdict(dict)
    for n in names:
        if not n.endswith(".weight"):
            continue
        mod = n[: -len(".weight")]
        parent, _, leaf = mod.rpartition(".")
        by_parent[parent][leaf] = n
    sets = []
    for leaves in by_parent.values():
        for group in FUSED_LAYER_NAMES:
            members = [leaves[g] for g in group if g in leaves]
            if len(members) > 1:
                sets.append(members)
    return sets


def build_module_tree(weights: Dict[str, torch.Tensor]) -> torch.nn.Module:
    """``{"a.b.c.weight": W}`` -> modules ``a``, ``a.b`` and a ``Linear`` at ``a.b.c``."""
    root = torch.nn.Module()
    for name, w in weights.items():
        mod = name[: -len(".weight")]
        node = root
        pieces = mod.split(".")
        for piece in pieces[:-1]:
            if not hasattr(node, piece):
                node.add_module(piece, torch.nn.Module())
            node = getattr(node, piece)
        node.add_module(pieces[-1], Linear(w))
    return root


def _is_weight_candidate(name: str, t: torch.Tensor) -> bool:
    if not name.endswith(".weight") or t.ndim != 2 or not t.is_floating_point():
        return False
    return not name[: -len(".weight")].endswith("norm")   # norms are ignored automatically


def process_shard(tensors: Dict[str, torch.Tensor], scheme, ignore: Iterable[str],
                  own: Optional[set] = None, run: Optional[Callable] = None, converter=None):
    """Quantise and compress the selected weights among ``tensors`` (already on the device).
    ``scheme``: one QuantizationScheme or ``{group name: QuantizationScheme}``.
    ``own``: names to keep in the result (default all); the others were only loaded as fused
    partners.  Returns ``(state_dict on cpu, quantization_config or None)``.

    ``run(model, modifier)`` drives the modifier (default: its data-free life cycle).
    ``converter``: see ``model_free_ptq``; applied after fused expert tensors have been split
    (process.py:107-112)."""
    from .oneshot import _run_data_free, compressed_state_dict

    tensors = split_fused_moe_experts(tensors)
    if converter is not None:
        before = set(tensors)
        if hasattr(converter, "validate"):
            converter.validate(tensors)
        converted = converter.process(tensors)
        tensors = tensors if converted is None else converted     # in place, or a new dict
        if own is not None:   # renamed or new tensors belong to this shard
            own = set(own) | (set(tensors) - before)
    weights = {n: t for n, t in tensors.items() if _is_weight_candidate(n, t)}
    model = build_module_tree(weights)
    groups = dict(scheme) if isinstance(scheme, dict) else {"group_0": scheme}
    targets = sorted({t for g in groups.values() for t in g.targets})
    modifier = QuantizationModifier(targets=targets, ignore=list(ignore), config_groups=groups)
    modifier.on_initialize(model)
    (run or (lambda m, mod: _run_data_free(m, [mod])))(model, modifier)
    modifier.on_finalize(model)
    state, qconfig = compressed_state_dict(model, compress=True)
    quantised = any(hasattr(m, "quantization_scheme") for m in model.modules())
    for n, t in tensors.items():
        if n not in weights:
            state[n] = t.detach().contiguous().cpu()
    if own is not None:
        keep = set()
        for n in own:
            keep.add(n)
            if n.endswith(".weight"):
                keep.add(n[: -len(".weight")])
        state = {k: v for k, v in state.items()
                 if k in keep or k.rpartition(".")[0] in keep}
    return state, (qconfig if quantised else None)


def _merge_configs(existing, new: Optional[dict]) -> Optional[dict]:
    """The converter's quantization config with this run's config groups appended and the ignore
    lists united; the format becomes "mixed-precision" when the two differ."""
    if existing is None:
        return new
    if hasattr(existing, "model_dump"):
        existing = existing.model_dump(mode="json")
    merged = dict(existing)
    merged.setdefault("quant_method", "compressed-tensors")
    if new is None:
        return merged
    groups = dict(merged.get("config_groups") or {})
    for name, g in new["config_groups"].items():
        key = name
        while key in groups:
            key = f"{key}_ptq"
        groups[key] = g
    merged["config_groups"] = groups
    merged["ignore"] = sorted(set(merged.get("ignore") or []) | set(new.get("ignore") or []))
    if merged.get("format") != new.get("format"):
        merged["format"] = "mixed-precision"
    merged["quantization_status"] = "compressed"
    return merged


def _weight_map(model_dir: str) -> Dict[str, str]:
    from safetensors import safe_open

    index = os.path.join(model_dir, INDEX_NAME)
    if os.path.exists(index):
        with open(index) as f:
            return dict(json.load(f)["weight_map"])
    out = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), framework="pt") as f:
                for k in f.keys():
                    out[k] = fn
    return out


def model_free_ptq(model_stub, save_directory, scheme=None, config=None, ignore: Iterable[str] = tuple(),
                   max_workers: int = 1, device=None, converter=None):
    """Quantise the safetensors checkpoint in directory ``model_stub`` into ``save_directory``.

    ``scheme``: preset name or QuantizationScheme, or ``config``: several schemes at once, given as
    ``{"config_groups": {name: scheme or preset name with "targets"}, "ignore": [...]}`` or an
    object with those attributes (a compressed-tensors ``QuantizationConfig``); the first group
    whose targets select a module applies to it.  ``ignore``: module names / ``re:`` patterns left
    alone (names ending in "norm" always are); ``device``: one device or a list (default: every
    visible GPU).  ``converter``: an object with ``process(tensors)`` (in place, or returning the new
    dict), optionally ``validate(tensors)`` and ``create_config()`` (compressed-tensors'
    ``Converter`` protocol): it turns a checkpoint of another format into the compressed-tensors
    layout shard by shard before the remaining floating-point weights are quantised, and its
    config is the starting point that this run's groups are appended to (save_utils.py:64-125)."""
    from safetensors import safe_open
    from safetensors.torch import load_file, save_file

    if (scheme is None) == (config is None):
        raise ValueError("Please specify either `config` or `scheme`")
    if not os.path.isdir(model_stub):
        raise ValueError(f"{model_stub} is not a directory (hub downloads are not available)")
    if config is not None:
        get = config.get if isinstance(config, dict) else (lambda k, d=None: getattr(config, k, d))
        scheme = {name: _group_scheme(g) for name, g in dict(get("config_groups") or {}).items()}
        if not scheme:
            raise ValueError("`config` holds no config_groups")
        ignore = list(ignore) + [i for i in (get("ignore") or []) if i not in ignore]
    else:
        scheme = validate_scheme(scheme)
    if device is None:
        n = torch.cuda.device_count()
        if n == 0:
            raise RuntimeError("model_free_ptq needs a CUDA device")
        devices = [torch.device("cuda", i) for i in range(n)]
    else:
        devices = [torch.device(d) for d in (device if isinstance(device, (list, tuple)) else [device])]
    os.makedirs(save_directory, exist_ok=True)

    wmap = _weight_map(model_stub)
    shards = sorted(set(wmap.values()))
    for fn in os.listdir(model_stub):   # configs, tokenizers, ...
        src = os.path.join(model_stub, fn)
        if os.path.isfile(src) and not fn.endswith(".safetensors") and fn != INDEX_NAME:
            shutil.copyfile(src, os.path.join(save_directory, fn))

    # fused sets that straddle shards: every owner's job also reads the partners
    partners = defaultdict(dict)   # shard -> {name: source shard}
    all_schemes = list(scheme.values()) if isinstance(scheme, dict) else [scheme]
    if any(sc.weights.strategy == "tensor_group" for sc in all_schemes):
        for members in fused_sets(wmap.keys()):
            for m in members:
                for other in members:
                    if wmap[other] != wmap[m]:
                        partners[wmap[m]][other] = wmap[other]

    def job(i: int, shard: str):
        dev = devices[i % len(devices)]
        with torch.cuda.device(dev):
            tensors = load_file(os.path.join(model_stub, shard), device=str(dev))
            own = set(tensors)
            for name, src in partners.get(shard, {}).items():
                with safe_open(os.path.join(model_stub, src), framework="pt", device=str(dev)) as f:
                    tensors[name] = f.get_tensor(name)
            state, qconfig = process_shard(tensors, scheme, ignore, own=own if partners.get(shard) else None,
                                           converter=converter)
            save_file(state, os.path.join(save_directory, shard), metadata={"format": "pt"})
        return shard, {k: shard for k in state}, sum(v.numel() * v.element_size() for v in state.values()), qconfig

    with ThreadPoolExecutor(max_workers=max(1, max_workers)) as pool:
        results = list(pool.map(lambda a: job(*a), enumerate(shards)))

    new_map, total, qconfig = {}, 0, None
    ignored = []
    for _shard, m, size, qc in results:
        new_map.update(m)
        total += size
        if qc is not None:
            ignored.extend(qc["ignore"])
            if qconfig is None:
                qconfig = qc
    if qconfig is not None:
        qconfig["ignore"] = sorted(set(ignored))
    if converter is not None and hasattr(converter, "create_config"):
        qconfig = _merge_configs(converter.create_config(), qconfig)
    if qconfig is not None:
        cfg_path = os.path.join(save_directory, "config.json")
        cfg = {}
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                cfg = json.load(f)
        from .oneshot import _ct_version
        cfg["quantization_config"] = {"version": _ct_version(), **qconfig}
        with open(cfg_path, "w") as f:
            json.dump(cfg, f, indent=2, default=str)
    if len(shards) > 1 or os.path.exists(os.path.join(model_stub, INDEX_NAME)):
        with open(os.path.join(save_directory, INDEX_NAME), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": new_map}, f, indent=2)
    return new_map
