"""Generate ``tests/golden/golden.pt`` from the real reference.

Run in a container that has an llm-compressor checkout and compressed-tensors installed, with
LLMC_REFERENCE_ROOT pointing at the checkout:

    LLMC_REFERENCE_ROOT=<checkout> TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py

What goes into the file
  known_answers  vectors held by the reference's OWN tests for this path, read out of
                 the test sources with ``ast`` (no numbers are typed in here):
                 tests/llmcompressor/modifiers/calibration/test_lifecycle.py:16-165,
                 tests/llmcompressor/observers/test_mse.py:9-42,
                 tests/llmcompressor/observers/test_min_max.py:8-30.
  ct_cases       seeded bf16 weights pushed through the reference observer
                 (memoryless_minmax) -> get_qparams -> compressed-tensors
                 fake_quantize / quantize -> the format's ``compress``.
  mse_cases      the reference ``memoryless_mse`` observer on seeded weights.
  hessian_cases  ``accumulate_hessian`` of gptq_quantize.py, unmodified.
  gptq_cases     ``quantize_weight`` of gptq_quantize.py, unmodified.

``sgpt_hessian.pt`` (a separate small file; ``--sgpt-only`` writes it alone) holds the
running-mean Hessian of modifiers/pruning/sparsegpt/sgpt_sparsify.py:20-56 after each of three
calls on seeded activations.  ``awq.pt`` (``--awq-only``) holds the AWQ grid search of
modifiers/transform/awq/base.py on small parent modules: per-candidate losses, chosen scales.
"""
from __future__ import annotations

import ast
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import torch  # noqa: E402

import ref_loader  # noqa: E402

SCHEMES = {
    # name: kwargs of QuantizationArgs (weight side)
    "w4a16_g128": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128),
    "w4a16_g32": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=32),
    "w4a16_asym_g128": dict(num_bits=4, type="int", symmetric=False, strategy="group", group_size=128),
    "w4_channel": dict(num_bits=4, type="int", symmetric=True, strategy="channel"),
    "w4_tensor": dict(num_bits=4, type="int", symmetric=True, strategy="tensor"),
    "w8a16_channel": dict(num_bits=8, type="int", symmetric=True, strategy="channel"),
    "w8_asym_channel": dict(num_bits=8, type="int", symmetric=False, strategy="channel"),
    "w8_g128": dict(num_bits=8, type="int", symmetric=True, strategy="group", group_size=128),
    "fp8_channel": dict(num_bits=8, type="float", symmetric=True, strategy="channel"),
    "fp8_tensor": dict(num_bits=8, type="float", symmetric=True, strategy="tensor"),
    "fp8_block": dict(num_bits=8, type="float", symmetric=True, strategy="block", block_structure=[16, 64]),
    "nvfp4": dict(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16,
                  scale_dtype=torch.float8_e4m3fn, zp_dtype=torch.float8_e4m3fn),
    "mxfp4": dict(num_bits=4, type="float", symmetric=True, strategy="group", group_size=32,
                  scale_dtype=torch.uint8, zp_dtype=torch.uint8),
    "mxfp8": dict(num_bits=8, type="float", symmetric=True, strategy="group", group_size=32,
                  scale_dtype=torch.uint8, zp_dtype=torch.uint8),
}


def synth_weight(N, K, seed, outliers=True, dtype=torch.bfloat16):
    """bf16 ~ N(0, 0.02) with 0.1 % N(0, 0.5) outliers, one all-zero run of 128 columns
    in row 0, a few exact zeros, one -0.0 and a few tiny negative values."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    if outliers:
        n_out = max(1, (N * K) // 1000)
        idx = torch.randperm(N * K, generator=g)[:n_out]
        w.view(-1)[idx] = torch.randn(n_out, generator=g) * 0.5
    w[0, : min(128, K)] = 0.0
    w[1, 3] = 0.0
    w[1, 5] = -0.0
    w[2, 7] = -1e-6
    w[2, 9] = 1e-6
    return w.to(dtype)


def _ct_args(kw, **over):
    from compressed_tensors.quantization import QuantizationArgs

    d = dict(kw)
    d.update(over)
    return QuantizationArgs(**d)


def _parse_known_answers():
    """Evaluate the parametrize lists of the reference tests."""
    from compressed_tensors.quantization import FP8_E4M3_DATA, QuantizationArgs

    root = os.path.join(ref_loader.REF_ROOT, "tests", "llmcompressor")
    ns = {"torch": torch, "QuantizationArgs": QuantizationArgs, "FP8_E4M3_DATA": FP8_E4M3_DATA}

    def params_of(path, func):
        tree = ast.parse(open(path).read())
        for node in tree.body:
            if isinstance(node, ast.FunctionDef) and node.name == func:
                for dec in node.decorator_list:
                    if isinstance(dec, ast.Call) and getattr(dec.func, "attr", "") == "parametrize":
                        return eval(compile(ast.Expression(dec.args[1]), path, "eval"), ns)
        raise KeyError(func)

    out = {}
    life = params_of(os.path.join(root, "modifiers/calibration/test_lifecycle.py"),
                     "test_static_weight_quantization")
    out["lifecycle_weight"] = [
        dict(args=_clean_args(a), exp_min=mn, exp_max=mx, exp_quant=q, exp_loss=l)
        for (a, mn, mx, q, l) in life
    ]
    out["mse_observer"] = [
        dict(strategy=s, symmetric=sym, exp_loss=l)
        for (s, sym, l) in params_of(os.path.join(root, "observers/test_mse.py"), "test_mse_observer")
    ]
    out["min_max_observer"] = [
        dict(symmetric=sym, scale=sc, zero_point=zp)
        for (sym, sc, zp) in params_of(os.path.join(root, "observers/test_min_max.py"), "test_min_max_observer")
    ]
    return out


def _clean_args(args):
    """QuantizationArgs -> plain python (enums to str, dtypes to their names)."""
    o = {}
    for k in ("num_bits", "type", "symmetric", "group_size", "strategy", "block_structure",
              "dynamic", "actorder", "scale_dtype", "zp_dtype", "observer", "observer_kwargs"):
        v = getattr(args, k)
        if hasattr(v, "value"):
            v = v.value
        if isinstance(v, torch.dtype):
            v = str(v)
        o[k] = v
    return o


def _ct_cases(ref):
    from compressed_tensors.compressors import BaseCompressor
    from compressed_tensors.compressors.format import infer_module_format
    from compressed_tensors.quantization import QuantizationScheme, fake_quantize

    Observer = ref.observers.Observer
    cases = {}
    for si, (name, kw) in enumerate(SCHEMES.items()):
        args = _ct_args(kw)
        N, K = (32, 256)
        w = synth_weight(N, K, seed=100 + si)
        obs = Observer.load_from_registry("memoryless_minmax", base_name="weight", args=args)
        obs(w)
        mn, mx = obs.min_vals.clone(), obs.max_vals.clone()
        qp = obs.get_qparams()
        scale, zp, gs = qp["scale"], qp["zero_point"], qp["global_scale"]
        fq = fake_quantize(w, scale, zp, args, global_scale=gs)
        scheme = QuantizationScheme(targets=["Linear"], weights=args)
        fmt = infer_module_format(torch.nn.Linear, scheme)
        comp = BaseCompressor.get_value_from_registry(fmt.value)
        # parameters as the module would hold them (calibration.py:151-162; CT initialize.py:164-254)
        sd = {"weight": w, "weight_scale": scale.to(w.dtype), "weight_zero_point": zp}
        if gs is not None:
            sd["weight_global_scale"] = gs
        out = comp.compress(sd, scheme)
        cases[name] = dict(
            args=_clean_args(args), weight=w, min=mn, max=mx, scale=scale,
            zero_point=zp, global_scale=gs, fake_quant=fq, format=fmt.value,
            compressed={k: v for k, v in out.items()},
        )
    # fused global scale (q/k/v): three weights share the absmax
    args = _ct_args(SCHEMES["nvfp4"])
    ws = [synth_weight(16, 64, seed=300 + i) * (1 + i) for i in range(3)]
    mods = [torch.nn.Linear(64, 16, bias=False) for _ in ws]
    obs = []
    for m, w in zip(mods, ws):
        m.weight.data = w
        obs.append(Observer.load_from_registry("memoryless_minmax", base_name="weight", args=args))
    ref.observers.FusionHandler.fuse(list(zip(obs, mods)))
    for o, m in zip(obs, mods):
        o(m.weight)
    qps = [o.get_qparams() for o in obs]
    cases["nvfp4_fused3"] = dict(
        args=_clean_args(args), weights=ws,
        scales=[q["scale"] for q in qps], global_scales=[q["global_scale"] for q in qps],
    )
    return cases


def _mse_cases(ref):
    Observer = ref.observers.Observer
    cases = {}
    specs = {
        "w4a16_g128": {},
        "w4a16_g128_grid100": dict(maxshrink=1.0, grid=100.0, norm=2.4),
        "w4_channel": {},
        "w8a16_channel": {},
        "w4a16_asym_g128": {},
        "fp8_channel": {},
        "nvfp4": {},
        "mxfp4": {},
    }
    for si, (name, okw) in enumerate(specs.items()):
        base = name.replace("_grid100", "")
        for dtype in (torch.bfloat16, torch.float32):
            args = _ct_args(SCHEMES[base], observer="memoryless_mse", observer_kwargs=dict(okw))
            w = synth_weight(16, 256, seed=500 + si).to(dtype)
            obs = Observer.load_from_registry("memoryless_mse", base_name="weight", args=args)
            obs(w)
            mn, mx = obs.min_vals.clone(), obs.max_vals.clone()
            qp = obs.get_qparams()
            cases[f"{name}_{str(dtype).split('.')[-1]}"] = dict(
                args=_clean_args(args), weight=w, min=mn, max=mx,
                scale=qp["scale"], zero_point=qp["zero_point"], global_scale=qp["global_scale"],
            )
    return cases


def synth_acts(B, S, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, K, generator=g)
    # columns with different energy so that act-order is a real permutation
    x = x * (0.25 + 2.0 * torch.rand(K, generator=g))
    return x.to(torch.bfloat16)


def _hessian_cases(ref):
    gq = ref.gptq_quantize
    cases = {}
    for name, (B, S, K) in {"b2_s96_k64": (2, 96, 64), "b1_s200_k160": (1, 200, 160),
                            "2d_s33_k48": (0, 33, 48)}.items():
        lin = torch.nn.Linear(K, 8, bias=False)
        x = synth_acts(max(B, 1), S, K, seed=700)
        if B == 0:
            x = x[0]
        H = gq.make_empty_hessian(lin)
        n = torch.zeros(())
        H, n = gq.accumulate_hessian(x, lin, H, n)
        H, n = gq.accumulate_hessian(x * 0.5, lin, H, n)
        cases[name] = dict(x=x, H=H.clone(), n=n.clone())
    return cases


def _gptq_cases(ref):
    gq = ref.gptq_quantize
    Observer = ref.observers.Observer
    cases = {}
    specs = [
        # name, scheme, (N, K), blocksize, extra args, tweaks
        ("w4a16_g128", "w4a16_g128", (32, 256), 128, {}, {}),
        ("w4a16_g32_bs64", "w4a16_g32", (24, 192), 64, {}, {}),
        ("w4a16_g128_actorder_weight", "w4a16_g128", (32, 256), 128, dict(actorder="weight"), {}),
        ("w4a16_g128_actorder_group", "w4a16_g128", (32, 256), 128, dict(actorder="group"), {}),
        ("w4a16_asym_g128", "w4a16_asym_g128", (32, 256), 128, {}, {}),
        ("w4_channel", "w4_channel", (20, 130), 128, {}, {}),
        ("w4_tensor", "w4_tensor", (8, 96), 32, {}, {}),
        ("w8a16_channel", "w8a16_channel", (32, 256), 128, {}, {}),
        ("fp8_channel", "fp8_channel", (32, 256), 128, {}, {}),
        ("nvfp4", "nvfp4", (32, 256), 128, {}, {}),
        ("mxfp4", "mxfp4", (32, 256), 128, {}, {}),
        ("w4a16_g128_dead_cols", "w4a16_g128", (32, 256), 128, {}, dict(dead=[3, 130, 255])),
        ("w4a16_g128_not_pd", "w4a16_g128", (16, 128), 128, {}, dict(not_pd=True)),
        ("w4a16_g128_mse", "w4a16_g128", (16, 256), 128, dict(observer="memoryless_mse"), {}),
        ("w4a16_g128_fp32w", "w4a16_g128", (16, 128), 128, {}, dict(dtype=torch.float32)),
    ]
    for ci, (name, sname, (N, K), bs, extra, tweak) in enumerate(specs):
        args = _ct_args(SCHEMES[sname], **extra)
        dtype = tweak.get("dtype", torch.bfloat16)
        w = synth_weight(N, K, seed=900 + ci).to(dtype)
        lin = torch.nn.Linear(K, N, bias=False)
        lin.weight.data = w.clone()
        x = synth_acts(4, 2 * K // 4 + 8, K, seed=950 + ci)
        if "dead" in tweak:
            x[..., tweak["dead"]] = 0
        H = gq.make_empty_hessian(lin)
        n = torch.zeros(())
        H, n = gq.accumulate_hessian(x, lin, H, n)
        Hn = H / n
        if tweak.get("not_pd"):
            Hn = Hn.clone()
            Hn[5, 5] = -10.0 * Hn.diag().mean()
        obs = Observer.load_from_registry(args.observer, base_name="weight", args=args)
        lin.weight_observer = obs
        obs(lin.weight)
        loss, out = gq.quantize_weight(lin, args, Hn.clone(), blocksize=bs, percdamp=0.01)
        cases[name] = dict(
            args=_clean_args(args), weight=w, hessian=Hn, blocksize=bs,
            percdamp=0.01, loss=loss, out=out,
        )
    return cases


def _sgpt_hessian_cases():
    """Outputs of ``accumulate_hessian`` of modifiers/pruning/sparsegpt/sgpt_sparsify.py (the
    running-mean Hessian of SparseGPT / Wanda), loaded from the reference checkout unmodified."""
    import importlib.util

    path = os.path.join(ref_loader.REF_ROOT, "src", "llmcompressor", "modifiers", "pruning", "sparsegpt",
                        "sgpt_sparsify.py")
    spec = importlib.util.spec_from_file_location("ref_sgpt_sparsify", path)
    sg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sg)
    cases = {}
    for name, (B, S, K) in {"b2_s96_k64": (2, 96, 64), "b3_s50_k160": (3, 50, 160), "2d_s33_k48": (0, 33, 48)}.items():
        lin = torch.nn.Linear(K, 8, bias=False)
        x = synth_acts(max(B, 1), S, K, seed=710)
        if B == 0:
            x = x[0]
        H = sg.make_empty_hessian(lin)
        n = 0
        steps = []
        for factor in (1.0, 0.5, 2.0):
            H, n = sg.accumulate_hessian(x * factor, lin, H, n)
            steps.append(dict(H=H.clone(), n=n))
        cases[name] = dict(x=x, factors=(1.0, 0.5, 2.0), steps=steps)
    return cases


def write_sgpt_fixture():
    assert ref_loader.reference_available(), "set LLMC_REFERENCE_ROOT to the llm-compressor checkout"
    path = os.path.join(HERE, "sgpt_hessian.pt")
    torch.save(dict(meta=dict(torch=torch.__version__), cases=_sgpt_hessian_cases()), path)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


def _awq_cases():
    """Outputs of the reference's ``AWQModifier._compute_best_scale`` (modifiers/transform/awq/base.py:607-763),
    ``_compute_layer_means`` (:907-973) and ``_get_grid_search_params`` (:802-836), run unmodified on the
    CPU over small parent modules.  ``accelerate`` is not installed here; the one name the import
    chain wants from it is provided by a stand-in module."""
    import importlib
    import types

    ref_loader.load_reference()
    if "accelerate" not in sys.modules:
        acc, acca = types.ModuleType("accelerate"), types.ModuleType("accelerate.accelerator")
        acca.get_state_dict_offloaded_model = lambda m: m.state_dict()
        acc.accelerator = acca
        sys.modules["accelerate"], sys.modules["accelerate.accelerator"] = acc, acca
    os.environ.setdefault("TQDM_DISABLE", "1")
    base = importlib.import_module("llmcompressor.modifiers.transform.awq.base")
    from compressed_tensors.quantization import QuantizationArgs, QuantizationScheme
    from compressed_tensors.quantization.lifecycle.initialize import initialize_module_for_quantization
    from llmcompressor.pipelines.cache import IntermediatesCache

    class MLP(torch.nn.Module):
        def __init__(self, K, N):
            super().__init__()
            self.gate_proj = torch.nn.Linear(K, N, bias=False)
            self.up_proj = torch.nn.Linear(K, N, bias=False)

        def forward(self, x):
            return torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x)

    specs = {
        "mlp_w4a16_duo": dict(kind="mlp", K=256, N=192, duo=True, n_grid=20, scheme="w4a16_g128"),
        "mlp_w4asym_both": dict(kind="mlp", K=256, N=160, duo="both", n_grid=12, scheme="w4a16_asym_g128"),
        "linear_w8channel_noduo": dict(kind="linear", K=192, N=96, duo=False, n_grid=10, scheme="w8a16_channel"),
        "mlp_nvfp4_duo": dict(kind="mlp", K=128, N=96, duo=True, n_grid=8, scheme="nvfp4"),
    }
    cases = {}
    for name, c in specs.items():
        g = torch.Generator().manual_seed(len(name) * 131)
        K, N = c["K"], c["N"]
        parent = MLP(K, N) if c["kind"] == "mlp" else torch.nn.Linear(K, N, bias=False)
        parent = parent.to(torch.bfloat16)
        layers = [parent.gate_proj, parent.up_proj] if c["kind"] == "mlp" else [parent]
        names = ["blk.mlp.gate_proj", "blk.mlp.up_proj"] if c["kind"] == "mlp" else ["blk.attn.o_proj"]
        args = _ct_args(SCHEMES[c["scheme"]])
        for layer in layers:
            layer.weight.data = (torch.randn(N, K, generator=g) * 0.05 *
                                 (0.5 + torch.rand(K, generator=g))).to(torch.bfloat16)
            initialize_module_for_quantization(layer, QuantizationScheme(targets=["Linear"], weights=args))
            layer.quantization_enabled = False     # as during calibration
        batches = [(torch.randn(2, 24, K, generator=g) * (0.25 + 2 * torch.rand(K, generator=g))).to(torch.bfloat16)
                   for _ in range(3)]
        mod = base.AWQModifier(duo_scaling=c["duo"], n_grid=c["n_grid"])
        smooth = torch.nn.LayerNorm(K, bias=False)
        mapping = base.ResolvedMapping("blk.norm", smooth, layers, balance_names=names, parent=parent,
                                       parent_name="blk.parent", activation_hook_target=None)
        cache = IntermediatesCache(None, None)
        key = "x" if c["kind"] == "mlp" else "input"
        for b in batches:
            cache.append({key: b})
        mod._parent_args_cache[parent] = cache
        x_sum = sum(b.abs().flatten(0, -2).float().sum(0) for b in batches)
        count = torch.tensor(sum(b.flatten(0, -2).size(0) for b in batches))
        mod._smooth_activation_stats["blk.norm"] = [x_sum.clone(), count.clone()]
        losses = []
        inner = mod._compute_loss

        def recording(a, b, inner=inner, losses=losses):
            v = inner(a, b)
            losses.append(v)
            return v
        object.__setattr__(mod, "_compute_loss", recording)
        weights = [layer.weight.data.clone() for layer in layers]
        with torch.no_grad():
            fp16 = mod._run_samples(parent)
            w_mean = base.AWQModifier._compute_layer_means(layers) if c["duo"] is not False else None
            best = mod._compute_best_scale(mapping, fp16, {layer: layer.weight.clone() for layer in layers})
        cases[name] = dict(kind=c["kind"], args=_clean_args(args), duo=c["duo"], n_grid=c["n_grid"],
                           weights=weights, batches=batches, x_sum=x_sum, count=int(count), w_mean=w_mean,
                           grid=mod._get_grid_search_params(), losses=losses, best_scales=best,
                           metrics=dict(mod._error_metrics[0]))
    return cases


def write_awq_fixture():
    assert ref_loader.reference_available(), "set LLMC_REFERENCE_ROOT to the llm-compressor checkout"
    path = os.path.join(HERE, "awq.pt")
    torch.save(dict(meta=dict(torch=torch.__version__), cases=_awq_cases()), path)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


def main():
    ref = ref_loader.load_reference()
    import compressed_tensors

    torch.manual_seed(0)
    gold = dict(
        meta=dict(torch=torch.__version__, compressed_tensors=compressed_tensors.__version__),
        known_answers=_parse_known_answers(),
        ct_cases=_ct_cases(ref),
        mse_cases=_mse_cases(ref),
        hessian_cases=_hessian_cases(ref),
        gptq_cases=_gptq_cases(ref),
    )
    path = os.path.join(HERE, "golden.pt")
    torch.save(gold, path)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    if "--sgpt-only" in sys.argv:
        write_sgpt_fixture()     # the small separate fixtures, without regenerating golden.pt
    elif "--awq-only" in sys.argv:
        write_awq_fixture()
    else:
        main()
        write_sgpt_fixture()
        write_awq_fixture()
