"""oneshot() through the modifiers on a tiny Llama-architecture model, checked against the
same layer-by-layer procedure driven with the CPU oracle (activations come from the same GPU
forward; Hessian, observer, GPTQ sweep and packing come from the oracle)."""
import copy

import pytest
import torch

import oracle
from helpers import mismatch
from llm_compressor_b200 import GPTQModifier, QuantizationModifier, oneshot, save_compressed_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def tiny_llama(seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=64, vocab_size=512, rms_norm_eps=1e-5, rope_theta=1e4,
                      tie_word_embeddings=False, max_position_embeddings=256)
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    for p in model.parameters():
        p.data.normal_(0, 0.02)
    for n, p in model.named_parameters():
        if "norm" in n:
            p.data.fill_(1.0)
    return model.to(DEV).eval()


def calib(n=16, length=128):
    g = torch.Generator().manual_seed(1)
    return torch.randint(0, 512, (n, length), generator=g)


def oracle_oneshot_gptq(model, data, spec):
    """Layer-by-layer GPTQ with the oracle doing every hot-path computation on CPU."""
    layers = list(model.model.layers)
    captured = []

    class Stop(Exception):
        pass

    def grab(_m, args, kwargs):
        captured.append((args, kwargs))
        raise Stop()
    h = layers[0].register_forward_pre_hook(grab, with_kwargs=True)
    with torch.no_grad():
        for row in data:
            try:
                model(input_ids=row[None].to(DEV))
            except Stop:
                pass
    h.remove()
    losses = {}
    for li, layer in enumerate(layers):
        lin = [(n, m) for n, m in layer.named_modules() if isinstance(m, torch.nn.Linear)]
        Hs = {m: [oracle.make_empty_hessian(m.weight.shape[1]), 0] for _, m in lin}
        hooks = []
        for _, m in lin:
            def hook(mod, args, _out):
                H, n = oracle.accumulate_hessian(args[0].detach().cpu(), Hs[mod][0], Hs[mod][1])
                Hs[mod] = [H, n]
            hooks.append(m.register_forward_hook(hook))
        with torch.no_grad():
            for args, kwargs in captured:
                layer(*args, **kwargs)
        for hk in hooks:
            hk.remove()
        for n, m in lin:
            H, cnt = Hs[m]
            loss, out = oracle.quantize_weight(m.weight.data.cpu(), spec, H / cnt)
            m.weight.data.copy_(out["weight"].to(DEV))
            m._oracle = out
            losses[f"model.layers.{li}.{n}"] = loss
        nxt = []
        with torch.no_grad():
            for args, kwargs in captured:
                o = layer(*args, **kwargs)
                nxt.append(((o[0] if isinstance(o, (tuple, list)) else o,) + tuple(args[1:]), kwargs))
        captured = nxt
    return losses


def test_oneshot_gptq_w4a16_matches_oracle_pipeline(tmp_path):
    base = tiny_llama()
    ref_model = copy.deepcopy(base)
    data = calib()
    spec = oracle.preset("W4A16")
    ref_losses = oracle_oneshot_gptq(ref_model, data, spec)

    recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder=None,
                          block_size=128, dampening_frac=0.01)
    model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data, num_calibration_samples=16,
                    output_dir=str(tmp_path / "ckpt"))
    lin = {n: m for n, m in model.named_modules() if isinstance(m, torch.nn.Linear) and n != "lm_head"}
    ref_lin = {n: m for n, m in ref_model.named_modules() if isinstance(m, torch.nn.Linear) and n != "lm_head"}
    assert len(lin) == 14
    for n, m in lin.items():
        r = ref_lin[n]
        layer0 = ".layers.0." in n
        # layer 0 sees identical inputs: the path's tolerances apply as they are.  Later layers
        # get activations that already differ in a few codes, and with 2048 calibration tokens
        # GPTQ amplifies that, so only a loose bound is checked there
        assert mismatch(m.weight.data, r.weight.data) <= (0.005 if layer0 else 0.15), n
        s, s_ref = m.weight_scale.data.float().cpu(), r._oracle["weight_scale"].float()
        assert torch.equal(s, s_ref), n
        assert recipe.losses[n] == pytest.approx(ref_losses[n], rel=0.01 if layer0 else 0.15), n
    assert not torch.equal(lin["model.layers.0.self_attn.q_proj"].weight.data,
                           base.model.layers[0].self_attn.q_proj.weight.data)
    # q/k/v and gate/up shared one Hessian accumulation each: 4 accumulations per layer, not 7
    # checkpoint layout
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "ckpt" / "model.safetensors"))
    key = "model.layers.0.self_attn.q_proj"
    assert sd[f"{key}.weight_packed"].dtype == torch.int32 and sd[f"{key}.weight_packed"].shape == (256, 32)
    assert sd[f"{key}.weight_scale"].shape == (256, 2) and f"{key}.weight_zero_point" not in sd
    assert sd[f"{key}.weight_shape"].tolist() == [256, 256]
    assert "lm_head.weight" in sd and f"{key}.weight" not in sd
    import json
    qc = json.load(open(tmp_path / "ckpt" / "config.json"))["quantization_config"]
    assert qc["format"] == "pack-quantized" and qc["quant_method"] == "compressed-tensors"
    assert "lm_head" in qc["ignore"]
    # the packed words decode to the oracle's codes
    packed_ref = oracle.compress_weight(
        {"weight": ref_lin[key].weight.data.cpu(), "weight_scale": ref_lin[key]._oracle["weight_scale"],
         "weight_zero_point": ref_lin[key]._oracle["weight_zero_point"]}, spec)
    a, b = sd[f"{key}.weight_packed"].view(torch.uint8), packed_ref["weight_packed"].view(torch.uint8)
    assert float((a != b).float().mean()) <= 0.01


def test_shared_hessians_equal_per_module_hessians():
    base = tiny_llama(seed=3)
    data = calib(8, 64)
    out = []
    for share in (True, False):
        recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder="static",
                              share_hessians=share)
        m = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data)
        out.append({n: p.data.clone() for n, p in m.named_parameters() if n.endswith("proj.weight")})
    for n in out[0]:
        assert torch.equal(out[0][n], out[1][n]), n


def test_concurrent_solves_equal_serial_solves():
    base = tiny_llama(seed=4)
    data = calib(8, 64)
    out = []
    for streams in (4, 1):
        recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder="static",
                              parallel_streams=streams)
        m = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data)
        out.append(({n: p.data.clone() for n, p in m.named_parameters() if "proj.weight" in n}, dict(recipe.losses)))
    assert len(out[0][0]) >= 28
    for n in out[0][0]:
        assert torch.equal(out[0][0][n], out[1][0][n]), n
    assert out[0][1] == out[1][1]


@pytest.mark.parametrize("scheme", ["NVFP4A16", "MXFP4A16", "W4A16", "FP8_DYNAMIC"])
def test_oneshot_rtn_data_free(scheme, tmp_path):
    base = tiny_llama(seed=5)
    model = oneshot(copy.deepcopy(base), recipe=QuantizationModifier(targets="Linear", scheme=scheme,
                                                                    ignore=["lm_head"]))
    spec = oracle.preset(scheme)
    attn = model.model.layers[0].self_attn
    ws = {n: getattr(attn, n).weight.data.cpu() for n in ("q_proj", "k_proj", "v_proj")}
    obs = {n: oracle.WeightObserver(spec) for n in ws}
    if spec.strategy == "tensor_group":
        for n, o in obs.items():
            o.fused = [p for k, p in obs.items() if k != n]
    for n, o in obs.items():
        o(ws[n])
    gss = {n: o.get_global_scale() for n, o in obs.items()}
    for n, o in obs.items():
        scale, zp = oracle.calculate_qparams(o.min_vals, o.max_vals, spec, global_scale=gss[n])
        got = getattr(attn, n).weight_scale.data.float().cpu()
        assert torch.equal(got, scale.float().reshape(got.shape)), (scheme, n)
        if gss[n] is not None:
            assert torch.equal(getattr(attn, n).weight_global_scale.data.cpu(), gss[n])
        assert torch.equal(getattr(attn, n).weight.data.cpu(), ws[n])  # RTN leaves the weight alone
    sd = save_compressed_model(model, str(tmp_path / scheme))
    key = "model.layers.0.self_attn.q_proj"
    st = {"weight": ws["q_proj"], "weight_scale": attn.q_proj.weight_scale.data.cpu(),
          "weight_zero_point": attn.q_proj.weight_zero_point.data.cpu()}
    if gss["q_proj"] is not None:
        st["weight_global_scale"] = gss["q_proj"]
    ref = oracle.compress_weight(st, spec, fmt=None if scheme != "FP8_DYNAMIC" else "float-quantized")
    for k, v in ref.items():
        got = sd[f"{key}.{k}"]
        if v.dtype == torch.float8_e4m3fn:
            assert torch.equal(got.view(torch.uint8), v.view(torch.uint8)), (scheme, k)
        else:
            assert torch.equal(got, v), (scheme, k)


def test_staged_hessian_accumulation_equals_per_batch_accumulation():
    """Gathering small calibration batches before the rank-k update changes the order of the
    float32 sums only: Hessians agree to rounding and the quantised models nearly everywhere."""
    base = tiny_llama(seed=5)
    data = calib(12, 96)
    out = []
    for stage in (0, 512, 100000):
        recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder=None,
                              hessian_stage_tokens=stage)
        m = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data)
        out.append({n: p.data.clone() for n, p in m.named_parameters() if n.endswith("proj.weight")})
    for other in out[1:]:
        for n in out[0]:
            layer0 = ".layers.0." in n
            assert mismatch(out[0][n], other[n]) <= (0.005 if layer0 else 0.15), n


class _Expert(torch.nn.Module):
    def __init__(self, h, i):
        super().__init__()
        self.gate_proj = torch.nn.Linear(h, i, bias=False)
        self.up_proj = torch.nn.Linear(h, i, bias=False)
        self.down_proj = torch.nn.Linear(i, h, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class _MoEBlock(torch.nn.Module):
    def __init__(self, h, i, experts):
        super().__init__()
        self.experts = torch.nn.ModuleList([_Expert(h, i) for _ in range(experts)])
        self.gate = torch.nn.Linear(h, experts, bias=False)

    def forward(self, x, **_):
        w = torch.softmax(self.gate(x), -1)
        return x + sum(w[..., e:e + 1] * ex(x) for e, ex in enumerate(self.experts))   # every expert sees every token


class _MoEModel(torch.nn.Module):
    def __init__(self, h=256, i=128, experts=6, layers=2):
        super().__init__()
        self.embed_tokens = torch.nn.Embedding(512, h)
        self.layers = torch.nn.ModuleList([_MoEBlock(h, i, experts) for _ in range(layers)])
        self.lm_head = torch.nn.Linear(h, 512, bias=False)

    def forward(self, input_ids=None, **_):
        x = self.embed_tokens(input_ids)
        for layer in self.layers:
            x = layer(x)
        return self.lm_head(x)


def test_all_expert_calibration_shares_one_hessian_per_layer():
    """All experts of a block see the same tokens: their gate / up projections share one Hessian
    accumulation and one factorisation, every down projection keeps its own; the blocks are found
    without a hint (longest ModuleList), the router is ignored by pattern."""
    torch.manual_seed(0)
    base = _MoEModel().to(torch.bfloat16).to(DEV)
    for p in base.parameters():
        p.requires_grad_(False)
    data = calib(8, 64)
    out = []
    for share in (True, False):
        recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head", "re:.*\\.gate$"],
                              actorder=None, share_hessians=share)
        m = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data)
        assert len(recipe.losses) == 2 * 6 * 3
        assert all(v == v and v < float("inf") for v in recipe.losses.values())
        assert not hasattr(m.layers[0].gate, "weight_scale")
        out.append({n: p.data.clone() for n, p in m.named_parameters() if n.endswith("proj.weight")})
    for n in out[0]:
        assert torch.equal(out[0][n], out[1][n]), n
    assert not torch.equal(out[0]["layers.0.experts.0.up_proj.weight"], base.layers[0].experts[0].up_proj.weight.data)


def _one_linear_modifier(K=256, N=64, actorder=None, scheme="W4A16"):
    torch.manual_seed(0)
    holder = torch.nn.Module()
    holder.proj = torch.nn.Linear(K, N, bias=False)
    holder = holder.to(torch.bfloat16).to(DEV)
    holder.proj.weight.data.normal_(0, 0.02)
    mod = GPTQModifier(targets="Linear", scheme=scheme, actorder=actorder)
    mod.on_initialize(holder)
    mod.on_calibration_start(holder)
    return holder, mod


@pytest.mark.parametrize("actorder", [None, "static", "group"])
def test_not_positive_definite_hessian_falls_back_to_rtn_through_the_modifier(actorder):
    """A Hessian whose factorisation fails (made on the host: a negative diagonal entry) must end in
    the reference's warning and a round-to-nearest result, for every act-order setting."""
    holder, mod = _one_linear_modifier(actorder=actorder)
    lin = holder.proj
    w0 = lin.weight.data.clone()
    x = torch.randn(2, 64, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    mod.calibrate_module(lin, (x,), None)
    grp = mod._groups[lin]
    grp.flush()
    grp.H.diagonal().copy_(-grp.H.diagonal().abs() - 1.0)   # not positive definite
    with pytest.warns(UserWarning, match="Falling back to round-to-nearest"):
        mod.on_sequential_epoch_end(holder, [lin])
    mod.on_calibration_end(holder)
    assert mod.on_finalize(holder)
    spec = oracle.preset("W4A16", actorder=actorder)
    # oracle: same Hessian -> Cholesky fails -> identity -> plain round to nearest (with the permutation applied)
    K = 256
    xs = x.cpu()
    H, n = oracle.accumulate_hessian(xs, oracle.make_empty_hessian(K), 0)
    d = H.diagonal().clone()
    H.diagonal().copy_(-d.abs() - 1.0)
    loss_ref, ref = oracle.quantize_weight(w0.cpu(), spec, H / n)
    assert torch.equal(lin.weight_scale.data.cpu(), ref["weight_scale"])
    assert mismatch(lin.weight.data, ref["weight"]) <= 0.005
    assert not torch.equal(lin.weight.data, w0)


def test_member_whose_input_diverges_is_reported():
    torch.manual_seed(0)
    holder = torch.nn.Module()
    holder.a = torch.nn.Linear(128, 32, bias=False)
    holder.b = torch.nn.Linear(128, 32, bias=False)
    holder = holder.to(torch.bfloat16).to(DEV)
    mod = GPTQModifier(targets="Linear", scheme="W8A16", actorder=None)
    mod.on_initialize(holder)
    mod.on_calibration_start(holder)
    x = torch.randn(1, 16, 128, device=DEV, dtype=torch.bfloat16)
    mod.calibrate_module(holder.a, (x,), None)
    mod.calibrate_module(holder.b, (x,), None)      # same tensor: one shared Hessian
    assert mod._groups[holder.a] is mod._groups[holder.b]
    y = torch.randn(1, 16, 128, device=DEV, dtype=torch.bfloat16)
    mod.calibrate_module(holder.a, (y,), None)
    with pytest.raises(RuntimeError, match="share_hessians=False"):
        mod.calibrate_module(holder.b, (y.clone(),), None)


def test_targeted_module_behind_the_blocks_is_calibrated_and_unreached_ones_are_reported(tmp_path):
    base = tiny_llama(seed=6)
    data = calib(8, 64)
    recipe = GPTQModifier(targets="Linear", scheme="W8A16", actorder=None)    # lm_head is NOT ignored
    model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data)
    assert "lm_head" in recipe.losses and len(recipe.losses) == 15
    assert not torch.equal(model.lm_head.weight.data, base.lm_head.weight.data)
    assert model.lm_head.quantization_status == "frozen"
    save_compressed_model(model, str(tmp_path / "ok"))
    # a targeted module that no forward pass reaches: finalisation reports it instead of leaving an
    # uninitialised scale in the checkpoint
    broken = copy.deepcopy(base)
    broken.orphan = torch.nn.Linear(256, 256, bias=False, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="never received calibration data"):
        oneshot(broken, recipe=GPTQModifier(targets="Linear", scheme="W8A16", ignore=["lm_head"], actorder=None),
                dataset=data)


def _capture_inputs(model, data, names):
    """{module name: [input of every calibration batch]} from a plain forward of the model."""
    got = {n: [] for n in names}
    mods = dict(model.named_modules())
    hooks = [mods[n].register_forward_pre_hook(lambda m, a, n=n: got[n].append(a[0].detach().float().cpu()))
             for n in names]
    with torch.no_grad():
        for row in data:
            model(input_ids=row[None].to(DEV))
    for h in hooks:
        h.remove()
    return got


def test_static_input_activation_scales_fp8_and_nvfp4(tmp_path):
    """Schemes that calibrate input activations: FP8 (static per-tensor scale from the moving
    average of the batches' min / max) and NVFP4 (global scale from the min / max over all batches)."""
    base = tiny_llama(seed=11)
    data = calib(6, 48)
    names = ["model.layers.0.self_attn.q_proj", "model.layers.0.mlp.down_proj", "model.layers.1.self_attn.o_proj"]
    acts = _capture_inputs(base, data, names)     # round-to-nearest leaves the weights as they are

    model = oneshot(copy.deepcopy(base), recipe=QuantizationModifier(targets="Linear", scheme="FP8", ignore=["lm_head"]),
                    dataset=data, output_dir=str(tmp_path / "fp8"))
    for n in names:
        m = dict(model.named_modules())[n]
        mn = mx = None
        for x in acts[n]:
            lo, hi = x.min().to(torch.bfloat16), x.max().to(torch.bfloat16)
            mn, mx = (lo, hi) if mn is None else (torch.lerp(mn, lo, 0.01), torch.lerp(mx, hi, 0.01))
        spec = oracle.QSpec(num_bits=8, type="float", symmetric=True, strategy="tensor")
        scale, _zp = oracle.calculate_qparams(mn.reshape(1), mx.reshape(1), spec)
        got = m.input_scale.data.float().cpu()
        assert abs(float(got) - float(scale)) <= 2.0 ** -7 * float(scale), (n, float(got), float(scale))
        assert not hasattr(m, "input_observer")
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "fp8" / "model.safetensors"))
    assert "model.layers.0.self_attn.q_proj.input_scale" in sd
    assert sd["model.layers.0.self_attn.q_proj.weight"].dtype == torch.float8_e4m3fn

    model = oneshot(copy.deepcopy(base), recipe=QuantizationModifier(targets="Linear", scheme="NVFP4", ignore=["lm_head"]),
                    dataset=data)
    for n in names:
        m = dict(model.named_modules())[n]
        lo = min(float(x.min().to(torch.bfloat16)) for x in acts[n])
        hi = max(float(x.max().to(torch.bfloat16)) for x in acts[n])
        ref = oracle.generate_gparam(torch.tensor([lo], dtype=torch.bfloat16), torch.tensor([hi], dtype=torch.bfloat16))
        assert torch.equal(m.input_global_scale.data.cpu(), ref), n
        assert not hasattr(m, "input_scale")


class _RecordingCache:
    """Records what an attention module hands to its cache (post-rotary keys, values)."""

    def __init__(self):
        self.keys, self.values = {}, {}

    def update(self, key_states, value_states, layer_idx, *args, **kwargs):
        self.keys.setdefault(layer_idx, []).append(key_states.detach().float().cpu())
        self.values.setdefault(layer_idx, []).append(value_states.detach().float().cpu())
        return key_states, value_states


@pytest.mark.parametrize("with_weights", [False, True])
def test_kv_cache_scales(tmp_path, with_weights):
    """``kv_cache_scheme``: FP8 per-tensor static scales of the cached keys and values, from the
    moving average of each calibration batch's min / max (the ``minmax`` observer), written to the
    attention modules as k_scale / v_scale and into the checkpoint."""
    base = tiny_llama(seed=5)
    data = calib(6, 48)
    rec = _RecordingCache()
    attn = [base.model.layers[i].self_attn for i in range(2)]
    hooks = [a.register_forward_pre_hook(lambda m, args, kwargs: (args, {**kwargs, "past_key_values": rec}),
                                         with_kwargs=True) for a in attn]
    with torch.no_grad():
        for row in data:
            base(input_ids=row[None].to(DEV), use_cache=False)
    for h in hooks:
        h.remove()
    kv = dict(num_bits=8, type="float", symmetric=True, strategy="tensor", dynamic=False)
    if with_weights:
        recipe = QuantizationModifier(targets="Linear", scheme="FP8_DYNAMIC", ignore=["lm_head"], kv_cache_scheme=kv)
    else:
        recipe = QuantizationModifier(targets=[], kv_cache_scheme=kv)
    model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data, output_dir=str(tmp_path / "kv"))
    spec = oracle.QSpec(num_bits=8, type="float", symmetric=True, strategy="tensor")
    for i in range(2):
        m = model.model.layers[i].self_attn
        for attr, seen in (("k_scale", rec.keys[i]), ("v_scale", rec.values[i])):
            mn = mx = None
            for x in seen:
                lo, hi = x.min().to(torch.bfloat16), x.max().to(torch.bfloat16)
                mn, mx = (lo, hi) if mn is None else (torch.lerp(mn, lo, 0.01), torch.lerp(mx, hi, 0.01))
            scale, _zp = oracle.calculate_qparams(mn.reshape(1), mx.reshape(1), spec)
            got = float(getattr(m, attr).data.float().cpu())
            # weights untouched (round to nearest leaves them): same activations, same statistics
            assert abs(got - float(scale)) <= 2.0 ** -7 * float(scale), (i, attr, got, float(scale))
        assert not hasattr(m, "k_observer") and not hasattr(m, "k_zero_point")
        assert m.quantization_status == "frozen"
    import json
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "kv" / "model.safetensors"))
    assert "model.layers.1.self_attn.k_scale" in sd and "model.layers.1.self_attn.v_scale" in sd
    cfg = json.load(open(tmp_path / "kv" / "config.json"))["quantization_config"]
    assert cfg["kv_cache_scheme"]["num_bits"] == 8 and cfg["kv_cache_scheme"]["type"] == "float"
    assert cfg["kv_cache_scheme"]["strategy"] == "tensor" and cfg["kv_cache_scheme"]["dynamic"] is False
    assert all("self_attn" not in t for g in cfg["config_groups"].values() for t in g["targets"])
    if with_weights:
        assert sd["model.layers.0.mlp.up_proj.weight"].dtype == torch.float8_e4m3fn


def test_kv_cache_scales_with_gptq():
    """The same calibration inside a GPTQ run: layer 0 sees unquantised inputs, so its scales are
    those of the plain model; later layers are calibrated on the quantised prefix."""
    base = tiny_llama(seed=6)
    data = calib(6, 48)
    rec = _RecordingCache()
    attn = base.model.layers[0].self_attn
    h = attn.register_forward_pre_hook(lambda m, args, kwargs: (args, {**kwargs, "past_key_values": rec}),
                                       with_kwargs=True)
    with torch.no_grad():
        for row in data:
            base(input_ids=row[None].to(DEV), use_cache=False)
    h.remove()
    kv = dict(num_bits=8, type="float", symmetric=True, strategy="tensor", dynamic=False)
    recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], kv_cache_scheme=kv)
    model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data)
    spec = oracle.QSpec(num_bits=8, type="float", symmetric=True, strategy="tensor")
    m = model.model.layers[0].self_attn
    for attr, seen in (("k_scale", rec.keys[0]), ("v_scale", rec.values[0])):
        mn = mx = None
        for x in seen:
            lo, hi = x.min().to(torch.bfloat16), x.max().to(torch.bfloat16)
            mn, mx = (lo, hi) if mn is None else (torch.lerp(mn, lo, 0.01), torch.lerp(mx, hi, 0.01))
        scale, _zp = oracle.calculate_qparams(mn.reshape(1), mx.reshape(1), spec)
        got = float(getattr(m, attr).data.float().cpu())
        assert abs(got - float(scale)) <= 2.0 ** -7 * float(scale), (attr, got, float(scale))
    last = model.model.layers[1].self_attn
    assert float(last.k_scale) > 0 and float(last.v_scale) > 0 and last.quantization_status == "frozen"
    assert model.model.layers[1].mlp.down_proj.quantization_status == "frozen"


def test_kv_cache_scheme_is_validated():
    with pytest.raises(NotImplementedError, match="per tensor"):
        QuantizationModifier(targets="Linear", kv_cache_scheme=dict(num_bits=8, type="float", strategy="channel",
                                                                     dynamic=False))
    mod = QuantizationModifier(targets=[], kv_cache_scheme=dict(num_bits=8, type="float", strategy="tensor",
                                                                dynamic=False))
    with pytest.raises(ValueError, match="no module matches"):
        mod.on_initialize(torch.nn.Sequential(torch.nn.Linear(8, 8)))


def _gptq_weights(model):
    return {n: p.data.clone() for n, p in model.named_parameters() if n.endswith("proj.weight")}


def test_activation_offload_and_prefetch_do_not_change_results():
    """Parking the blocks' inputs in pinned host memory between uses, with or without prefetching
    the next batch on a copy stream, moves data only."""
    base = tiny_llama(seed=21)
    data = calib(12, 640)      # [1, 640, 256] bf16 hidden states are below the 1 MiB parking limit ...
    batch = 4                  # ... four sequences per batch are above it

    def run(**kw):
        recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"])
        return _gptq_weights(oneshot(copy.deepcopy(base), recipe=recipe, dataset=data, batch_size=batch, **kw))

    from llm_compressor_b200 import ops
    before = ops.set_reproducible(True)     # no atomics across token splits: equal inputs, equal bits
    try:
        ref = run()
        for kw in (dict(sequential_offload_device="cpu"),
                   dict(sequential_offload_device="cpu", sequential_prefetch=True)):
            got = run(**kw)
            for n in ref:
                assert torch.equal(ref[n], got[n]), (kw, n)
    finally:
        ops.set_reproducible(before)


def test_activation_store_parks_large_tensors_on_the_host():
    from llm_compressor_b200.oneshot import _ActivationStore
    store = _ActivationStore(torch.device(DEV), "cpu", prefetch=True)
    big = torch.randn(4, 640, 256, device=DEV).to(torch.bfloat16)
    small = torch.arange(640, device=DEV)
    for i in range(3):
        store.append(((big + i,), {"position_ids": small, "flag": True, "pair": (small, None)}))
    store.settle()
    (parked,), kw = store.items[0]
    assert parked.device.type == "cpu" and parked.is_pinned() and kw["position_ids"].is_cuda
    seen = list(store.batches(release=True))
    assert all(x is None for x in store.items)
    for i, ((t,), kw) in enumerate(seen):
        assert t.is_cuda and torch.equal(t, big + i) and kw["flag"] is True and kw["pair"][1] is None


def test_propagate_error_false_feeds_unquantised_outputs():
    """Without error propagation block 1 is calibrated on the outputs of the unquantised block 0:
    the same as a run that quantises block 1 only."""
    from llm_compressor_b200 import ops
    before = ops.set_reproducible(True)
    try:
        _check_propagate_error_false()
    finally:
        ops.set_reproducible(before)


def _check_propagate_error_false():
    base = tiny_llama(seed=22)
    data = calib(8, 64)
    both = oneshot(copy.deepcopy(base), recipe=GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"]),
                   dataset=data, propagate_error=False)
    only1 = oneshot(copy.deepcopy(base), dataset=data, recipe=GPTQModifier(
        targets="Linear", scheme="W4A16", ignore=["lm_head", "re:.*layers\\.0\\..*"]))
    default = oneshot(copy.deepcopy(base), dataset=data,
                      recipe=GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"]))
    a, b, c = _gptq_weights(both), _gptq_weights(only1), _gptq_weights(default)
    differs = 0
    for n in a:
        if ".layers.1." in n:
            assert torch.equal(a[n], b[n]), n
            differs += int(not torch.equal(a[n], c[n]))
        else:
            assert torch.equal(a[n], c[n]), n     # block 0 sees the same inputs either way
    assert differs > 0
