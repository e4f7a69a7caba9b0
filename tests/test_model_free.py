"""model_free_ptq: host logic on CPU, whole flow against the in-memory QuantizationModifier path on GPU."""
import json
import os

import pytest
import torch

from llm_compressor_b200 import model_free as mf
from llm_compressor_b200.quant_args import preset_name_to_scheme


def test_split_fused_moe_experts():
    t = {"mlp.experts.gate_up_proj": torch.arange(2 * 6 * 4, dtype=torch.float32).reshape(2, 6, 4),
         "mlp.experts.down_proj": torch.ones(2, 4, 3), "mlp.router.weight": torch.zeros(2, 4)}
    out = mf.split_fused_moe_experts(t)
    assert set(out) == {"mlp.experts.0.gate_proj.weight", "mlp.experts.0.up_proj.weight",
                        "mlp.experts.1.gate_proj.weight", "mlp.experts.1.up_proj.weight",
                        "mlp.experts.0.down_proj.weight", "mlp.experts.1.down_proj.weight", "mlp.router.weight"}
    assert torch.equal(out["mlp.experts.1.up_proj.weight"], t["mlp.experts.gate_up_proj"][1, 3:])
    assert out["mlp.experts.0.down_proj.weight"].shape == (4, 3)
    with pytest.raises(ValueError, match="divisible"):
        mf.split_fused_moe_experts({"x.gate_up_proj": torch.zeros(2, 5, 4)})


def test_fused_sets_and_tree():
    names = ["m.l0.attn.q_proj.weight", "m.l0.attn.k_proj.weight", "m.l0.attn.v_proj.weight",
             "m.l0.attn.o_proj.weight", "m.l0.mlp.gate_proj.weight", "m.l0.mlp.up_proj.weight",
             "m.l0.mlp.down_proj.weight", "m.l1.attn.q_proj.weight", "m.norm.weight"]
    sets = mf.fused_sets(names)
    assert sorted(map(sorted, sets)) == sorted(map(sorted, [names[0:3], names[4:6]]))
    tree = mf.build_module_tree({n: torch.zeros(2, 8) for n in names[:4]})
    mods = dict(tree.named_modules())
    assert type(mods["m.l0.attn.q_proj"]).__name__ == "Linear"
    assert mods["m.l0.attn.o_proj"].in_features == 8 and mods["m.l0.attn.o_proj"].out_features == 2


def test_validate_scheme():
    s = mf.validate_scheme("FP8_DYNAMIC")
    assert s.targets == ["Linear"] and s.weights.num_bits == 8
    with pytest.raises(ValueError, match="Unknown preset"):
        mf.validate_scheme("W3A3")
    with pytest.raises(ValueError):
        mf.model_free_ptq("/nonexistent", "/tmp/x", scheme="W4A16")
    with pytest.raises(ValueError, match="either"):
        mf.model_free_ptq("/tmp", "/tmp/x")


class _Attn(torch.nn.Module):
    def __init__(self, h):
        super().__init__()
        self.q_proj = torch.nn.Linear(h, h, bias=False)
        self.k_proj = torch.nn.Linear(h, h // 2, bias=False)
        self.v_proj = torch.nn.Linear(h, h // 2, bias=False)
        self.o_proj = torch.nn.Linear(h, h, bias=False)


class _Mlp(torch.nn.Module):
    def __init__(self, h, i):
        super().__init__()
        self.gate_proj = torch.nn.Linear(h, i, bias=False)
        self.up_proj = torch.nn.Linear(h, i, bias=False)
        self.down_proj = torch.nn.Linear(i, h, bias=False)


class _Layer(torch.nn.Module):
    def __init__(self, h, i):
        super().__init__()
        self.self_attn, self.mlp = _Attn(h), _Mlp(h, i)
        self.input_layernorm = torch.nn.LayerNorm(h)


class _Model(torch.nn.Module):
    def __init__(self, h=128, i=256, layers=2):
        super().__init__()
        self.layers = torch.nn.ModuleList([_Layer(h, i) for _ in range(layers)])
        self.lm_head = torch.nn.Linear(h, 64, bias=False)


@pytest.mark.gpu
@pytest.mark.parametrize("scheme", ["NVFP4A16", "W4A16", "FP8_DYNAMIC", "MXFP4A16"])
def test_model_free_matches_in_memory_path(tmp_path, scheme):
    from safetensors.torch import load_file, save_file

    from llm_compressor_b200 import QuantizationModifier, oneshot

    torch.manual_seed(0)
    model = _Model().to(torch.bfloat16)
    for p in model.parameters():
        p.requires_grad_(False)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    # two shards; the q/k/v set of layer 0 and the gate/up set of layer 1 straddle them
    a = {k: v for k, v in sd.items() if k.startswith("layers.0.") and "k_proj" not in k and "v_proj" not in k}
    a["layers.1.mlp.up_proj.weight"] = sd["layers.1.mlp.up_proj.weight"]
    b = {k: v for k, v in sd.items() if k not in a}
    src = tmp_path / "src"
    src.mkdir()
    save_file(a, str(src / "model-00001-of-00002.safetensors"))
    save_file(b, str(src / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in a}
    wm.update({k: "model-00002-of-00002.safetensors" for k in b})
    (src / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    (src / "config.json").write_text(json.dumps({"architectures": ["X"]}))

    out = tmp_path / "out"
    new_map = mf.model_free_ptq(str(src), str(out), scheme=scheme, ignore=["lm_head"], device="cuda:0")

    ref_dir = tmp_path / "ref"
    oneshot(model.to("cuda:0"), recipe=QuantizationModifier(targets="Linear", scheme=scheme, ignore=["lm_head"]),
            output_dir=str(ref_dir))
    ref = load_file(str(ref_dir / "model.safetensors"))
    got = {}
    for fn in ("model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"):
        part = load_file(str(out / fn))
        assert not set(part) & set(got)
        got.update(part)
    assert set(got) == set(ref) == set(new_map)
    for k in ref:
        assert got[k].dtype == ref[k].dtype and got[k].shape == ref[k].shape, k
        assert torch.equal(got[k].view(torch.uint8), ref[k].view(torch.uint8)), k
    # tensors stay in the shard they came from
    assert new_map["layers.0.self_attn.k_proj.weight_packed" if scheme != "FP8_DYNAMIC"
                   else "layers.0.self_attn.k_proj.weight"] == "model-00002-of-00002.safetensors"
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["architectures"] == ["X"]
    qc = cfg["quantization_config"]
    assert qc["quant_method"] == "compressed-tensors" and "lm_head" in qc["ignore"]
    assert qc["format"] == json.loads((ref_dir / "config.json").read_text())["quantization_config"]["format"]
    assert os.path.exists(out / "model.safetensors.index.json")


@pytest.mark.gpu
def test_model_free_moe_experts(tmp_path):
    from safetensors.torch import load_file, save_file

    torch.manual_seed(1)
    t = {"mlp.experts.gate_up_proj": (torch.randn(3, 256, 128) * 0.02).to(torch.bfloat16),
         "mlp.experts.down_proj": (torch.randn(3, 128, 128) * 0.02).to(torch.bfloat16),
         "mlp.gate.weight": torch.randn(3, 128).to(torch.bfloat16)}
    src = tmp_path / "src"
    src.mkdir()
    save_file(t, str(src / "model.safetensors"))
    out = tmp_path / "out"
    mf.model_free_ptq(str(src), str(out), scheme="FP8_DYNAMIC", ignore=["re:.*mlp.gate$"], device="cuda:0")
    got = load_file(str(out / "model.safetensors"))
    assert got["mlp.experts.2.up_proj.weight"].dtype == torch.float8_e4m3fn
    assert got["mlp.experts.2.up_proj.weight"].shape == (128, 128)
    assert got["mlp.experts.0.down_proj.weight_scale"].shape == (128, 1)
    assert torch.equal(got["mlp.gate.weight"], t["mlp.gate.weight"])
    assert "mlp.experts.gate_up_proj" not in got


@pytest.mark.gpu
def test_model_free_against_the_oracle_and_with_two_groups(tmp_path):
    """Every tensor the shard jobs write equals what the CPU oracle makes of the same weight
    (observer -> qparams -> compressor), for a config with two groups: attention W4A16, MLP FP8."""
    from safetensors.torch import load_file, save_file

    import oracle

    torch.manual_seed(2)
    model = _Model().to(torch.bfloat16)
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    src = tmp_path / "src"
    src.mkdir()
    save_file(sd, str(src / "model.safetensors"))
    config = {"config_groups": {"attn": {"scheme": "W4A16", "targets": ["re:.*self_attn\\..*_proj"]},
                                "mlp": {"scheme": "FP8_DYNAMIC", "targets": ["re:.*mlp\\..*_proj"]}},
              "ignore": ["lm_head"]}
    out = tmp_path / "out"
    mf.model_free_ptq(str(src), str(out), config=config, device="cuda:0")
    got = load_file(str(out / "model.safetensors"))
    specs = {"self_attn": (oracle.preset("W4A16"), None), "mlp": (oracle.preset("FP8_DYNAMIC"), "float-quantized")}
    checked = 0
    for name, w in sd.items():
        kind = "self_attn" if "self_attn" in name else ("mlp" if "mlp" in name else None)
        if kind is None or not name.endswith("_proj.weight"):
            assert torch.equal(got[name], w), name     # untouched (norms, lm_head)
            continue
        spec, fmt = specs[kind]
        qp = oracle.WeightObserver(spec)(w).get_qparams()
        ref = oracle.compress_weight({"weight": w, "weight_scale": qp["scale"].to(w.dtype),
                                      "weight_zero_point": qp["zero_point"]}, spec, fmt=fmt)
        base = name[: -len(".weight")]
        for k, v in ref.items():
            g = got[f"{base}.{k}"]
            assert g.dtype == v.dtype and g.shape == v.shape, (name, k)
            assert torch.equal(g.view(torch.uint8), v.view(torch.uint8)), (name, k)
        checked += 1
    assert checked == 14
    qc = json.loads((out / "config.json").read_text())["quantization_config"]
    assert len(qc["config_groups"]) == 2 and qc["format"] == "mixed-precision" and "version" in qc


class _RenamingConverter:
    """A converter in the shape of compressed-tensors' ``Converter`` protocol: the source checkpoint
    calls its tensors ``transformer.*`` and holds the attention projections already compressed in a
    foreign layout (``.qweight`` int8 + ``.scales``), which become ``weight`` / ``weight_scale``."""

    def __init__(self):
        self.validated = 0

    def validate(self, tensors):
        self.validated += 1
        if not any(k.startswith("transformer.") for k in tensors):
            raise ValueError("not a checkpoint of the foreign format")

    def process(self, tensors):
        out = {}
        for k, v in tensors.items():
            k = k.replace("transformer.", "", 1)
            if k.endswith(".qweight"):
                k = k[: -len(".qweight")] + ".weight"
            elif k.endswith(".scales"):
                k = k[: -len(".scales")] + ".weight_scale"
            out[k] = v
        return out

    def create_config(self):
        return {"quant_method": "compressed-tensors", "format": "int-quantized", "quantization_status": "compressed",
                "config_groups": {"group_0": {"targets": ["re:.*self_attn\\..*_proj"], "format": "int-quantized",
                                              "weights": {"num_bits": 8, "type": "int", "symmetric": True,
                                                          "strategy": "channel"}}},
                "ignore": ["lm_head"], "kv_cache_scheme": None}


@pytest.mark.gpu
def test_model_free_with_a_converter(tmp_path):
    from safetensors.torch import load_file, save_file

    import oracle

    torch.manual_seed(4)
    model = _Model(layers=1).to(torch.bfloat16)
    sd = {}
    for k, v in model.state_dict().items():
        if "self_attn" in k:     # "already compressed" by the foreign tool
            base = k[: -len(".weight")]
            scale = (v.float().abs().amax(dim=1, keepdim=True) / 127).to(torch.bfloat16)
            sd[f"transformer.{base}.qweight"] = torch.round(v.float() / scale.float()).clamp(-128, 127).to(torch.int8)
            sd[f"transformer.{base}.scales"] = scale
        else:
            sd[f"transformer.{k}"] = v.detach().clone()
    src, out = tmp_path / "src", tmp_path / "out"
    src.mkdir()
    save_file(sd, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"model_type": "toy"}))
    conv = _RenamingConverter()
    mf.model_free_ptq(str(src), str(out), scheme="FP8_DYNAMIC", ignore=["lm_head"], device="cuda:0", converter=conv)
    assert conv.validated == 1
    got = load_file(str(out / "model.safetensors"))
    assert not any(k.startswith("transformer.") for k in got)
    # converted tensors pass through under their new names, untouched
    q = "layers.0.self_attn.q_proj"
    assert torch.equal(got[f"{q}.weight"], sd[f"transformer.{q}.qweight"])
    assert torch.equal(got[f"{q}.weight_scale"], sd[f"transformer.{q}.scales"])
    # the floating-point weights that were left are quantised by this run, as the oracle does it
    spec = oracle.preset("FP8_DYNAMIC")
    w = sd["transformer.layers.0.mlp.down_proj.weight"]
    qp = oracle.WeightObserver(spec)(w).get_qparams()
    ref = oracle.compress_weight({"weight": w, "weight_scale": qp["scale"].to(w.dtype),
                                  "weight_zero_point": qp["zero_point"]}, spec, fmt="float-quantized")
    for k, v in ref.items():
        g = got[f"layers.0.mlp.down_proj.{k}"]
        assert g.dtype == v.dtype and torch.equal(g.view(torch.uint8), v.view(torch.uint8)), k
    assert torch.equal(got["lm_head.weight"], sd["transformer.lm_head.weight"])
    qc = json.loads((out / "config.json").read_text())["quantization_config"]
    assert set(qc["config_groups"]) == {"group_0", "group_0_ptq"} and qc["format"] == "mixed-precision"
    assert qc["config_groups"]["group_0"]["weights"]["num_bits"] == 8
    assert "lm_head" in qc["ignore"] and "version" in qc
