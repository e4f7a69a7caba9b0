"""The checkpoint writer against compressed-tensors' own readers: what ``save_compressed_model``
writes is parsed with the installed package's ``QuantizationConfig`` and decompressed module by
module with its compressors; the result must be the fake-quantised weight, bit for bit."""
import copy
import json
import os

import pytest
import torch

from llm_compressor_b200 import GPTQModifier, QuantizationModifier, oneshot, ops
from test_gpu_oneshot import calib, tiny_llama

pytestmark = pytest.mark.gpu
ct = pytest.importorskip("compressed_tensors")


def _load(dirname):
    from safetensors.torch import load_file
    files = [f for f in os.listdir(dirname) if f.endswith(".safetensors")]
    sd = {}
    for f in files:
        sd.update(load_file(os.path.join(dirname, f)))
    cfg = json.load(open(os.path.join(dirname, "config.json")))
    return sd, cfg


def _decompress_all(sd, qc):
    """{module name: dequantised weight} through compressed-tensors' compressor classes."""
    from compressed_tensors.compressors import BaseCompressor
    from compressed_tensors.quantization import QuantizationConfig
    conf = QuantizationConfig.model_validate({k: v for k, v in qc.items() if k != "version"})
    assert conf.quantization_status.value == "compressed"
    names = sorted({k.rsplit(".", 1)[0] for k in sd if k.endswith((".weight_packed", ".weight_scale"))})
    out = {}
    for name in names:
        scheme = next(iter(conf.config_groups.values()))
        fmt = scheme.format or conf.format
        comp = BaseCompressor.load_from_registry(fmt)
        local = {k[len(name) + 1:]: v for k, v in sd.items() if k.startswith(name + ".")}
        out[name] = comp.decompress(local, scheme)["weight"]
    return out


# (MXFP4: the installed compressed-tensors writes the format but cannot read it back)
@pytest.mark.parametrize("scheme", ["W4A16", "W4A16_ASYM", "W8A16", "NVFP4A16", "MXFP8A16"])
def test_rtn_checkpoint_decompresses_to_the_fake_quantised_weight(scheme, tmp_path):
    base = tiny_llama(seed=7)
    recipe = QuantizationModifier(targets="Linear", scheme=scheme, ignore=["lm_head"])
    model = oneshot(copy.deepcopy(base), recipe=recipe, output_dir=str(tmp_path / scheme))
    sd, cfg = _load(str(tmp_path / scheme))
    qc = cfg["quantization_config"]
    assert qc["version"] == ct.__version__ and qc["quant_method"] == "compressed-tensors"
    assert os.path.exists(tmp_path / scheme / "recipe.yaml")
    deq = _decompress_all(sd, qc)
    assert len(deq) == 14
    for name, w in deq.items():
        m = dict(model.named_modules())[name]
        args = m.quantization_scheme.weights
        gs = m.weight_global_scale.data if hasattr(m, "weight_global_scale") else None
        fq = ops.fake_quantize(m.weight.data, m.weight_scale.data, m.weight_zero_point.data, args, global_scale=gs)
        # equal as numbers: a code of zero decompresses to +0, the fake-quantised value may be -0
        assert w.dtype == fq.dtype and torch.equal(w.to(fq.device), fq), (scheme, name)


def test_gptq_checkpoint_decompresses_to_the_quantised_model_and_shards(tmp_path):
    base = tiny_llama(seed=8)
    recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder="group")
    model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=calib(8, 64))
    from llm_compressor_b200 import save_compressed_model
    out = str(tmp_path / "sharded")
    save_compressed_model(model, out, recipe=[recipe], max_shard_size="300KB")
    index = json.load(open(os.path.join(out, "model.safetensors.index.json")))
    files = set(index["weight_map"].values())
    assert len(files) > 1 and all(os.path.exists(os.path.join(out, f)) for f in files)
    sd, cfg = _load(out)
    assert set(sd) == set(index["weight_map"])
    deq = _decompress_all(sd, cfg["quantization_config"])
    for name, w in deq.items():
        m = dict(model.named_modules())[name]
        # GPTQ leaves the fake-quantised weight in the module.  Act-order "group" derives its scales
        # from the float32 working copy (gptq_quantize.py:111-115), so the weight was formed with the
        # float32 scale and the checkpoint holds the bf16 one: the same codes, values one bf16 ulp apart
        a, b = w.to(m.weight.device).float(), m.weight.data.float()
        assert bool(((a - b).abs() <= b.abs() * 2.0 ** -7).all()), name
        assert f"{name}.weight_g_idx" in sd
    import yaml
    rec = yaml.safe_load(open(os.path.join(out, "recipe.yaml")))
    args = rec["default_stage"]["default_modifiers"]["GPTQModifier"]
    assert args["scheme"] == "W4A16" and args["actorder"] == "group" and args["block_size"] == 128


def test_gptq_static_order_checkpoint_is_exact(tmp_path):
    base = tiny_llama(seed=8)
    recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder="static")
    model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=calib(8, 64), output_dir=str(tmp_path / "s"))
    sd, cfg = _load(str(tmp_path / "s"))
    for name, w in _decompress_all(sd, cfg["quantization_config"]).items():
        m = dict(model.named_modules())[name]
        assert torch.equal(w.to(m.weight.device, m.weight.dtype), m.weight.data), name
        assert f"{name}.weight_g_idx" not in sd


def test_tied_embeddings_are_written_once(tmp_path):
    base = tiny_llama(seed=9)
    base.lm_head.weight = base.model.embed_tokens.weight     # one table
    model = oneshot(base, recipe=QuantizationModifier(targets="Linear", scheme="W8A16", ignore=["lm_head"]),
                    output_dir=str(tmp_path / "tied"))
    sd, cfg = _load(str(tmp_path / "tied"))
    assert "model.embed_tokens.weight" in sd and "lm_head.weight" not in sd
    assert cfg["tie_word_embeddings"] is True
