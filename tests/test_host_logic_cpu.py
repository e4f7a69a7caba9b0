"""Host logic that needs no GPU: AWQ mapping resolution and grid, the activation store of the
sequential driver, the kv-cache plumbing, the merge of a converter's config."""
import pytest
import torch

import oracle
from llm_compressor_b200 import awq
from llm_compressor_b200.model_free import _merge_configs
from llm_compressor_b200.modifiers import QuantizationModifier, _ObservingCache, _observing_cache_hook
from llm_compressor_b200.oneshot import _ActivationStore, _tree_map, _with_hidden
from llm_compressor_b200.quant_args import QuantizationArgs, QuantizationScheme


def _tiny_llama(kv_heads, layers=2):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=layers, num_attention_heads=4,
                      num_key_value_heads=kv_heads, head_dim=16, vocab_size=64, tie_word_embeddings=False,
                      max_position_embeddings=64)
    return LlamaForCausalLM(cfg)


def _attach(model, **args):
    scheme = QuantizationScheme(targets=["Linear"], weights=QuantizationArgs(**args))
    for n, m in model.named_modules():
        if isinstance(m, torch.nn.Linear) and "lm_head" not in n:
            m.quantization_scheme = scheme


@pytest.mark.parametrize("kv_heads,per_layer", [(4, 4), (2, 3)])
def test_awq_mapping_resolution(kv_heads, per_layer):
    model = _tiny_llama(kv_heads)
    _attach(model, num_bits=4, type="int", symmetric=True, strategy="group", group_size=32)
    mod = awq.AWQModifier()
    mod.on_initialize(model)
    if kv_heads == 2:    # v_proj is narrower than o_proj's input under grouped-query attention
        with pytest.warns(UserWarning, match="incompatible shapes"):
            mod._set_resolved_mappings(model)
    else:
        mod._set_resolved_mappings(model)
    res = mod._resolved
    assert len(res) == 2 * per_layer
    by_smooth = {m.smooth_name: m for m in res}
    first = by_smooth["model.layers.0.input_layernorm"]
    assert first.balance_names == [f"model.layers.0.self_attn.{p}_proj" for p in "qkv"]
    assert first.parent_name == "model.layers.0.self_attn"
    up = by_smooth["model.layers.1.mlp.up_proj"]
    assert up.balance_names == ["model.layers.1.mlp.down_proj"] and up.parent_name == "model.layers.1.mlp.down_proj"
    gate = by_smooth["model.layers.1.post_attention_layernorm"]
    assert gate.parent_name == "model.layers.1.mlp" and len(gate.balance_layers) == 2
    assert ("model.layers.0.self_attn.v_proj" in by_smooth) == (kv_heads == 4)


def test_awq_skips_mappings_without_quantised_layers():
    model = _tiny_llama(4, layers=1)
    mod = awq.AWQModifier()
    mod.on_initialize(model)
    with pytest.warns(UserWarning, match="no layers are targeted"):
        mod._set_resolved_mappings(model)
    assert mod._resolved == []
    with pytest.raises(NotImplementedError):
        awq.AWQModifier(mappings=[awq.AWQMapping("a", ["b"], activation_hook_target="x")]).on_initialize(model)


def test_awq_grid_scales_and_means_follow_the_oracle():
    g = torch.Generator().manual_seed(0)
    for duo, n in ((True, 20), (False, 7), ("both", 12)):
        assert awq.grid_search_params(duo, n) == oracle.awq.grid_search_params(duo, n)
    with pytest.raises(ValueError):
        awq.grid_search_params("maybe", 4)
    x_mean = torch.rand(96, generator=g) + 0.01
    layers = []
    for args in (dict(num_bits=4, type="int", strategy="group", group_size=32),
                 dict(num_bits=8, type="int", strategy="channel"),
                 dict(num_bits=8, type="float", strategy="block", block_structure=[16, 32])):
        lin = torch.nn.Linear(96, 64, bias=False)
        lin.quantization_scheme = QuantizationScheme(targets=["Linear"], weights=QuantizationArgs(**args))
        layers.append(lin)
    specs = [oracle.QSpec(**{k: v for k, v in vars(l.quantization_scheme.weights).items()
                              if k in ("num_bits", "type", "symmetric", "strategy", "group_size", "block_structure")})
             for l in layers]
    w_mean = awq.compute_layer_means(layers)
    assert torch.equal(w_mean, oracle.awq.layer_means([l.weight.data for l in layers], specs))
    for ratio, duo in ((0.0, False), (0.5, True), (1.0, True)):
        assert torch.equal(awq.candidate_scales(x_mean, w_mean, ratio, duo),
                           oracle.awq.candidate_scales(x_mean, w_mean, ratio, duo))


def test_activation_store_without_a_gpu():
    store = _ActivationStore("cpu", offload="cpu", prefetch=True)     # same device: nothing to park, no stream
    assert store.offload is None and store.prefetch is False
    items = [((torch.full((2, 3), float(i)),), {"mask": None, "pos": (torch.arange(3), 5)}) for i in range(3)]
    for it in items:
        store.append(it)
    store.settle()
    seen = list(store.batches(release=True))
    assert all(x is None for x in store.items) and len(seen) == 3
    assert seen[1][0][0] is items[1][0][0] and seen[2][1]["pos"][1] == 5
    assert _tree_map(lambda t: t + 1, {"a": [torch.zeros(1), (torch.ones(1), "s")]})["a"][1][0].item() == 2.0
    h = torch.ones(2)
    assert _with_hidden((torch.zeros(2), 7), {"k": 1}, h) == ((h, 7), {"k": 1})
    assert _with_hidden((), {"hidden_states": torch.zeros(2), "k": 1}, h)[1]["hidden_states"] is h
    with pytest.raises(ValueError):
        _with_hidden((), {"x": 1}, h)


def test_observing_cache_feeds_the_observers_and_the_wrapped_cache():
    calls = []

    class Attn(torch.nn.Module):
        def forward(self, hidden_states, past_key_values=None):
            return hidden_states

    class Inner:
        def update(self, k, v, layer_idx):
            calls.append(("inner", layer_idx))
            return k + 1, v + 1

        def get_seq_length(self):
            return 9

    m = Attn()
    m.k_observer = lambda t: calls.append(("k", float(t.sum())))
    m.v_observer = lambda t: calls.append(("v", float(t.sum())))
    _, kwargs = _observing_cache_hook(m, (), {"past_key_values": Inner()})
    cache = kwargs["past_key_values"]
    assert isinstance(cache, _ObservingCache) and cache.get_seq_length() == 9
    k, v = cache.update(torch.ones(2), torch.full((2,), 2.0), 3)
    assert calls == [("k", 2.0), ("v", 4.0), ("inner", 3)] and float(k[0]) == 2.0 and float(v[0]) == 3.0
    _, kwargs = _observing_cache_hook(m, (), {})
    k, v = kwargs["past_key_values"].update(torch.ones(2), torch.ones(2), 0)
    assert float(k.sum()) == 2.0
    with pytest.raises(AttributeError):
        kwargs["past_key_values"].get_seq_length()


def test_kv_cache_scheme_attaches_scales_to_attention_modules():
    model = _tiny_llama(2, layers=1)
    mod = QuantizationModifier(targets=[], kv_cache_scheme=dict(num_bits=8, type="float", strategy="tensor",
                                                                dynamic=False))
    mod.on_initialize(model)
    attn = model.model.layers[0].self_attn
    assert attn.k_scale.shape == (1,) and attn.v_scale.shape == (1,) and not hasattr(attn, "k_zero_point")
    assert attn.quantization_scheme.weights is None and attn.quantization_status == "initialized"
    assert mod.calibrates_activations and mod.requires_calibration_data
    assert mod.recipe_args()["kv_cache_scheme"]["num_bits"] == 8
    asym = QuantizationModifier(targets=[], kv_cache_scheme=dict(num_bits=8, type="int", symmetric=False,
                                                                 strategy="tensor", dynamic=False))
    model2 = _tiny_llama(2, layers=1)
    asym.on_initialize(model2)
    assert model2.model.layers[0].self_attn.k_zero_point.dtype == torch.int8


def test_converter_config_merge():
    new = {"quant_method": "compressed-tensors", "format": "float-quantized", "quantization_status": "compressed",
           "config_groups": {"group_0": {"targets": ["Linear"]}}, "ignore": ["lm_head", "x"]}
    assert _merge_configs(None, new) is new
    old = {"format": "int-quantized", "config_groups": {"group_0": {"targets": ["re:.*attn.*"]}}, "ignore": ["lm_head"]}
    merged = _merge_configs(old, new)
    assert set(merged["config_groups"]) == {"group_0", "group_0_ptq"} and merged["format"] == "mixed-precision"
    assert merged["ignore"] == ["lm_head", "x"] and merged["quant_method"] == "compressed-tensors"
    assert _merge_configs(old, None)["format"] == "int-quantized"
    same = _merge_configs({"format": "float-quantized", "config_groups": {}}, new)
    assert same["format"] == "float-quantized" and list(same["config_groups"]) == ["group_0"]
