"""AWQModifier against the fixtures made with the reference's own AWQ search (tests/golden/awq.pt),
the CPU oracle, and end to end on a tiny Llama-architecture model.

What is bit-exact: Q(W * s) / s for given candidate scales (the kernels' part).  The search itself
runs the parent module on the GPU, whose matmuls round differently from the CPU's, so its losses
are compared within 2 % and its choice must be the fixture's best candidate or one whose
fixture loss is within 1 % of the best."""
import copy

import pytest
import torch

import oracle
from helpers import args_from, bits_equal
from llm_compressor_b200 import AWQMapping, AWQModifier, QuantizationModifier, awq, oneshot
from llm_compressor_b200.quant_args import QuantizationScheme
from test_oracle_golden import spec_from

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class _MLP(torch.nn.Module):
    def __init__(self, K, N):
        super().__init__()
        self.gate_proj = torch.nn.Linear(K, N, bias=False)
        self.up_proj = torch.nn.Linear(K, N, bias=False)

    def forward(self, x):
        return torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x)


def _build(case):
    """(parent module on the GPU, its balance layers) of a fixture case, schemes attached."""
    N, K = case["weights"][0].shape
    parent = _MLP(K, N) if case["kind"] == "mlp" else torch.nn.Linear(K, N, bias=False)
    parent = parent.to(torch.bfloat16).to(DEV)
    layers = [parent.gate_proj, parent.up_proj] if case["kind"] == "mlp" else [parent]
    for layer, w in zip(layers, case["weights"]):
        layer.weight.data = w.to(DEV)
        layer.quantization_scheme = QuantizationScheme(targets=["Linear"], weights=args_from(case["args"]))
    return parent, layers


def test_scaled_fake_quantize_is_bit_exact(awq_golden):
    for name, c in awq_golden["cases"].items():
        spec = spec_from(c["args"])
        specs = [spec] * len(c["weights"])
        parent, layers = _build(c)
        x_mean = c["x_sum"] / c["count"]
        for ratio, duo in c["grid"]:
            scales = oracle.awq.candidate_scales(x_mean, c["w_mean"], ratio, duo)
            ref = oracle.awq.scaled_fake_quantize(c["weights"], scales, specs, fused=spec.strategy == "tensor_group")
            got = awq.scaled_fake_quantize([w.to(DEV) for w in c["weights"]], scales.to(DEV), layers, parent)
            for g, r in zip(got, ref):
                assert bits_equal(g, r), (name, ratio, duo)
        for layer, w in zip(layers, c["weights"]):
            assert torch.equal(layer.weight.data.cpu(), w) and not hasattr(layer, "weight_observer")


def test_layer_means_and_grid(awq_golden):
    for name, c in awq_golden["cases"].items():
        _, layers = _build(c)
        assert awq.grid_search_params(c["duo"], c["n_grid"]) == c["grid"], name
        if c["w_mean"] is not None:
            got = awq.compute_layer_means(layers).cpu()
            assert got.dtype == c["w_mean"].dtype
            assert torch.allclose(got, c["w_mean"], rtol=1e-12, atol=0), name


def test_best_scale_search_against_the_reference(awq_golden):
    for name, c in awq_golden["cases"].items():
        parent, layers = _build(c)
        mod = AWQModifier(duo_scaling=c["duo"], n_grid=c["n_grid"])
        smooth = torch.nn.LayerNorm(layers[0].in_features, bias=False).to(DEV)
        mapping = awq.ResolvedMapping("blk.norm", smooth, layers, ["blk.a"] * len(layers), parent, "blk.parent")
        key = "x" if c["kind"] == "mlp" else "input"
        mod._parent_args_cache[parent] = [{key: b.to(DEV)} for b in c["batches"]]
        mod._smooth_activation_stats["blk.norm"] = [c["x_sum"].to(DEV), c["count"]]
        with torch.no_grad():
            fp16 = mod._run_samples(parent)
            best = mod._compute_best_scale(mapping, fp16, {layer: layer.weight.data.clone() for layer in layers})
        metrics = mod.error_metrics[0]
        losses = [h["error"] for h in metrics["history"]]
        assert len(losses) == len(c["losses"])
        for a, b in zip(losses, c["losses"]):
            assert a == pytest.approx(b, rel=0.02), name
        ours = min(range(len(losses)), key=losses.__getitem__)
        assert c["losses"][ours] <= min(c["losses"]) * 1.01, (name, ours)
        if c["losses"][ours] == min(c["losses"]) and c["losses"].index(min(c["losses"])) == ours:
            assert best.dtype == c["best_scales"].dtype
            assert torch.allclose(best.cpu(), c["best_scales"], rtol=1e-5), name
        for layer, w in zip(layers, c["weights"]):
            assert torch.equal(layer.weight.data.cpu(), w), "the search must leave the weights as they were"


def _tiny_llama(kv_heads):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=kv_heads, head_dim=64, vocab_size=512, rms_norm_eps=1e-5, rope_theta=1e4,
                      tie_word_embeddings=False, max_position_embeddings=256)
    torch.manual_seed(3)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    for n, p in model.named_parameters():
        if "norm" in n:
            p.data.fill_(1.0)
        else:
            p.data = (torch.randn(p.shape, generator=g) * 0.03 * (0.3 + 2 * torch.rand(p.shape[-1], generator=g))
                      ).to(torch.bfloat16)
    return model.to(DEV).eval()


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_oneshot_awq_then_rtn(kv_heads, tmp_path):
    base = _tiny_llama(kv_heads)
    g = torch.Generator().manual_seed(1)
    data = torch.randint(0, 512, (8, 64), generator=g)
    probe = data[:2].to(DEV)
    with torch.no_grad():
        before = base(input_ids=probe).logits.float()
    awq_mod = AWQModifier(n_grid=10)
    recipe = [awq_mod, QuantizationModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"])]
    with pytest.warns(UserWarning) if kv_heads == 2 else _no_warning():
        model = oneshot(copy.deepcopy(base), recipe=recipe, dataset=data, output_dir=str(tmp_path / "awq"))
    # v_proj -> o_proj is skipped under grouped-query attention (widths differ)
    per_layer = 4 if kv_heads == 4 else 3
    assert len(awq_mod.error_metrics) == 2 * per_layer
    for m in awq_mod.error_metrics:
        assert m["best_error"] <= m["initial_error"], m["layer_name"]
    assert any(m["best_ratio"] > 0 for m in awq_mod.error_metrics)
    # the smoothing is function-preserving up to rounding: the weights moved, the logits did not
    moved = sum(int(not torch.equal(a.data, b.data)) for a, b in zip(model.parameters(), base.parameters()))
    assert moved >= 2 * (per_layer + 3)
    with torch.no_grad():
        after = model(input_ids=probe).logits.float()
    assert float((after - before).norm() / before.norm()) < 0.03
    # and the quantisation that follows sees the smoothed weights
    lin = model.model.layers[0].mlp.down_proj
    ref = oracle.WeightObserver(oracle.preset("W4A16"))(lin.weight.data.cpu()).get_qparams()
    assert bits_equal(lin.weight_scale.data, ref["scale"])
    assert (tmp_path / "awq" / "recipe.yaml").exists()
    assert "AWQModifier" in (tmp_path / "awq" / "recipe.yaml").read_text()


class _no_warning:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def test_awq_validation():
    with pytest.raises(ValueError, match="duo_scaling"):
        AWQModifier(duo_scaling="sometimes")
    mod = AWQModifier(mappings=[dict(smooth_layer="re:.*norm$", balance_layers=["re:.*fc$"])])
    assert isinstance(mod.mappings[0], AWQMapping)
    model = torch.nn.ModuleDict({"norm": torch.nn.LayerNorm(16), "fc": torch.nn.Linear(16, 8)}).to(DEV)
    model.fc.quantization_scheme = QuantizationScheme(
        targets=["Linear"], weights=args_from(dict(num_bits=8, type="int", symmetric=True, strategy="tensor")))
    mod.on_initialize(model)
    with pytest.raises(ValueError, match="duo_scaling is only supported with per-channel"):
        mod.on_calibration_start(model)
