"""The CPU oracle against outputs of the real reference (tests/golden/golden.pt) and
against the known-answer vectors of the reference's own tests."""
import pytest
import torch

import oracle
from oracle import QSpec


def spec_from(d):
    keys = ("num_bits", "type", "symmetric", "strategy", "group_size", "block_structure",
            "scale_dtype", "zp_dtype", "actorder", "observer", "observer_kwargs")
    kw = {k: d[k] for k in keys if k in d and d[k] is not None}
    kw.setdefault("observer_kwargs", {})
    return QSpec(**kw)


def same(a, b):
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    if a.dtype in (torch.float8_e4m3fn,):
        return torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    if a.is_floating_point():
        # bit equality including the sign of zero
        n = a.element_size()
        it = {2: torch.int16, 4: torch.int32}[n]
        return torch.equal(a.contiguous().view(it), b.contiguous().view(it))
    return torch.equal(a, b)


# ---------------------------------------------------------------- known answers
def test_lifecycle_known_answers(golden):
    for case in golden["known_answers"]["lifecycle_weight"]:
        args = spec_from(case["args"])
        w = torch.arange(24, dtype=torch.bfloat16).reshape(4, 6)
        obs = oracle.WeightObserver(args)
        obs(w)
        assert torch.equal(obs.min_vals, case["exp_min"].to(obs.min_vals.dtype)), args
        assert torch.equal(obs.max_vals, case["exp_max"].to(obs.max_vals.dtype)), args
        qp = obs.get_qparams()
        fq = oracle.fake_quantize(w, qp["scale"].to(torch.bfloat16) if qp["global_scale"] is None else qp["scale"].to(torch.bfloat16),
                                  qp["zero_point"], args, global_scale=qp["global_scale"])
        assert torch.allclose(fq.to(torch.bfloat16), case["exp_quant"].to(torch.bfloat16)), (args, fq)
        assert torch.nn.functional.mse_loss(fq.float(), w.float()) <= case["exp_loss"]


def test_mse_known_answers(golden):
    for case in golden["known_answers"]["mse_observer"]:
        st = case["strategy"]
        args = QSpec(num_bits=8, strategy=st, symmetric=case["symmetric"],
                     group_size=2 if st == "group" else None,
                     block_structure=[3, 2] if st == "block" else None, observer="mse")
        t = torch.arange(24).reshape(6, 4) / 24
        obs = oracle.WeightObserver(args)
        qp = obs(t).get_qparams()
        fq = oracle.fake_quantize(t, qp["scale"], qp["zero_point"], args)
        loss = torch.sum((t - fq).abs().pow(2)) / t.numel()
        assert float(loss) == pytest.approx(case["exp_loss"], abs=1e-10), case


def test_minmax_known_answers(golden):
    for case in golden["known_answers"]["min_max_observer"]:
        args = QSpec(num_bits=8, symmetric=case["symmetric"], observer="minmax")
        t = torch.tensor([1.0, 1, 1, 1, 1]).reshape(1, 5)
        qp = oracle.WeightObserver(args)(t).get_qparams()
        assert round(qp["scale"].item(), 4) == case["scale"]
        assert round(qp["zero_point"].item(), 4) == case["zero_point"]


# ---------------------------------------------------------------- compressed-tensors
def test_ct_cases(golden):
    for name, c in golden["ct_cases"].items():
        if name == "nvfp4_fused3":
            continue
        args = spec_from(c["args"])
        w = c["weight"]
        mn, mx = oracle.observe_minmax(w, args)
        assert same(mn, c["min"]) and same(mx, c["max"]), name
        obs = oracle.WeightObserver(args)
        qp = obs(w).get_qparams()
        assert same(qp["scale"], c["scale"]), name
        assert same(qp["zero_point"], c["zero_point"]), name
        if c["global_scale"] is None:
            assert qp["global_scale"] is None
        else:
            assert same(qp["global_scale"], c["global_scale"]), name
        fq = oracle.fake_quantize(w, qp["scale"], qp["zero_point"], args, global_scale=qp["global_scale"])
        assert same(fq, c["fake_quant"]), name
        assert oracle.infer_format(args) == c["format"], name
        sd = {"weight": w, "weight_scale": qp["scale"].to(w.dtype), "weight_zero_point": qp["zero_point"]}
        if qp["global_scale"] is not None:
            sd["weight_global_scale"] = qp["global_scale"]
        out = oracle.compress_weight(sd, args)
        assert set(out) == set(c["compressed"]), (name, set(out), set(c["compressed"]))
        for k, v in c["compressed"].items():
            assert same(out[k], v), (name, k)


def test_fused_global_scale(golden):
    c = golden["ct_cases"]["nvfp4_fused3"]
    args = spec_from(c["args"])
    obs = [oracle.WeightObserver(args) for _ in c["weights"]]
    for o in obs:
        o.fused = [p for p in obs if p is not o]
    for o, w in zip(obs, c["weights"]):
        o(w)
    # statistics are consumed by get_qparams: read all global scales first, as the
    # reference's cooperative deletion allows
    gss = [o.get_global_scale() for o in obs]
    for o, gs, s_ref, g_ref in zip(obs, gss, c["scales"], c["global_scales"]):
        assert same(gs, g_ref)
        scale, _ = oracle.calculate_qparams(o.min_vals, o.max_vals, args, global_scale=gs)
        assert same(scale, s_ref)


def test_mse_cases(golden):
    for name, c in golden["mse_cases"].items():
        args = spec_from(c["args"])
        obs = oracle.WeightObserver(args, kind="memoryless_mse")
        obs(c["weight"])
        assert same(obs.min_vals, c["min"]) and same(obs.max_vals, c["max"]), name
        qp = obs.get_qparams()
        assert same(qp["scale"], c["scale"]), name


# ---------------------------------------------------------------- GPTQ
def test_hessian_cases(golden):
    for name, c in golden["hessian_cases"].items():
        K = c["x"].shape[-1]
        H = oracle.make_empty_hessian(K)
        n = torch.zeros(())
        H, n = oracle.accumulate_hessian(c["x"], H, n)
        H, n = oracle.accumulate_hessian(c["x"] * 0.5, H, n)
        assert torch.equal(n, c["n"]), name
        assert torch.equal(H, c["H"]), name


def test_running_mean_hessian_cases(sgpt_golden):
    """The oracle's running-mean Hessian against outputs of the reference's sgpt_sparsify.py."""
    for name, c in sgpt_golden["cases"].items():
        K = c["x"].shape[-1]
        H, n = oracle.make_empty_hessian(K), 0
        for factor, step in zip(c["factors"], c["steps"]):
            H, n = oracle.accumulate_hessian_running_mean(c["x"] * factor, H, n)
            assert n == step["n"], name
            assert same(H, step["H"]), name


def test_gptq_cases(golden):
    for name, c in golden["gptq_cases"].items():
        args = spec_from(c["args"])
        loss, out = oracle.quantize_weight(c["weight"], args, c["hessian"].clone(),
                                           blocksize=c["blocksize"], percdamp=c["percdamp"])
        ref = c["out"]
        assert set(out) == set(ref), (name, set(out), set(ref))
        for k in ref:
            assert same(out[k], ref[k]), (name, k)
        assert loss == pytest.approx(c["loss"], rel=1e-6), name


# ---------------------------------------------------------------- rounding rules
def test_rounding_rules_match_torch_casts():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(20000, generator=g) * torch.logspace(-12, 3, 20000)
    assert torch.equal(oracle.bf16_round(x), x.to(torch.bfloat16).float())
    y = torch.clamp(x, -448, 448)
    assert torch.equal(oracle.cast_e4m3(y), y.to(torch.float8_e4m3fn).float())
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.1, 0.0, -0.0, 7.0, -5.0])
    exp = torch.tensor([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, -0.0, -0.0, 0.0, 0.0, 6.0, -4.0])
    got = oracle.cast_e2m1(ties)
    assert torch.equal(got, exp)
    assert torch.equal(torch.signbit(got), torch.signbit(exp))


# ---------------------------------------------------------------- AWQ
def awq_parent(case):
    """``run_parent(weights) -> outputs`` of a fixture case: the parent modules the fixture was made with."""
    import torch.nn.functional as F
    if case["kind"] == "mlp":
        return lambda ws: [F.silu(F.linear(x, ws[0])) * F.linear(x, ws[1]) for x in case["batches"]]
    return lambda ws: [F.linear(x, ws[0]) for x in case["batches"]]


def test_awq_cases(awq_golden):
    """The oracle's AWQ search against the reference's own ``_compute_best_scale``: the same
    per-candidate losses and the same chosen scales, bit for bit (both run on the CPU)."""
    for name, c in awq_golden["cases"].items():
        spec = spec_from(c["args"])
        specs = [spec] * len(c["weights"])
        assert oracle.awq.grid_search_params(c["duo"], c["n_grid"]) == c["grid"], name
        if c["w_mean"] is not None:
            assert torch.equal(oracle.awq.layer_means(c["weights"], specs), c["w_mean"]), name
        best, losses = oracle.awq.best_scale(c["x_sum"], c["count"], c["weights"], specs, awq_parent(c),
                                             duo_scaling=c["duo"], n_grid=c["n_grid"],
                                             fused=spec.strategy == "tensor_group")
        assert losses == c["losses"], name
        assert best.dtype == c["best_scales"].dtype and torch.equal(best, c["best_scales"]), name
