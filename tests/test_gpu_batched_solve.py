"""Batched solve of many small problems (b200q_gptq_factor_batched, b200q_gptq_sweep_batched and
the GPTQModifier path that uses them) against float64, the single-problem kernels and the CPU
oracle.  Same tolerances as the single-problem tests: factors within a small multiple of the
float32 chain's own error, GPTQ weights with at least 99.5 % identical values, identical scales,
loss within 1 %."""
import warnings

import pytest
import torch

import oracle
from helpers import args_from, bits_equal, mismatch, synth_acts, synth_weight
from llm_compressor_b200 import GPTQModifier, gptq, observers, ops
from test_oracle_golden import spec_from

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CODE_MATCH = 0.995
LOSS_RTOL = 0.01


def _spd(K, seed):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(4 * K, K, generator=g) * (0.25 + 2 * torch.rand(K, generator=g))
    H = (2 * X.t() @ X / 4).float()
    H[torch.arange(K), torch.arange(K)] += 0.01 * H.diag().mean()
    return H


@pytest.mark.parametrize("K,count", [(32, 3), (128, 5), (130, 2), (200, 4), (768, 6), (1000, 2), (2048, 2)])
def test_batched_factor_matches_float64(K, count):
    Hs = [_spd(K, 100 * K + i) for i in range(count)]
    dev = [H.clone().to(DEV) for H in Hs]
    status = ops.gptq_factor_batched(dev).cpu()
    assert int(status.abs().max()) == 0
    for H, Hg in zip(Hs, dev):
        Hd = H.double()
        U_ref = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(Hd)), upper=True)
        U = Hg.cpu().double()
        assert float(U.tril(-1).abs().max()) == 0.0
        err = float((U - U_ref).norm() / U_ref.norm())
        U32 = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H.clone())), upper=True).double()
        err32 = float((U32 - U_ref).norm() / U_ref.norm())
        assert err < max(5e-5, 4 * err32), (err, err32)


def test_batched_factor_agrees_with_the_single_problem_kernel():
    K = 640
    Hs = [_spd(K, 7 + i).to(DEV) for i in range(3)]
    single = [H.clone() for H in Hs]
    for H in single:
        assert ops.gptq_factor(H) == 0
    ops.gptq_factor_batched(Hs)
    for a, b in zip(Hs, single):
        assert float((a - b).norm() / b.norm()) < 2e-5


def test_batched_factor_reports_the_failing_problem_only():
    K = 256
    Hs = [_spd(K, i) for i in range(4)]
    Hs[2][200, 200] = -5.0
    dev = [H.clone().to(DEV) for H in Hs]
    status = ops.gptq_factor_batched(dev).cpu()
    assert status[:, 0].tolist() == [0, 0, 1, 0]
    # reversed column order: column 200 of H is column K - 1 - 200 of the factored matrix
    assert int(status[2, 1]) == K - 1 - 200 + 1
    U_ref = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(Hs[3].double())), upper=True)
    assert float((dev[3].cpu().double() - U_ref).norm() / U_ref.norm()) < 5e-5


def _problem(N, K, seed, tokens_factor=2):
    w = synth_weight(N, K, seed=seed)
    S = min(K // 2, 512)
    x = synth_acts(max(8, -(-tokens_factor * K // S)), S, K, seed=seed + 1)
    H, n = oracle.accumulate_hessian(x, oracle.make_empty_hessian(K), 0)
    return w, H / n


def _lin(w, args):
    N, K = w.shape
    lin = torch.nn.Linear(K, N, bias=False, device=DEV, dtype=w.dtype)
    lin.weight.data = w.to(DEV)
    lin.weight_observer = observers.Observer.load_from_registry(args.observer, base_name="weight", args=args)
    lin.weight_observer(lin.weight.data)
    return lin


SCHEMES = {
    "W4A16": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128),
    "W4A16_ASYM": dict(num_bits=4, type="int", symmetric=False, strategy="group", group_size=128),
    "W8_CHANNEL": dict(num_bits=8, type="int", symmetric=True, strategy="channel"),
    "W4_ACTORDER_WEIGHT": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128,
                               actorder="weight"),
    "W4_ACTORDER_GROUP": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128,
                              actorder="group"),
}


@pytest.mark.parametrize("N,K,scheme,count", [(96, 256, "W4A16", 3), (200, 768, "W4A16", 3), (128, 640, "W4A16_ASYM", 2),
                                              (130, 384, "W8_CHANNEL", 2), (64, 1152, "W4_ACTORDER_WEIGHT", 2),
                                              (64, 512, "W4_ACTORDER_GROUP", 2), (300, 2048, "W4A16", 2)])
def test_batched_gptq_vs_oracle(N, K, scheme, count):
    args = args_from(SCHEMES[scheme])
    problems = [_problem(N, K, seed=31 * N + K + 5 * i) for i in range(count)]
    mods = [_lin(w, args) for w, _ in problems]
    factors = gptq.factor_hessians_batched([H.clone().to(DEV) for _, H in problems], 0.01, args.actorder)
    done = gptq.quantize_weights_batched(mods, args, factors)
    gptq.resolve_factors(factors)
    assert all(f.ok for f in factors)
    for (w, H), (loss, out) in zip(problems, done):
        loss_ref, ref = oracle.quantize_weight(w, _oracle_spec(scheme), H.clone())
        assert bits_equal(out["weight_scale"], ref["weight_scale"])
        assert bits_equal(out["weight_zero_point"], ref["weight_zero_point"])
        if "weight_g_idx" in ref:
            assert torch.equal(out["weight_g_idx"].cpu().long(), ref["weight_g_idx"].long())
        mm = mismatch(out["weight"], ref["weight"])
        assert mm <= 1 - CODE_MATCH, mm
        assert float(loss) == pytest.approx(loss_ref, rel=LOSS_RTOL)


def _oracle_spec(scheme):
    return spec_from(dict(SCHEMES[scheme]))


def test_batched_sweep_agrees_with_the_single_problem_kernel():
    N, K = 160, 896
    args = args_from(SCHEMES["W4A16"])
    problems = [_problem(N, K, seed=11 + i) for i in range(3)]
    single = []
    for w, H in problems:
        lin = _lin(w, args)
        single.append(gptq.quantize_weight(lin, args, H.clone().to(DEV)))
    mods = [_lin(w, args) for w, _ in problems]
    factors = gptq.factor_hessians_batched([H.clone().to(DEV) for _, H in problems], 0.01, None)
    done = gptq.quantize_weights_batched(mods, args, factors)
    for (loss_a, a), (loss_b, b) in zip(done, single):
        assert bits_equal(a["weight_scale"], b["weight_scale"])
        assert mismatch(a["weight"], b["weight"]) <= 1 - CODE_MATCH
        assert float(loss_a) == pytest.approx(loss_b, rel=LOSS_RTOL)


def test_batched_sweep_without_factor_equals_the_single_problem_fallback():
    # no factor: the identity stands in for U (round to nearest); no trailing update runs, so the
    # two kernels must agree bit for bit
    N, K = 70, 256
    args = args_from(SCHEMES["W4A16"])
    ws = [synth_weight(N, K, seed=i) for i in range(2)]
    mods = [_lin(w, args) for w in ws]
    wf = [ops.gather_columns_f32(m.weight.data) for m in mods]
    qp = [m.weight_observer.get_qparams() for m in mods]
    losses = ops.gptq_sweep_batched(wf, None, [q["scale"] for q in qp], [q["zero_point"] for q in qp], args)
    for i, (m, f, q) in enumerate(zip(mods, wf, qp)):
        ref = ops.gather_columns_f32(m.weight.data)
        ref_losses = ops.gptq_sweep(ref, None, q["scale"], q["zero_point"], args)
        assert torch.equal(f, ref)
        assert torch.allclose(losses[i], ref_losses, rtol=1e-5, atol=0)


class _Experts(torch.nn.Module):
    def __init__(self, count, hidden, inter):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.up = torch.nn.ModuleList(torch.nn.Linear(hidden, inter, bias=False) for _ in range(count))
        self.down = torch.nn.ModuleList(torch.nn.Linear(inter, hidden, bias=False) for _ in range(count))
        for m in list(self.up) + list(self.down):
            m.weight.data = torch.randn(m.weight.shape, generator=g) * 0.05

    def forward(self, x):
        # every expert sees its own slice of the tokens
        parts = x.chunk(len(self.up), dim=1)
        return torch.cat([d(torch.nn.functional.silu(u(p))) for u, d, p in zip(self.up, self.down, parts)], dim=1)


@pytest.mark.parametrize("fail_one", [False, True])
def test_modifier_takes_the_batched_path_for_many_small_hessians(fail_one):
    count, hidden, inter = 6, 256, 384
    torch.manual_seed(0)
    x = (torch.randn(4, count * 640, hidden) * (0.5 + torch.rand(hidden))).to(torch.bfloat16).to(DEV)

    def run(batch):
        model = _Experts(count, hidden, inter).to(torch.bfloat16).to(DEV)
        mod = GPTQModifier(targets="Linear", scheme="W4A16", batch_small_hessians=batch)
        events = []
        mod.trace = lambda e, m=None: events.append(e)
        mod.on_initialize(model)
        mod.on_calibration_start(model)
        with torch.no_grad():
            model(x)
        if fail_one:
            g = mod._groups[model.up[2]]
            g.flush()
            g.H.zero_()
            g.H.diagonal().fill_(1.0)
            g.H[3, 3] = -4.0
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            mod.on_sequential_epoch_end(model, list(model.up) + list(model.down))
        mod.on_calibration_end(model)
        mod.on_finalize(model)
        return model, mod, events, [str(w.message) for w in caught]

    base_model, base, base_events, base_warn = run(0)
    model, mod, events, warned = run(4)
    # one factor event per Hessian either way; the batched run raises them before any sweep
    assert events.count("job_factored") == 2 * count
    assert events.count("job_start") == 1 and base_events.count("job_start") == 2 * count
    assert any("round-to-nearest" in w for w in warned) == fail_one
    assert any("round-to-nearest" in w for w in base_warn) == fail_one
    for (name, a), (_, b) in zip(model.named_modules(), base_model.named_modules()):
        if not isinstance(a, torch.nn.Linear):
            continue
        assert a.quantization_status == "frozen"
        assert bits_equal(a.weight_scale, b.weight_scale)
        assert mismatch(a.weight.data, b.weight.data) <= 1 - CODE_MATCH, name
    for name, loss in mod.losses.items():
        assert loss == pytest.approx(base.losses[name], rel=LOSS_RTOL, abs=1e-9), name
