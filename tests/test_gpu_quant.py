"""Observer / qparams / quantize / pack kernels against the golden fixtures (outputs of
the reference on the same inputs) and against the CPU oracle on larger seeded inputs.
Everything goes through the C ABI (ctypes) and must be bit-exact."""
import pytest
import torch

import oracle
from helpers import args_from, bits_equal, mismatch, synth_weight
from llm_compressor_b200 import compressors, observers, ops
from test_oracle_golden import spec_from

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SCHEMES = ["w4a16_g128", "w4a16_g32", "w4a16_asym_g128", "w4_channel", "w4_tensor", "w8a16_channel",
           "w8_asym_channel", "w8_g128", "fp8_channel", "fp8_tensor", "fp8_block", "nvfp4", "mxfp4",
           "mxfp8"]


@pytest.mark.parametrize("name", SCHEMES)
def test_golden_observer_qparams_quantize_pack(golden, name):
    c = golden["ct_cases"][name]
    args = args_from(c["args"])
    w = c["weight"].to(DEV)
    mn, mx = ops.observe_minmax(w, args)
    assert bits_equal(mn, c["min"]) and bits_equal(mx, c["max"])
    obs = observers.Observer.load_from_registry("memoryless_minmax", base_name="weight", args=args)
    qp = obs(w).get_qparams()
    assert bits_equal(qp["scale"], c["scale"])
    assert bits_equal(qp["zero_point"], c["zero_point"])
    if c["global_scale"] is None:
        assert qp["global_scale"] is None
    else:
        assert bits_equal(qp["global_scale"], c["global_scale"])
    fq = ops.fake_quantize(w, qp["scale"], qp["zero_point"], args, global_scale=qp["global_scale"])
    assert bits_equal(fq, c["fake_quant"].to(w.dtype)), mismatch(fq, c["fake_quant"].to(w.dtype))
    assert compressors.infer_module_format(args) == c["format"]
    sd = {"weight": w, "weight_scale": qp["scale"].to(w.dtype), "weight_zero_point": qp["zero_point"]}
    if qp["global_scale"] is not None:
        sd["weight_global_scale"] = qp["global_scale"]
    out = compressors.compress_state_dict(sd, args)
    assert set(out) == set(c["compressed"])
    for k, v in c["compressed"].items():
        assert bits_equal(out[k], v), (k, mismatch(out[k], v))


@pytest.mark.parametrize("name", SCHEMES)
@pytest.mark.parametrize("shape", [(256, 1024), (7, 40), (64, 2048)])
def test_oracle_parity_larger(golden, name, shape):
    args = args_from(golden["ct_cases"][name]["args"])
    N, K = shape
    if args.strategy in ("group", "tensor_group") and K % args.group_size:
        pytest.skip("group size does not divide K")
    spec = spec_from(golden["ct_cases"][name]["args"])
    w = synth_weight(N, K, seed=N * 7 + K)
    wd = w.to(DEV)
    o = oracle.WeightObserver(spec)
    o(w)
    omn, omx = o.min_vals.clone(), o.max_vals.clone()
    oqp = o.get_qparams()
    mn, mx = ops.observe_minmax(wd, args)
    assert bits_equal(mn, omn) and bits_equal(mx, omx)
    obs = observers.MemorylessMinMaxObserver("weight", args)
    qp = obs(wd).get_qparams()
    assert bits_equal(qp["scale"], oqp["scale"])
    assert bits_equal(qp["zero_point"], oqp["zero_point"])
    ofq = oracle.fake_quantize(w, oqp["scale"], oqp["zero_point"], spec, global_scale=oqp["global_scale"])
    fq = ops.fake_quantize(wd, qp["scale"], qp["zero_point"], args, global_scale=qp["global_scale"])
    assert bits_equal(fq, ofq.to(w.dtype)), mismatch(fq, ofq.to(w.dtype))
    if args.type == "float" and args.num_bits == 4 and K % 2:
        return
    sd = {"weight": w, "weight_scale": oqp["scale"].to(w.dtype), "weight_zero_point": oqp["zero_point"]}
    if oqp["global_scale"] is not None:
        sd["weight_global_scale"] = oqp["global_scale"]
    ref = oracle.compress_weight(sd, spec)
    out = compressors.compress_state_dict({k: v.to(DEV) for k, v in sd.items()}, args)
    assert set(out) == set(ref)
    for k, v in ref.items():
        assert bits_equal(out[k], v), (k, mismatch(out[k], v))


@pytest.mark.parametrize("name", ["w4a16_g128", "w4a16_g32", "w4a16_asym_g128", "w8_g128", "w8a16_channel",
                                  "w4_channel", "fp8_channel", "mxfp4", "mxfp8"])
def test_fused_rtn_matches_unfused(golden, name):
    """One-pass statistics -> qparams -> codes equals the observer + compressor sequence."""
    args = args_from(golden["ct_cases"][name]["args"])
    spec = spec_from(golden["ct_cases"][name]["args"])
    w = synth_weight(128, 1024, seed=11)
    o = oracle.WeightObserver(spec)
    oqp = o(w).get_qparams()
    sd = {"weight": w, "weight_scale": oqp["scale"].to(w.dtype), "weight_zero_point": oqp["zero_point"]}
    ref = oracle.compress_weight(sd, spec)
    r = ops.rtn_quantize_pack(w.to(DEV), args)
    assert bits_equal(r["scale"], oqp["scale"].to(w.dtype))
    assert bits_equal(r["zero_point"], oqp["zero_point"])
    codes = r["codes"]
    if "weight_packed" in ref:
        assert bits_equal(codes, ref["weight_packed"]), mismatch(codes, ref["weight_packed"])
    else:
        exp = ref["weight"]
        if exp.dtype == torch.int8:  # fused path packs int8 four to a word
            exp = oracle.pack_int32(exp, 8)
        assert bits_equal(codes, exp), mismatch(codes, exp)
    if args.is_mx:
        assert bits_equal(r["scale_store"], ref["weight_scale"])


@pytest.mark.parametrize("name", ["fp8_channel", "w4_channel", "w8a16_channel"])
@pytest.mark.parametrize("N,K", [(3, 8), (5, 2056), (33, 14336), (3, 28672), (4, 40960)])
def test_fused_rtn_channel_row_lengths(golden, name, N, K):
    """Rows from one chunk to more than the register-resident kernel holds (which falls back)."""
    args = args_from(golden["ct_cases"][name]["args"])
    spec = spec_from(golden["ct_cases"][name]["args"])
    w = synth_weight(N, K, seed=N + K)
    oqp = oracle.WeightObserver(spec)(w).get_qparams()
    ref = oracle.compress_weight({"weight": w, "weight_scale": oqp["scale"].to(w.dtype),
                                  "weight_zero_point": oqp["zero_point"]}, spec)
    r = ops.rtn_quantize_pack(w.to(DEV), args)
    assert bits_equal(r["scale"], oqp["scale"].to(w.dtype))
    assert bits_equal(r["zero_point"], oqp["zero_point"])
    if "weight_packed" in ref:
        assert bits_equal(r["codes"], ref["weight_packed"])
    else:
        exp = ref["weight"]
        if exp.dtype == torch.int8:
            exp = oracle.pack_int32(exp, 8)
        assert bits_equal(r["codes"], exp)


def test_fused_nvfp4_and_shared_global_scale(golden):
    c = golden["ct_cases"]["nvfp4_fused3"]
    args = args_from(c["args"])
    mods = []
    for w in c["weights"]:
        m = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device=DEV, dtype=w.dtype)
        m.weight.data = w.to(DEV)
        m.weight_observer = observers.MemorylessMinMaxObserver("weight", args)
        mods.append(m)
    observers.fuse_observers([(m.weight_observer, m) for m in mods])
    for m in mods:
        m.weight_observer(m.weight.data)
    qps = [m.weight_observer.get_qparams() for m in mods]
    for qp, s_ref, g_ref in zip(qps, c["scales"], c["global_scales"]):
        assert bits_equal(qp["global_scale"], g_ref)
        assert bits_equal(qp["scale"], s_ref)
    assert all(not m.weight_observer.has_statistics for m in mods)
    # one-pass NVFP4 with the shared scale equals the oracle's compress
    spec = spec_from(c["args"])
    for m, qp in zip(mods, qps):
        w = m.weight.data.cpu()
        sd = {"weight": w, "weight_scale": qp["scale"].cpu().to(w.dtype),
              "weight_zero_point": qp["zero_point"].cpu(), "weight_global_scale": qp["global_scale"].cpu()}
        ref = oracle.compress_weight(sd, spec)
        r = ops.nvfp4_quantize_pack(m.weight.data, qp["global_scale"])
        assert bits_equal(r["codes"], ref["weight_packed"])
        assert bits_equal(r["scale_store"], ref["weight_scale"])


def test_actorder_g_idx_pack(golden):
    """pack with a column -> group map (act-order "group") equals the oracle."""
    spec = oracle.preset("W4A16")
    args = args_from(dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128))
    w = synth_weight(32, 512, seed=5)
    g = torch.Generator().manual_seed(0)
    perm = torch.randperm(512, generator=g)
    g_idx = (torch.arange(512) // 128)[torch.argsort(perm)].to(torch.int32)
    o = oracle.WeightObserver(spec)
    oqp = o(w[:, perm].contiguous()).get_qparams()
    sd = {"weight": w, "weight_scale": oqp["scale"], "weight_zero_point": oqp["zero_point"], "weight_g_idx": g_idx}
    ref = oracle.compress_weight(sd, spec)
    out = compressors.compress_state_dict({k: v.to(DEV) for k, v in sd.items()}, args)
    assert bits_equal(out["weight_packed"], ref["weight_packed"])


def test_rejects_cpu_tensors():
    from llm_compressor_b200._lib import B200QError
    args = args_from(dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128))
    with pytest.raises(B200QError):
        ops.observe_minmax(torch.zeros(4, 128, dtype=torch.bfloat16), args)


@pytest.mark.parametrize("name", ["w4a16_g128", "w4a16_g32", "w4a16_asym_g128", "w8_g128", "w8a16_channel", "w4_channel",
                                  "fp8_channel", "mxfp4", "mxfp8"])
@pytest.mark.parametrize("seed", [0, 1])
def test_fused_rtn_on_rounding_boundaries(golden, name, seed):
    """Weights placed on (and one bf16 step beside) the rounding boundaries of the code grid: the
    reciprocal-multiply fast paths must fall back to the exact division wherever it matters."""
    args = args_from(golden["ct_cases"][name]["args"])
    spec = spec_from(golden["ct_cases"][name]["args"])
    g = torch.Generator().manual_seed(100 + seed)
    N, K = 64, 1024
    base = torch.rand(N, 1, generator=g) * 0.05 + 1e-3                      # per-row magnitude
    steps = torch.randint(-31, 32, (N, K), generator=g).float() * 0.5       # multiples of half a code step
    w = (steps * base / 7.5).to(torch.bfloat16)
    # neighbours one bf16 ulp up / down on a third of the entries each
    bits = w.view(torch.int16).clone()
    sel = torch.randint(0, 3, (N, K), generator=g) * (w != 0)               # zeros stay zeros (no NaN patterns)
    bits = torch.where(sel == 1, bits + 1, torch.where(sel == 2, bits - 1, bits))
    w = bits.view(torch.bfloat16).clone()
    assert bool(torch.isfinite(w.float()).all())
    w[:, 0] = (base[:, 0] * 2.0).to(torch.bfloat16)                         # a row maximum that fixes the scale
    w[0, 5] = -0.0
    w[1, 7] = 0.0
    o = oracle.WeightObserver(spec)
    oqp = o(w).get_qparams()
    ref = oracle.compress_weight({"weight": w, "weight_scale": oqp["scale"].to(w.dtype),
                                  "weight_zero_point": oqp["zero_point"]}, spec)
    r = ops.rtn_quantize_pack(w.to(DEV), args)
    assert bits_equal(r["scale"], oqp["scale"].to(w.dtype))
    assert bits_equal(r["zero_point"], oqp["zero_point"])
    if "weight_packed" in ref:
        assert bits_equal(r["codes"], ref["weight_packed"]), mismatch(r["codes"], ref["weight_packed"])
    else:
        exp = ref["weight"]
        if exp.dtype == torch.int8:
            exp = oracle.pack_int32(exp, 8)
        assert bits_equal(r["codes"], exp), mismatch(r["codes"], exp)
    # the unfused path (observer -> qparams -> quantize_pack) on the same data
    mn, mx = ops.observe_minmax(w.to(DEV), args)
    scale, zp = ops.qparams(mn, mx, args)
    packed = ops.quantize_pack(w.to(DEV), scale, zp, args, pack_int8=True)
    a, b = packed.contiguous().view(torch.uint8).flatten(), r["codes"].contiguous().view(torch.uint8).flatten()
    assert a.numel() == b.numel() and torch.equal(a, b)


def test_nvfp4_on_rounding_boundaries():
    spec = oracle.preset("NVFP4A16")
    g = torch.Generator().manual_seed(7)
    N, K = 64, 1024
    grid = torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0])
    idx = torch.randint(0, len(grid), (N, K), generator=g)
    sign = torch.randint(0, 2, (N, K), generator=g).float() * 2 - 1
    blk = (torch.rand(N, K // 16, generator=g) * 0.04 + 1e-3).repeat_interleave(16, dim=1)
    w = (grid[idx] * sign * blk / 6.0).to(torch.bfloat16)
    bits = w.view(torch.int16).clone()
    sel = torch.randint(0, 3, (N, K), generator=g) * (w != 0)
    w = torch.where(sel == 1, bits + 1, torch.where(sel == 2, bits - 1, bits)).view(torch.bfloat16).clone()
    assert bool(torch.isfinite(w.float()).all())
    w[:, ::16] = blk[:, ::16].to(torch.bfloat16)          # block maxima
    o = oracle.WeightObserver(spec)
    oqp = o(w).get_qparams()
    ref = oracle.compress_weight({"weight": w, "weight_scale": oqp["scale"], "weight_zero_point": oqp["zero_point"],
                                  "weight_global_scale": oqp["global_scale"]}, spec)
    r = ops.nvfp4_quantize_pack(w.to(DEV), oqp["global_scale"].to(DEV))
    assert bits_equal(r["codes"], ref["weight_packed"]), mismatch(r["codes"], ref["weight_packed"])
    assert bits_equal(r["scale_store"], ref["weight_scale"])


def test_pack_fp4_to_uint8_helper():
    """The stand-alone packing helper on every E2M1 value of both signs (-0.0 included)."""
    from llm_compressor_b200 import compressors
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    vals = torch.cat([vals, -vals])
    g = torch.Generator().manual_seed(3)
    x = vals[torch.randint(0, 16, (37, 96), generator=g)]
    for dtype in (torch.bfloat16, torch.float32):
        got = compressors.pack_fp4_to_uint8(x.to(dtype).to(DEV))
        assert got.dtype == torch.uint8 and tuple(got.shape) == (37, 48)
        assert torch.equal(got.cpu(), oracle.pack_fp4(x.to(dtype)))
    with pytest.raises(ValueError, match="even number of columns"):
        compressors.pack_fp4_to_uint8(x[:, :5].to(DEV))


@pytest.mark.parametrize("N,K", [(64, 512), (300, 1024)])
def test_nvfp4_two_pass_equals_observer_then_compressor(N, K):
    """amax pass + fused NVFP4 pass (alone, and with fused partners sharing the global scale) equals
    observer -> calculate_qparams -> NVFP4 compressor of the oracle, bit for bit."""
    spec = oracle.preset("NVFP4A16")
    w = synth_weight(N, K, seed=N + K)
    p = synth_weight(N // 2, K, seed=N + K + 1) * 3
    for partners in ([], [p]):
        obs = [oracle.WeightObserver(spec) for _ in range(1 + len(partners))]
        for i, o in enumerate(obs):
            o.fused = [q for j, q in enumerate(obs) if j != i]
        for o, t in zip(obs, [w] + partners):
            o(t)
        qp = obs[0].get_qparams()
        ref = oracle.compress_weight({"weight": w, "weight_scale": qp["scale"].to(w.dtype),
                                      "weight_zero_point": qp["zero_point"],
                                      "weight_global_scale": qp["global_scale"]}, spec)
        r = ops.nvfp4_two_pass(w.to(DEV), [t.to(DEV) for t in partners])
        assert bits_equal(r["global_scale"], qp["global_scale"])
        assert bits_equal(r["codes"], ref["weight_packed"])
        assert bits_equal(r["scale_store"], ref["weight_scale"])


@pytest.mark.parametrize("name", ["w4a16_g128", "w4a16_g32", "w4a16_asym_g128", "w8_g128", "mxfp4", "mxfp8"])
@pytest.mark.parametrize("N,K", [(5, 2048), (300, 4096), (64, 14336)])
def test_fused_rtn_whole_tile_rows(golden, name, N, K):
    """Rows made of whole 2048-element tiles take the TMA-fed kernel: same bits as the oracle."""
    args = args_from(golden["ct_cases"][name]["args"])
    spec = spec_from(golden["ct_cases"][name]["args"])
    w = synth_weight(N, K, seed=N + K + 1)
    oqp = oracle.WeightObserver(spec)(w).get_qparams()
    ref = oracle.compress_weight({"weight": w, "weight_scale": oqp["scale"].to(w.dtype),
                                  "weight_zero_point": oqp["zero_point"]}, spec)
    r = ops.rtn_quantize_pack(w.to(DEV), args)
    assert bits_equal(r["scale"], oqp["scale"].to(w.dtype))
    assert bits_equal(r["zero_point"], oqp["zero_point"])
    if "weight_packed" in ref:
        assert bits_equal(r["codes"], ref["weight_packed"]), mismatch(r["codes"], ref["weight_packed"])
    else:
        exp = ref["weight"]
        if exp.dtype == torch.int8:
            exp = oracle.pack_int32(exp, 8)
        assert bits_equal(r["codes"], exp), mismatch(r["codes"], exp)
    if args.is_mx:
        assert bits_equal(r["scale_store"], ref["weight_scale"])
    from llm_compressor_b200 import _lib
    assert _lib.load().b200q_take_wait_status() == 0


@pytest.mark.parametrize("N,K", [(7, 2048), (130, 6144)])
def test_fused_nvfp4_whole_tile_rows(N, K):
    spec = oracle.preset("NVFP4A16")
    w = synth_weight(N, K, seed=N + K)
    obs = oracle.WeightObserver(spec)
    obs(w)
    qp = obs.get_qparams()
    ref = oracle.compress_weight({"weight": w, "weight_scale": qp["scale"].to(w.dtype), "weight_zero_point": qp["zero_point"],
                                  "weight_global_scale": qp["global_scale"]}, spec)
    r = ops.nvfp4_quantize_pack(w.to(DEV), qp["global_scale"].to(DEV))
    assert bits_equal(r["codes"], ref["weight_packed"])
    assert bits_equal(r["scale_store"], ref["weight_scale"])
    assert bits_equal(r["scale"], qp["scale"].to(w.dtype))


def test_bounded_wait_that_runs_out_is_reported_and_nothing_hangs(monkeypatch):
    """Failure made on the host: one warp of the TMA-fed kernel is told to leave out one of its tile
    requests, so its wait for that tile runs into the bound (about a second).  The kernel must
    return, the library must report B200Q_ERR_DEVICE once, and the next call must work."""
    from llm_compressor_b200 import _lib
    lib = _lib.load()
    args = args_from(dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128))
    w = synth_weight(4096, 4096, seed=1).to(DEV)     # several tiles per warp
    good = ops.rtn_quantize_pack(w, args)
    assert lib.b200q_take_wait_status() == 0
    monkeypatch.setenv("B200Q_TEST_DROP_TILE", "1")
    bad = ops.rtn_quantize_pack(w, args)
    torch.cuda.synchronize()
    monkeypatch.delenv("B200Q_TEST_DROP_TILE")
    assert lib.b200q_take_wait_status() == _lib.C.c_int(-4).value      # B200Q_ERR_DEVICE, once
    assert lib.b200q_take_wait_status() == 0
    del bad                                                             # incomplete by construction
    again = ops.rtn_quantize_pack(w, args)
    assert torch.equal(again["codes"], good["codes"]) and lib.b200q_take_wait_status() == 0
