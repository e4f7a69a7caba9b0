"""Host logic of the modifiers, matching rules and the multi-rank plumbing (gloo, CPU)."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from llm_compressor_b200 import dist as bdist
from llm_compressor_b200.modifiers import GPTQModifier, QuantizationModifier, match_named_modules


class Attn(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = torch.nn.Linear(256, 256, bias=False)
        self.k_proj = torch.nn.Linear(256, 64, bias=False)
        self.v_proj = torch.nn.Linear(256, 64, bias=False)


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = torch.nn.Embedding(10, 256)
        self.attn = Attn()
        self.gate = torch.nn.Linear(256, 8, bias=False)
        self.lm_head = torch.nn.Linear(256, 10, bias=False)


def test_match_named_modules_rules():
    m = Tiny()
    names = [n for n, _ in match_named_modules(m, ["Linear"], ["lm_head"])]
    assert names == ["attn.q_proj", "attn.k_proj", "attn.v_proj", "gate"]
    names = [n for n, _ in match_named_modules(m, ["Linear"], ["lm_head", "re:.*gate$"])]
    assert "gate" not in names
    assert [n for n, _ in match_named_modules(m, ["re:attn\\..*"], [])] == ["attn.q_proj", "attn.k_proj", "attn.v_proj"]
    assert [n for n, _ in match_named_modules(m, ["attn.q_proj"], [])] == ["attn.q_proj"]


def test_scheme_resolution_and_actorder_defaults():
    g = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"])
    groups = g.resolve_quantization_config()
    assert list(groups) == ["group_0"]
    assert groups["group_0"].weights.actorder == "weight"  # reference default "static"
    assert GPTQModifier(scheme="W4A16", actorder=None).resolve_quantization_config()["group_0"].weights.actorder is None
    assert GPTQModifier(scheme="W4A16", actorder="group").resolve_quantization_config()["group_0"].weights.actorder == "group"
    # channel strategy: static permutes, group falls back to None
    assert GPTQModifier(scheme="FP8_DYNAMIC").resolve_quantization_config()["group_0"].weights.actorder == "weight"
    with pytest.warns(UserWarning):
        a = GPTQModifier(scheme="W8A16", actorder="group").resolve_quantization_config()["group_0"].weights.actorder
    assert a is None
    with pytest.raises(ValueError):
        GPTQModifier(scheme="W4A16", config_groups={"g": {"targets": ["Linear"]}}).resolve_quantization_config()
    with pytest.raises(ValueError):
        QuantizationModifier(scheme="W4A16", weight_observer="mse", observer={"weights": "mse"}).resolve_quantization_config()
    q = QuantizationModifier(scheme="W4A16", weight_observer="mse").resolve_quantization_config()
    assert q["group_0"].weights.observer == "mse"


def test_initialize_attaches_params_and_checks_divisibility():
    m = Tiny().to(torch.bfloat16)
    mod = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head", "gate"])
    mod.on_initialize(m)
    assert m.attn.q_proj.weight_scale.shape == (256, 2) and m.attn.q_proj.weight_scale.dtype == torch.bfloat16
    assert m.attn.k_proj.weight_zero_point.dtype == torch.int8
    assert not hasattr(m.lm_head, "weight_scale") and not hasattr(m.embed, "weight_scale")
    m2 = Tiny()
    m2.odd = torch.nn.Linear(200, 8, bias=False)
    with pytest.raises(ValueError, match="not divisible"):
        GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"]).on_initialize(m2)
    m3 = Tiny()
    nv = QuantizationModifier(targets="Linear", scheme="NVFP4A16", ignore=["lm_head"])
    nv.on_initialize(m3)
    assert m3.attn.q_proj.weight_global_scale.dtype == torch.float32


def test_gptq_requires_targets():
    m = Tiny()
    mod = GPTQModifier(targets="Conv2d", scheme="W4A16")
    mod.on_initialize(m)
    with pytest.raises(ValueError):
        mod.on_calibration_start(m)


def test_greedy_bin_packing_and_partition():
    items = ["a", "b", "c", "d", "e"]
    w = {"a": 4096, "b": 14336, "c": 4096, "d": 4096, "e": 1024}
    it, bins, where = bdist.greedy_bin_packing(items, 2, item_weight_fn=lambda k: w[k])
    assert it[0] == "b" and where["b"] == 0
    assert sum(w[k] for k in bins[0]) == 14336 and sum(w[k] for k in bins[1]) == 4096 * 3 + 1024
    assert [len(bdist.partition_samples(10, r, 4)) for r in range(4)] == [2, 3, 2, 3]
    assert list(bdist.partition_samples(10, 1, 4)) == [2, 3, 4]


class _G:
    def __init__(self, K, val):
        self.H = torch.full((K, K), float(val))
        self.n = 3.0
        self.device = torch.device("cpu")

    def __hash__(self):
        return id(self)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    try:
        groups = [_G(8, rank + 1), _G(16, 10 * (rank + 1))]
        items, bins, where = bdist.greedy_bin_packing(list(groups), world, item_weight_fn=lambda g: g.H.shape[0])
        order = {id(g): i for i, g in enumerate(groups)}
        everyone = _G(4, 100 * (rank + 1))      # a Hessian every rank wants (owner None): all-reduced
        where[everyone] = None
        bdist.reduce_hessians(items + [everyone], where)
        assert float(everyone.H[0, 0]) == 300.0 and everyone.n == 6.0
        res = {}
        for g in groups:
            owner = where[g]
            if owner == rank:
                res[order[id(g)]] = (float(g.H[0, 0]), g.n)
            else:
                assert g.H is None
        # activation statistics: min / max observers combine with MIN / MAX, moving averages with AVG
        from llm_compressor_b200.observers import MinMaxObserver, StaticMinMaxObserver
        from llm_compressor_b200.quant_args import QuantizationArgs
        act = QuantizationArgs(num_bits=8, type="float", strategy="tensor", dynamic=False)
        so, mo = StaticMinMaxObserver("input", act), MinMaxObserver("input", act)
        for o in (so, mo):
            o.min_vals, o.max_vals = torch.tensor([-1.0 - rank]), torch.tensor([2.0 + 2 * rank])
        bdist.wait_for_comms(so.sync_activation_stats() + mo.sync_activation_stats())
        assert (float(so.min_vals), float(so.max_vals)) == (-2.0, 4.0)
        assert (float(mo.min_vals), float(mo.max_vals)) == (-1.5, 3.0)
        lin = torch.nn.Linear(4, 4, bias=False)
        lin.weight.data.fill_(float(rank + 5))
        lin.weight_scale = torch.nn.Parameter(torch.full((4, 1), float(rank)), requires_grad=False)
        bdist.broadcast_module_params([lin], {lin: 1}, ("weight", "weight_scale", "weight_g_idx"))
        # many tensors of two owners, mixed dtypes (float8 travels as bytes), one non-contiguous, and a
        # bucket limit small enough to need several buckets per owner
        g = torch.Generator().manual_seed(7)
        mods, owner = [], {}
        for i in range(6):
            m = torch.nn.Module()
            src = torch.randn(5, 3 + i, generator=g)
            m.weight = torch.nn.Parameter((src if rank == i % 2 else torch.zeros_like(src)).to(torch.bfloat16),
                                          requires_grad=False)
            sc = torch.rand(5, 1, generator=g) + 0.5
            m.weight_scale = torch.nn.Parameter(sc if rank == i % 2 else torch.zeros_like(sc), requires_grad=False)
            zp = (torch.rand(5, 1, generator=g) * 4).to(torch.float8_e4m3fn)
            m.weight_zero_point = torch.nn.Parameter(zp if rank == i % 2 else torch.zeros_like(zp), requires_grad=False)
            gi = torch.arange(2 * (3 + i), dtype=torch.int32)[::2]          # not contiguous
            m.weight_g_idx = torch.nn.Parameter(gi if rank == i % 2 else torch.zeros_like(gi), requires_grad=False)
            m.expect = (src.to(torch.bfloat16), sc, zp, gi.clone())
            mods.append(m)
            owner[m] = i % 2
        old_limit, bdist._BUCKET_BYTES = bdist._BUCKET_BYTES, 96
        try:
            bdist.broadcast_module_params(mods, owner, ("weight", "weight_scale", "weight_zero_point", "weight_g_idx"))
        finally:
            bdist._BUCKET_BYTES = old_limit
        for m in mods:
            w, sc, zp, gi = m.expect
            assert torch.equal(m.weight.data, w) and torch.equal(m.weight_scale.data, sc)
            assert torch.equal(m.weight_zero_point.data.view(torch.uint8), zp.view(torch.uint8))
            assert torch.equal(m.weight_g_idx.data, gi)
        q.put((rank, res, float(lin.weight[0, 0]), float(lin.weight_scale[0, 0])))
    finally:
        torch.distributed.destroy_process_group()


def test_reduce_and_broadcast_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    merged = {}
    for rank, res, w, s in out:
        merged.update(res)
        assert w == 6.0 and s == 1.0  # values of rank 1 everywhere
    assert merged[0] == (3.0, 6.0)    # 1 + 2, samples 3 + 3
    assert merged[1] == (30.0, 6.0)   # 10 + 20


def _failing_worker(rank, world, port, q):
    """Rank 1 raises before the reduction (a host-made failure); rank 0 must get an error from the
    collective within the process group's timeout instead of waiting forever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world,
                                         timeout=datetime.timedelta(seconds=5))
    t0 = time.time()
    try:
        if rank == 1:
            raise RuntimeError("calibration failed on this rank")
        groups = [_G(8, 1.0)]
        bdist.reduce_hessians(groups, {groups[0]: 0})
        q.put((rank, "completed", time.time() - t0))
    except RuntimeError as e:
        q.put((rank, "error: " + str(e)[:80], time.time() - t0))


def test_rank_that_fails_before_the_reduction_does_not_hang_the_others():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 7) % 1000
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict((r, (what, dt)) for r, what, dt in [q.get(timeout=120) for _ in procs])
    for p in procs:
        p.join(timeout=60)
    assert out[1][0].startswith("error: calibration failed")
    assert out[0][0].startswith("error"), out[0]      # the survivor's collective ended with an error ...
    assert out[0][1] < 60, out[0]                      # ... within the short timeout, not the default 30 minutes
