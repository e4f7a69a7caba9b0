"""Benchmark of the calibrate-and-quantize hot path on B200.

Workload (BASELINE.json configs[2]): GPTQ W4A16, symmetric int4, group 128, block 128,
dampening 0.01, no act-order, on a Llama-3-8B-shaped decoder (hidden 4096, intermediate
14336, 32 query / 8 KV heads, 32 layers) with 512 x 2048 calibration tokens.

One STEP is the hot path of one decoder layer: accumulate the Hessians of its four distinct
Linear inputs over all 1,048,576 calibration tokens, then for its seven Linear modules observe,
factor, sweep and pack to int4.  Weights and activations are synthetic (seeded normal,
per-column scales); every layer has the same shapes, so the metric - wall seconds of the hot
path for the 32-layer model - is 32 x the mean step time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Under torchrun (N > 1) the calibration sequences are split across ranks, partial Hessians are
sum-reduced (NCCL) to the rank that owns each Hessian, owners solve and pack, and the
fake-quantised weights are broadcast back (strong scaling: total work fixed).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, KV_OUT, LAYERS = 4096, 14336, 1024, 32
SEQS, SEQ_LEN = 512, 2048
METRIC = "gptq_w4a16_llama3_8b_hotpath_wall_s"
# (name, out_features, input group)
MODULES = [("q_proj", HIDDEN, "attn_in"), ("k_proj", KV_OUT, "attn_in"), ("v_proj", KV_OUT, "attn_in"),
           ("o_proj", HIDDEN, "o_in"), ("gate_proj", INTER, "mlp_in"), ("up_proj", INTER, "mlp_in"),
           ("down_proj", HIDDEN, "down_in")]
GROUP_K = {"attn_in": HIDDEN, "o_in": HIDDEN, "mlp_in": HIDDEN, "down_in": INTER}


# DRAM traffic of one rank-k update launch (dram__bytes_read.sum + dram__bytes_write.sum of ncu
# captures at the launch sizes of the layer step, 32768 tokens): 620 MB at K = 4096, 10.3 GB at
# K = 14336 (four token splits per tile: 8.7 GB read, 1.6 GB written).  A step runs 96 launches of
# width 4096 and 32 of width 14336.
SYRK_TRAFFIC = {
    "K4096": 0.62e9, "K14336": 10.3e9,
    "per_launch_weighted": (96 * 0.62e9 + 32 * 10.3e9) / 128,
    "note": "mean bytes per launch over a step's 96 K=4096 launches (0.62e9 each, algorithmic 0.34e9) and 32 "
            "K=14336 launches (10.3e9 each, algorithmic 1.76e9): X panels are re-read by every band of 8 block "
            "rows and the partial tiles of the four token splits are added into H; DRAM stays at 19-27 % of its "
            "peak, the kernel is tensor bound",
}


def f_syrk(tokens: int, K: int) -> float:
    """Algorithmic flops of a symmetric rank-k update: one multiply-add per token for each of
    the K(K+1)/2 distinct entries."""
    return float(tokens) * K * (K + 1)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=p.get("bf16_tflops_sustained", 1394.5), hbm=p.get("hbm_gbs", 6538.0), source="measured")
    return dict(tflops=1400.0, hbm=6650.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ready = threading.Event()   # set once NVML is initialised and the first sample is in

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            }
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:  # noqa: BLE001
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
                self.ready.set()
                time.sleep(0.2)
        except Exception as e:  # noqa: BLE001
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")
        finally:
            self.ready.set()

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ======================================================================================
# CPU arm: the oracle (a port of the reference's torch code) on the host cores
# ======================================================================================
def cpu_reference_step_seconds(sample_scale: float = 1.0):
    """Time a bounded sample of one layer's hot path with the CPU oracle and extrapolate to
    the full layer.  Returns (seconds_per_layer, cores, description)."""
    import torch

    import oracle

    torch.manual_seed(0)
    # all host cores this process may use (torchrun presets OMP_NUM_THREADS=1 for its workers)
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    if torch.get_num_threads() < avail:
        torch.set_num_threads(avail)
    cores = torch.get_num_threads()
    spec = oracle.preset("W4A16")
    t_h = {}
    for K in (HIDDEN, INTER):
        x = torch.randn(1, SEQ_LEN, K).to(torch.bfloat16)
        H = oracle.make_empty_hessian(K)
        oracle.accumulate_hessian(x[:, :64], H, 0)  # warm the BLAS threads
        t0 = time.perf_counter()
        oracle.accumulate_hessian(x, H, 0)
        t_h[K] = time.perf_counter() - t0
        del H
    # the reference keeps one Hessian per Linear: 6 of width 4096 and 1 of width 14336 per layer
    hess_layer = SEQS * (6 * t_h[HIDDEN] + t_h[INTER])
    # observe + quantize_weight + pack on the real q_proj shape, timed in full; the other modules
    # are scaled by their share of the solve's arithmetic (N K^2 sweep + 4/3 K^3 factorisations)
    N_s, K_s = HIDDEN, HIDDEN
    w = (torch.randn(N_s, K_s) * 0.02).to(torch.bfloat16)
    xs = torch.randn(1, SEQ_LEN, K_s).to(torch.bfloat16)
    Hs, ns = oracle.accumulate_hessian(xs, oracle.make_empty_hessian(K_s), 0)
    Hs[torch.arange(K_s), torch.arange(K_s)] += 0.1 * Hs.diag().mean()  # 2048 tokens < K: keep it PD
    t0 = time.perf_counter()
    obs = oracle.WeightObserver(spec)
    obs(w)
    _, out = oracle.quantize_weight(w, spec, Hs / ns, observer=obs)
    oracle.compress_weight({"weight": out["weight"], "weight_scale": out["weight_scale"],
                            "weight_zero_point": out["weight_zero_point"]}, spec)
    t_q = time.perf_counter() - t0

    def work(n_out, K):
        return n_out * K * K + 4.0 / 3.0 * K ** 3

    solve_layer = sum(t_q * work(n_out, GROUP_K[grp]) / work(N_s, K_s) for _, n_out, grp in MODULES)
    desc = (f"oracle on {cores} host threads: accumulate_hessian on one 2048-token sequence at K=4096 "
            f"({t_h[HIDDEN]:.2f} s) and K=14336 ({t_h[INTER]:.2f} s), x512 sequences x (6+1) modules; "
            f"observe+quantize_weight+pack on a 4096x4096 module ({t_q:.2f} s) scaled to the seven "
            f"modules by N*K^2 + 4/3*K^3")
    return hess_layer + solve_layer, cores, desc


def run_reference(args):
    """`--impl reference`: the reference's CPU path (the oracle port) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        sec, cores, desc = cpu_reference_step_seconds()
        if i >= args.warmup:
            vals.append(sec)
    step_s = sum(vals) / len(vals)
    value = step_s * LAYERS
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.seqs, args.tokens_per_call),
        "step_note": "one decoder layer (bounded CPU sample, extrapolated)",
        "cpu_baseline": {"value": value, "unit": "s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ======================================================================================
# GPU arm
# ======================================================================================
def workload_config(seqs=SEQS, tokens_per_call=32768):
    """The `config` object of both arms' JSON lines."""
    return {"workload": "configs[2]: GPTQ W4A16 g128 (sym int4, block 128, damp 0.01, no act-order), "
                        "Llama-3-8B shapes, %d x %d calibration tokens" % (seqs, SEQ_LEN),
            "step": "one decoder layer: 4 Hessians over all tokens + 7 modules observe/factor/sweep/pack",
            "layers": LAYERS, "tokens_per_syrk_call": tokens_per_call,
            "l2": "inputs larger than L2 (tens of GB streamed per step)",
            "calibration_scale": SEQS / seqs}


class _Layer:
    """Seven Linear modules with the shapes of one Llama-3-8B decoder layer."""

    def __init__(self, torch, device):
        gw = torch.Generator(device=device).manual_seed(0)
        self.module = torch.nn.Module()
        self.mods = []
        for name, n_out, grp in MODULES:
            lin = torch.nn.Linear(GROUP_K[grp], n_out, bias=False, device=device, dtype=torch.bfloat16)
            lin.weight.data = (torch.randn(n_out, GROUP_K[grp], generator=gw, device=device) * 0.02).to(torch.bfloat16)
            lin.requires_grad_(False)
            setattr(self.module, name, lin)
            self.mods.append((name, lin, grp))
        self.W0 = {name: lin.weight.data.clone() for name, lin, _ in self.mods}


class LayerBench:
    """One step = the product's own calls for one decoder layer: ``GPTQModifier.calibrate_module``
    (the forward hook) for every module and calibration chunk, ``on_sequential_epoch_end`` (observe,
    and ``compress_modules``: owner assignment, Hessian reduction, solves, broadcast - all of
    llm_compressor_b200.dist), then the int4 pack of the layer's modules."""

    def __init__(self, rank, world, tokens_per_call, seqs, device, solve_streams=4):
        import torch

        from llm_compressor_b200 import GPTQModifier

        self.torch = torch
        self.rank, self.world, self.dev = rank, world, device
        # this rank's share of the calibration sequences (src/llmcompressor/datasets/utils.py:244-253)
        lo, hi = (seqs * rank) // world, (seqs * (rank + 1)) // world
        self.local_seqs, self.total_seqs = hi - lo, seqs
        self.local_tokens = self.local_seqs * SEQ_LEN
        self.tokens_per_call = min(tokens_per_call, self.local_tokens)
        g = torch.Generator(device=device).manual_seed(1 + rank)
        self.X = {}
        for name, K in GROUP_K.items():
            x = torch.empty(self.local_tokens, K, dtype=torch.bfloat16, device=device)
            colscale = 0.25 + 2.0 * torch.rand(K, generator=g, device=device)
            for t0 in range(0, self.local_tokens, 65536):
                t1 = min(self.local_tokens, t0 + 65536)
                x[t0:t1] = (torch.randn(t1 - t0, K, generator=g, device=device) * colscale).to(torch.bfloat16)
            self.X[name] = x
        self.layer = _Layer(torch, device)
        self.modifier = GPTQModifier(targets="Linear", scheme="W4A16", actorder=None, block_size=128,
                                     dampening_frac=0.01, parallel_streams=solve_streams,
                                     hessian_stage_tokens=self.tokens_per_call)
        self.modifier.on_initialize(self.layer.module)
        self.qargs = self.layer.mods[0][1].quantization_scheme.weights
        self.syrk_events, self.phase_events, self.job_events = [], [], []
        self._record = False
        self.modifier.trace = self._trace

    def _trace(self, event, module):
        if not self._record:
            return
        ev = self.torch.cuda.Event(enable_timing=True)
        ev.record()
        if event.startswith("job_"):
            grp = next(g_ for _, lin, g_ in self.layer.mods if lin is module)
            self.job_events.append((self._step_index, grp, event[4:], ev))
        else:
            self.phase_events.append((self._step_index, event, ev))

    def step(self, from_host=None, record=False, index=0):
        """One decoder layer.  `from_host`: HostFeeder supplying activation chunks from pinned
        host memory (end-to-end arm); otherwise activations are resident in HBM."""
        torch = self.torch
        from llm_compressor_b200 import compressors

        self._record, self._step_index = record, index
        mod = self.modifier
        for name, lin, _ in self.layer.mods:   # the previous step left its quantised weights here
            lin.weight.data.copy_(self.layer.W0[name])
        self._trace("begin", None)
        mod.on_calibration_start(self.layer.module)
        for g_, K in GROUP_K.items():
            X = self.X[g_]
            members = [lin for _, lin, grp in self.layer.mods if grp == g_]
            for t0 in range(0, self.local_tokens, self.tokens_per_call):
                t1 = min(self.local_tokens, t0 + self.tokens_per_call)
                chunk = from_host.next_chunk(g_, t0, t1) if from_host is not None else X[t0:t1]
                batch = chunk.view((t1 - t0) // SEQ_LEN, SEQ_LEN, K)
                if record:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                for lin in members:   # the hook of every module that receives this tensor
                    mod.calibrate_module(lin, (batch,), None)
                if record:
                    e1.record()
                    self.syrk_events.append((e0, e1, t1 - t0, K))
                if from_host is not None:
                    from_host.release(chunk)
        mod.on_sequential_epoch_end(self.layer.module, list(self.layer.module.modules()))
        mod.on_calibration_end(self.layer.module)
        results = {}
        if self.rank == 0:   # the save path packs on the writing rank
            for name, lin, _ in self.layer.mods:
                packed = compressors.compress_state_dict(
                    {"weight": lin.weight.data, "weight_scale": lin.weight_scale.data,
                     "weight_zero_point": lin.weight_zero_point.data}, self.qargs)
                results[name] = (mod.losses.get(name), lin.weight.data, packed)
        self._trace("end", None)
        return results


class HostFeeder:
    """Pinned host copies of the activations, streamed to the device in double-buffered
    chunks on a copy stream (the end-to-end arm's host->device leg)."""

    def __init__(self, bench: LayerBench, budget_bytes: int):
        torch = bench.torch
        self.torch, self.b = torch, bench
        self.copy_stream = torch.cuda.Stream()
        self.host, self.cycle = {}, {}
        need = sum(x.numel() * 2 for x in bench.X.values())
        frac = min(1.0, budget_bytes / need)
        for g_, x in bench.X.items():
            rows = max(bench.tokens_per_call, int(x.shape[0] * frac) // bench.tokens_per_call * bench.tokens_per_call)
            rows = min(rows, x.shape[0])
            h = torch.empty(rows, x.shape[1], dtype=torch.bfloat16, pin_memory=True)
            h.copy_(x[:rows])
            self.host[g_], self.cycle[g_] = h, rows
        self.pool_fraction = frac
        self.bufs = {}
        self.h2d_bytes = 0
        self.pending = None

    def _buf(self, K, slot):
        key = (K, slot)
        if key not in self.bufs:
            self.bufs[key] = (self.torch.empty(self.b.tokens_per_call, K, dtype=self.torch.bfloat16, device=self.b.dev),
                              self.torch.cuda.Event(), self.torch.cuda.Event())
        return self.bufs[key]

    def start_step(self):
        self.slot, self.h2d_bytes = 0, 0

    def next_chunk(self, g_, t0, t1):
        torch = self.torch
        K = GROUP_K[g_]
        buf, ready, free = self._buf(K, self.slot & 1)
        self.slot += 1
        rows = t1 - t0
        src0 = t0 % self.cycle[g_]
        if src0 + rows > self.cycle[g_]:
            src0 = 0
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(free)  # the kernel that last read this buffer is done
            buf[:rows].copy_(self.host[g_][src0:src0 + rows], non_blocking=True)
            ready.record(self.copy_stream)
        torch.cuda.current_stream().wait_event(ready)
        self.h2d_bytes += rows * K * 2
        out = buf[:rows]
        out._feeder_free = free
        return out

    def release(self, chunk):
        chunk._feeder_free.record(self.torch.cuda.current_stream())


def parity_check(bench, snapshot, losses):
    """Ties the timed numbers to verified output: k_proj (1024 x 4096) of the last timed step against
    the CPU oracle on the same weight and the same calibration tokens, and the rank-k update against
    the oracle's Hessian on a 4096-token sample.  Runs after the timed regions, on every rank for the
    collective and on rank 0 for the comparison."""
    import torch
    import torch.distributed as dist

    import oracle
    from llm_compressor_b200 import gptq

    t_start = time.perf_counter()
    K = HIDDEN
    X = bench.X["attn_in"]
    H = torch.zeros(K, K, dtype=torch.float32, device=bench.dev)
    for t0 in range(0, bench.local_tokens, bench.tokens_per_call):
        t1 = min(bench.local_tokens, t0 + bench.tokens_per_call)
        gptq.accumulate_hessian_lower(X[t0:t1].view(-1, SEQ_LEN, K), H, 0)
    if bench.world > 1:
        dist.all_reduce(H)
    gptq.finalize_hessian(H, bench.total_seqs)
    if bench.rank != 0:
        return None
    spec = oracle.preset("W4A16")
    w0 = bench.layer.W0["k_proj"].cpu()
    loss_ref, ref = oracle.quantize_weight(w0, spec, H.cpu())
    wq, scale = snapshot
    code_match = float((wq.cpu().view(torch.int16) == ref["weight"].view(torch.int16)).float().mean())
    scale_equal = bool(torch.equal(scale.cpu().view(torch.int16), ref["weight_scale"].view(torch.int16)))
    loss = losses.get("k_proj")
    # Hessian of a 4096-token sample, oracle on the host against the kernel
    xs = X[:4096]
    Hs = torch.zeros(K, K, dtype=torch.float32, device=bench.dev)
    gptq.accumulate_hessian_lower(xs.view(2, SEQ_LEN, K), Hs, 0)
    gptq.finalize_hessian(Hs, 1)
    Ho, _ = oracle.accumulate_hessian(xs.cpu().view(2, SEQ_LEN, K), oracle.make_empty_hessian(K), 0)
    herr = float((Hs.cpu().double() - Ho.double()).norm() / Ho.double().norm())
    return {"module": "k_proj 1024x4096 of the last timed step, against the CPU oracle",
            "code_match": round(code_match, 6), "scale_equal": scale_equal,
            "loss_rel": None if loss is None else round(abs(loss - loss_ref) / abs(loss_ref), 6),
            "hessian_rel_fro_4096_tokens": herr,
            "ok": bool(code_match >= 0.995 and scale_equal and herr < 1e-3 and
                       (loss is None or abs(loss - loss_ref) <= 0.01 * abs(loss_ref))),
            "seconds": round(time.perf_counter() - t_start, 1)}


def run_b200(args):
    import torch
    import torch.distributed as dist

    from llm_compressor_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    peaks = load_peaks()
    seqs = args.seqs
    bench = LayerBench(rank, world, args.tokens_per_call, seqs, dev, solve_streams=args.solve_streams)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # L2 is defeated by size: every step streams tens of GB of activations (>> 126 MB)
    # warm-up keeps the previous step's results alive while the next step runs, exactly like the
    # timed loop, so that the allocator pools of the solve streams reach their steady state here
    results = None
    for _ in range(args.warmup):
        results = bench.step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    # NVML initialisation takes driver locks for a few hundred milliseconds: let it finish before
    # the timed region (it used to land on one of the first timed steps)
    sampler.ready.wait(timeout=10)
    launches0 = lib.b200q_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bench.syrk_events, bench.phase_events, bench.job_events = [], [], []
    barrier()
    e0.record()
    for i in range(args.steps):
        results = bench.step(record=True, index=i)
    e1.record()
    barrier()
    launches = lib.b200q_launch_count() - launches0
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = ms_per_step / 1e3 * LAYERS
    # what the parity check compares: k_proj as the last timed step left it
    kp = dict((n, l) for n, l, _ in bench.layer.mods)["k_proj"]
    snapshot = (kp.weight.data.clone(), kp.weight_scale.data.clone())
    losses = dict(bench.modifier.losses)
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, losses)
        losses = {k: v for d in gathered for k, v in d.items()}

    # dominant kernel: the SYRK; achieved = algorithmic flops / CUDA-event time of its launches
    syrk_ms = sum(a.elapsed_time(b) for a, b, _, _ in bench.syrk_events)
    syrk_flops = sum(f_syrk(t, K) for _, _, t, K in bench.syrk_events)
    achieved = syrk_flops / (syrk_ms * 1e-3) / 1e12 if syrk_ms > 0 else 0.0
    roofline = {"bound": "tensor", "kernel": "syrk_pair_kernel (tcgen05 cta_group::2)", "achieved": achieved, "peak": peaks["tflops"],
                "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                # dram__bytes_read.sum + dram__bytes_write.sum of ncu-captured launches, weighted by
                # how often each width runs in a step
                "traffic": SYRK_TRAFFIC["per_launch_weighted"], "traffic_note": SYRK_TRAFFIC["note"],
                "peak_source": peaks["source"] + " bf16_tflops_sustained",
                "share_of_step": syrk_ms / ms if ms else None,
                "launches": len(bench.syrk_events)}

    # device time of the step's phases (mean per step): Hessian accumulation (hook calls, weight
    # observers), the reduction to the owners, the solve (factorise, sweep) and the broadcast + pack
    phases = {"hessian": 0.0, "reduce": 0.0, "solve": 0.0, "broadcast_pack": 0.0}
    solve_steps = []
    by_step = {}
    for idx, name, ev in bench.phase_events:
        by_step.setdefault(idx, {})[name] = ev
    for idx in sorted(by_step):
        evs = by_step[idx]
        if not {"begin", "solve", "done", "end"} <= set(evs):
            continue
        first = evs.get("reduce", evs["solve"])
        phases["hessian"] += evs["begin"].elapsed_time(first) / args.steps
        if "reduce" in evs:
            phases["reduce"] += evs["reduce"].elapsed_time(evs["solve"]) / args.steps
        solve_end = evs.get("broadcast", evs["done"])
        phases["solve"] += evs["solve"].elapsed_time(solve_end) / args.steps
        phases["broadcast_pack"] += solve_end.elapsed_time(evs["end"]) / args.steps
        solve_steps.append(round(evs["solve"].elapsed_time(solve_end), 1))

    # device time line of the last timed step's solve jobs on this rank, ms after the solve phase
    # began: {group: [start, factored, swept]}
    jobs = {}
    last = args.steps - 1
    if last in by_step and "solve" in by_step[last]:
        t0 = by_step[last]["solve"]
        for step_i, g_, what, ev in bench.job_events:
            if step_i == last:
                jobs.setdefault(g_, []).append(round(t0.elapsed_time(ev), 1))

    # end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        import psutil
        avail = psutil.virtual_memory().available
        budget = int(min(0.25 * avail, 64 * 2**30))
        feeder = HostFeeder(bench, budget)
        d2h_bytes = 0
        host_out = {}
        barrier()
        steps_e2e = max(1, min(args.steps, args.e2e_steps))
        for it in range(1 + steps_e2e):
            if it == 1:
                barrier()
                t0 = torch.cuda.Event(enable_timing=True)
                t1 = torch.cuda.Event(enable_timing=True)
                t0.record()
            feeder.start_step()
            res = bench.step(from_host=feeder)
            d2h_bytes = 0
            for name, (loss, wq, packed) in res.items():
                for k, v in packed.items():
                    key = (name, k)
                    if key not in host_out:
                        host_out[key] = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                    host_out[key].copy_(v, non_blocking=True)
                    d2h_bytes += v.numel() * v.element_size()
        t1.record()
        barrier()
        ms_e2e = t0.elapsed_time(t1) / steps_e2e
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        e2e = {"value": ms_e2e / 1e3 * LAYERS, "unit": "s", "h2d_bytes_per_step": feeder.h2d_bytes,
               "d2h_bytes_per_step": d2h_bytes, "steps": steps_e2e,
               "host_pool_fraction": round(feeder.pool_fraction, 3)}
        del feeder, host_out

    parity = None
    if not args.no_parity:
        try:
            parity = parity_check(bench, snapshot, losses)
        except Exception as e:  # noqa: BLE001 - the timing line must still be printed
            parity = {"ok": False, "error": f"{type(e).__name__}: {e}"}

    # quantize / pack kernels (the metric's "pack GB/s"), rank 0, after the timed region
    pack = None
    if rank == 0 and not args.no_pack:
        del results
        bench.X.clear()
        flush = torch.empty(8, dtype=torch.uint8, device=dev)
        pack = {r["kernel"]: {"gbs": round(r["gbs"], 1), "frac_of_hbm_peak": round(r["frac_of_hbm_peak"], 3),
                              "bytes_per_elem": r["bytes_per_elem"], "moved_bytes_per_elem": r.get("moved_bytes_per_elem")}
                for r in pack_micro(5, peaks, make_timed(flush), torch.Generator(device=dev).manual_seed(0), dev)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sec, cores, desc = cpu_reference_step_seconds()
        cpu = {"value": sec * LAYERS, "unit": "s", "cores": cores, "kind": "port", "sample": desc}

    # the whole oneshot() run on the 8B-architecture model (after everything above has been measured)
    oneshot_line = None
    if not args.no_oneshot:
        results = None
        del bench
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            oneshot_line = run_oneshot_arm(rank, world, dev, args.oneshot_seqs, args.oneshot_batch)
        except Exception as e:  # noqa: BLE001 - the hot-path line must still be printed
            oneshot_line = {"error": f"{type(e).__name__}: {e}"[:400]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(seqs, args.tokens_per_call),
            "product_path": "GPTQModifier.calibrate_module / on_sequential_epoch_end / compress_modules "
                            "(llm_compressor_b200.dist owner assignment, reduction, broadcast)",
            "phases_ms": phases, "solve_ms_per_step": solve_steps, "solve_jobs_ms": jobs, "roofline": roofline,
            "parity_check": parity, "pack_gbs": pack, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "oneshot": oneshot_line,
            "clocks": clocks,
            "published_reference": {"value": 745.03, "unit": "s", "note": "whole oneshot incl. model forwards, "
                                    "GPU not stated (docs/guides/big_models_and_distributed/distributed_oneshot.md:107-111)"},
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_oneshot_arm(rank, world, dev, seqs, batch_size):
    """The metric as BASELINE.json words it: wall seconds of ``oneshot()`` with ``GPTQModifier`` (W4A16,
    g128, block 128, damp 0.01, no act-order, lm_head ignored, sequential pipeline) on a random-init
    Llama-3-8B-architecture ``LlamaForCausalLM`` with 512 x 2048 random calibration tokens.  Under
    torchrun every rank holds the model and calibrates its share of the sequences; Hessians are
    reduced to their owners, owners solve, results are broadcast (the product path, as it is).
    Returns the dict for the JSON line (rank 0) or None."""
    import torch
    import torch.distributed as dist
    from transformers import LlamaConfig, LlamaForCausalLM

    from llm_compressor_b200 import GPTQModifier, oneshot
    from llm_compressor_b200 import compressors

    cfg = LlamaConfig(hidden_size=HIDDEN, intermediate_size=INTER, num_hidden_layers=LAYERS, num_attention_heads=32,
                      num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=8192, tie_word_embeddings=False)
    torch.manual_seed(0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    model.eval().requires_grad_(False)
    data = torch.randint(0, cfg.vocab_size, (seqs, SEQ_LEN), generator=torch.Generator().manual_seed(1))
    recipe = GPTQModifier(targets="Linear", scheme="W4A16", ignore=["lm_head"], actorder=None, block_size=128,
                          dampening_frac=0.01)
    phases = {}
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    oneshot(model, recipe=recipe, dataset=data, num_calibration_samples=seqs, batch_size=batch_size,
            phase_times=phases)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    # packing of every quantised module on the device (what the checkpoint writer runs before it copies out)
    t1 = time.perf_counter()
    n_packed = 0
    if rank == 0:
        for _n, m in model.named_modules():
            if hasattr(m, "quantization_scheme") and hasattr(m, "weight_scale"):
                compressors.compress_state_dict({"weight": m.weight.data, "weight_scale": m.weight_scale.data,
                                                 "weight_zero_point": m.weight_zero_point.data}, m.quantization_scheme)
                n_packed += 1
        torch.cuda.synchronize()
    pack_s = time.perf_counter() - t1
    t = torch.tensor([wall], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    losses = list(recipe.losses.values())
    finite = all(v == v and v < float("inf") for v in losses)
    if rank != 0:
        return None
    return {"metric": "gptq_w4a16_llama3_8b_oneshot_wall_s", "wall_s": float(t.item()), "unit": "s",
            "phases_s": {k: round(v, 2) for k, v in phases.items()}, "pack_s": round(pack_s, 3),
            "modules_packed": n_packed, "modules_solved_on_rank0": len(losses), "losses_finite": finite,
            "config": {"workload": "configs[2] through oneshot(): random-init Llama-3-8B-architecture LlamaForCausalLM, "
                                   "GPTQModifier W4A16 g128, %d x %d calibration tokens" % (seqs, SEQ_LEN),
                       "batch_size": batch_size, "pipeline": "sequential, activations resident in HBM"},
            "published_reference_s": {"1_gpu": 745.03, "2_gpu": 372.0, "4_gpu": 264.0,
                                      "note": "docs/guides/big_models_and_distributed/distributed_oneshot.md:107-113, GPU not stated"}}


# ======================================================================================
# configs[3]: GPTQ FP8 (per-channel scales) of one Qwen3-30B-A3B-shaped MoE decoder layer
# ======================================================================================
def run_moe(args):
    """One layer of the MoE configuration through GPTQModifier: hidden 2048, 32 / 4 heads of 128
    (q 4096 x 2048, k / v 512 x 2048, o 2048 x 4096), 128 experts with gate / up 768 x 2048 and
    down 2048 x 768, 256 x 2048 calibration tokens, all-expert calibration (every expert sees every
    token, so all 256 gate / up projections share ONE Hessian and every down projection has its
    own), FP8 E4M3 weights with per-channel scales, act-order "static".  Under torchrun the token
    shards are reduced, the experts' Hessians go to owners and the shared one to every rank."""
    import torch
    import torch.distributed as dist

    import oracle
    from llm_compressor_b200 import GPTQModifier, compressors

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    H_, QO, KV, E, MI, MOE_LAYERS = 2048, 4096, 512, args.experts, 768, 48
    seqs = args.seqs if args.seqs != SEQS else 256
    lo, hi = (seqs * rank) // world, (seqs * (rank + 1)) // world
    tokens = (hi - lo) * SEQ_LEN
    chunk = min(args.tokens_per_call, tokens)
    g = torch.Generator(device=dev).manual_seed(1 + rank)

    def acts(K):
        x = torch.empty(tokens + 8 * E, K, dtype=torch.bfloat16, device=dev)
        cs = 0.25 + 2.0 * torch.rand(K, generator=g, device=dev)
        for t0 in range(0, x.shape[0], 65536):
            t1 = min(x.shape[0], t0 + 65536)
            x[t0:t1] = (torch.randn(t1 - t0, K, generator=g, device=dev) * cs).to(torch.bfloat16)
        return x
    X = {"hidden": acts(H_), "o_in": acts(QO), "down_in": acts(MI)}
    gw = torch.Generator(device=dev).manual_seed(0)
    layer = torch.nn.Module()
    mods = []   # (name, module, input key, row offset into the input buffer)

    def add(name, n_out, k_in, key, off=0):
        lin = torch.nn.Linear(k_in, n_out, bias=False, device=dev, dtype=torch.bfloat16)
        lin.weight.data = (torch.randn(n_out, k_in, generator=gw, device=dev) * 0.02).to(torch.bfloat16)
        lin.requires_grad_(False)
        setattr(layer, name, lin)
        mods.append((name, lin, key, off))
    add("q_proj", QO, H_, "hidden"); add("k_proj", KV, H_, "hidden"); add("v_proj", KV, H_, "hidden")
    add("o_proj", H_, QO, "o_in")
    for e in range(E):
        # every expert's gate / up see the block input; each down projection has its own input
        # (a window of the shared buffer shifted by 8 rows per expert: distinct tensors)
        add(f"experts_{e}_gate_proj", MI, H_, "mlp", 8); add(f"experts_{e}_up_proj", MI, H_, "mlp", 8)
        add(f"experts_{e}_down_proj", H_, MI, "down_in", 8 * e)
    W0 = {name: lin.weight.data.clone() for name, lin, _, _ in mods}
    mod = GPTQModifier(targets="Linear", scheme="FP8_DYNAMIC", actorder="static", block_size=128, dampening_frac=0.01,
                       parallel_streams=args.solve_streams, hessian_stage_tokens=chunk)
    mod.on_initialize(layer)
    events = {}

    def trace(ev, _m):
        if ev in ("reduce", "solve", "broadcast", "done"):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            events[ev] = e
    mod.trace = trace

    def step():
        for name, lin, _, _ in mods:
            lin.weight.data.copy_(W0[name])
        e0 = torch.cuda.Event(enable_timing=True)
        e0.record()
        mod.on_calibration_start(layer)
        for t0 in range(0, tokens, chunk):
            t1 = min(tokens, t0 + chunk)
            views = {}
            for name, lin, key, off in mods:
                src = X["hidden"] if key == "mlp" else X[key]
                vk = (key, off)
                if vk not in views:
                    views[vk] = src[off + t0: off + t1].view((t1 - t0) // SEQ_LEN, SEQ_LEN, src.shape[1])
                mod.calibrate_module(lin, (views[vk],), None)
        mod.on_sequential_epoch_end(layer, list(layer.modules()))
        mod.on_calibration_end(layer)
        if rank == 0:
            for name, lin, _, _ in mods:
                compressors.compress_state_dict({"weight": lin.weight.data, "weight_scale": lin.weight_scale.data,
                                                 "weight_zero_point": lin.weight_zero_point.data},
                                                lin.quantization_scheme)
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record()
        return e0, e1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(args.warmup):
        step()
    barrier()
    t_wall = time.perf_counter()
    marks = [step() for _ in range(args.steps)]
    barrier()
    wall_ms = (time.perf_counter() - t_wall) * 1e3 / args.steps
    ms = sum(a.elapsed_time(b) for a, b in marks) / args.steps
    first = events.get("reduce", events["solve"])
    phases = {"hessian_ms": marks[-1][0].elapsed_time(first),
              "reduce_ms": events["reduce"].elapsed_time(events["solve"]) if "reduce" in events else 0.0,
              "solve_ms": events["solve"].elapsed_time(events.get("broadcast", events["done"])),
              "rest_ms": events.get("broadcast", events["done"]).elapsed_time(marks[-1][1])}
    tms = torch.tensor([ms, wall_ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    # parity against the CPU oracle of one expert's down projection (K = 768, its own Hessian) and
    # of one gate projection (K = 2048, the Hessian all experts share): both go through the batched
    # factor / fused sweep launches
    parity = None
    if rank == 0 and world == 1:
        from llm_compressor_b200 import gptq
        spec = oracle.preset("FP8_DYNAMIC", actorder="static")
        parity = {"ok": True, "modules": []}
        for wanted in ("experts_3_down_proj", "experts_5_gate_proj"):
            name, lin, key, off = next(m for m in mods if m[0] == wanted)
            src = X["hidden"] if key == "mlp" else X[key]
            K_ = src.shape[1]
            Hh = torch.zeros(K_, K_, device=dev)
            for t0 in range(0, tokens, chunk):
                t1 = min(tokens, t0 + chunk)
                gptq.accumulate_hessian_lower(src[off + t0: off + t1].view(-1, SEQ_LEN, K_), Hh, 0)
            gptq.finalize_hessian(Hh, seqs)
            loss_ref, ref = oracle.quantize_weight(W0[name].cpu(), spec, Hh.cpu())
            match = float((lin.weight.data.cpu().view(torch.int16) == ref["weight"].view(torch.int16)).float().mean())
            one = {"module": name, "code_match": round(match, 6),
                   "scale_equal": bool(torch.equal(lin.weight_scale.data.cpu().view(torch.int16).flatten(),
                                                   ref["weight_scale"].view(torch.int16).flatten())),
                   "loss_rel": round(abs(mod.losses[name] - loss_ref) / abs(loss_ref), 6)}
            one["ok"] = one["code_match"] >= 0.995 and one["scale_equal"] and one["loss_rel"] <= 0.01
            parity["modules"].append(one)
            parity["ok"] = parity["ok"] and one["ok"]
    if rank == 0:
        print(json.dumps({
            "metric": "gptq_fp8_qwen3_30b_a3b_layer_ms", "value": float(tms[0]), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(tms[0]), "host_wall_ms_per_step": float(tms[1]),
            "model_estimate_s": float(tms[1]) * MOE_LAYERS / 1e3, "higher_is_better": False, "scaling": "strong",
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[3]: GPTQ FP8 E4M3 per-channel, act-order static, one Qwen3-30B-A3B-shaped MoE layer "
                                   "(%d experts, all-expert calibration), %d x %d calibration tokens" % (E, seqs, SEQ_LEN),
                       "modules": len(mods), "distinct_hessians": 3 + E, "layers_in_model": MOE_LAYERS},
            "phases": {k: round(v, 2) for k, v in phases.items()}, "parity_check": parity,
        }))
    if world > 1:
        dist.destroy_process_group()


# ======================================================================================
# configs[4]: the Llama-3-70B widths (8192 / 28672), act-order and the 100-step MSE observer
# ======================================================================================
def run_70b(args):
    """Kernel-level figures at the widths of the 70B configuration, one module of each kind on one
    GPU (the model itself is layer-sharded over 8 GPUs, so one GPU never holds more than this):
    Hessian update at K = 8192 and 28672, the factorisation at both widths, act-order "group" GPTQ of
    a 1024-row slice of down_proj (8192 x 28672) with the 100-candidate MSE observer, and that
    observer on the full 8192 x 28672 weight.  The factor is checked through its defining property
    (U^T U H v = v on random probes, in float64 on the device)."""
    import torch

    from llm_compressor_b200 import gptq, observers, ops
    from llm_compressor_b200.quant_args import QuantizationArgs

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(8, dtype=torch.uint8, device=dev)
    timed = make_timed(flush)
    g = torch.Generator(device=dev).manual_seed(0)
    out = {"metric": "gptq_w4a16_llama3_70b_module_ms", "config": {"workload": "configs[4]: Llama-3-70B widths, W4A16 g128, "
           "act-order group, memoryless_mse with 100 candidates (maxshrink 1.0, grid 100, norm 2.4)"}, "results": {}}
    peaks = load_peaks()
    T = 32768
    for K in (8192, 28672):
        x = torch.randn(T, K, generator=g, device=dev).to(torch.bfloat16)
        H = torch.zeros(K, K, device=dev)
        ms = timed(lambda: ops.hessian_syrk(x, H, 2.0), args.steps, do_flush=False)
        out["results"][f"syrk_K{K}_T{T}"] = {"ms": round(ms, 3), "tflops": round(f_syrk(T, K) / ms / 1e9, 1),
                                             "frac_of_burst_peak": round(f_syrk(T, K) / ms / 1e9 / 1661.0, 3)}
        # a well conditioned Hessian from 4 such calls, then the factorisation
        H.zero_()
        for i in range(4):
            x.copy_(torch.randn(T, K, generator=g, device=dev).to(torch.bfloat16))
            ops.hessian_syrk(x, H, 2.0)
        del x
        ops.hessian_finalize(H, 1.0 / 64)
        ops.gptq_prepare(H, None, 0.01)
        U = H.clone()
        st = ops.gptq_factor_async(U)
        assert ops.gptq_factor_status(st) == 0
        v = torch.randn(K, 2, generator=g, device=dev, dtype=torch.float64)
        r = U.double().t() @ (U.double() @ (H.double() @ v)) - v
        resid = float(r.norm() / v.norm())
        Hw = torch.empty_like(H)

        def fac():
            Hw.copy_(H)
            ops.gptq_factor(Hw)
        ms = timed(fac, max(2, args.steps // 2), do_flush=False)
        out["results"][f"factor_K{K}"] = {"ms": round(ms, 2), "workspace_gb": round(_lib_ws(K) / 2**30, 2),
                                          "residual_UtUH_minus_I": resid, "ok": resid < 1e-3}
        if K == 28672:
            a = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128, actorder="group",
                                 observer="memoryless_mse", observer_kwargs={"maxshrink": 1.0, "grid": 100.0, "norm": 2.4})
            rows = 1024
            lin = torch.nn.Linear(K, rows, bias=False, device=dev, dtype=torch.bfloat16)
            lin.weight.data = (torch.randn(rows, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)

            def solve():
                lin.weight_observer = observers.Observer.load_from_registry("memoryless_mse", base_name="weight", args=a)
                lin.weight_observer(lin.weight.data)
                return gptq.quantize_weight(lin, a, H.clone(), blocksize=128, percdamp=0.0)
            loss, res = solve()
            ms = timed(lambda: solve(), 2, do_flush=False)
            out["results"]["gptq_actorder_group_mse100_down_proj_1024rows"] = {
                "ms": round(ms, 2), "loss": loss, "g_idx_is_permutation_of_groups": bool(
                    torch.equal(torch.sort(res["weight_g_idx"]).values.cpu(), (torch.arange(K) // 128).to(torch.int32)))}
            del lin
            w = (torch.randn(8192, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            for cand, kw in ((20, {}), (100, {"maxshrink": 1.0, "grid": 100.0, "norm": 2.4})):
                am = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128,
                                      observer="memoryless_mse", observer_kwargs=kw)
                ms = timed(lambda: ops.observe_mse(w, am, **kw), 3, do_flush=False)
                out["results"][f"observe_mse_8192x28672_{cand}cand"] = {
                    "ms": round(ms, 2), "g_element_steps_per_s": round(8192 * K * cand / ms / 1e6, 1)}
            del w
        del H, U, Hw
        torch.cuda.empty_cache()
    out["peaks"] = peaks
    print(json.dumps(out))


def _lib_ws(K):
    from llm_compressor_b200 import _lib
    return _lib.load().b200q_gptq_factor_workspace_bytes(K)


def pack_micro(steps, peaks, timed, g, dev):
    """Quantize / pack kernels on a 16384 x 8192 bf16 matrix, and the NVFP4 / MXFP4 weight path on
    the two large Llama-3-8B matrices with 0.1 % outliers: GB/s of ALGORITHMIC bytes (the weight
    read, the codes and the stored scale bytes; the bf16 copy of the scales that the module keeps
    is extra and listed as moved bytes) and the fraction of the measured HBM copy bandwidth."""
    import torch

    from llm_compressor_b200 import ops
    from llm_compressor_b200.quant_args import QuantizationArgs, preset_name_to_scheme

    results = []

    def add(name, N, K, ms, bpe, moved):
        gbs = bpe * N * K / (ms * 1e-3) / 1e9
        results.append({"kernel": name, "N": N, "K": K, "ms": ms, "gbs": gbs, "bytes_per_elem": bpe,
                        "moved_bytes_per_elem": moved, "frac_of_hbm_peak": gbs / peaks["hbm"]})

    # two 256 MiB inputs used in turn: each launch reads data the previous launch evicted
    # from L2 (126 MB); an explicit flush would leave dirty lines whose write-back would be
    # charged to these short kernels
    N, K = 16384, 8192
    ws = [(torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(2)]
    turn = [0]

    def nxt():
        turn[0] ^= 1
        return ws[turn[0]]
    w = ws[0]
    # (name, preset, algorithmic bytes per element, bytes actually moved per element)
    cases = [("rtn_int4_g128", "W4A16", 2 + 0.5 + 2 / 128, 2 + 0.5 + 2 / 128 + 1 / 128),
             ("rtn_mxfp4", "MXFP4A16", 2 + 0.5 + 1 / 32, 2 + 0.5 + 1 / 32 + 2 / 32 + 1 / 32),
             ("rtn_mxfp8", "MXFP8A16", 2 + 1 + 1 / 32, 2 + 1 + 1 / 32 + 2 / 32 + 1 / 32),
             ("rtn_fp8_channel", "FP8_DYNAMIC", 3.0, 3.0)]
    for name, preset, bpe, moved in cases:
        a = preset_name_to_scheme(preset, ["Linear"]).weights
        ms = timed(lambda: ops.rtn_quantize_pack(nxt(), a), steps, do_flush=False)
        add(name, N, K, ms, bpe, moved)
    a4 = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128)
    mn, mx = ops.observe_minmax(w, a4)
    scale, zp = ops.qparams(mn, mx, a4)
    ms = timed(lambda: ops.quantize_pack(nxt(), scale, zp, a4), steps, do_flush=False)
    add("pack_int4_g128_given_scale", N, K, ms, 2 + 0.5 + 2 / 128, 2 + 0.5 + 2 / 128)
    ms = timed(lambda: ops.observe_minmax(nxt(), a4), steps, do_flush=False)
    add("observe_minmax_g128", N, K, ms, 2.0, 2.0 + 4 / 128)
    gs = torch.tensor([1000.0], device=dev)
    ms = timed(lambda: ops.nvfp4_quantize_pack(nxt(), gs), steps, do_flush=False)
    add("nvfp4_given_global_scale", N, K, ms, 2 + 0.5 + 1 / 16, 2 + 0.5 + 1 / 16 + 2 / 16)
    del ws, w, mn, mx, scale, zp

    # the data-free FP4 weight path on the MLP matrices of Llama-3-8B (0.1 % of the entries replaced
    # by N(0, 0.5) outliers): NVFP4 needs the tensor-wide amax first, hence two reads of the weight
    for (n_, k_) in ((INTER, HIDDEN), (HIDDEN, INTER)):
        pair = []
        for _ in range(3):   # 3 x 117 MB: each launch reads a matrix that has left L2
            m = torch.randn(n_, k_, generator=g, device=dev) * 0.02
            idx = torch.randint(0, n_ * k_, (n_ * k_ // 1000,), generator=g, device=dev)
            m.view(-1)[idx] = torch.randn(idx.numel(), generator=g, device=dev) * 0.5
            pair.append(m.to(torch.bfloat16))
        cyc = [0]

        def nx():
            cyc[0] = (cyc[0] + 1) % len(pair)
            return pair[cyc[0]]
        ms = timed(lambda: ops.nvfp4_two_pass(nx()), steps, do_flush=False)
        add(f"nvfp4_two_pass_{n_}x{k_}", n_, k_, ms, 2 * 2 + 0.5 + 1 / 16, 2 * 2 + 0.5 + 1 / 16 + 2 / 16)
        amx = preset_name_to_scheme("MXFP4A16", ["Linear"]).weights
        ms = timed(lambda: ops.rtn_quantize_pack(nx(), amx), steps, do_flush=False)
        add(f"rtn_mxfp4_{n_}x{k_}", n_, k_, ms, 2 + 0.5 + 1 / 32, 2 + 0.5 + 1 / 32 + 2 / 32 + 1 / 32)
        del pair
    return results


def make_timed(flush):
    import torch

    def timed(fn, iters, do_flush=True):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            # keep the GPU busy while the host queues the flush, the events and the launch, so the
            # interval between the events holds the kernel and not the host's launch overhead
            torch.cuda._sleep(3_000_000)
            if do_flush:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)
    return timed


def run_micro(args):
    """Kernel-level figures on small cases (also the cases ncu captures are taken on):
    Hessian SYRK TFLOP/s and quantize/pack GB/s against their rooflines.  One JSON line."""
    import torch

    from llm_compressor_b200 import ops
    from llm_compressor_b200.quant_args import QuantizationArgs, preset_name_to_scheme

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=dev)  # > L2 (126 MB)
    out = {"micro": args.micro, "peaks": peaks, "results": []}

    timed = make_timed(flush)

    g = torch.Generator(device=dev).manual_seed(0)
    if args.micro in ("syrk", "all"):
        for K, T in ((4096, 32768), (14336, 16384)) if args.micro == "all" else ((args.micro_k, args.micro_t),):
            x = torch.randn(T, K, generator=g, device=dev).to(torch.bfloat16)
            H = torch.zeros(K, K, device=dev)
            ms = timed(lambda: ops.hessian_syrk(x, H, 2.0), args.steps)
            tf = f_syrk(T, K) / (ms * 1e-3) / 1e12
            out["results"].append({"kernel": "syrk", "K": K, "T": T, "ms": ms, "tflops": tf,
                                   "frac_of_burst_peak": tf / 1661.0 if peaks["source"] == "measured" else None})
            del x, H
    if args.micro in ("pack", "all"):
        out["results"].extend(pack_micro(args.steps, peaks, timed, g, dev))
    if args.micro in ("mse", "all"):
        import time as _time

        from llm_compressor_b200 import observers
        from llm_compressor_b200.quant_args import QuantizationArgs
        for (N, K) in ((4096, 4096), (14336, 4096)):
            w = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            for kw in ({}, {"maxshrink": 1.0, "grid": 100.0, "norm": 2.4}):
                a = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128,
                                     observer="memoryless_mse", observer_kwargs=kw)
                ts = []
                for _ in range(max(3, args.steps)):
                    obs = observers.Observer.load_from_registry("memoryless_mse", base_name="weight", args=a)
                    torch.cuda.synchronize()
                    t0 = _time.perf_counter()
                    obs(w)
                    torch.cuda.synchronize()
                    ts.append((_time.perf_counter() - t0) * 1e3)
                ms = statistics.median(ts)
                steps = int(kw.get("maxshrink", 0.2) * kw.get("grid", 100.0))
                out["results"].append({"kernel": "observe_mse_int4_g128", "N": N, "K": K, "candidates": steps, "ms": ms,
                                       "g_element_steps_per_s": N * K * steps / ms / 1e6})
    if args.micro in ("factor", "all"):
        K = args.micro_k if args.micro == "factor" else 4096
        xx = torch.randn(2 * K, K, generator=g, device=dev)
        H0 = (xx.t() @ xx) / K + 0.01 * torch.eye(K, device=dev)
        Hw = H0.clone()

        def f():
            Hw.copy_(H0)
            ops.gptq_factor(Hw)
        ms = timed(f, args.steps)
        out["results"].append({"kernel": "gptq_factor", "K": K, "ms": ms,
                               "tflops_fp32": (2.0 / 3.0) * K ** 3 / (ms * 1e-3) / 1e12})
    if args.micro == "sweep":
        # the column sweep of one module (N = 4096 rows) with its tensor-core trailing updates
        K = args.micro_k
        N = 4096
        xx = torch.randn(2 * K, K, generator=g, device=dev)
        U = (xx.t() @ xx) / K + 0.01 * torch.eye(K, device=dev)
        del xx
        assert ops.gptq_factor(U) == 0
        a4 = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128)
        w = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        mn, mx = ops.observe_minmax(w, a4)
        scale, zp = ops.qparams(mn, mx, a4)
        wf = torch.empty(N, K, device=dev)

        def f():
            wf.copy_(w)
            ops.gptq_sweep(wf, U, scale, zp, a4)
        ms = timed(f, args.steps)
        out["results"].append({"kernel": "gptq_sweep", "N": N, "K": K, "ms": ms,
                               "tflops_fp32": (float(N) * K * K + 128.0 * N * K) / (ms * 1e-3) / 1e12})
    if args.micro == "small":
        # the batched kernels for many small problems, on the expert shapes of the MoE configuration:
        # `count` Hessians of K columns factored by one launch, `count` weights [N, K] swept by one launch
        K, count = args.micro_k, args.micro_count
        N = 2048 if K <= 1024 else 768
        xx = torch.randn(2 * K, K, generator=g, device=dev)
        H0 = (xx.t() @ xx) / K + 0.01 * torch.eye(K, device=dev)
        del xx
        Hs = [H0.clone() for _ in range(count)]

        def ff():
            for H in Hs:
                H.copy_(H0)
            ops.gptq_factor_batched(Hs)
        ms = timed(ff, args.steps) - timed(lambda: [H.copy_(H0) for H in Hs], args.steps)
        out["results"].append({"kernel": "gptq_factor_batched", "K": K, "count": count, "ms": ms,
                               "tflops_fp32": count * (2.0 / 3.0) * K ** 3 / (ms * 1e-3) / 1e12})
        a8 = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel")
        ws = [(torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(count)]
        qp = [ops.qparams(*ops.observe_minmax(w, a8), a8) for w in ws]
        wfs = [torch.empty(N, K, device=dev) for _ in range(count)]

        def restore():
            for wf, w in zip(wfs, ws):
                wf.copy_(w)

        def fs():
            restore()
            ops.gptq_sweep_batched(wfs, Hs, [q[0] for q in qp], None, a8)
        ms = timed(fs, args.steps) - timed(restore, args.steps)
        out["results"].append({"kernel": "gptq_sweep_batched", "N": N, "K": K, "count": count, "ms": ms,
                               "tflops_fp32": count * (float(N) * K * K + 128.0 * N * K) / (ms * 1e-3) / 1e12})
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", default=None, choices=["syrk", "pack", "factor", "sweep", "mse", "small", "all"],
                    help="kernel-level micro benchmark instead of the layer step")
    ap.add_argument("--micro-k", type=int, default=4096)
    ap.add_argument("--micro-t", type=int, default=32768)
    ap.add_argument("--micro-count", type=int, default=128, help="problems per launch of --micro small")
    ap.add_argument("--workload", default="llama8b", choices=["llama8b", "moe", "70b"],
                    help="llama8b: the headline layer step (configs[2]); moe: one Qwen3-30B-A3B-shaped layer "
                         "(configs[3]); 70b: module-level figures at the Llama-3-70B widths (configs[4])")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens-per-call", type=int, default=32768)
    ap.add_argument("--seqs", type=int, default=SEQS, help="calibration sequences (512 = the named config)")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--solve-streams", type=int, default=4,
                    help="CUDA streams the factorisations / sweeps of one layer are spread over")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-pack", action="store_true", help="skip the quantize/pack kernel figures")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the last timed step")
    ap.add_argument("--no-oneshot", action="store_true", help="skip the whole-model oneshot() run")
    ap.add_argument("--oneshot-seqs", type=int, default=SEQS)
    ap.add_argument("--oneshot-batch", type=int, default=8, help="sequences per calibration batch of the oneshot run")
    args = ap.parse_args()
    if args.workload == "moe":
        run_moe(args)
    elif args.workload == "70b":
        run_70b(args)
    elif args.micro:
        run_micro(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
