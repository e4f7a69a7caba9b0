"""torch-tensor front end of the C-ABI kernels: one function per entry point.

torch is used for device memory and the current stream only; every computation is a call
into ``libb200q.so``.  All tensors must live on a CUDA device.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .quant_args import QuantizationArgs

_DT = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"b200q kernels take bfloat16 or float32 tensors, got {t.dtype}") from None


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.B200QError("b200q kernels need CUDA tensors; there is no CPU path")


def _2d(w: torch.Tensor):
    if w.ndim != 2 or w.stride(1) != 1:
        raise ValueError("expected a 2-D tensor with contiguous rows")
    return w.shape[0], w.shape[1], w.stride(0)


def _zp_storage(args: QuantizationArgs):
    return args.zp_dtype


# ------------------------------------------------------------------------------ observers
def observe_minmax(w: torch.Tensor, args: QuantizationArgs):
    """(min_vals, max_vals) of qparam shape, in w's dtype."""
    _need_cuda(w)
    lib = _lib.load()
    N, K, ld = _2d(w)
    qa = args.c_struct()
    shape = args.qparam_shape(N, K)
    mn = torch.empty(shape, dtype=w.dtype, device=w.device)
    mx = torch.empty(shape, dtype=w.dtype, device=w.device)
    nbytes = lib.b200q_observe_minmax_workspace_bytes(N, K, qa)
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=w.device)
    check(lib.b200q_observe_minmax(ptr(w), _dt(w), N, K, ld, qa, ptr(mn), ptr(mx), ptr(scratch),
                                   stream_ptr()), "b200q_observe_minmax")
    return mn, mx


def observe_mse(w, args, maxshrink=0.20, patience=5, grid=100.0, norm=2.4, expand=1.0):
    _need_cuda(w)
    lib = _lib.load()
    N, K, ld = _2d(w)
    if args.strategy == "tensor_group" and args.scale_dtype is not None:
        args = args.model_copy(update={"scale_dtype": None})
    qa = args.c_struct()
    shape = args.qparam_shape(N, K)
    mn = torch.empty(shape, dtype=w.dtype, device=w.device)
    mx = torch.empty(shape, dtype=w.dtype, device=w.device)
    steps = lib.b200q_observe_mse_steps(float(maxshrink), float(grid))
    if steps < 0:
        raise ValueError(f"maxshrink * grid = {maxshrink * grid} is not a valid number of candidates")
    nbytes = lib.b200q_observe_mse_workspace_bytes(N, K, qa, steps)
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=w.device)
    check(lib.b200q_observe_mse(ptr(w), _dt(w), N, K, ld, qa, float(maxshrink), int(patience),
                                float(grid), float(norm), float(expand), ptr(mn), ptr(mx),
                                ptr(scratch), stream_ptr()), "b200q_observe_mse")
    return mn, mx


def observe_mse_noalloc(w, args, mn: torch.Tensor, mx: torch.Tensor, maxshrink=0.20, patience=5,
                        grid=100.0, norm=2.4, expand=1.0):
    """MSE grid search into caller-provided ``mn`` / ``mx`` without allocating anything on the
    device: for callers that must not touch an allocator (memory fully committed to a cache
    pool, allocator callbacks).  The scratch is a fixed array inside the library, so at most
    1023 shrink candidates are accepted, and calls that overlap on the GPU would race on it:
    keep them on one stream.  Make the first call on a device outside stream capture."""
    _need_cuda(w, mn, mx)
    N, K, ld = _2d(w)
    if args.strategy == "tensor_group" and args.scale_dtype is not None:
        args = args.model_copy(update={"scale_dtype": None})
    shape = tuple(args.qparam_shape(N, K))
    for t in (mn, mx):
        if tuple(t.shape) != shape or t.dtype != w.dtype or not t.is_contiguous():
            raise ValueError(f"min/max outputs must be contiguous {shape} tensors of dtype {w.dtype}")
    lib = _lib.load()
    rc = lib.b200q_observe_mse_noalloc(ptr(w), _dt(w), N, K, ld, args.c_struct(), float(maxshrink),
                                       int(patience), float(grid), float(norm), float(expand), ptr(mn),
                                       ptr(mx), stream_ptr())
    if rc == -1 and lib.b200q_observe_mse_steps(float(maxshrink), float(grid)) > 1023:
        raise _lib.B200QError("b200q_observe_mse_noalloc: int(maxshrink*grid) = %d candidates exceed the "
                              "built-in scratch of 1023; use observe_mse" % int(maxshrink * grid))
    check(rc, "b200q_observe_mse_noalloc")
    return mn, mx


def absmax_accumulate(mn, mx, absmax: torch.Tensor):
    _need_cuda(mn, mx, absmax)
    assert absmax.dtype == torch.float32
    check(_lib.load().b200q_absmax_accumulate(ptr(mn), ptr(mx), _dt(mn), mn.numel(), ptr(absmax),
                                              stream_ptr()), "b200q_absmax_accumulate")


def global_scale_from_absmax(absmax: torch.Tensor, stat_dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(1, dtype=torch.float32, device=absmax.device)
    check(_lib.load().b200q_global_scale_finalize(ptr(absmax), _DT[stat_dtype], ptr(out),
                                                  stream_ptr()), "b200q_global_scale_finalize")
    return out


def qparams(mn, mx, args: QuantizationArgs, global_scale=None):
    """(scale, zero_point) of the statistics' shape."""
    _need_cuda(mn, mx, global_scale)
    mn, mx = mn.contiguous(), mx.contiguous()
    sdt = torch.float32 if global_scale is not None else mn.dtype
    scale = torch.empty(mn.shape, dtype=sdt, device=mn.device)
    zp = torch.empty(mn.shape, dtype=_zp_storage(args), device=mn.device)
    check(_lib.load().b200q_qparams(ptr(mn), ptr(mx), _dt(mn), mn.numel(), args.c_struct(),
                                    ptr(global_scale), ptr(scale), ptr(zp), stream_ptr()),
          "b200q_qparams")
    return scale, zp


# ------------------------------------------------------------------------ quantize / pack
def _prep_params(w, scale, zp, g_idx, global_scale):
    _need_cuda(w, scale, zp, g_idx, global_scale)
    scale = scale.contiguous()
    zp = None if zp is None else zp.contiguous()
    if g_idx is not None:
        g_idx = g_idx.to(torch.int32).contiguous()
        if bool((g_idx < 0).any()):
            g_idx = None  # uninitialised g_idx means column order
    if global_scale is not None:
        global_scale = global_scale.to(torch.float32).contiguous()
    return scale, zp, g_idx, global_scale


def fake_quantize(w, scale, zp, args: QuantizationArgs, g_idx=None, global_scale=None):
    scale, zp, g_idx, global_scale = _prep_params(w, scale, zp, g_idx, global_scale)
    N, K, ld = _2d(w)
    out = torch.empty((N, K), dtype=w.dtype, device=w.device)
    check(_lib.load().b200q_fake_quantize(ptr(w), _dt(w), N, K, ld, ptr(scale), _dt(scale), ptr(zp),
                                          ptr(g_idx), ptr(global_scale), args.c_struct(), ptr(out),
                                          out.stride(0), stream_ptr()), "b200q_fake_quantize")
    return out


def quantize_pack(w, scale, zp, args: QuantizationArgs, g_idx=None, global_scale=None,
                  pack_int8=False):
    """Storage codes: int32 words (int4, or int8 with pack_int8), int8 / float8 bytes, or
    uint8 nibble pairs (FP4)."""
    scale, zp, g_idx, global_scale = _prep_params(w, scale, zp, g_idx, global_scale)
    N, K, ld = _2d(w)
    dev = w.device
    if args.type == "int" and args.num_bits == 4:
        out = torch.empty((N, -(-K // 8)), dtype=torch.int32, device=dev)
    elif args.type == "int" and args.num_bits == 8:
        out = (torch.empty((N, -(-K // 4)), dtype=torch.int32, device=dev) if pack_int8
               else torch.empty((N, K), dtype=torch.int8, device=dev))
    elif args.type == "float" and args.num_bits == 8:
        out = torch.empty((N, K), dtype=torch.float8_e4m3fn, device=dev)
    elif args.type == "float" and args.num_bits == 4:
        out = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
    else:
        raise ValueError(f"unsupported code type {args.type}{args.num_bits}")
    check(_lib.load().b200q_quantize_pack(ptr(w), _dt(w), N, K, ld, ptr(scale), _dt(scale), ptr(zp),
                                          ptr(g_idx), ptr(global_scale), args.c_struct(),
                                          int(pack_int8), ptr(out), stream_ptr()),
          "b200q_quantize_pack")
    return out


def pack_zero_points(zp: torch.Tensor, num_bits: int) -> torch.Tensor:
    _need_cuda(zp)
    zp = zp.to(torch.int8).contiguous()
    N, G = zp.shape
    pf = 32 // num_bits
    out = torch.empty((-(-N // pf), G), dtype=torch.int32, device=zp.device)
    check(_lib.load().b200q_pack_zero_points(ptr(zp), N, G, num_bits, ptr(out), stream_ptr()),
          "b200q_pack_zero_points")
    return out


def compress_scale(scale: torch.Tensor, kind: str) -> torch.Tensor:
    """kind "fp8" -> float8_e4m3fn tensor, "e8m0" -> uint8 biased exponents."""
    _need_cuda(scale)
    scale = scale.contiguous()
    out = torch.empty(scale.shape, dtype=torch.uint8, device=scale.device)
    k = {"fp8": _lib.SCALE_FP8, "e8m0": _lib.SCALE_E8M0}[kind]
    check(_lib.load().b200q_compress_scale(ptr(scale), _dt(scale), scale.numel(), k, ptr(out),
                                           stream_ptr()), "b200q_compress_scale")
    return out.view(torch.float8_e4m3fn) if kind == "fp8" else out


def _code_buffer(args, N, K, dev):
    if args.num_bits == 4:
        if args.type == "int":
            return torch.empty((N, K // 8), dtype=torch.int32, device=dev)
        return torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
    if args.type == "int":
        return torch.empty((N, K // 4), dtype=torch.int32, device=dev)
    return torch.empty((N, K), dtype=torch.float8_e4m3fn, device=dev)


def rtn_quantize_pack(w, args: QuantizationArgs):
    """One pass: statistics -> qparams -> codes.  Returns dict(scale, zero_point,
    scale_store, codes); int8 codes come packed four to an int32 word."""
    _need_cuda(w)
    N, K, ld = _2d(w)
    dev = w.device
    shape = args.qparam_shape(N, K)
    scale = torch.empty(shape, dtype=w.dtype, device=dev)
    zp = torch.empty(shape, dtype=_zp_storage(args), device=dev)
    store = torch.empty(shape, dtype=torch.uint8, device=dev) if args.is_mx else None
    out = _code_buffer(args, N, K, dev)
    check(_lib.load().b200q_rtn_quantize_pack(ptr(w), _dt(w), N, K, ld, args.c_struct(), ptr(scale),
                                              ptr(zp), ptr(store), ptr(out), stream_ptr()),
          "b200q_rtn_quantize_pack")
    return dict(scale=scale, zero_point=zp, scale_store=store, codes=out)


def nvfp4_quantize_pack(w, global_scale: torch.Tensor):
    _need_cuda(w, global_scale)
    N, K, ld = _2d(w)
    dev = w.device
    scale = torch.empty((N, K // 16), dtype=w.dtype, device=dev)
    store = torch.empty((N, K // 16), dtype=torch.uint8, device=dev)
    out = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
    gs = global_scale.to(torch.float32).contiguous()
    check(_lib.load().b200q_nvfp4_quantize_pack(ptr(w), _dt(w), N, K, ld, ptr(gs), ptr(scale),
                                                ptr(store), ptr(out), stream_ptr()),
          "b200q_nvfp4_quantize_pack")
    return dict(scale=scale, scale_store=store.view(torch.float8_e4m3fn), codes=out)


def nvfp4_two_pass(w, partners=()):
    """NVFP4 weight quantisation from nothing but the weight: pass 1 finds the tensor-wide
    largest magnitude (over ``w`` and the ``partners`` that share its global scale: q/k/v,
    gate/up) and turns it into the global scale, pass 2 is ``nvfp4_quantize_pack``.  Returns its
    dict plus ``global_scale``."""
    from .quant_args import QuantizationArgs
    _need_cuda(w, *partners)
    targs = QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor")
    absmax = torch.zeros(1, dtype=torch.float32, device=w.device)
    lib = _lib.load()
    for t in (w, *partners):
        N, K, ld = _2d(t)
        rc = lib.b200q_absmax_accumulate_weight(ptr(t), _dt(t), N, K, ld, ptr(absmax), stream_ptr())
        if rc == -2:   # shape / dtype the streaming kernel does not take
            mn, mx = observe_minmax(t, targs)
            absmax_accumulate(mn, mx, absmax)
        else:
            check(rc, "b200q_absmax_accumulate_weight")
    gs = global_scale_from_absmax(absmax, w.dtype)
    out = nvfp4_quantize_pack(w, gs)
    out["global_scale"] = gs
    return out


# ------------------------------------------------------------------------------- Hessian
def hessian_syrk(x: torch.Tensor, H: torch.Tensor, alpha: float = 2.0, status=None):
    """H_lower += alpha * x^T x ; x [T,K] bf16 with contiguous rows.  ``status`` (int32 device
    tensor, optional) becomes non-zero if a bounded wait inside the kernel ran out."""
    _need_cuda(x, H)
    if x.dtype != torch.bfloat16:
        raise TypeError("hessian_syrk takes bfloat16 activations")
    T, K, ld = _2d(x)
    assert H.dtype == torch.float32 and H.shape == (K, K) and H.stride(1) == 1
    if K % 8 or H.stride(0) % 4:
        # the kernel's tiles need 16-byte rows: widths that are not a multiple of 8 go through a
        # zero-padded copy (the reference accepts any width)
        Kp = -(-K // 8) * 8
        xp = torch.zeros((T, Kp), dtype=x.dtype, device=x.device)
        xp[:, :K] = x
        Hp = torch.zeros((Kp, Kp), dtype=torch.float32, device=H.device)
        hessian_syrk(xp, Hp, alpha, status)
        H += Hp[:K, :K]
        return H
    check(_lib.load().b200q_hessian_syrk(ptr(x), T, K, ld, ptr(H), H.stride(0), float(alpha),
                                         ptr(status), stream_ptr()), "b200q_hessian_syrk")
    return H


def hessian_finalize(H: torch.Tensor, scale: float = 1.0):
    _need_cuda(H)
    K = H.shape[0]
    check(_lib.load().b200q_hessian_finalize(ptr(H), K, H.stride(0), float(scale), stream_ptr()),
          "b200q_hessian_finalize")
    return H


# ---------------------------------------------------------------------------- GPTQ solve
def set_reproducible(on: bool) -> bool:
    """Bitwise reproducible Hessian accumulation (no atomics across token splits) for all later
    calls in this process; returns the previous setting."""
    lib = _lib.load()
    before = bool(lib.b200q_get_reproducible())
    lib.b200q_set_reproducible(int(bool(on)))
    return before


def actorder_perm(H: torch.Tensor) -> torch.Tensor:
    _need_cuda(H)
    K = H.shape[0]
    perm = torch.empty(K, dtype=torch.int32, device=H.device)
    check(_lib.load().b200q_actorder_perm(ptr(H), K, H.stride(0), ptr(perm), stream_ptr()),
          "b200q_actorder_perm")
    return perm


def gather_columns_f32(w: torch.Tensor, perm=None) -> torch.Tensor:
    _need_cuda(w, perm)
    N, K, ld = _2d(w)
    out = torch.empty((N, K), dtype=torch.float32, device=w.device)
    check(_lib.load().b200q_gather_columns_f32(ptr(w), _dt(w), N, K, ld, ptr(perm), ptr(out),
                                               out.stride(0), stream_ptr()),
          "b200q_gather_columns_f32")
    return out


def permute_hessian(H: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    _need_cuda(H, perm)
    K = H.shape[0]
    out = torch.empty_like(H)
    check(_lib.load().b200q_permute_hessian(ptr(H), K, H.stride(0), ptr(perm), ptr(out),
                                            out.stride(0), stream_ptr()), "b200q_permute_hessian")
    return out


def scatter_columns_cast(wf: torch.Tensor, dtype: torch.dtype, perm=None) -> torch.Tensor:
    _need_cuda(wf, perm)
    N, K, ld = _2d(wf)
    out = torch.empty((N, K), dtype=dtype, device=wf.device)
    check(_lib.load().b200q_scatter_columns_cast(ptr(wf), N, K, ld, ptr(perm), ptr(out), _DT[dtype],
                                                 out.stride(0), stream_ptr()),
          "b200q_scatter_columns_cast")
    return out


def gptq_prepare(H: torch.Tensor, wf: torch.Tensor, percdamp: float):
    _need_cuda(H, wf)
    K = H.shape[0]
    N, ldf = (wf.shape[0], wf.stride(0)) if wf is not None else (0, K)
    check(_lib.load().b200q_gptq_prepare(ptr(H), K, H.stride(0), ptr(wf), N, ldf,
                                         float(percdamp), stream_ptr()), "b200q_gptq_prepare")


def gptq_zero_dead_columns(diag: torch.Tensor, wf: torch.Tensor):
    _need_cuda(diag, wf)
    assert diag.dtype == torch.float32 and diag.ndim == 1
    check(_lib.load().b200q_gptq_zero_dead_columns(ptr(diag), diag.stride(0), diag.numel(), ptr(wf),
                                                   wf.shape[0], wf.stride(0), stream_ptr()),
          "b200q_gptq_zero_dead_columns")


def gptq_factor_async(H: torch.Tensor) -> torch.Tensor:
    """In place H -> U (upper, U^T U = H^-1) without waiting for the result.  Returns the device
    status words for ``gptq_factor_status``; U is meaningless when the status is not 0."""
    _need_cuda(H)
    lib = _lib.load()
    K = H.shape[0]
    ws = torch.empty(max(lib.b200q_gptq_factor_workspace_bytes(K), 4), dtype=torch.uint8,
                     device=H.device)
    status = torch.zeros(4, dtype=torch.int32, device=H.device)
    check(lib.b200q_gptq_factor(ptr(H), K, H.stride(0), ptr(ws), ptr(status), stream_ptr()),
          "b200q_gptq_factor")
    return status


def gptq_factor_status(status: torch.Tensor) -> int:
    """Waits for a factorisation: 0, or NOT_POSITIVE_DEFINITE; raises on a device error."""
    st = status.tolist()
    if st[2] != 0:
        raise _lib.B200QError("b200q_gptq_factor: a bounded wait inside the GEMM kernel expired")
    return int(st[0])


def gptq_factor(H: torch.Tensor) -> int:
    """In place H -> U (upper, U^T U = H^-1).  Returns 0, or NOT_POSITIVE_DEFINITE."""
    return gptq_factor_status(gptq_factor_async(H))


def gptq_sweep(wf, U, scale, zp, args: QuantizationArgs, blocksize=128, col_group=None,
               global_scale=None, return_status: bool = False):
    """Runs the column sweep in place on wf; returns per-row losses, and with ``return_status``
    also the call's device status word (int32 [1]; non-zero: a bounded wait inside a
    trailing-update GEMM ran out and wf is incomplete)."""
    _need_cuda(wf, U, scale, zp, col_group, global_scale)
    lib = _lib.load()
    N, K, ld = _2d(wf)
    scale = scale.contiguous()
    zp = None if zp is None else zp.contiguous()
    if col_group is not None:
        col_group = col_group.to(torch.int32).contiguous()
    if global_scale is not None:
        global_scale = global_scale.to(torch.float32).contiguous()
    losses = torch.empty(N, dtype=torch.float32, device=wf.device)
    ws = torch.empty(max(lib.b200q_gptq_sweep_workspace_bytes(N, K, blocksize), 4) + 16,
                     dtype=torch.uint8, device=wf.device)
    check(lib.b200q_gptq_sweep(ptr(wf), N, K, ld, ptr(U), 0 if U is None else U.stride(0),
                               ptr(scale), _dt(scale), ptr(zp), ptr(col_group), ptr(global_scale),
                               args.c_struct(), int(blocksize), ptr(losses), ptr(ws), stream_ptr()),
          "b200q_gptq_sweep")
    if return_status:
        return losses, ws[:4].view(torch.int32)
    return losses


def _pointer_table(rows) -> torch.Tensor:
    """Device int64 [len(rows), count]: row r holds the addresses of the tensors in rows[r]
    (a row that is None becomes a row of zeros and is passed to the library as NULL)."""
    first = next(r for r in rows if r is not None)
    table = [[0] * len(first) if r is None else [t.data_ptr() for t in r] for r in rows]
    return torch.tensor(table, dtype=torch.int64, device=first[0].device)


def gptq_factor_batched(Hs) -> torch.Tensor:
    """In place H -> U for a list of small Hessians of one size, one thread block each, in one
    launch.  Returns the device status words, int32 [count, 4] (see ``gptq_factor_async``)."""
    _need_cuda(*Hs)
    lib = _lib.load()
    K, ld = Hs[0].shape[0], Hs[0].stride(0)
    for H in Hs:
        if H.shape != (K, K) or H.stride(0) != ld or H.stride(1) != 1 or H.dtype != torch.float32:
            raise ValueError("batched factorisation needs float32 Hessians of one size and one layout")
    count = len(Hs)
    scratch = torch.empty((count, K * K), dtype=torch.float32, device=Hs[0].device)
    status = torch.empty((count, 4), dtype=torch.int32, device=Hs[0].device)
    table = _pointer_table([Hs, list(scratch.unbind(0))])
    check(lib.b200q_gptq_factor_batched(ptr(table[0]), ptr(table[1]), count, K, ld, ptr(status), stream_ptr()),
          "b200q_gptq_factor_batched")
    return status


def gather_columns_f32_batched(ws, perms=None, dead_diags=None) -> torch.Tensor:
    """float32 copies [count, N, K] of weights of one shape, columns permuted by ``perms[i]`` and the
    columns with ``dead_diags[i][c] == 0`` zeroed, in one launch (either list may be None)."""
    count = len(ws)
    N, K, ld = _2d(ws[0])
    for w in ws:
        if _2d(w) != (N, K, ld) or w.dtype != ws[0].dtype:
            raise ValueError("batched gather needs weights of one shape, layout and dtype")
    _need_cuda(*ws)
    out = torch.empty((count, N, K), dtype=torch.float32, device=ws[0].device)
    if perms is not None:
        perms = [p.to(torch.int32).contiguous() for p in perms]
    if dead_diags is not None:
        dead_diags = [d.to(torch.float32).contiguous() for d in dead_diags]
    table = _pointer_table([ws, perms, dead_diags, list(out.unbind(0))])
    check(_lib.load().b200q_gather_columns_f32_batched(
        ptr(table[0]), _dt(ws[0]), ptr(table[1]) if perms is not None else None,
        ptr(table[2]) if dead_diags is not None else None, ptr(table[3]), count, N, K, ld, K, stream_ptr()),
        "b200q_gather_columns_f32_batched")
    return out


def scatter_columns_cast_batched(wfs, dtype: torch.dtype, perms=None) -> torch.Tensor:
    """The way back: [count, N, K] in ``dtype`` with ``out[i][:, perms[i][c]] = wfs[i][:, c]``."""
    count = len(wfs)
    N, K, ld = _2d(wfs[0])
    for w in wfs:
        if _2d(w) != (N, K, ld) or w.dtype != torch.float32:
            raise ValueError("batched scatter needs float32 matrices of one shape and layout")
    _need_cuda(*wfs)
    out = torch.empty((count, N, K), dtype=dtype, device=wfs[0].device)
    if perms is not None:
        perms = [p.to(torch.int32).contiguous() for p in perms]
    table = _pointer_table([wfs, perms, list(out.unbind(0))])
    check(_lib.load().b200q_scatter_columns_cast_batched(
        ptr(table[0]), ptr(table[1]) if perms is not None else None, ptr(table[2]), _DT[dtype], count, N, K, ld, K,
        stream_ptr()), "b200q_scatter_columns_cast_batched")
    return out


def gptq_sweep_batched(wfs, Us, scales, zps, args: QuantizationArgs, col_groups=None, global_scales=None,
                       blocksize=128) -> torch.Tensor:
    """The column sweep, in place, on a list of float32 weights of one shape that share the
    quantisation scheme, in one launch.  ``Us``, ``zps``, ``col_groups``, ``global_scales``: a list
    with one tensor per weight, or None for all.  Returns the per-row losses [count, N]."""
    count = len(wfs)
    N, K, ld = _2d(wfs[0])
    dev = wfs[0].device
    scales = [s.contiguous() for s in scales]
    sdt = _dt(scales[0])
    zps = None if zps is None else [z.contiguous() for z in zps]
    col_groups = None if col_groups is None else [c.to(torch.int32).contiguous() for c in col_groups]
    global_scales = None if global_scales is None else [g.to(torch.float32).contiguous() for g in global_scales]
    for lst in (wfs, Us, scales, zps, col_groups, global_scales):
        if lst is not None:
            if len(lst) != count:
                raise ValueError("one tensor per weight, or None for all")
            _need_cuda(*lst)
    for w in wfs:
        if _2d(w) != (N, K, ld) or w.dtype != torch.float32:
            raise ValueError("batched sweep needs float32 weights of one shape and one layout")
    ldu = 0
    if Us is not None:
        ldu = Us[0].stride(0)
        for U in Us:
            if U.shape != (K, K) or U.stride(0) != ldu or U.stride(1) != 1:
                raise ValueError("batched sweep needs factors of one size and one layout")
    if any(_dt(s) != sdt or s.numel() != scales[0].numel() for s in scales):
        raise ValueError("batched sweep needs scales of one dtype and one shape")
    losses = torch.empty((count, N), dtype=torch.float32, device=dev)
    table = _pointer_table([wfs, Us, scales, zps, col_groups, global_scales, list(losses.unbind(0))])

    def row(i, present):
        return ptr(table[i]) if present is not None else None

    check(_lib.load().b200q_gptq_sweep_batched(
        ptr(table[0]), row(1, Us), ptr(table[2]), sdt, row(3, zps), row(4, col_groups), row(5, global_scales),
        ptr(table[6]), count, N, K, ld, ldu, args.c_struct(), int(blocksize), stream_ptr()),
        "b200q_gptq_sweep_batched")
    return losses


def gemm_tf32x3(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, trans_b: bool, alpha=1.0, beta=0.0,
                lower_tiles=False, workspace: "torch.Tensor | None" = None) -> torch.Tensor:
    """c = beta*c + alpha * a @ (b.T if trans_b else b) on the tensor cores with float32 accuracy;
    a [M,Kd], Kd <= 128.  ``workspace`` (uint8, 16-byte aligned) is allocated when not given."""
    _need_cuda(a, b, c)
    lib = _lib.load()
    M, Kd = a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    need = lib.b200q_gemm_tf32x3_workspace_bytes(M, N, Kd)
    ws = workspace if workspace is not None else torch.empty(need + 16, dtype=torch.uint8, device=a.device)
    if ws.numel() < need:
        raise ValueError(f"workspace holds {ws.numel()} bytes, {need} needed")
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    check(lib.b200q_gemm_tf32x3(int(trans_b), ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(c), c.stride(0), M, N, Kd,
                                float(alpha), float(beta), int(lower_tiles), ptr(ws), ptr(status), stream_ptr()),
          "b200q_gemm_tf32x3")
    if int(status.item()) != 0:
        raise _lib.B200QError("b200q_gemm_tf32x3: a bounded wait inside the kernel expired")
    return c
