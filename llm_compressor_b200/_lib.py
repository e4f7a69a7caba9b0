"""ctypes binding of ``libb200q.so`` (declared in ``include/b200q.h``).

The library is the only compute path of this package: if it is missing or a call
returns a non-zero status the caller gets an exception; nothing falls back to torch
ops or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200Q_LIBRARY") or os.path.join(_PKG, "libb200q.so")

# enums of include/b200q.h
BF16, F32, F16 = 0, 1, 2
QINT, QFLOAT = 0, 1
TENSOR, CHANNEL, GROUP, TENSOR_GROUP, BLOCK = 0, 1, 2, 3, 4
SCALE_PLAIN, SCALE_FP8, SCALE_E8M0 = 0, 1, 2
ZP_INT8, ZP_FP8, ZP_UINT8 = 0, 1, 2
NOT_POSITIVE_DEFINITE = 1

_STATUS = {
    -1: "bad argument (pointer / shape / alignment)",
    -2: "unsupported combination",
    -3: "CUDA error",
    -4: "device-side error (bounded wait expired)",
}


class QArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_bits", "qtype", "symmetric", "strategy", "group_size", "block_h", "block_w",
        "scale_kind", "zp_kind")]


class B200QError(RuntimeError):
    pass


_p, _i, _i64, _f, _d = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double
_qa = C.POINTER(QArgs)

# name -> (restype, argtypes); must list every symbol of include/b200q.h
SIGNATURES = {
    "b200q_version": (C.c_char_p, []),
    "b200q_last_error": (C.c_char_p, []),
    "b200q_launch_count": (C.c_longlong, []),
    "b200q_take_wait_status": (_i, []),
    "b200q_observe_minmax_workspace_bytes": (C.c_size_t, [_i64, _i64, _qa]),
    "b200q_observe_minmax": (_i, [_p, _i, _i64, _i64, _i64, _qa, _p, _p, _p, _p]),
    "b200q_absmax_accumulate": (_i, [_p, _p, _i, _i64, _p, _p]),
    "b200q_global_scale_finalize": (_i, [_p, _i, _p, _p]),
    "b200q_absmax_accumulate_weight": (_i, [_p, _i, _i64, _i64, _i64, _p, _p]),
    "b200q_qparams": (_i, [_p, _p, _i, _i64, _qa, _p, _p, _p, _p]),
    "b200q_observe_mse_workspace_bytes": (C.c_size_t, [_i64, _i64, _qa, _i]),
    "b200q_observe_mse_steps": (_i, [_d, _d]),
    "b200q_observe_mse": (_i, [_p, _i, _i64, _i64, _i64, _qa, _d, _i, _d, _f, _f, _p, _p, _p, _p]),
    "b200q_observe_mse_noalloc": (_i, [_p, _i, _i64, _i64, _i64, _qa, _d, _i, _d, _f, _f, _p, _p, _p]),
    "b200q_fake_quantize": (_i, [_p, _i, _i64, _i64, _i64, _p, _i, _p, _p, _p, _qa, _p, _i64, _p]),
    "b200q_quantize_pack": (_i, [_p, _i, _i64, _i64, _i64, _p, _i, _p, _p, _p, _qa, _i, _p, _p]),
    "b200q_pack_zero_points": (_i, [_p, _i64, _i64, _i, _p, _p]),
    "b200q_compress_scale": (_i, [_p, _i, _i64, _i, _p, _p]),
    "b200q_rtn_quantize_pack": (_i, [_p, _i, _i64, _i64, _i64, _qa, _p, _p, _p, _p, _p]),
    "b200q_nvfp4_quantize_pack": (_i, [_p, _i, _i64, _i64, _i64, _p, _p, _p, _p, _p]),
    "b200q_hessian_syrk": (_i, [_p, _i64, _i64, _i64, _p, _i64, _f, _p, _p]),
    "b200q_hessian_finalize": (_i, [_p, _i64, _i64, _f, _p]),
    "b200q_set_reproducible": (None, [_i]),
    "b200q_get_reproducible": (_i, []),
    "b200q_actorder_perm": (_i, [_p, _i64, _i64, _p, _p]),
    "b200q_gather_columns_f32": (_i, [_p, _i, _i64, _i64, _i64, _p, _p, _i64, _p]),
    "b200q_permute_hessian": (_i, [_p, _i64, _i64, _p, _p, _i64, _p]),
    "b200q_scatter_columns_cast": (_i, [_p, _i64, _i64, _i64, _p, _p, _i, _i64, _p]),
    "b200q_gptq_prepare": (_i, [_p, _i64, _i64, _p, _i64, _i64, _f, _p]),
    "b200q_gptq_zero_dead_columns": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p]),
    "b200q_gptq_factor_workspace_bytes": (C.c_size_t, [_i64]),
    "b200q_gptq_factor": (_i, [_p, _i64, _i64, _p, _p, _p]),
    "b200q_gemm_tf32x3_workspace_bytes": (C.c_size_t, [_i64, _i64, _i64]),
    "b200q_gemm_tf32x3": (_i, [_i, _p, _i64, _p, _i64, _p, _i64, _i64, _i64, _i64, _f, _f, _i, _p, _p, _p]),
    "b200q_gptq_sweep_workspace_bytes": (C.c_size_t, [_i64, _i64, _i]),
    "b200q_gptq_sweep": (_i, [_p, _i64, _i64, _i64, _p, _i64, _p, _i, _p, _p, _p, _qa, _i, _p, _p, _p]),
    "b200q_gptq_factor_batched_workspace_bytes": (C.c_size_t, [_i64, _i]),
    "b200q_gptq_factor_batched": (_i, [_p, _p, _i, _i64, _i64, _p, _p]),
    "b200q_gather_columns_f32_batched": (_i, [_p, _i, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _p]),
    "b200q_scatter_columns_cast_batched": (_i, [_p, _p, _p, _i, _i, _i64, _i64, _i64, _i64, _p]),
    "b200q_gptq_sweep_batched": (_i, [_p, _p, _p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _qa, _i, _p]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen the kernel library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200QError(
                f"{LIB_PATH} not found: build it with `python -m llm_compressor_b200.build` "
                "(there is no fallback path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> int:
    """Raise on negative (error) status; positive numeric statuses are returned."""
    if rc < 0:
        detail = load().b200q_last_error().decode() if rc == -3 else ""
        raise B200QError(f"{what}: {_STATUS.get(rc, rc)} {detail}")
    return rc


def ptr(t):
    """Device pointer of a torch tensor (or None)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
