"""The allocation-free MSE observer entry point against the ordinary one.

Some users of this library cannot allocate device memory when they observe a weight: a server
that has given all of its memory to a cache pool, or code that runs inside an allocator
callback.  ``b200q_observe_mse_noalloc`` keeps its scratch in an array inside the library, and
must return exactly what ``b200q_observe_mse`` returns.  The array is shared by every call, so
two calls in a row (with different candidate counts, the second shorter) check that what one
call leaves behind does not leak into the next.  This file is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from helpers import synth_weight
from llm_compressor_b200 import _lib, ops
from llm_compressor_b200.quant_args import QuantizationArgs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference(w, args, **kw):
    return ops.observe_mse(w, args, **kw)


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    args = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128)
    shape = args.qparam_shape(64, 1024)
    calls = [
        (synth_weight(64, 1024, seed=41).to(DEV), dict(maxshrink=0.8, grid=100.0, patience=5, norm=2.4)),
        (synth_weight(64, 1024, seed=42).to(DEV), dict(maxshrink=0.2, grid=100.0, patience=2, norm=2.0)),
    ]
    # outputs are allocated up front: the calls under test allocate nothing themselves
    outs = [(torch.empty(shape, dtype=torch.bfloat16, device=DEV), torch.empty(shape, dtype=torch.bfloat16, device=DEV))
            for _ in calls]
    expected = [_reference(w, args, **kw) for w, kw in calls]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    for (w, kw), (mn, mx) in zip(calls, outs):
        ops.observe_mse_noalloc(w, args, mn, mx, **kw)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    for (mn, mx), (emn, emx) in zip(outs, expected):
        assert torch.equal(mn, emn) and torch.equal(mx, emx)


def test_noalloc_channel_strategy_and_fp32_weights():
    args = QuantizationArgs(num_bits=8, type="int", symmetric=False, strategy="channel")
    w = synth_weight(48, 512, seed=7, dtype=torch.float32).to(DEV)
    emn, emx = _reference(w, args)
    mn, mx = torch.empty_like(emn), torch.empty_like(emx)
    ops.observe_mse_noalloc(w, args, mn, mx)
    ops.observe_mse_noalloc(w, args, mn, mx)  # same call again over the used scratch
    assert torch.equal(mn, emn) and torch.equal(mx, emx)


def test_noalloc_rejects_more_candidates_than_its_scratch_holds():
    args = QuantizationArgs(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128)
    w = synth_weight(8, 256, seed=1).to(DEV)
    mn = torch.empty(args.qparam_shape(8, 256), dtype=torch.bfloat16, device=DEV)
    mx = torch.empty_like(mn)
    with pytest.raises(_lib.B200QError, match="1023"):
        ops.observe_mse_noalloc(w, args, mn, mx, maxshrink=1.0, grid=2000.0)
    # straight through the C ABI: error status and a message, nothing launched
    lib = _lib.load()
    rc = lib.b200q_observe_mse_noalloc(C.c_void_p(w.data_ptr()), _lib.BF16, 8, 256, 256, args.c_struct(), 1.0, 5,
                                       2000.0, 2.4, 1.0, C.c_void_p(mn.data_ptr()), C.c_void_p(mx.data_ptr()),
                                       _lib.stream_ptr())
    assert rc == -1
    assert b"1023" in lib.b200q_last_error()
