"""CPU-side checks: the C-ABI library is built, loads, and exports every symbol that
include/b200q.h declares; host-side argument handling."""
import os
import re

import pytest
import torch

from llm_compressor_b200 import _lib, compressors, ops
from llm_compressor_b200.quant_args import QuantizationArgs, preset_name_to_scheme

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200q.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)
    assert b"sm_100a" in lib.b200q_version()


def test_no_cpu_fallback():
    args = QuantizationArgs(num_bits=4, strategy="group", group_size=128)
    with pytest.raises(_lib.B200QError):
        ops.observe_minmax(torch.zeros(4, 128, dtype=torch.bfloat16), args)


def test_quant_args_aliases_and_presets():
    a = QuantizationArgs(num_bits=4, group_size=128, actorder="static")
    assert a.strategy == "group" and a.actorder == "weight" and a.observer == "memoryless_minmax"
    assert QuantizationArgs(num_bits=4, group_size=128, actorder=True).actorder == "group"
    with pytest.raises(ValueError):
        QuantizationArgs(num_bits=4, strategy="channel", actorder="group")
    with pytest.raises(ValueError):
        QuantizationArgs(num_bits=4, strategy="group")
    s = preset_name_to_scheme("W4A16", ["Linear"])
    assert s.weights.group_size == 128 and s.input_activations is None
    assert preset_name_to_scheme("nvfp4a16", ["Linear"]).weights.scale_dtype == torch.float8_e4m3fn
    assert preset_name_to_scheme("MXFP4", ["Linear"]).weights.is_mx


def test_format_inference_priority():
    f = compressors.infer_module_format
    assert f(preset_name_to_scheme("W4A16", ["Linear"])) == "pack-quantized"
    assert f(preset_name_to_scheme("W8A16", ["Linear"])) == "pack-quantized"
    assert f(preset_name_to_scheme("W8A8", ["Linear"])) == "int-quantized"
    assert f(preset_name_to_scheme("FP8_DYNAMIC", ["Linear"])) == "float-quantized"
    assert f(preset_name_to_scheme("NVFP4A16", ["Linear"])) == "nvfp4-pack-quantized"
    assert f(preset_name_to_scheme("MXFP4A16", ["Linear"])) == "mxfp4-pack-quantized"
    assert f(preset_name_to_scheme("MXFP8A16", ["Linear"])) == "mxfp8-quantized"
    assert f(QuantizationArgs(num_bits=8, type="float", strategy="channel")) == "naive-quantized"


def test_accepts_compressed_tensors_args():
    ct = pytest.importorskip("compressed_tensors.quantization")
    a = QuantizationArgs.of(ct.QuantizationArgs(num_bits=4, type="int", strategy="group", group_size=128,
                                                actorder="static"))
    assert (a.num_bits, a.strategy, a.group_size, a.actorder) == (4, "group", 128, "weight")
    c = a.c_struct()
    assert (c.num_bits, c.strategy, c.group_size) == (4, _lib.GROUP, 128)


def test_run_concurrent_keeps_order_and_raises():
    from llm_compressor_b200.streams import run_concurrent

    assert run_concurrent([lambda i=i: i * i for i in range(6)], "cpu", 4) == [0, 1, 4, 9, 16, 25]
    assert run_concurrent([], "cpu") == []

    def bad():
        raise RuntimeError("boom")
    with pytest.raises(RuntimeError, match="boom"):
        run_concurrent([lambda: 1, bad], "cpu")
