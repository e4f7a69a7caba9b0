"""Load the runnable parts of the reference (llm-compressor) for fixture generation.

Only used by ``make_golden.py`` in a container where the reference checkout is
present; nothing here runs in the GPU tests.  The reference package does not
import as a whole against compressed-tensors 0.15 (it wants newer symbols), so a
temporary copy with an emptied top-level ``__init__`` is put on ``sys.path`` and
the few missing ``compressed_tensors`` names are provided by an in-process shim
whose semantics follow ``src/llmcompressor/utils/dist.py:20-52``.
"""
import importlib
import importlib.util
import os
import shutil
import sys
import tempfile
import types

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

# the llm-compressor checkout to load (fixture generation and the plug-in test need one):
# LLMC_REFERENCE_ROOT, else a checkout named "reference" next to this repository if there is one
_SIBLING = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))
REF_ROOT = os.environ.get("LLMC_REFERENCE_ROOT", "") or (
    _SIBLING if os.path.isdir(os.path.join(_SIBLING, "src", "llmcompressor")) else "")


def reference_available() -> bool:
    return bool(REF_ROOT) and os.path.isdir(os.path.join(REF_ROOT, "src", "llmcompressor"))


def _install_shim():
    import torch.distributed as dist
    import compressed_tensors

    if "compressed_tensors.distributed" not in sys.modules:
        m = types.ModuleType("compressed_tensors.distributed")

        def greedy_bin_packing(items, num_bins, item_weight_fn=lambda x: 1):
            items.sort(key=item_weight_fn, reverse=True)
            bins = [[] for _ in range(num_bins)]
            loads = [0] * num_bins
            where = {}
            for it in items:
                b = loads.index(min(loads))
                bins[b].append(it)
                loads[b] += item_weight_fn(it)
                where[it] = b
            return items, bins, where

        def wait_for_comms(pending):
            for w in list(pending):
                w.wait()
            pending.clear()

        def is_distributed():
            return dist.is_available() and dist.is_initialized()

        def is_source_process():
            return (not is_distributed()) or dist.get_rank() == 0

        m.greedy_bin_packing = greedy_bin_packing
        m.wait_for_comms = wait_for_comms
        m.is_distributed = is_distributed
        m.is_source_process = is_source_process
        sys.modules["compressed_tensors.distributed"] = m
        compressed_tensors.distributed = m
    import compressed_tensors.offload.dist_utils as du

    if not hasattr(du, "is_source_process"):
        du.is_source_process = sys.modules["compressed_tensors.distributed"].is_source_process


_loaded = {}


def load_reference():
    """Returns a namespace with gptq_quantize (module), observers (package), calibration."""
    if _loaded:
        return _loaded["ns"]
    assert reference_available(), "reference checkout not present"
    _install_shim()
    tmp = tempfile.mkdtemp(prefix="llmc_ref_")
    dst = os.path.join(tmp, "llmcompressor")
    shutil.copytree(os.path.join(REF_ROOT, "src", "llmcompressor"), dst)
    with open(os.path.join(dst, "__init__.py"), "w") as f:
        f.write("")
    sys.path.insert(0, tmp)
    importlib.import_module("llmcompressor.core")
    observers = importlib.import_module("llmcompressor.observers")
    spec = importlib.util.spec_from_file_location(
        "ref_gptq_quantize", os.path.join(dst, "modifiers", "gptq", "gptq_quantize.py")
    )
    gq = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gq)
    ns = types.SimpleNamespace(gptq_quantize=gq, observers=observers, tmp=tmp)
    try:
        ns.calibration = importlib.import_module("llmcompressor.modifiers.quantization.calibration")
    except Exception as e:  # noqa: BLE001
        ns.calibration = None
        ns.calibration_error = repr(e)
    _loaded["ns"] = ns
    return ns
