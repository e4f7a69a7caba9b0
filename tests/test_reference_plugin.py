"""The plug-in for an unmodified llm-compressor: ``b200_minmax`` / ``b200_mse`` registered with the
REFERENCE's observer registry and driven through the reference's own ``Observer.forward`` ->
``flatten_for_calibration`` -> ``update_statistics_from_observed`` -> ``get_qparams`` chain.

Runs where an llm-compressor checkout is available (LLMC_REFERENCE_ROOT, or a checkout named
"reference" next to the repository).  There is no GPU there,
so the two kernel calls are stood in for by the CPU oracle: what is under test is the seam - the
registration, the shapes handed to the kernels for every strategy, and that the reference's
qparams come out identical to its own observers'."""
import os
import sys

import pytest
import torch

import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import ref_loader  # noqa: E402

pytestmark = pytest.mark.skipif(not ref_loader.reference_available(),
                                reason="needs LLMC_REFERENCE_ROOT (an llm-compressor checkout)")


@pytest.fixture(scope="module")
def plugin(monkeysession):
    from llm_compressor_b200 import ops, reference_plugin
    from test_oracle_golden import spec_from

    ref = ref_loader.load_reference()
    seen = []

    def spec_of(args):
        return spec_from({k: getattr(args, k) for k in ("num_bits", "type", "symmetric", "strategy", "group_size",
                                                         "block_structure", "scale_dtype", "zp_dtype")})

    def fake_minmax(w, args):
        seen.append(("minmax", tuple(w.shape), args.strategy, args.group_size))
        return oracle.observe_minmax(w, spec_of(args))

    def fake_mse(w, args, **kw):
        seen.append(("mse", tuple(w.shape), args.strategy, args.group_size))
        return oracle.observe_mse(w, spec_of(args), **kw)

    monkeysession.setattr(ops, "observe_minmax", fake_minmax)
    monkeysession.setattr(ops, "observe_mse", fake_mse)
    classes = reference_plugin.register_observers(ref.observers.Observer)
    return ref, classes, seen


@pytest.fixture(scope="module")
def monkeysession():
    mp = pytest.MonkeyPatch()
    yield mp
    mp.undo()


def _ct_args(**kw):
    from compressed_tensors.quantization import QuantizationArgs
    return QuantizationArgs(**kw)


CASES = {
    "group": dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128),
    "group_asym": dict(num_bits=4, type="int", symmetric=False, strategy="group", group_size=32),
    "channel": dict(num_bits=8, type="int", symmetric=True, strategy="channel"),
    "tensor": dict(num_bits=8, type="float", symmetric=True, strategy="tensor"),
    "block": dict(num_bits=8, type="float", symmetric=True, strategy="block", block_structure=[64, 64]),
    "nvfp4": dict(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16,
                  scale_dtype=torch.float8_e4m3fn, zp_dtype=torch.float8_e4m3fn),
}


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("kind", ["minmax", "mse"])
def test_registered_observers_match_the_reference_observers(plugin, case, kind):
    ref, _classes, seen = plugin
    Observer = ref.observers.Observer
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(192, 256, generator=g) * 0.05).to(torch.bfloat16)
    ours = Observer.load_from_registry(f"b200_{kind}", base_name="weight", args=_ct_args(**CASES[case]))
    theirs = Observer.load_from_registry(f"memoryless_{kind}", base_name="weight", args=_ct_args(**CASES[case]))
    seen.clear()
    a = ours(w).get_qparams()
    b = theirs(w).get_qparams()
    assert seen and seen[0][0] == kind
    assert not ours.has_statistics
    for key in ("scale", "zero_point", "global_scale"):
        if b[key] is None:
            assert a[key] is None
        else:
            x, y = a[key], b[key]
            assert x.shape == y.shape and x.dtype == y.dtype, (case, key)
            assert torch.equal(x.float(), y.float()), (case, key)
    # what the kernels were handed: 2-D, groups side by side where the group kernels apply
    _, shape, strategy, gsize = seen[0]
    assert len(shape) == 2
    if case in ("group", "group_asym", "nvfp4"):
        assert strategy == "group" and shape == (192, 256) and gsize == CASES[case]["group_size"]
    elif case == "tensor":
        assert strategy == "tensor" and shape == (1, 192 * 256)
    elif case == "block":
        assert strategy == "channel" and shape == (3 * 4, 64 * 64)
    else:
        assert strategy == "channel" and shape == (192, 256)


def test_registering_twice_is_rejected_by_the_reference_registry(plugin):
    from llm_compressor_b200 import reference_plugin
    ref, _classes, _ = plugin
    with pytest.raises(Exception):
        reference_plugin.register_observers(ref.observers.Observer)


def test_patch_gptq_rebinds_the_three_names():
    import types

    from llm_compressor_b200 import gptq, reference_plugin
    base = types.SimpleNamespace(make_empty_hessian=None, accumulate_hessian=None, quantize_weight=None)
    reference_plugin.patch_gptq(base)
    assert base.accumulate_hessian is gptq.accumulate_hessian and base.quantize_weight is gptq.quantize_weight
    assert base.make_empty_hessian is gptq.make_empty_hessian
