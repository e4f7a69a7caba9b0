"""Plug the b200q kernels into an unmodified llm-compressor installation.

Two seams of the reference are used, both as it defines them:

* observers: ``@Observer.register("name")`` subclasses that implement
  ``update_statistics_from_observed(observed)`` with ``observed`` of shape
  ``(num_observations, *qparam_shape, group_size)`` and leave ``min_vals`` / ``max_vals`` on
  the instance (src/llmcompressor/observers/base.py:29-76).  ``register_observers()`` adds
  ``b200_minmax`` and ``b200_mse``; a recipe selects them with ``weight_observer="b200_minmax"``.
  New names are needed because re-registering an existing name with another class raises
  (compressed_tensors/registry/registry.py:216-220).
* GPTQ math: ``llmcompressor.modifiers.gptq.base`` binds ``make_empty_hessian``,
  ``accumulate_hessian`` and ``quantize_weight`` at import (gptq/base.py:27-31);
  ``patch_gptq()`` rebinds those three names there.

Nothing in this module is imported by the rest of the package.
"""
from __future__ import annotations

import math

import torch

from . import gptq, ops
from .quant_args import QuantizationArgs

__all__ = ["register_observers", "patch_gptq", "observed_as_matrix"]


def observed_as_matrix(observed: torch.Tensor, args: QuantizationArgs):
    """``observed`` (num_observations, *qparam_shape, group) -> (matrix [rows, cols], kernel args,
    qparam shape): a view whose per-group / per-row statistics are the statistics over
    (0, -1) of ``observed``.  Weight observations have num_observations == 1."""
    if observed.shape[0] != 1:
        raise NotImplementedError("b200 observers take weight observations (one observation)")
    qshape = tuple(observed.shape[1:-1])
    group = observed.shape[-1]
    if not observed.is_contiguous():
        observed = observed.contiguous()     # BLOCK flattening transposes
    inner = qshape[-1] if qshape else 1
    rows = math.prod(qshape[:-1]) if len(qshape) > 1 else 1
    if rows * inner == 1:
        # one group over everything (TENSOR strategy): the whole-tensor kernels
        kargs = args.model_copy(update={"strategy": "tensor", "group_size": None, "actorder": None,
                                        "block_structure": None})
        return observed.reshape(1, group), kargs, qshape
    pow2 = group >= 8 and group <= 256 and (group & (group - 1)) == 0
    if inner > 1 and pow2:
        # groups that lie side by side in memory: the streaming group kernels
        kargs = args.model_copy(update={"strategy": "group", "group_size": group, "actorder": None})
        return observed.reshape(rows, inner * group), kargs, qshape
    kargs = args.model_copy(update={"strategy": "channel", "group_size": None, "actorder": None,
                                    "block_structure": None})
    return observed.reshape(rows * inner, group), kargs, qshape


def register_observers(observer_base=None):
    """Register ``b200_minmax`` and ``b200_mse`` with the reference's observer registry
    (``observer_base`` defaults to ``llmcompressor.observers.base.Observer``).  Returns the two
    classes."""
    if observer_base is None:
        from llmcompressor.observers.base import Observer as observer_base   # noqa: N813

    @observer_base.register("b200_minmax")
    class B200MinMaxObserver(observer_base):
        """Memoryless min / max of a weight on the b200q kernels."""

        def update_statistics_from_observed(self, observed: torch.Tensor) -> None:
            mat, kargs, qshape = observed_as_matrix(observed, QuantizationArgs.of(self.args))
            mn, mx = ops.observe_minmax(mat, kargs)
            self.min_vals, self.max_vals = mn.reshape(qshape), mx.reshape(qshape)

    @observer_base.register("b200_mse")
    class B200MSEObserver(observer_base):
        """Memoryless MSE shrink-grid search of a weight on the b200q kernels; takes the
        reference's observer_kwargs (maxshrink, patience, grid, norm, expand)."""

        def update_statistics_from_observed(self, observed: torch.Tensor) -> None:
            kw = dict(maxshrink=0.20, patience=5, grid=100.0, norm=2.4, expand=1.0)
            kw.update({k: v for k, v in (self.args.observer_kwargs or {}).items() if k in kw})
            if kw["expand"] < 1.0:
                raise ValueError(f"expand value must be at least 1.0, got {kw['expand']}")
            own = QuantizationArgs.of(self.args)
            if own.strategy == "tensor_group" and own.scale_dtype is not None:
                own = own.model_copy(update={"scale_dtype": None})   # mse_quant.py:52-57
            mat, kargs, qshape = observed_as_matrix(observed, own)
            mn, mx = ops.observe_mse(mat, kargs, **kw)
            self.min_vals, self.max_vals = mn.reshape(qshape), mx.reshape(qshape)

    return B200MinMaxObserver, B200MSEObserver


def patch_gptq(gptq_base=None):
    """Rebind the three GPTQ math functions of ``llmcompressor.modifiers.gptq.base`` to the b200q
    implementations (same signatures and return values).  Returns the module that was patched."""
    if gptq_base is None:
        import llmcompressor.modifiers.gptq.base as gptq_base
    gptq_base.make_empty_hessian = gptq.make_empty_hessian
    gptq_base.accumulate_hessian = gptq.accumulate_hessian
    gptq_base.quantize_weight = gptq.quantize_weight
    return gptq_base
