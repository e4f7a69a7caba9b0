"""GPTQ math functions with the reference's names and contracts, on b200q kernels.

Drop-in for ``make_empty_hessian`` / ``accumulate_hessian`` / ``quantize_weight`` of
src/llmcompressor/modifiers/gptq/gptq_quantize.py (:19-25, :28-64, :67-264).

Two things go beyond the reference's per-module functions, both without changing results:
``accumulate_hessian_lower`` / ``finalize_hessian`` keep only the lower triangle current
between hook calls (the mirror and the division by the sample count happen once), and
``factor_hessian`` lets modules that see the same input (q/k/v, gate/up, the experts of an
all-expert calibration) share one permutation and one factor U instead of recomputing them.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, ops
from .observers import Observer
from .quant_args import QuantizationArgs

__all__ = ["make_empty_hessian", "accumulate_hessian", "accumulate_hessian_lower",
           "finalize_hessian", "factor_hessian", "factor_hessians_batched", "resolve_factors",
           "HessianFactor", "quantize_weight", "quantize_weights_batched", "GPTQ_PRECISION"]

GPTQ_PRECISION = torch.float32

_NOT_PD_MESSAGE = (
    "Failed to invert hessian due to numerical instability. Consider increasing "
    "GPTQModifier.dampening_frac, increasing the number of calibration samples, or shuffling "
    "the calibration dataset. Falling back to round-to-nearest for this module.")


def make_empty_hessian(module: torch.nn.Module, device=None) -> torch.Tensor:
    weight = module.weight
    num_columns = weight.shape[1]
    device = device if device is not None else weight.device
    return torch.zeros((num_columns, num_columns), device=device, dtype=GPTQ_PRECISION)


def _tokens_2d(inp: torch.Tensor, device) -> tuple[torch.Tensor, int]:
    """[B,S,K] / [S,K] / [B,...,K] activations -> ([tokens, K] bf16 contiguous rows, B)."""
    inp = inp.to(device=device)
    if inp.ndim == 2:
        inp = inp.unsqueeze(0)
    elif inp.ndim > 3:
        inp = inp.reshape(inp.shape[0], -1, inp.shape[-1])
    num_added = inp.shape[0]
    x = inp.reshape(-1, inp.shape[-1])
    if x.dtype != torch.bfloat16:
        # the kernel contracts bf16 operands; float16/float32 activations are rounded once here
        x = x.to(torch.bfloat16)
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    return x, num_added


def accumulate_hessian_lower(inp: torch.Tensor, H: torch.Tensor, num_samples):
    """Hook-path accumulation: H_lower += 2 X^T X (tiles on and below the diagonal only),
    sample count += number of sequences.  ``finalize_hessian`` mirrors and normalises once,
    before the solve.  ``num_samples`` may be a python number or a tensor."""
    x, added = _tokens_2d(inp, H.device)
    ops.hessian_syrk(x, H, alpha=2.0)
    num_samples += added
    return H, num_samples


def finalize_hessian(H: torch.Tensor, num_samples) -> torch.Tensor:
    """Mirror the lower triangle and divide by the sample count (base.py:336), in place."""
    n = float(num_samples)
    ops.hessian_finalize(H, 1.0 / n if n else 1.0)
    return H


def accumulate_hessian(inp, module, H, num_samples):
    """Same contract as the reference: mutates and returns (H, num_samples) with H the full
    symmetric matrix after every call.  Only Linear-like modules (weight [out, in]) are
    handled; the sample count grows by the number of sequences, not tokens."""
    if isinstance(module, torch.nn.Conv2d):
        raise NotImplementedError("Conv2d Hessians are outside this package's path")
    H, num_samples = accumulate_hessian_lower(inp, H, num_samples)
    ops.hessian_finalize(H, 1.0)
    return H, num_samples


def accumulate_hessian_running_mean(inp, module, H, num_samples):
    """The SparseGPT / Wanda consumers' Hessian: the running mean of 2 X^T X over the samples
    seen so far (src/llmcompressor/modifiers/pruning/sparsegpt/sgpt_sparsify.py:20-56), same
    contract as ``accumulate_hessian`` (mutates and returns the full symmetric H and the sample
    count).  The same rank-k kernel with alpha = 2 / n after the stored part has been rescaled."""
    if isinstance(module, torch.nn.Conv2d):
        raise NotImplementedError("Conv2d Hessians are outside this package's path")
    x, added = _tokens_2d(inp, H.device)
    ops.hessian_finalize(H, num_samples / (num_samples + added))   # H *= n / (n + added)
    num_samples += added
    ops.hessian_syrk(x, H, alpha=2.0 / num_samples)
    ops.hessian_finalize(H, 1.0)
    return H, num_samples


@dataclass
class HessianFactor:
    """What the sweep needs from one Hessian: the act-order permutation (or None), the
    diagonal before dead-column patching, and U (upper, U^T U = (H + damp I)^-1) or None
    when the factorisation failed and the identity stands in for it.

    A deferred factor (``factor_hessian(..., defer=True)``) has ``ok is None`` until
    ``resolve()`` has waited for the device status; its U must not be trusted before that."""
    K: int
    perm: Optional[torch.Tensor]
    diag: torch.Tensor
    U: Optional[torch.Tensor]
    ok: Optional[bool]
    status: Optional[torch.Tensor] = None

    def resolve(self) -> "HessianFactor":
        if self.ok is None:
            st = ops.gptq_factor_status(self.status)
            self.ok = st != _lib.NOT_POSITIVE_DEFINITE
            if not self.ok:
                warnings.warn(_NOT_PD_MESSAGE)
                self.U = None
        return self


def factor_hessian(hessian: torch.Tensor, percdamp: float = 0.01, actorder=None,
                   defer: bool = False) -> HessianFactor:
    """Permute (act-order), patch dead columns, dampen and factor ``hessian`` (consumed).
    ``defer``: do not wait for the factorisation's status (see ``HessianFactor.resolve``)."""
    H, perm, diag = _factor_prologue(hessian, percdamp, actorder)
    factor = HessianFactor(H.shape[0], perm, diag, H, None, ops.gptq_factor_async(H))
    return factor if defer else factor.resolve()


def _factor_prologue(hessian: torch.Tensor, percdamp: float, actorder):
    """Everything of ``factor_hessian`` before the factorisation itself: (H ready to factor,
    permutation or None, diagonal before the dead-column patch)."""
    H = hessian
    K = H.shape[0]
    if H.shape != (K, K) or H.dtype != torch.float32:
        raise ValueError("hessian must be a square float32 matrix")
    perm = None
    if actorder:
        perm = ops.actorder_perm(H)
        H = ops.permute_hessian(H, perm)
    diag = H.diagonal().clone()
    ops.gptq_prepare(H, None, percdamp)
    return H, perm, diag


def factor_hessians_batched(hessians, percdamp: float = 0.01, actorder=None):
    """``factor_hessian(..., defer=True)`` for a list of small Hessians of one size, with all the
    factorisations in one launch (one thread block per matrix).  The matrices are consumed.
    Returns the deferred factors; ``resolve_factors`` reads all their status words at once."""
    parts = [_factor_prologue(H, percdamp, actorder) for H in hessians]
    status = ops.gptq_factor_batched([H for H, _, _ in parts])
    return [HessianFactor(H.shape[0], perm, diag, H, None, status[i]) for i, (H, perm, diag) in enumerate(parts)]


def resolve_factors(factors) -> None:
    """``HessianFactor.resolve`` for many factors with one wait for the device."""
    pending = [f for f in factors if f.ok is None]
    if not pending:
        return
    words = torch.stack([f.status.reshape(-1)[:4] for f in pending]).tolist()
    for f, st in zip(pending, words):
        if st[2] != 0:
            raise _lib.B200QError("b200q_gptq_factor: a bounded wait inside the GEMM kernel expired")
        f.ok = st[0] != _lib.NOT_POSITIVE_DEFINITE
        if not f.ok:
            warnings.warn(_NOT_PD_MESSAGE)
            f.U = None


@dataclass
class _SweepInput:
    """One module's operands of the column sweep, and what the epilogue needs."""
    args: QuantizationArgs
    actorder: Optional[str]
    factor: HessianFactor
    W: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    global_scale: Optional[torch.Tensor]
    col_group: Optional[torch.Tensor]
    g_idx: Optional[torch.Tensor]
    final_dtype: torch.dtype


def _sweep_input(module, quant_args, hessian, percdamp, factor, W=None) -> _SweepInput:
    """``W``: the float32 copy of the weight, already permuted and with its dead columns zeroed (the
    batched path makes it for all modules at once); made here when not given."""
    args = QuantizationArgs.of(quant_args)
    strategy, actorder = args.strategy, args.actorder
    weight = module.weight.data if isinstance(module.weight, torch.nn.Parameter) else module.weight
    observer: Observer = module.weight_observer
    N, K = weight.shape
    if strategy not in ("tensor", "channel", "group", "tensor_group", "block"):
        raise ValueError(f"Quantization strategy is not supported for GPTQ: {strategy}")

    if actorder == "group" and strategy not in ("group", "tensor_group"):
        warnings.warn("ActivationOrdering.GROUP requires a grouped quantization strategy; "
                      "falling back to actorder=None for this module.")
        actorder = None

    if factor is None:
        if hessian is None or hessian.shape != (K, K):
            raise ValueError("hessian must be float32 [in_features, in_features]")
        factor = factor_hessian(hessian, percdamp, actorder)
    elif factor.K != K or (factor.perm is not None) != bool(actorder):
        raise ValueError("factor does not match this module / act-order setting")
    perm = factor.perm

    prepared = W is not None
    if not prepared:
        W = ops.gather_columns_f32(weight, perm)

    if actorder == "group":
        observer.delete_statistics(check_fused=False)
        observer(W)
    elif not observer.has_statistics:
        observer(weight)     # memoryless: the statistics of the weight as it is now

    col_group = None
    g_idx = None
    if strategy in ("group", "tensor_group", "block"):
        divisor = args.group_size if strategy != "block" else args.block_structure[1]
        g_idx = torch.arange(K, device=W.device, dtype=torch.int32) // divisor
        if actorder == "weight":
            g_idx = g_idx[perm.long()]
            col_group = g_idx

    qparams = observer.get_qparams()
    if not prepared:
        ops.gptq_zero_dead_columns(factor.diag, W)
    return _SweepInput(args, actorder, factor, W, qparams["scale"], qparams["zero_point"], qparams["global_scale"],
                       col_group, g_idx, weight.dtype)


def _sweep_output(inp: _SweepInput, weight=None) -> dict:
    """``weight``: the swept weight already scattered back and cast (batched path)."""
    perm = inp.factor.perm
    out = {
        "weight": weight if weight is not None else ops.scatter_columns_cast(inp.W, inp.final_dtype, perm),
        "weight_scale": inp.scale.to(inp.final_dtype),
        "weight_zero_point": inp.zero_point.to(inp.args.zp_dtype),
    }
    if inp.global_scale is not None:
        out["weight_global_scale"] = inp.global_scale.to(inp.final_dtype)
    if inp.actorder == "group":
        K = inp.W.shape[1]
        invperm = torch.empty_like(perm)
        invperm[perm.long()] = torch.arange(K, device=perm.device, dtype=perm.dtype)
        out["weight_g_idx"] = inp.g_idx[invperm.long()]
    return out


def quantize_weight(module, quant_args, hessian: Optional[torch.Tensor], blocksize: int = 128,
                    percdamp: float = 0.01, factor: Optional[HessianFactor] = None, defer: bool = False):
    """GPTQ-quantise ``module.weight`` given its Hessian (already divided by the sample
    count).  Returns ``(loss, dict)`` with the fake-quantised weight in the original dtype,
    ``weight_scale``, ``weight_zero_point`` and, where they apply, ``weight_global_scale`` and
    ``weight_g_idx``.  ``hessian`` is consumed.  ``module.weight_observer`` is asked to
    observe the weight if it holds no statistics yet (act-order "group" always re-observes the
    permuted weight); ``module.weight`` is not touched.

    ``factor`` (from ``factor_hessian`` with the same ``percdamp`` and act-order setting) may
    be passed instead of ``hessian`` when several modules share one Hessian.

    ``defer``: nothing waits for the device; the loss comes back as a 0-dim device tensor, a
    deferred ``factor`` is used as it is, and the dict carries one extra entry ``"_status"``
    (the sweep's int32 device status word, non-zero after an expired bounded wait) that the
    caller must pop and check.  The caller must also ``factor.resolve()`` afterwards and repeat
    the call without ``defer`` (after re-observing the weight) if the factorisation turned out
    to have failed."""
    inp = _sweep_input(module, quant_args, hessian, percdamp, factor)
    losses, status = ops.gptq_sweep(inp.W, inp.factor.U, inp.scale, inp.zero_point, inp.args, blocksize=blocksize,
                                    col_group=inp.col_group, global_scale=inp.global_scale, return_status=True)
    out = _sweep_output(inp)
    if defer:
        loss = losses.sum()
        out["_status"] = status   # the sweep's device status word; the caller checks and removes it
    else:
        loss, st = torch.stack([losses.sum(), status[0].to(torch.float32)]).tolist()
        if st != 0:
            raise _lib.B200QError("b200q_gptq_sweep: a bounded wait inside the GEMM kernel expired")
    return loss, out


def quantize_weights_batched(modules, quant_args, factors, blocksize: int = 128, percdamp: float = 0.01):
    """``quantize_weight(..., defer=True)`` for many small modules of one weight shape and one
    quantisation scheme, each with its own (deferred) factor, with all the column sweeps in one
    launch.  Returns ``[(loss, dict), ...]`` in the order of ``modules``: the losses are 0-dim
    device tensors and the dicts carry no ``"_status"`` (the batched sweep has no bounded wait).
    As with the deferred single call, the caller resolves the factors afterwards and redoes the
    modules whose factorisation failed."""
    weights = [m.weight.data if isinstance(m.weight, torch.nn.Parameter) else m.weight for m in modules]
    perms = [f.perm for f in factors]
    if any((p is None) != (perms[0] is None) for p in perms):
        raise ValueError("the factors of a batch must all carry a permutation or none")
    # one launch: float32 copies, permuted, dead columns zeroed
    Wf = ops.gather_columns_f32_batched(weights, None if perms[0] is None else perms, [f.diag for f in factors])
    inputs = [_sweep_input(m, quant_args, None, percdamp, f, W=Wf[k])
              for k, (m, f) in enumerate(zip(modules, factors))]
    first = inputs[0]

    def column(name):
        vals = [getattr(i, name) for i in inputs]
        if any((v is None) != (vals[0] is None) for v in vals):
            raise ValueError(f"{name} must be present for all modules of a batch or for none")
        return None if vals[0] is None else vals

    losses = ops.gptq_sweep_batched([i.W for i in inputs], [i.factor.U for i in inputs], column("scale"),
                                    column("zero_point"), first.args, col_groups=column("col_group"),
                                    global_scales=column("global_scale"), blocksize=blocksize)
    sums = losses.sum(dim=1)
    back = ops.scatter_columns_cast_batched([i.W for i in inputs], first.final_dtype,
                                            None if perms[0] is None else perms)
    return [(sums[k], _sweep_output(i, weight=back[k])) for k, i in enumerate(inputs)]
