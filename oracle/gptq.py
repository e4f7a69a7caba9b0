"""GPTQ Hessian accumulation and the blockwise quantisation sweep on CPU tensors
(test infrastructure only).

Restates ``make_empty_hessian`` / ``accumulate_hessian`` / ``quantize_weight`` /
``_apply_activation_ordering`` of src/llmcompressor/modifiers/gptq/gptq_quantize.py
(:19-25, :28-64, :67-264, :267-278).  The sweep is written block-vectorised where the
reference loops in Python, but every value goes through the same sequence of float32 /
bf16 operations in the same order per column, so the results are bit-identical on CPU.
"""
from __future__ import annotations

import math

import torch

from .observers import WeightObserver
from .qparams import qrange
from .quantize import _round_codes


def make_empty_hessian(num_columns: int) -> torch.Tensor:
    return torch.zeros((num_columns, num_columns), dtype=torch.float32)


def accumulate_hessian(inp: torch.Tensor, H: torch.Tensor, num_samples):
    """H += (sqrt2 X)^T (sqrt2 X) with X = inp flattened to [tokens, K]; the sample count
    grows by the number of SEQUENCES (leading dimension), gptq_quantize.py:34-64."""
    if inp.ndim == 2:
        inp = inp.unsqueeze(0)
    elif inp.ndim > 3:
        inp = inp.reshape(inp.shape[0], -1, inp.shape[-1])
    added = inp.shape[0]
    x = inp.reshape(-1, inp.shape[-1]).t()
    num_samples = num_samples + added
    x = x.to(torch.float32)
    x = math.sqrt(2) * x
    H += x.matmul(x.t())
    return H, num_samples


def accumulate_hessian_running_mean(inp: torch.Tensor, H: torch.Tensor, num_samples):
    """The SparseGPT / Wanda variant: H is the running mean of 2 X^T X over the samples seen so
    far (src/llmcompressor/modifiers/pruning/sparsegpt/sgpt_sparsify.py:20-56)."""
    if inp.ndim == 2:
        inp = inp.unsqueeze(0)
    added = inp.shape[0]
    x = inp.reshape(-1, inp.shape[-1]).t()
    H *= num_samples / (num_samples + added)
    num_samples = num_samples + added
    x = x.to(torch.float32)
    x = math.sqrt(2 / num_samples) * x
    H += x.matmul(x.t())
    return H, num_samples


def hessian_inverse_factor(H: torch.Tensor, percdamp: float):
    """Upper factor U with U^T U = (H + damp I)^-1, computed as the reference does:
    Cholesky, Cholesky-inverse, upper Cholesky (gptq_quantize.py:150-156).  Returns
    (U, ok); ok False means the factorisation failed and U is the identity (:157-164)."""
    K = H.shape[0]
    try:
        damp = percdamp * torch.mean(torch.diag(H))
        idx = torch.arange(K)
        H[idx, idx] += damp
        L = torch.linalg.cholesky(H)
        Hinv = torch.cholesky_inverse(L)
        U = torch.linalg.cholesky(Hinv, upper=True)
        return U, True
    except torch._C._LinAlgError:
        return torch.eye(K, dtype=H.dtype), False


def _column_quant(w, scale_col, zp_col, args, global_scale):
    """fake-quantise one float32 column with per-row parameters: the reference's
    channel-wise call inside the sweep (gptq_quantize.py:184-225)."""
    s = scale_col / global_scale if global_scale is not None else scale_col
    v = w / s
    if zp_col is not None:
        v = v + zp_col.to(w.dtype)
    q = _round_codes(v, args)
    d = q.to(s.dtype)
    if zp_col is not None:
        d = d - zp_col.to(s.dtype)
    return d * s


def quantize_weight(
    weight: torch.Tensor,
    args,
    hessian: torch.Tensor,
    blocksize: int = 128,
    percdamp: float = 0.01,
    observer: WeightObserver | None = None,
):
    """Returns (loss, dict) like the reference; ``hessian`` is consumed.

    ``observer`` must already hold statistics of ``weight`` (the modifier observes before
    it compresses, src/llmcompressor/modifiers/gptq/base.py:243-247); when omitted a
    memoryless observer of the kind named in ``args`` is created and run here."""
    strategy, actorder = args.strategy, args.actorder
    final_shape, final_dtype = weight.shape, weight.dtype
    if observer is None:
        observer = WeightObserver(args)
        observer(weight)
    W = weight.clone().to(torch.float32)
    H = hessian
    N, K = W.shape
    if actorder == "group" and strategy not in ("group", "tensor_group"):
        actorder = None
    perm = None
    if actorder:
        perm = torch.argsort(torch.diag(H), descending=True)
        W = W[:, perm]
        H = H[perm][:, perm]
    if actorder == "group":
        observer.delete_statistics()
        observer(W)
    g_idx = None
    if strategy in ("group", "tensor_group", "block"):
        div = args.group_size if strategy != "block" else args.block_structure[1]
        g_idx = torch.arange(K, dtype=torch.int) // div
        if actorder == "weight":
            g_idx = g_idx[perm]
    qp = observer.get_qparams()
    scale, zp, gscale = qp["scale"], qp["zero_point"], qp["global_scale"]

    losses = torch.zeros(N)
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    U, _ok = hessian_inverse_factor(H, percdamp)

    if strategy == "block":
        bh = args.block_structure[0]
        row_block = torch.arange(N) // bh

    for i1 in range(0, K, blocksize):
        i2 = min(i1 + blocksize, K)
        W1 = W[:, i1:i2].clone()
        Q1 = torch.zeros_like(W1)
        E1 = torch.zeros_like(W1)
        L1 = torch.zeros_like(W1)
        U1 = U[i1:i2, i1:i2]
        for i in range(i2 - i1):
            w = W1[:, i]
            d = U1[i, i]
            if strategy == "tensor":
                q = _column_quant(w, scale, zp, args, gscale)
            elif strategy == "channel":
                q = _column_quant(w, scale[:, 0], zp[:, 0], args, gscale)
            elif strategy in ("group", "tensor_group"):
                g = int(g_idx[i1 + i])
                q = _column_quant(w, scale[:, g], zp[:, g], args, gscale)
            elif strategy == "block":
                g = int(g_idx[i1 + i])
                q = _column_quant(w, scale[row_block, g], zp[row_block, g], args, gscale)
            else:
                raise ValueError(f"Quantization strategy is not supported for GPTQ: {strategy}")
            Q1[:, i] = q
            L1[:, i] = (w - q) ** 2 / d**2
            err = (w - q) / d
            W1[:, i:] -= err.unsqueeze(1).matmul(U1[i, i:].unsqueeze(0))
            E1[:, i] = err
        W[:, i1:i2] = Q1
        losses += torch.sum(L1, 1) / 2
        W[:, i2:] -= E1.matmul(U[i1:i2, i2:])

    invperm = None
    if actorder:
        invperm = torch.argsort(perm)
        W = W[:, invperm]
    W = W.reshape(final_shape).to(final_dtype)
    loss = torch.sum(losses).item()
    out = {
        "weight": W,
        "weight_scale": scale.to(final_dtype),
        "weight_zero_point": zp.to(args.zp_dtype),
    }
    if gscale is not None and bool(gscale):
        out["weight_global_scale"] = gscale.to(final_dtype)
    if actorder == "group":
        out["weight_g_idx"] = g_idx[invperm]
    return loss, out
