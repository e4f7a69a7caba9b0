"""CPU restatement of the AWQ scale search (test infrastructure only).

Follows src/llmcompressor/modifiers/transform/awq/base.py: ``_compute_layer_means`` (:907-973),
``_get_grid_search_params`` (:802-836), the candidate scales and Q(W * s) / s of
``_compute_best_scale`` (:607-763) and the mean-squared output error of ``_compute_loss``
(:765-800).  Pinned by ``tests/golden/awq.pt`` (outputs of the reference's own functions).
"""
from __future__ import annotations

import torch

from .observers import WeightObserver
from .quantize import fake_quantize

HIGH_PRECISION = torch.float64     # src/llmcompressor/utils/dev.py:175-181


def layer_means(weights, specs) -> torch.Tensor:
    """Mean over the rows of all weights of |w| / max|w| of its quantisation chunk."""
    total, count = 0, 0
    for weight, spec in zip(weights, specs):
        weight = weight.clone()
        shape = weight.shape
        inter = None
        if spec.strategy == "tensor":
            chunk = weight.numel()
        elif spec.strategy == "channel":
            chunk = weight.size(1)
        elif spec.strategy in ("group", "tensor_group"):
            chunk = spec.group_size
        elif spec.strategy == "block":
            bh, bw = spec.block_structure
            weight = weight.unflatten(0, (-1, bh)).unflatten(-1, (-1, bw)).transpose(1, 2)
            inter = weight.shape
            chunk = bh * bw
        else:
            raise ValueError(spec.strategy)
        weight = weight.reshape(-1, chunk)
        weight.abs_()
        weight.div_(weight.amax(dim=1, keepdim=True) + 1e-6)
        if inter is not None:
            weight = weight.view(inter).transpose(1, 2)
        weight = weight.reshape(shape)
        count += weight.size(0)
        total = total + weight.sum(0, dtype=HIGH_PRECISION)
    return total / count


def grid_search_params(duo_scaling, n_grid):
    if duo_scaling == "both":
        n = int(n_grid / 2)
        return [(i / (n - 1), duo) for i in range(n) for duo in (False, True)]
    if duo_scaling is False:
        return [(i / (n_grid - 1), False) for i in range(n_grid)]
    if duo_scaling is True:
        return [(0.0, False)] + [(i / (n_grid - 2), True) for i in range(n_grid - 1)]
    raise ValueError(duo_scaling)


def candidate_scales(x_mean, w_mean, ratio, duo):
    if duo:
        scales = (x_mean.pow(ratio) / (w_mean.pow(1 - ratio) + 1e-4)).clamp(min=1e-4)
    else:
        scales = x_mean.pow(ratio).clamp(min=1e-4).view(-1)
    scales = scales / (scales.max() * scales.min()).sqrt()
    scales[torch.isinf(scales)] = 1
    scales[torch.isnan(scales)] = 1
    return scales


def scaled_fake_quantize(weights, scales, specs, fused: bool = False):
    """[Q(W * s) / s] in the weights' dtype; ``fused``: the weights share one NVFP4 global scale."""
    view = scales.view(1, -1)
    scaled = [(w * view).to(w.dtype) for w in weights]
    observers = [WeightObserver(spec, "memoryless_minmax") for spec in specs]
    for obs, ws in zip(observers, scaled):
        obs(ws)
    if fused:
        for obs in observers:
            obs.fused = [o for o in observers if o is not obs]
    # every observer's global scale needs the statistics of all of them: read them first
    gscales = [obs.get_global_scale() for obs in observers]
    out = []
    for obs, gs, ws, w, spec in zip(observers, gscales, scaled, weights, specs):
        obs.get_global_scale = lambda gs=gs: gs
        qp = obs.get_qparams()
        fq = fake_quantize(ws, qp["scale"], qp["zero_point"], spec, global_scale=qp["global_scale"])
        out.append((fq / view).to(w.dtype))
    return out


def output_error(reference_outputs, outputs) -> float:
    loss = torch.tensor(0.0)
    n = 0
    for a, b in zip(reference_outputs, outputs):
        loss += torch.nn.functional.mse_loss(a, b, reduction="sum")
        n += a.numel()
    return (loss / n).item()


def best_scale(x_sum, count, weights, specs, run_parent, duo_scaling=True, n_grid=20, fused=False):
    """The search: ``run_parent(list of weights) -> list of outputs`` evaluates the parent module
    with the balance weights replaced.  Returns (best scales, [loss per grid point])."""
    x_mean = x_sum / count
    w_mean = layer_means(weights, specs) if duo_scaling else None
    reference_outputs = run_parent(weights)
    best_error, best, losses = float("inf"), None, []
    for ratio, duo in grid_search_params(duo_scaling, n_grid):
        scales = candidate_scales(x_mean, w_mean, ratio, duo)
        loss = output_error(reference_outputs, run_parent(scaled_fake_quantize(weights, scales, specs, fused)))
        losses.append(loss)
        if loss < best_error:
            best_error, best = loss, scales.clone()
    return best, losses
