"""Multi-GPU plumbing of the compress step: owner assignment, Hessian reduction to owners,
result broadcast.  One process per GPU, ``torch.distributed`` (NCCL on GPUs, gloo on CPU in
tests).  Mirrors src/llmcompressor/utils/dist.py:20-88 and
src/llmcompressor/modifiers/gptq/base.py:345-370.
"""
from __future__ import annotations

from typing import Callable, Hashable, Sequence, TypeVar

import torch
import torch.distributed as dist

T = TypeVar("T", bound=Hashable)

__all__ = ["is_distributed", "rank", "world_size", "greedy_bin_packing", "wait_for_comms",
           "reduce_hessians", "broadcast_module_params", "partition_samples"]


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def rank() -> int:
    return dist.get_rank() if is_distributed() else 0


def world_size() -> int:
    return dist.get_world_size() if is_distributed() else 1


def greedy_bin_packing(items: list, num_bins: int, item_weight_fn: Callable = lambda x: 1):
    """Sort ``items`` in place by descending weight and give each to the least-loaded bin.
    Returns (items, bin_to_items, item_to_bin)."""
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


def wait_for_comms(pending: list) -> None:
    for w in list(pending):
        w.wait()
    pending.clear()


def partition_samples(num_samples: int, r: int, world: int) -> range:
    """Calibration samples of rank r: [floor(S r / R), floor(S (r+1) / R))
    (src/llmcompressor/datasets/utils.py:244-253)."""
    return range((num_samples * r) // world, (num_samples * (r + 1)) // world)


def reduce_hessians(groups: Sequence, group_to_rank: dict) -> None:
    """Sum each group's partial Hessian and sample count onto its owner; other ranks drop
    theirs.  A group whose ``group_to_rank`` entry is None is wanted by every rank (its member
    modules are spread over all of them) and is all-reduced instead.  ``groups`` have attributes
    ``H`` (float32 [K,K]) and ``n``."""
    me = rank()
    pending = []
    if not groups:
        return
    dev = None
    for g in groups:
        dst = group_to_rank[g]
        H = g.H if g.H.device.type != "cpu" or dist.get_backend() == "gloo" else g.H.to(g.device)
        g.H = H
        dev = H.device
        if dst is None:
            pending.append(dist.all_reduce(H, op=dist.ReduceOp.SUM, async_op=True))
        else:
            pending.append(dist.reduce(H, dst=dst, op=dist.ReduceOp.SUM, async_op=True))
    # every sample count in one collective and one read
    counts = torch.tensor([float(g.n) for g in groups], dtype=torch.float32, device=dev)
    pending.append(dist.all_reduce(counts, op=dist.ReduceOp.SUM, async_op=True))
    wait_for_comms(pending)
    totals = counts.tolist()
    for g, n in zip(groups, totals):
        if group_to_rank[g] in (me, None):
            g.n = n
        else:
            g.H = None


def _as_broadcastable(t: torch.Tensor) -> torch.Tensor:
    # NCCL has no float8 type: send the bytes
    return t.view(torch.uint8) if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else t


def broadcast_module_params(modules: Sequence, module_to_rank: dict, names: Sequence[str]) -> None:
    """Broadcast the named parameters of every module from its owner."""
    pending = []
    for m in modules:
        src = module_to_rank[m]
        for name in names:
            p = getattr(m, name, None)
            if p is None:
                continue
            pending.append(dist.broadcast(_as_broadcastable(p.data), src=src, async_op=True))
    wait_for_comms(pending)
