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


_BUCKET_BYTES = 256 << 20     # parameters of one owner travel in buckets of at most this size


def broadcast_module_params(modules: Sequence, module_to_rank: dict, names: Sequence[str]) -> None:
    """Broadcast the named parameters of every module from its owner.  The parameters of one
    owner are packed into byte buckets (one collective per bucket instead of one per tensor: a
    layer of a mixture of experts has more than a thousand small tensors); a tensor larger than a
    bucket goes by itself.  Which tensor travels in which collective depends on the tensors' sizes
    only, never on a rank's local memory layout."""
    me = rank()
    by_src: dict = {}
    for m in modules:
        src = module_to_rank[m]
        for name in names:
            p = getattr(m, name, None)
            if p is not None:
                by_src.setdefault(src, []).append(p.data)
    pending, after = [], []

    def as_bytes(t):
        return t.contiguous().reshape(-1).view(torch.uint8)      # a copy when t is not contiguous

    def alone(t, src):
        buf = t if t.is_contiguous() else t.contiguous()
        pending.append(dist.broadcast(_as_broadcastable(buf), src=src, async_op=True))
        if buf is not t and me != src:
            after.append(lambda: t.copy_(buf))

    def packed(bucket, src):
        offsets, total = [], 0
        for t in bucket:
            offsets.append(total)
            total += (t.numel() * t.element_size() + 15) // 16 * 16
        buf = torch.empty(total, dtype=torch.uint8, device=bucket[0].device)
        views = [buf[o: o + t.numel() * t.element_size()] for o, t in zip(offsets, bucket)]
        if me == src:
            torch._foreach_copy_(views, [as_bytes(t) for t in bucket])
        pending.append(dist.broadcast(buf, src=src, async_op=True))
        if me != src:
            def unpack():
                dense = [(t, v) for t, v in zip(bucket, views) if t.is_contiguous()]
                if dense:
                    torch._foreach_copy_([as_bytes(t) for t, _ in dense], [v for _, v in dense])
                for t, v in zip(bucket, views):
                    if not t.is_contiguous():
                        t.copy_(v.view(t.dtype).view(t.shape))
            after.append(unpack)

    for src in sorted(by_src):
        bucket, size = [], 0
        for t in by_src[src]:
            nbytes = t.numel() * t.element_size()
            if nbytes == 0:
                continue
            if nbytes > _BUCKET_BYTES:
                alone(t, src)
                continue
            if size + nbytes > _BUCKET_BYTES and bucket:
                (alone(bucket[0], src) if len(bucket) == 1 else packed(bucket, src))
                bucket, size = [], 0
            bucket.append(t)
            size += nbytes
        if bucket:
            (alone(bucket[0], src) if len(bucket) == 1 else packed(bucket, src))
    wait_for_comms(pending)
    for fn in after:
        fn()
