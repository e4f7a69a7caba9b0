"""Run independent jobs of the solve concurrently, each on its own CUDA stream.

The Hessian factorisation and the column sweep of one module are long chains of small,
dependent kernel launches that leave most of the GPU idle; the chains of different Hessians
are independent of each other.  Each job gets a host thread (the C library releases the
interpreter lock during its calls and keeps its caches per thread) and a side stream.

Ordering contract: side streams start after everything already queued on the caller's
current stream and the caller's stream waits for every side stream before this function
returns, so callers need no extra synchronisation.  Side streams are used nowhere else,
which also makes the caching allocator's per-stream block reuse safe for tensors that are
allocated in a job and consumed by the caller afterwards.
"""
from __future__ import annotations

import os as _os
import threading
from typing import Callable, List, Sequence

import torch

_STREAMS: dict = {}
_LOCK = threading.Lock()


def _side_streams(device: torch.device, n: int) -> List["torch.cuda.Stream"]:
    with _LOCK:
        have = _STREAMS.setdefault((device.type, device.index), [])
        while len(have) < n:
            # the first stream runs the longest job: give it priority over the others
            have.append(torch.cuda.Stream(device=device, priority=(-1 if not have and _os.environ.get('B200Q_STREAM_PRIORITY', '1') == '1' else 0)))
        return have[:n]


def run_concurrent(jobs: Sequence[Callable[[], object]], device, max_streams: int = 4) -> list:
    """Call every job; returns their results in order.  Jobs are started in the order given
    (put the longest first).  The first exception raised by a job is re-raised here after all
    jobs have ended."""
    jobs = list(jobs)
    device = torch.device(device)
    if len(jobs) <= 1 or max_streams <= 1 or device.type != "cuda":
        return [job() for job in jobs]
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    n = min(max_streams, len(jobs))
    streams = _side_streams(device, n)
    main = torch.cuda.current_stream(device)
    ready = torch.cuda.Event()
    ready.record(main)
    # static assignment, worker i runs jobs i, i + n, ...: the first job gets the priority stream and
    # every job meets the same stream (and its allocator pool) on every call
    results: list = [None] * len(jobs)
    errors: list = []
    grad = torch.is_grad_enabled()

    def worker(first, stream):
        torch.cuda.set_device(device)
        with torch.cuda.stream(stream), torch.set_grad_enabled(grad):
            stream.wait_event(ready)
            for i in range(first, len(jobs), n):
                try:
                    results[i] = jobs[i]()
                except BaseException as e:  # noqa: BLE001 - re-raised by the caller below
                    errors.append(e)
                    return

    threads = [threading.Thread(target=worker, args=(i, s), daemon=True) for i, s in enumerate(streams)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for s in streams:
        main.wait_stream(s)
    if errors:
        raise errors[0]
    return results
