"""Device-side timing: CUDA events on the launching stream, L2 flush between iterations,
max over ranks. Never wall clock for kernels.

The reference times its EP steps the same way, one CUDA-event pair per iteration
(`DeepEP_v1/deepep_v1_dispatch.py:186-248`), and its copy-engine loops by wall clock around the
enqueue loop plus one stream synchronise (`Copy_Engine/nvlink_copy_engine_test.py:548-560`; that
form lives in `csrc/copy/ce_copy.cpp`, where the copies are not kernels). Added here: the L2 flush
between iterations and the reduction to the slowest rank."""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from . import dist as D

L2_BYTES = 126 * 1024 * 1024


class L2Flusher:
    """Writes a buffer twice the L2 size so the next iteration starts cold."""

    def __init__(self, device=None, nbytes: int = 2 * L2_BYTES):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")

    def __call__(self):
        self.buf.fill_(1)


def time_steps(step: Callable[[], None], steps: int, warmup: int, *, flush: Optional[Callable] = None,
               before: Optional[Callable] = None, group=None) -> dict:
    """Run `warmup` untimed + `steps` timed calls. Each timed call is bracketed by its own event
    pair (the optional L2 flush and the optional `before` hook run outside the pair).
    Returns per-step ms list (this rank), mean ms and the max over ranks of the mean."""
    for _ in range(warmup):
        if flush:
            flush()
        if before:
            before()
        step()
    torch.cuda.synchronize()
    D.barrier(group)
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        if flush:
            flush()
        if before:
            before()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    D.barrier(group)
    torch.cuda.synchronize()
    ms: List[float] = [a.elapsed_time(b) for a, b in evs]
    mean = sum(ms) / max(len(ms), 1)
    return dict(ms=ms, mean_ms=mean, max_rank_mean_ms=D.all_reduce_scalar(mean, "max", group),
                min_ms=min(ms) if ms else 0.0)
