"""Shared scaffolding of the copy benchmark CLIs.

One process per GPU. Each rank owns one symmetric region (CUDA IPC) that holds its receive
area; a source rank reaches a peer's receive area through the mapped pointer. Without a
torchrun environment the CLIs run as a single rank that copies to itself (the reference's
single-process debugging mode, `Copy_Engine/nvlink_copy_engine_test.py:385-387`).

Timing follows the reference for copy-engine paths (steady clock around enqueue + stream
synchronise, `Copy_Engine/nvlink_copy_engine_test.py:549-560`) and additionally reports the
device time (CUDA events) for SM kernels; the slowest rank defines the aggregate.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional

import torch

from ..parallel.symm import LocalWorld, ProcessWorld, SymmetricRegion
from ..utils import dist as D
from ..utils.sizes import fmt_bytes

GIB = float(1 << 30)


class CopyWorld:
    """Rank info + one symmetric receive region per rank."""

    def __init__(self, recv_bytes: int):
        self.rank, self.size, self.local_rank = D.init_distributed()
        self.device = torch.device("cuda", torch.cuda.current_device())
        if D.is_dist():
            self.world = ProcessWorld(None, self.device)
        else:
            self.world = LocalWorld.make(1, self.device)[0]
        self.recv_bytes = int(recv_bytes)
        self.region = SymmetricRegion(self.world, max(self.recv_bytes, 256))
        self.recv = self.region.view(0, (max(self.recv_bytes, 256),), "uint8")
        D.barrier()

    def peer_ptr(self, peer: int) -> int:
        return self.region.peer_ptrs[peer]

    def peer_device(self, peer: int) -> int:
        """CUDA ordinal of `peer` as seen from this process (ranks map to ordinals on one node)."""
        return peer % max(torch.cuda.device_count(), 1) if D.is_dist() else self.device.index

    def peer_view(self, peer: int, nbytes: int) -> torch.Tensor:
        """A uint8 tensor aliasing the first nbytes of `peer`'s receive area (mapped pointer)."""
        return self.region.C.view_tensor(self.peer_ptr(peer), [nbytes], "uint8", self.device.index)

    def close(self):
        torch.cuda.synchronize()
        D.barrier()
        self.region.close()
        D.shutdown()


def add_common_flags(ap: argparse.ArgumentParser, *, nbytes_default: str, iters: int = 100,
                     warmup: int = 10) -> None:
    from ..utils.sizes import parse_nbytes
    ap.add_argument("--nbytes", "--copy-size", dest="nbytes", type=parse_nbytes,
                    default=parse_nbytes(nbytes_default), help="bytes per copy (K/M/G binary, KB/MB/GB decimal)")
    ap.add_argument("--iters", type=int, default=iters)
    ap.add_argument("--warmup", type=int, default=warmup)
    ap.add_argument("--check", action="store_true", help="verify destination contents after timing")
    ap.add_argument("--sleep-before", type=float, default=0.0, help="seconds to sleep before warm-up")
    ap.add_argument("--jsonl", default=None, help="append one JSON record per run to this file (rank 0)")


def sleep_phase(seconds: float) -> None:
    D.barrier()
    if seconds > 0:
        time.sleep(seconds)
    D.barrier()


def device_timed(fn, stream: Optional[torch.cuda.Stream] = None) -> float:
    """Run fn() between two events on `stream`; returns elapsed seconds (device time)."""
    st = stream or torch.cuda.current_stream()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(st)
    fn()
    b.record(st)
    b.synchronize()
    return a.elapsed_time(b) * 1e-3


def report(world_rank: int, line: str, *, elapsed: float, bytes_moved: float, extra: dict,
           jsonl: Optional[str], title: str, expectation: str) -> None:
    """Ordered per-rank lines, then the rank-0 aggregate (sum of bytes / slowest rank)."""
    slowest = D.all_reduce_max_float(elapsed)
    total = D.all_reduce_sum_float(bytes_moved)
    D.ordered_print(line)
    if world_rank == 0:
        agg = total / GIB / slowest if slowest > 0 else 0.0
        print(f"[aggregate] {title}: total={fmt_bytes(total)} slowest_elapsed={slowest * 1e3:.3f} ms "
              f"aggregate_bw={agg:.3f} GiB/s ({agg * GIB / 1e9:.2f} GB/s)")
        print(f"[profiler expectation] {expectation}")
        rec = dict(title=title, slowest_elapsed_s=slowest, total_bytes=total, aggregate_gib_s=agg, **extra)
        if jsonl:
            with open(jsonl, "a") as f:
                f.write(json.dumps(rec) + "\n")
        sys.stdout.flush()


def bw(nbytes: float, seconds: float) -> float:
    return nbytes / GIB / seconds if seconds > 0 else 0.0


def position_pattern(nbytes: int, seed: int, device) -> torch.Tensor:
    """Position-dependent bytes (so a permutation inside a chunk is detected), never 252/253."""
    idx = torch.arange(nbytes, device=device, dtype=torch.int64)
    return ((idx * 131 + seed * 7919 + (idx >> 11) * 17) % 251).to(torch.uint8)
