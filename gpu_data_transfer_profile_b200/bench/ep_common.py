"""Shared pieces of the dispatch / combine / MoE-loop CLIs: flags, validation, fake tokens and
router, buffer construction, device timing with max over ranks, result records.

Flag parity: `DeepEP_v1/deepep_v1_dispatch.py:59-121` (shared by the combine and Megatron-loop
scripts). `--ep 1` is accepted here (single-GPU runs); the reference requires EP > 1.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Callable, Optional

import torch

from ..parallel.buffer import Buffer
from ..parallel.symm import LocalWorld
from ..ref.cpu_oracle import make_routing
from ..utils import dist as D

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def add_ep_flags(ap: argparse.ArgumentParser, num_sms_default: int = 24) -> None:
    ap.add_argument("--num-local-tokens", type=int, required=True)
    ap.add_argument("--token-hidden", type=int, required=True)
    ap.add_argument("--num-of-experts", type=int, required=True)
    ap.add_argument("--topk", type=int, required=True)
    ap.add_argument("--ep", type=int, required=True)
    ap.add_argument("--dtype", choices=tuple(DTYPES), default="bf16")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--warmup-iters", type=int, default=5)
    ap.add_argument("--benchmark-iters", type=int, default=20)
    ap.add_argument("--deepep-num-sms", "--num-sms", dest="num_sms", type=int, default=num_sms_default)
    ap.add_argument("--print-timing", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--check-correctness", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--async-finish", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--allocate-on-comm-stream", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--zipf", type=float, default=0.0, help="Zipf exponent of the expert popularity (0 = uniform)")
    ap.add_argument("--use-fp8", action="store_true", help="fp8 e4m3 dispatch with 1x128 scales (cast fused)")
    ap.add_argument("--jsonl", default=None)


def validate_args(args, world_size: int) -> None:
    checks = [
        (args.num_local_tokens > 0, "--num-local-tokens must be positive."),
        (args.token_hidden > 0, "--token-hidden must be positive."),
        (args.num_of_experts > 0, "--num-of-experts must be positive."),
        (args.topk > 0, "--topk must be positive."),
        (args.ep >= 1, "--ep must be at least 1."),
        (world_size % args.ep == 0, "--ep must divide torchrun WORLD_SIZE."),
        (args.num_of_experts % args.ep == 0, "--num-of-experts must be divisible by --ep."),
        (args.topk <= args.num_of_experts, "--topk cannot exceed --num-of-experts."),
        (args.topk <= 32, "--topk above 32 is not supported."),
        (args.warmup_iters >= 0, "--warmup-iters cannot be negative."),
        (args.benchmark_iters >= 1, "--benchmark-iters must be at least 1."),
        (args.async_finish or not args.allocate_on_comm_stream, "--allocate-on-comm-stream requires --async-finish."),
        ((args.token_hidden * DTYPES[args.dtype].itemsize) % 16 == 0, "token row must be a multiple of 16 bytes."),
    ]
    for ok, msg in checks:
        if not ok:
            raise ValueError(msg)


class EpContext:
    """Rank info, EP group, buffer, fake tokens and routing."""

    def __init__(self, args, *, group_by_expert: bool = False, extra_tokens: int = 0):
        self.rank, self.world, self.local_rank = D.init_distributed()
        validate_args(args, self.world)
        self.args = args
        self.group, self.ep_rank, self.group_index = D.create_ep_group(args.ep)
        self.device = torch.device("cuda", torch.cuda.current_device())
        Buffer.set_num_sms(args.num_sms)
        self.dtype = DTYPES[args.dtype]
        T, H, E, K = args.num_local_tokens, args.token_hidden, args.num_of_experts, args.topk
        hidden_bytes = H * max(self.dtype.itemsize, 2)
        need = 0
        for cfg in (Buffer.get_dispatch_config(args.ep, T + extra_tokens, K, E, group_by_expert),
                    Buffer.get_combine_config(args.ep, T + extra_tokens, K, E, group_by_expert)):
            cfg.combine_elem_bytes = self.dtype.itemsize
            need = max(need, cfg.get_nvl_buffer_size_hint(hidden_bytes, args.ep),
                       cfg.get_rdma_buffer_size_hint(hidden_bytes, args.ep))
        world = None if D.is_dist() else LocalWorld.make(1, self.device)[0]
        self.buffer = Buffer(self.group, need, 0, world=world)
        g = torch.Generator().manual_seed(args.seed + self.rank)
        self.x = torch.randn(T, H, generator=g).to(self.dtype).to(self.device)
        self.reroute(0)

    def reroute(self, it: int) -> None:
        a = self.args
        idx, w = make_routing(a.num_local_tokens, a.num_of_experts, a.topk,
                              seed=a.seed * 7 + self.rank + 1000 * it, zipf_s=a.zipf)
        self.topk_idx, self.topk_weights = idx.to(self.device), w.to(self.device)

    def close(self) -> None:
        self.buffer.destroy()
        D.shutdown()


def timed_loop(fn: Callable[[], None], warmup: int, iters: int, *, before: Optional[Callable] = None,
               group=None) -> dict:
    """Per-iteration CUDA-event timing; returns mean/min ms of this rank and the max over ranks."""
    for _ in range(warmup):
        if before:
            before()
        fn()
    torch.cuda.synchronize()
    D.barrier(group)
    ev = []
    for _ in range(iters):
        if before:
            before()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        ev.append((a, b))
    torch.cuda.synchronize()
    D.barrier(group)
    ms = [a.elapsed_time(b) for a, b in ev]
    mean = sum(ms) / len(ms)
    return dict(mean_ms=mean, min_ms=min(ms), max_over_ranks_ms=D.all_reduce_scalar(mean, "max", group))


def emit(rank: int, record: dict, jsonl: Optional[str]) -> None:
    if rank == 0:
        print("[record] " + json.dumps(record), flush=True)
        if jsonl:
            with open(jsonl, "a") as f:
                f.write(json.dumps(record) + "\n")


def remote_rows(in_rank: torch.Tensor, rank: int) -> int:
    r = in_rank.clone()
    r[:, rank] = False
    return int(r.sum().item())
