"""Batch address-layout benchmark: N copies between one pair of GPUs with gaps inserted
between the chunks on the source side, the destination side, or both.

Capability parity: `Copy_Engine/nvlink_batch_address_layout_test.py:1-383` (flags `:193-219`,
layout construction `:89-115`, per-chunk fill values `:134-135`, gap sentinels must survive
`:156-189`). The check here compares every chunk completely (position-dependent bytes) and
every destination gap completely.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.layout_copy \
        --layout both-discontinuous --nbytes 2048K --copies-per-iter 4 --check
"""
from __future__ import annotations

import argparse

import torch

from ..ops.copy import CopyEngine
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import fmt_bytes, parse_nbytes, parse_size_list
from . import copy_common as CC
from .copy_engine import resolve_sizes


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    CC.add_common_flags(ap, nbytes_default="1M")
    ap.add_argument("--copies-per-iter", type=int, default=8)
    ap.add_argument("--non-uniform-copy-size", action="store_true")
    ap.add_argument("--copy-sizes", type=parse_size_list, default=None)
    ap.add_argument("--layout", choices=list(P.LAYOUTS), default="contiguous")
    ap.add_argument("--gap-size", type=parse_nbytes, default=parse_nbytes("64K"))
    ap.add_argument("--copy-mode", choices=["separate", "batch"], default="batch")
    ap.add_argument("--batch-impl", choices=["graph", "kernel"], default="graph")
    ap.add_argument("--mode", choices=list(P.PAIR_MODES), default="ring")
    ap.add_argument("--no-proxy-thread", action="store_true")
    return ap


def fill_source(lay: P.GapLayout, rank: int, device) -> torch.Tensor:
    src = torch.full((lay.src_bytes,), P.SRC_GAP_SENTINEL, dtype=torch.uint8, device=device)
    for i, (o, s) in enumerate(zip(lay.src_offsets, lay.sizes)):
        src[o:o + s] = CC.position_pattern(s, seed=rank * 17 + i, device=device)
    return src


def check_destination(recv: torch.Tensor, lay: P.GapLayout, writer: int) -> bool:
    ok = True
    for i, (o, s) in enumerate(zip(lay.dst_offsets, lay.sizes)):
        ok = ok and bool(torch.equal(recv[o:o + s], CC.position_pattern(s, seed=writer * 17 + i, device=recv.device)))
    for o, ln in lay.dst_gaps():
        ok = ok and bool((recv[o:o + ln] == P.DST_GAP_SENTINEL).all())
    return ok


def main() -> int:
    args = build_parser().parse_args()
    if args.gap_size < 0:
        raise ValueError("--gap-size must be >= 0")
    sizes = resolve_sizes(args)
    lay = P.build_layout(args.layout, sizes, args.gap_size)
    w = CC.CopyWorld(lay.dst_bytes)
    _, dst_rank = P.choose_pair(w.rank, w.size, args.mode) if w.size > 1 else (0, 0)
    src = fill_source(lay, w.rank, w.device)
    w.recv.fill_(P.DST_GAP_SENTINEL)
    torch.cuda.synchronize()
    D.barrier()
    dst_ptr = w.peer_ptr(dst_rank)
    copies = [(dst_ptr + do, w.peer_device(dst_rank), src.data_ptr() + so, w.device.index, s)
              for so, do, s in zip(lay.src_offsets, lay.dst_offsets, lay.sizes)]
    mode = "separate" if args.copy_mode == "separate" else args.batch_impl
    eng = CopyEngine(copies, mode, stream_device=w.peer_device(dst_rank), use_proxy=not args.no_proxy_thread)
    CC.sleep_phase(args.sleep_before)
    if args.warmup:
        eng.run(args.warmup)
    D.barrier()
    r = eng.run(args.iters)
    D.barrier()
    elapsed, total = r["wall_seconds"], sum(sizes)
    moved = float(total) * args.iters
    ok = True
    if args.check:
        torch.cuda.synchronize()
        D.barrier()
        writers = [s for s in range(w.size) if (P.choose_pair(s, w.size, args.mode)[1] if w.size > 1 else 0) == w.rank]
        if writers:
            ok = check_destination(w.recv, lay, writers[0])
    line = (f"[rank {w.rank}] layout={args.layout} gap={fmt_bytes(args.gap_size)} copy_mode={args.copy_mode}({mode}) "
            f"copies/iter={len(sizes)} bytes/iter={fmt_bytes(total)} iters={args.iters} "
            f"elapsed={elapsed * 1e3:.3f} ms local_bw={CC.bw(moved, elapsed):.3f} GiB/s"
            + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(w.rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl,
              title="batch address-layout copy",
              extra=dict(bench="layout_copy", world=w.size, layout=args.layout, gap=args.gap_size,
                         copy_mode=mode, sizes=list(sizes), iters=args.iters),
              expectation="chunks of one submission may be coalesced by the copy engine when contiguous")
    all_ok = D.all_ranks_boolean(ok)
    del eng
    w.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
