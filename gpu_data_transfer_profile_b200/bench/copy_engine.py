"""Pairwise copy-engine (DMA) benchmark: one source -> one destination per rank.

Capability parity: `Copy_Engine/nvlink_copy_engine_test.py:430-628` (flags `:431-453`).
N chunks per iteration, uniform or per-copy sizes; `--copy-mode separate` issues N peer
memcpys per iteration, `--copy-mode batch` issues ONE submission per iteration
(`--batch-impl graph`: a CUDA graph of N memcpy nodes on the copy engines;
`--batch-impl kernel`: one SM kernel over a descriptor table). The submission loop is native
and, by default, runs on a proxy thread.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.copy_engine --nbytes 8M --check
"""
from __future__ import annotations

import argparse

import torch

from ..ops.copy import CopyEngine
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import contiguous_offsets, default_nonuniform_sizes, fmt_bytes, parse_size_list
from . import copy_common as CC


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    CC.add_common_flags(ap, nbytes_default="1G")
    ap.add_argument("--copies-per-iter", type=int, default=1)
    ap.add_argument("--non-uniform-copy-size", action="store_true")
    ap.add_argument("--copy-sizes", type=parse_size_list, default=None)
    ap.add_argument("--copy-mode", choices=["separate", "batch"], default="separate")
    ap.add_argument("--batch-impl", choices=["graph", "kernel"], default="graph")
    ap.add_argument("--mode", choices=list(P.PAIR_MODES), default="ring")
    ap.add_argument("--no-proxy-thread", action="store_true", help="submit from the calling thread")
    return ap


def resolve_sizes(args) -> tuple:
    if args.copies_per_iter <= 0:
        raise ValueError("--copies-per-iter must be positive")
    if args.copy_sizes is not None:
        if len(args.copy_sizes) != args.copies_per_iter:
            raise ValueError("--copy-sizes needs exactly --copies-per-iter entries")
        return tuple(args.copy_sizes)
    if args.non_uniform_copy_size:
        return default_nonuniform_sizes(args.nbytes * args.copies_per_iter, args.copies_per_iter)
    return tuple(args.nbytes for _ in range(args.copies_per_iter))


def engine_mode(args) -> str:
    return "separate" if args.copy_mode == "separate" else args.batch_impl


def main() -> int:
    args = build_parser().parse_args()
    if args.iters <= 0 or args.warmup < 0:
        raise ValueError("--iters must be > 0 and --warmup >= 0")
    sizes = resolve_sizes(args)
    offs = contiguous_offsets(sizes)
    total = sum(sizes)
    w = CC.CopyWorld(total)
    src_dev, dst_rank = P.choose_pair(w.rank, w.size, args.mode) if w.size > 1 else (0, 0)
    src = torch.full((total,), P.pair_fill_value(w.rank), dtype=torch.uint8, device=w.device)
    w.recv.fill_(P.pair_prefill_value(w.rank))
    torch.cuda.synchronize()
    D.barrier()
    dst_ptr = w.peer_ptr(dst_rank)
    copies = [(dst_ptr + o, w.peer_device(dst_rank), src.data_ptr() + o, w.device.index, s)
              for o, s in zip(offs, sizes)]
    # the copy stream lives on the destination device, as in the reference's pair benchmark
    eng = CopyEngine(copies, engine_mode(args), stream_device=w.peer_device(dst_rank),
                     use_proxy=not args.no_proxy_thread)
    CC.sleep_phase(args.sleep_before)
    if args.warmup:
        eng.run(args.warmup)
    D.barrier()
    r = eng.run(args.iters)
    D.barrier()
    elapsed = r["wall_seconds"]
    moved = float(total) * args.iters
    ok = True
    if args.check:
        torch.cuda.synchronize()
        D.barrier()
        # my receive area was written by the rank whose destination is me
        writers = [s for s in range(w.size) if (P.choose_pair(s, w.size, args.mode)[1] if w.size > 1 else 0) == w.rank]
        if writers:
            want = torch.full((total,), P.pair_fill_value(writers[0]), dtype=torch.uint8, device=w.device)
            ok = bool(torch.equal(w.recv[:total], want))
    line = (f"[rank {w.rank}] GPU{w.device.index} -> GPU{w.peer_device(dst_rank)} mode={args.mode} "
            f"copy_mode={args.copy_mode}({engine_mode(args)}) copies/iter={len(sizes)} bytes/iter={fmt_bytes(total)} "
            f"iters={args.iters} elapsed={elapsed * 1e3:.3f} ms submit={r['submit_seconds'] * 1e3:.3f} ms "
            f"local_bw={CC.bw(moved, elapsed):.3f} GiB/s" + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(w.rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl,
              title="pairwise copy-engine copy",
              extra=dict(bench="copy_engine", world=w.size, mode=args.mode, copy_mode=engine_mode(args),
                         sizes=list(sizes), iters=args.iters),
              expectation=("one peer-to-peer memcpy per chunk per iteration" if args.copy_mode == "separate" else
                           "one graph launch (N memcpy nodes) per iteration" if args.batch_impl == "graph" else
                           "one batched_copy_kernel launch per iteration"))
    all_ok = D.all_ranks_boolean(ok)
    del eng
    w.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
