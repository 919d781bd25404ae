"""Peer-copy bandwidth sweep: copy engines vs LSU peer stores vs TMA-staged-local + LSU peer
stores, for message sizes 4 KiB .. 1 GiB (powers of two) and three traffic patterns:

  one-to-one   ring neighbour copy (every rank sends to rank+1)
  all-to-all   every rank sends a private chunk of `size` bytes to every other rank
  round-robin  one source range of `size` bytes cut into 8 KiB chunks dealt over all peers

One process per GPU; all variants of one size run back to back inside this process, so a whole
sweep is one launch (the reference loops a profiler over separate launches,
`Copy_Engine/sample_run.sh:4-32`). SM kernels are timed with CUDA events, copy-engine variants
with a steady clock around submit + stream synchronise; the slowest rank defines the time.
The best variant per (pattern, size) is written as a selector table that `ops/variants.py` loads.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.copy_sweep \
        --min-bytes 4K --max-bytes 1G --jsonl copy_sweep.jsonl --table variant_table.json
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from ..ops import copy as K
from ..parallel.symm import SymmetricRegion
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import fmt_bytes, parse_nbytes, pow2_sweep
from . import copy_common as CC


def iters_for(nbytes: int) -> int:
    return int(max(5, min(200, (1 << 31) // max(nbytes, 1))))


def time_kernel(fn, iters: int) -> float:
    """fn(launches) enqueues `launches` back-to-back launches from a native loop."""
    fn(2)
    torch.cuda.synchronize()
    D.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn(iters)
    b.record()
    b.synchronize()
    D.barrier()
    return a.elapsed_time(b) * 1e-3 / iters


def time_engine(copies, mode: str, dev: int, iters: int, ctas_per_copy: int = 8) -> float:
    eng = K.CopyEngine(copies, mode, stream_device=dev, use_proxy=True, kernel_ctas_per_copy=ctas_per_copy)
    eng.run(2)
    D.barrier()
    r = eng.run(iters)
    D.barrier()
    del eng
    return r["wall_seconds"] / iters


def time_engine_python(copies, dev: int, iters: int) -> float:
    """One peer memcpy per runtime call from the Python thread (how the reference submits)."""
    eng = K.CopyEngine(copies, "separate", stream_device=dev, use_proxy=False)
    eng.run_from_python(2)
    D.barrier()
    secs = eng.run_from_python(iters)
    D.barrier()
    del eng
    return secs / iters


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--min-bytes", dest="min", type=parse_nbytes, default=parse_nbytes("4K"))
    ap.add_argument("--max-bytes", dest="max", type=parse_nbytes, default=parse_nbytes("1G"))
    ap.add_argument("--patterns", default="one-to-one,all-to-all,round-robin")
    ap.add_argument("--num-sms", type=int, default=0, help="CTAs for SM kernels (0 = sized per message)")
    ap.add_argument("--rr-bytes", type=parse_nbytes, default=8192)
    ap.add_argument("--no-multimem", action="store_true", help="skip the NVSwitch multicast variant")
    ap.add_argument("--jsonl", default=None)
    ap.add_argument("--resume", action="store_true",
                    help="skip (pattern, size) pairs that the --jsonl file already holds (continue an interrupted sweep)")
    ap.add_argument("--table", default=None)
    args = ap.parse_args()
    rank, world, _ = D.env_rank_info()
    sizes = pow2_sweep(args.min, args.max)
    peers = max(world - 1, 1)
    w = CC.CopyWorld(max(sizes) * (world if world > 1 else 1))       # slot s = bytes received from rank s
    src = torch.empty(max(sizes), dtype=torch.uint8, device=w.device)
    src.copy_(CC.position_pattern(src.numel(), rank, w.device))
    status = K.StagedStatus(w.device)
    sms = K.sm_count(w.device)
    mc = None
    if world > 1 and "all-to-all" in args.patterns and not args.no_multimem:
        mc = K.MulticastBuffer(max(sizes) * world)
        if not D.all_ranks_boolean(mc.available):
            if rank == 0:
                print(f"[sweep] multimem variant skipped: {mc.why or 'no multicast mapping on a peer'}", flush=True)
            mc = None
    records, table = [], {}

    def ctas_for(n: int) -> int:
        if args.num_sms:
            return args.num_sms
        return int(max(1, min(sms, n // 16384)))

    def emit(pattern, n, variant, secs, moved):
        slow = D.all_reduce_max_float(secs)
        tot = D.all_reduce_sum_float(float(moved))
        rec = dict(bench="copy_sweep", world=world, pattern=pattern, nbytes=n, variant=variant,
                   seconds_slowest=slow, aggregate_gb_s=tot / slow / 1e9, per_rank_gb_s=tot / slow / 1e9 / world)
        records.append(rec)
        if rank == 0:
            print(f"[sweep] {pattern:11s} {fmt_bytes(n):>11s} {variant:12s} {slow * 1e6:10.2f} us  "
                  f"{rec['per_rank_gb_s']:8.2f} GB/s per rank", flush=True)
            if args.jsonl:
                with open(args.jsonl, "a") as f:
                    f.write(json.dumps(rec) + "\n")

    done = set()
    if args.resume and args.jsonl:
        import os
        if os.path.exists(args.jsonl):
            for line in open(args.jsonl):
                if line.strip():
                    r = json.loads(line)
                    if r.get("world") == world:
                        done.add((r["pattern"], r["nbytes"]))
                        records.append(r)
    for pattern in args.patterns.split(","):
        for n in sizes:
            if (pattern, n) in done:
                prev = [r for r in records if r["pattern"] == pattern and r["nbytes"] == n]
                b = min(prev, key=lambda r: r["seconds_slowest"])
                table.setdefault(pattern, []).append({"nbytes": n, "variant": b["variant"], "seconds": b["seconds_slowest"]})
                continue
            it = iters_for(n)
            s_t = src[:n]
            if pattern == "one-to-one":
                dst_rank = P.choose_pair(rank, world, "ring")[1] if world > 1 else 0
                d_t = w.peer_view(dst_rank, n)
                c = ctas_for(n)
                ce = [(d_t.data_ptr(), w.peer_device(dst_rank), s_t.data_ptr(), w.device.index, n)]
                variants = {
                    "ce": lambda: time_engine(ce, "separate", w.device.index, it),
                    "ce_python": lambda: time_engine_python(ce, w.device.index, it),
                    "lsu16": lambda: time_kernel(lambda L: K.lsu_copy(d_t, s_t, n, ctas=c, threads=512, vec_bytes=16, launches=L), it),
                    "lsu32": lambda: time_kernel(lambda L: K.lsu_copy(d_t, s_t, n, ctas=c, threads=512, vec_bytes=32, launches=L), it),
                    "lsu16_overlap": lambda: time_kernel(lambda L: K.lsu_copy(
                        d_t, s_t, n, ctas=c, threads=512, vec_bytes=16, launches=L, overlap_launches=True), it),
                }
                if n % 16 == 0:
                    tile = min(32768, max(1024, n // max(c, 1) // 16 * 16)) if n >= 16384 else max(16, n)
                    variants["tma_staged"] = lambda: time_kernel(
                        lambda L: K.tma_staged_copy([d_t], s_t, n, tile=tile, stages=K.pick_stages(tile), ctas=c,
                                                    threads=288, status=status, launches=L), it)
                moved = n
            elif pattern == "all-to-all":
                if world < 2:
                    continue
                order = P.destination_order(rank, world, True)
                views = [w.region.C.view_tensor(w.peer_ptr(d) + rank * n, [n], "uint8", w.device.index) for d in order]
                c = max(1, ctas_for(n * peers) // peers)
                ce = [(v.data_ptr(), w.peer_device(d), s_t.data_ptr(), w.device.index, n) for v, d in zip(views, order)]

                def lsu_all(vec, L):
                    for _ in range(L):
                        for v in views:
                            K.lsu_copy(v, s_t, n, ctas=c, threads=512, vec_bytes=vec)
                variants = {
                    "ce": lambda: time_engine(ce, "separate", w.device.index, it),
                    "ce_python": lambda: time_engine_python(ce, w.device.index, it),
                    "ce_graph": lambda: time_engine(ce, "graph", w.device.index, it),
                    "sm_batched": lambda: time_engine(ce, "kernel", w.device.index, it, ctas_per_copy=max(c, 1)),
                    "lsu16": lambda: time_kernel(lambda L: lsu_all(16, L), it),
                }
                if mc is not None and n % 16 == 0:
                    cm = ctas_for(n)
                    variants["multimem"] = lambda: time_kernel(
                        lambda L: mc.broadcast(s_t, n, offset=rank * n, ctas=cm, threads=512, launches=L), it)
                moved = n * peers
            else:  # round-robin
                if world < 2 or n % 16 or n < args.rr_bytes:
                    continue
                order = P.rr_destinations(rank, world, "ring")
                views = [w.region.C.view_tensor(w.peer_ptr(d) + rank * n, [n], "uint8", w.device.index) for d in order]
                c = ctas_for(n)
                chunks = P.rr_chunks(n, args.rr_bytes, len(order))
                variants = {
                    "lsu_rr": lambda: time_kernel(lambda L: K.lsu_rr_copy(views, s_t, n, args.rr_bytes, ctas=c, threads=512, launches=L), it),
                    "tma_rr": lambda: time_kernel(lambda L: K.tma_staged_copy(
                        views, s_t, n, rr_bytes=args.rr_bytes, tile=32768, stages=4, ctas=c, threads=288, status=status,
                        launches=L), it),
                }
                if len(chunks) <= 1024:
                    ce = [(views[sl].data_ptr() + off, w.peer_device(order[sl]), s_t.data_ptr() + off, w.device.index, ln)
                          for sl, off, ln in chunks]
                    variants["ce_graph"] = lambda: time_engine(ce, "graph", w.device.index, max(5, it // 4))
                moved = n
            best = None
            for name, fn in variants.items():
                secs = fn()
                emit(pattern, n, name, secs, moved)
                slow = records[-1]["seconds_slowest"]
                if name == "ce_python":
                    continue            # comparator column only, never a selectable variant
                if best is None or slow < best[1]:
                    best = (name, slow)
            status.check()
            table.setdefault(pattern, []).append({"nbytes": n, "variant": best[0], "seconds": best[1]})
    if rank == 0 and args.table:
        with open(args.table, "w") as f:
            json.dump({"world": world, "measured": time.strftime("%Y-%m-%d"), "table": table}, f, indent=1)
    w.close()
    return 0


if __name__ == "__main__":
    D.run_main(main)
