"""Multi-source all-to-all batched copy benchmark: N logical source buffers (A, B, C, ...)
separated by a gap, each cut into world-1 sub-buffers; sub-buffer k of every source goes to
GPU (rank+k+1) % world, and every destination is served by ONE submission of N copies.

Capability parity: `Copy_Engine/nvlink_multi_source_all_to_all_batch_test.py:1-449`
(flags `:157-188`, mapping `:74-102`, chunk values `:78-79`, source- or destination-indexed
sizes `:231-247`). The check compares every (source, destination) chunk completely.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.msrc_copy --nbytes 512K --check
"""
from __future__ import annotations

import argparse

import torch

from ..ops.copy import CopyEngine
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import fmt_bytes, parse_nbytes, parse_size_list
from . import copy_common as CC


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    CC.add_common_flags(ap, nbytes_default="1M")
    ap.add_argument("--num-source-buffers", type=int, default=4)
    ap.add_argument("--source-buffer-sizes", type=parse_size_list, default=None,
                    help="one sub-buffer size per SOURCE buffer (same for every destination)")
    ap.add_argument("--destination-buffer-sizes", type=parse_size_list, default=None,
                    help="one sub-buffer size per DESTINATION (same for every source)")
    ap.add_argument("--source-buffer-gap-size", type=parse_nbytes, default=parse_nbytes("64K"))
    ap.add_argument("--copy-mode", choices=["separate", "batch"], default="batch")
    ap.add_argument("--batch-impl", choices=["graph", "kernel"], default="graph")
    ap.add_argument("--no-proxy-thread", action="store_true")
    return ap


def _seed(rank: int, source: int, slot: int) -> int:
    return P.msrc_chunk_value(rank, source, slot) + 251 * (rank + 1)


def main() -> int:
    args = build_parser().parse_args()
    rank, world, _ = D.env_rank_info()
    if world < 2:
        raise ValueError("the multi-source benchmark needs world_size >= 2 (launch with torchrun)")
    if args.num_source_buffers <= 0:
        raise ValueError("--num-source-buffers must be positive")
    table = P.msrc_sizes(world, args.num_source_buffers, args.nbytes, args.source_buffer_sizes,
                         args.destination_buffer_sizes)
    plan = P.build_multi_source_plan(rank, world, table, args.source_buffer_gap_size)
    # every rank receives, from the peer that is k+1 steps behind it, that peer's slot-k chunks.
    # receive area: one region per sender, sized for the largest destination total.
    per_sender = max(plan.dst_bytes)
    w = CC.CopyWorld(per_sender * world)
    src = torch.full((plan.src_bytes,), P.SRC_GAP_SENTINEL, dtype=torch.uint8, device=w.device)
    for k, peer, entries in plan.batches():
        for s, (so, _, nb) in enumerate(entries):
            src[so:so + nb] = CC.position_pattern(nb, seed=_seed(rank, s, k), device=w.device)
    w.recv.fill_(P.DST_GAP_SENTINEL)
    torch.cuda.synchronize()
    D.barrier()
    mode = "separate" if args.copy_mode == "separate" else args.batch_impl
    engines = []
    for k, peer, entries in plan.batches():
        base = w.peer_ptr(peer) + rank * per_sender
        copies = [(base + do, w.peer_device(peer), src.data_ptr() + so, w.device.index, nb)
                  for so, do, nb in entries]
        engines.append(CopyEngine(copies, mode, stream_device=w.device.index,
                                  use_proxy=not args.no_proxy_thread))
    CC.sleep_phase(args.sleep_before)

    def run(iters: int) -> float:
        # one submission per destination per iteration; engines own separate streams, so the
        # destinations proceed concurrently as in the reference's per-destination batches
        import concurrent.futures as cf
        with cf.ThreadPoolExecutor(len(engines)) as ex:
            rs = list(ex.map(lambda e: e.run(iters), engines))
        return max(r["wall_seconds"] for r in rs)

    if args.warmup:
        run(args.warmup)
    D.barrier()
    elapsed = run(args.iters)
    D.barrier()
    per_iter = sum(sum(r) for r in table)
    moved = float(per_iter) * args.iters
    ok = True
    if args.check:
        torch.cuda.synchronize()
        D.barrier()
        for sender in range(world):
            if sender == rank:
                continue
            k = (rank - sender - 1) % world            # my slot index in the sender's plan
            sp = P.build_multi_source_plan(sender, world, table, args.source_buffer_gap_size)
            base = sender * per_sender
            for s in range(args.num_source_buffers):
                do, nb = sp.dst_offsets[s][k], sp.sub_sizes[s][k]
                want = CC.position_pattern(nb, seed=_seed(sender, s, k), device=w.device)
                ok = ok and bool(torch.equal(w.recv[base + do:base + do + nb], want))
    line = (f"[rank {rank}] sources={args.num_source_buffers} copy_mode={args.copy_mode}({mode}) "
            f"bytes/iter={fmt_bytes(per_iter)} submissions/iter={world - 1} iters={args.iters} "
            f"elapsed={elapsed * 1e3:.3f} ms egress_bw={CC.bw(moved, elapsed):.3f} GiB/s"
            + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl,
              title="multi-source all-to-all batched copy",
              extra=dict(bench="msrc_copy", world=world, copy_mode=mode, table=[list(r) for r in table],
                         gap=args.source_buffer_gap_size, iters=args.iters),
              expectation=f"{world - 1} submissions per iteration, {args.num_source_buffers} copies each")
    all_ok = D.all_ranks_boolean(ok)
    engines.clear()
    w.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
