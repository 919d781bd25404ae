"""SM-driven round-robin copy benchmark: the source range is cut into chunks of
`--round-robin-bytes`; chunk c goes to peer table[c % n_peers] at the same byte offset.

Capability parity: `LSU_TMA/nvlink_lsu_tma_round_robin_copy_test.py:1-1211` (flags `:973-1015`;
source executor only `:1039-1040`; `--mode pair` rejected `:863-864`; destinations pre-filled
with distinct wrong values and checked only where they own a chunk `:891-924`, `:1091`).
The check here compares, for every destination, ALL owned chunks byte for byte and verifies
that every byte it does not own still holds the pre-fill value.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.rr_copy --method tma \
        --nbytes 1M --round-robin-bytes 8K --num-sms 4 --persistent-kernel --check
"""
from __future__ import annotations

import argparse

import torch

from ..ops import copy as K
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import fmt_bytes, parse_nbytes
from . import copy_common as CC
from .sm_copy import add_sm_flags, staged_threads


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    CC.add_common_flags(ap, nbytes_default="1G")
    add_sm_flags(ap, "src")
    ap.add_argument("--round-robin-bytes", "--round-robin-size", dest="rr_bytes", type=parse_nbytes,
                    default=parse_nbytes("8K"))
    return ap


def prefill_value(dst_rank: int, src_rank: int) -> int:
    return (200 + dst_rank * 3 + src_rank) % 251


def owned_mask(nbytes: int, rr_bytes: int, n_dst: int, slot: int, device) -> torch.Tensor:
    off = torch.arange(nbytes, device=device, dtype=torch.int64)
    return ((off // rr_bytes) % n_dst) == slot


def main() -> int:
    args = build_parser().parse_args()
    if args.executor != "src":
        raise ValueError("round-robin copies run on the source GPU only (--executor src)")
    rank, world, _ = D.env_rank_info()
    if world < 2:
        raise ValueError("the round-robin benchmark needs world_size >= 2 (launch with torchrun)")
    if args.rr_bytes <= 0:
        raise ValueError("--round-robin-bytes must be positive")
    n, c = args.nbytes, args.copies_per_iter
    piece = args.tma_inter_tile_bytes or args.tma_tile_bytes
    stages = args.tma_stages or K.pick_stages(args.tma_tile_bytes)
    if args.method == "tma":
        K.check_staged_constraints(n, args.tma_tile_bytes, piece, stages, args.rr_bytes)
    dsts = P.rr_destinations(rank, world, args.mode)          # raises for --mode pair
    # receive area: one slot of n*c bytes per source rank
    w = CC.CopyWorld(n * c * world)
    src = torch.empty(n * c, dtype=torch.uint8, device=w.device)
    for i in range(c):
        src[i * n:(i + 1) * n] = CC.position_pattern(n, seed=rank * 31 + i, device=w.device)
    for s in range(world):
        w.recv[s * n * c:(s + 1) * n * c] = prefill_value(rank, s)
    torch.cuda.synchronize()
    D.barrier()
    dst_views = [w.region.C.view_tensor(w.peer_ptr(d) + rank * n * c, [n * c], "uint8", w.device.index)
                 for d in dsts]
    status = K.StagedStatus(w.device)
    ctas = K.resolve_num_ctas(args.num_sms, w.device)

    def launch(k_iters: int, launches: int = 1):
        for i in range(c):
            sv = src[i * n:(i + 1) * n]
            dv = [d[i * n:(i + 1) * n] for d in dst_views]
            if args.method == "lsu":
                K.lsu_rr_copy(dv, sv, n, args.rr_bytes, ctas=ctas, threads=args.threads_per_cta, iters=k_iters, launches=launches)
            else:
                K.tma_staged_copy(dv, sv, n, rr_bytes=args.rr_bytes, tile=args.tma_tile_bytes, piece=piece,
                                  stages=stages, ctas=ctas, threads=staged_threads(args.threads_per_cta),
                                  iters=k_iters, status=status, launches=launches)

    def phase(iters: int):
        if args.persistent_kernel:
            launch(iters)
        elif c == 1:
            launch(1, iters)          # native back-to-back launches, no interpreter in between
        else:
            for _ in range(iters):
                launch(1)

    launch(1)
    torch.cuda.synchronize()
    CC.sleep_phase(args.sleep_before)
    if args.warmup:
        phase(args.warmup)
    torch.cuda.synchronize()
    D.barrier()
    elapsed = CC.device_timed(lambda: phase(args.iters))
    D.barrier()
    status.check()
    moved = float(n) * c * args.iters
    ok = True
    if args.check:
        torch.cuda.synchronize()
        D.barrier()
        for s in range(world):
            if s == rank:
                continue
            slot = P.rr_destinations(s, world, args.mode).index(rank)
            mask = owned_mask(n, args.rr_bytes, world - 1, slot, w.device)
            for i in range(c):
                got = w.recv[s * n * c + i * n: s * n * c + (i + 1) * n]
                want = CC.position_pattern(n, seed=s * 31 + i, device=w.device)
                ok = ok and bool(torch.equal(got[mask], want[mask]))
                ok = ok and bool((got[~mask] == prefill_value(rank, s)).all())
    kern = "lsu_rr_copy_kernel" if args.method == "lsu" else "tma_staged_push_kernel"
    line = (f"[rank {rank}] method={args.method} rr={fmt_bytes(args.rr_bytes)} dsts={list(dsts)} ctas={ctas} "
            f"persistent={args.persistent_kernel} bytes/copy={fmt_bytes(n)} iters={args.iters} "
            f"device_time={elapsed * 1e3:.3f} ms bw={CC.bw(moved, elapsed):.3f} GiB/s"
            + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl, title="SM round-robin copy",
              expectation=f"kernel {kern}", extra=dict(
                  bench="rr_copy", world=world, method=args.method, ctas=ctas, nbytes=n, rr_bytes=args.rr_bytes,
                  iters=args.iters, persistent=args.persistent_kernel, tile=args.tma_tile_bytes, stages=stages))
    all_ok = D.all_ranks_boolean(ok)
    w.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
