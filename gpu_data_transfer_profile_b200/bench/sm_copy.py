"""SM-driven pair copy benchmark: LSU ld/st versus the shared-memory staged ("TMA") pipeline.

Capability parity: `LSU_TMA/nvlink_lsu_tma_copy_test.py:1-828` (flags `:615-652`): `--method
lsu|tma`, `--executor src|dst` (push from the source GPU or pull from the destination GPU),
`--num-sms` as the CTA count (0 = all SMs), `--threads-per-cta`, stage ("intra") and store
("inter") tile sizes, `--persistent-kernel` (one launch that loops `iters` times on the device),
`--copies-per-iter`, pair topology, `--check`. Added here: `--vec-bytes 16|32` for the LSU
path and `--tma-stages` for the pipeline depth. In the staged method the bulk-copy engine
only touches the executor's own memory; NVLink traffic is always LSU.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.sm_copy --method tma \
        --nbytes 1M --num-sms 4 --persistent-kernel --executor src --check
"""
from __future__ import annotations

import argparse

import torch

from ..ops import copy as K
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import fmt_bytes, parse_nbytes
from . import copy_common as CC


def add_sm_flags(ap: argparse.ArgumentParser, executor_default: str) -> None:
    ap.add_argument("--copies-per-iter", type=int, default=1)
    ap.add_argument("--method", choices=["lsu", "tma"], default="lsu")
    ap.add_argument("--executor", choices=["src", "dst"], default=executor_default)
    ap.add_argument("--num-sms", type=int, default=0, help="CTAs to launch (0 = one per SM)")
    ap.add_argument("--threads-per-cta", type=int, default=256)
    ap.add_argument("--vec-bytes", type=int, choices=[16, 32], default=16)
    ap.add_argument("--tma-tile-bytes", "--tma-intra-tile-bytes", dest="tma_tile_bytes", type=parse_nbytes,
                    default=parse_nbytes("64K"))
    ap.add_argument("--tma-inter-tile-bytes", type=parse_nbytes, default=None)
    ap.add_argument("--tma-stages", type=int, default=0, help="pipeline depth (0 = as many as fit, max 4)")
    ap.add_argument("--persistent-kernel", action="store_true")
    ap.add_argument("--overlap-launches", action="store_true",
                    help="LSU method: let consecutive launches overlap (programmatic dependent launch)")
    ap.add_argument("--mode", choices=list(P.PAIR_MODES), default="ring")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    CC.add_common_flags(ap, nbytes_default="1G")
    add_sm_flags(ap, "dst")
    return ap


def staged_threads(threads_per_cta: int) -> int:
    """One producer warp + consumer warps; the flag counts the consumer threads."""
    t = max(32, (threads_per_cta // 32) * 32)
    return min(32 + t, 1024)


def main() -> int:
    args = build_parser().parse_args()
    if args.copies_per_iter <= 0 or args.iters <= 0:
        raise ValueError("--copies-per-iter and --iters must be positive")
    n, c = args.nbytes, args.copies_per_iter
    piece = args.tma_inter_tile_bytes or args.tma_tile_bytes
    stages = args.tma_stages or K.pick_stages(args.tma_tile_bytes)
    if args.method == "tma":
        K.check_staged_constraints(n, args.tma_tile_bytes, piece, stages)
    w = CC.CopyWorld(n * c)
    pair = (lambda r: P.choose_pair(r, w.size, args.mode)[1]) if w.size > 1 else (lambda r: 0)
    dst_rank = pair(w.rank)
    src_rank = next((s for s in range(w.size) if pair(s) == w.rank), w.rank)
    # src executor: I push my local source into dst_rank's receive area.
    # dst executor: the receive area is MINE and I pull from src_rank's source, which therefore
    # has to be peer-visible: sources live in a second symmetric region.
    from ..parallel.symm import SymmetricRegion
    src_region = SymmetricRegion(w.world, max(n * c, 256))
    src = src_region.view(0, (n * c,), "uint8")
    for i in range(c):
        src[i * n:(i + 1) * n] = CC.position_pattern(n, seed=w.rank * 31 + i, device=w.device)
    w.recv.fill_(P.pair_prefill_value(w.rank))
    torch.cuda.synchronize()
    D.barrier()
    if args.executor == "src":
        s_t, d_t = src, w.peer_view(dst_rank, n * c)
    else:
        s_t = w.region.C.view_tensor(src_region.peer_ptrs[src_rank], [n * c], "uint8", w.device.index)
        d_t = w.recv
    status = K.StagedStatus(w.device)
    ctas = K.resolve_num_ctas(args.num_sms, w.device)

    def launch(iters_in_kernel: int, launches: int = 1):
        for i in range(c):
            sv, dv = s_t[i * n:(i + 1) * n], d_t[i * n:(i + 1) * n]
            if args.method == "lsu":
                K.lsu_copy(dv, sv, n, ctas=ctas, threads=args.threads_per_cta, iters=iters_in_kernel,
                           vec_bytes=args.vec_bytes, executor=w.device, launches=launches,
                           overlap_launches=args.overlap_launches)
            else:
                K.tma_staged_copy([dv], sv, n, pull=args.executor == "dst", tile=args.tma_tile_bytes,
                                  piece=piece, stages=stages, ctas=ctas,
                                  threads=staged_threads(args.threads_per_cta), iters=iters_in_kernel,
                                  status=status, launches=launches)

    def phase(iters: int):
        if args.persistent_kernel:
            launch(iters)
        elif c == 1:
            launch(1, iters)          # native back-to-back launches, no interpreter in between
        else:
            for _ in range(iters):
                launch(1)

    launch(1)                      # first launch outside the timed phase (module load)
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
        for i in range(c):
            want = CC.position_pattern(n, seed=src_rank * 31 + i, device=w.device)
            ok = ok and bool(torch.equal(w.recv[i * n:(i + 1) * n], want))
    kern = ("lsu_copy_kernel" if args.method == "lsu" else
            "tma_staged_pull_kernel" if args.executor == "dst" else "tma_staged_push_kernel")
    line = (f"[rank {w.rank}] method={args.method} executor={args.executor} ctas={ctas} threads={args.threads_per_cta} "
            f"persistent={args.persistent_kernel} bytes/copy={fmt_bytes(n)} copies/iter={c} iters={args.iters} "
            f"device_time={elapsed * 1e3:.3f} ms bw={CC.bw(moved, elapsed):.3f} GiB/s "
            f"({moved / elapsed / 1e9 if elapsed else 0:.2f} GB/s)" + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(w.rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl,
              title="SM pair copy", expectation=f"kernel {kern}: "
              + (f"1 launch of {args.iters} iterations" if args.persistent_kernel else f"{args.iters * c} launches"),
              extra=dict(bench="sm_copy", world=w.size, method=args.method, executor=args.executor, ctas=ctas,
                         threads=args.threads_per_cta, nbytes=n, copies=c, iters=args.iters,
                         persistent=args.persistent_kernel, tile=args.tma_tile_bytes, piece=piece, stages=stages,
                         vec_bytes=args.vec_bytes))
    all_ok = D.all_ranks_boolean(ok)
    torch.cuda.synchronize()
    D.barrier()
    src_region.close()
    w.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
