"""Fan-out ("all-to-all") copy-engine benchmark: every active source rank copies the SAME
source buffer into its private slot on every other GPU.

Capability parity: `Copy_Engine/nvlink_all_to_all_copy_engine_test.py:1-306` (flags `:107-128`,
destination order `:66-71`, active-source subset `:149-170`, copy stream on the source device
`:213-214`, three samples per destination in the check `:91-103`; here the check compares the
whole slot).

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.a2a_copy --nbytes 16M --check
"""
from __future__ import annotations

import argparse

import torch

from ..ops.copy import CopyEngine
from ..utils import dist as D
from ..utils import patterns as P
from ..utils.sizes import fmt_bytes, parse_gpu_ids
from . import copy_common as CC


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    CC.add_common_flags(ap, nbytes_default="16M")
    ap.add_argument("--copy-mode", choices=["separate", "batch", "multimem"], default="separate",
                    help="multimem: one store stream through the NVSwitch multicast address (NVLS)")
    ap.add_argument("--num-sms", type=int, default=0, help="CTAs of the multimem kernel (0 = one per SM)")
    ap.add_argument("--batch-impl", choices=["graph", "kernel"], default="graph")
    ap.add_argument("--rotate-destination-order", action="store_true")
    ap.add_argument("--active-source-gpus", nargs="?", const="0", default=None,
                    help="comma-separated ranks that send (bare flag = rank 0 only; default = all)")
    ap.add_argument("--no-proxy-thread", action="store_true")
    return ap


def run_multimem(args, w, src, active, is_src, order) -> int:
    """Fan-out by switch multicast: rank r stores its source ONCE to slot r of a multicast-mapped
    buffer; the switch replicates it into slot r of every GPU (the sender's own copy included)."""
    from ..ops.copy import MulticastBuffer
    n = args.nbytes
    mc = MulticastBuffer(n * w.size)
    if not D.all_ranks_boolean(mc.available):
        D.ordered_print(f"[rank {w.rank}] multimem unavailable: {mc.why or 'a peer has no multicast mapping'}")
        w.close()
        return 3
    mc.tensor.fill_(P.DST_GAP_SENTINEL)
    torch.cuda.synchronize()
    D.barrier()

    def phase(k):
        if is_src:
            mc.broadcast(src, n, offset=w.rank * n, ctas=args.num_sms, launches=k)

    CC.sleep_phase(args.sleep_before)
    phase(max(args.warmup, 1))
    torch.cuda.synchronize()
    D.barrier()
    elapsed = CC.device_timed(lambda: phase(args.iters)) if is_src else 0.0
    torch.cuda.synchronize()
    D.barrier()
    moved = float(n) * len(order) * args.iters if is_src else 0.0
    ok = True
    if args.check:
        for s in range(w.size):
            slot = mc.tensor[s * n:(s + 1) * n]
            want = CC.position_pattern(n, seed=s, device=w.device) if s in active else None
            ok = ok and (bool(torch.equal(slot, want)) if want is not None else bool((slot == P.DST_GAP_SENTINEL).all()))
    line = (f"[rank {w.rank}] source={'yes' if is_src else 'no '} copy_mode=multimem bytes/dst={fmt_bytes(n)} "
            f"iters={args.iters} device_time={elapsed * 1e3:.3f} ms delivered_bw={CC.bw(moved, elapsed):.3f} GiB/s "
            f"link_bw={CC.bw(float(n) * args.iters if is_src else 0.0, elapsed):.3f} GiB/s"
            + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(w.rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl, title="fan-out by switch multicast",
              extra=dict(bench="a2a_copy", world=w.size, copy_mode="multimem", nbytes=n, iters=args.iters, active=list(active)),
              expectation="kernel multimem_bcast_kernel: one store stream per source, replicated in the switch")
    all_ok = D.all_ranks_boolean(ok)
    torch.cuda.synchronize()
    D.barrier()
    w.close()
    return 0 if all_ok else 2


def main() -> int:
    args = build_parser().parse_args()
    n = args.nbytes
    rank, world, _ = D.env_rank_info()
    if world < 2:
        raise ValueError("the fan-out benchmark needs world_size >= 2 (launch with torchrun)")
    w = CC.CopyWorld(n * world)            # slot s of my receive area belongs to source rank s
    active = parse_gpu_ids(args.active_source_gpus, w.size)
    is_src = w.rank in active
    src = CC.position_pattern(n, seed=w.rank, device=w.device)
    w.recv.fill_(P.DST_GAP_SENTINEL)
    torch.cuda.synchronize()
    D.barrier()
    order = P.destination_order(w.rank, w.size, args.rotate_destination_order)
    if args.copy_mode == "multimem":
        return run_multimem(args, w, src, active, is_src, order)
    copies = [(w.peer_ptr(d) + w.rank * n, w.peer_device(d), src.data_ptr(), w.device.index, n) for d in order]
    mode = "separate" if args.copy_mode == "separate" else args.batch_impl
    eng = CopyEngine(copies, mode, stream_device=w.device.index, use_proxy=not args.no_proxy_thread) if is_src else None
    CC.sleep_phase(args.sleep_before)
    if eng and args.warmup:
        eng.run(args.warmup)
    D.barrier()
    r = eng.run(args.iters) if eng else dict(wall_seconds=0.0, submit_seconds=0.0)
    D.barrier()
    elapsed = r["wall_seconds"]
    moved = float(n) * len(order) * args.iters if is_src else 0.0
    ok = True
    if args.check:
        torch.cuda.synchronize()
        D.barrier()
        for s in range(w.size):
            slot = w.recv[s * n:(s + 1) * n]
            if s == w.rank or s not in active:
                ok = ok and bool((slot == P.DST_GAP_SENTINEL).all())
            else:
                ok = ok and bool(torch.equal(slot, CC.position_pattern(n, seed=s, device=w.device)))
    line = (f"[rank {w.rank}] source={'yes' if is_src else 'no '} dsts={list(order)} copy_mode={args.copy_mode}({mode}) "
            f"bytes/dst={fmt_bytes(n)} iters={args.iters} elapsed={elapsed * 1e3:.3f} ms "
            f"egress_bw={CC.bw(moved, elapsed):.3f} GiB/s" + (f" check={'OK' if ok else 'FAIL'}" if args.check else ""))
    CC.report(w.rank, line, elapsed=elapsed, bytes_moved=moved, jsonl=args.jsonl,
              title="fan-out copy-engine copy",
              extra=dict(bench="a2a_copy", world=w.size, copy_mode=mode, nbytes=n, iters=args.iters,
                         active=list(active), rotate=args.rotate_destination_order),
              expectation=f"{len(order)} peer-to-peer memcpys per iteration on every active source GPU")
    all_ok = D.all_ranks_boolean(ok)
    del eng
    w.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
