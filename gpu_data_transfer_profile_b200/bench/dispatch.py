"""EP dispatch benchmark with fake tokens and a fake router.

Capability parity: `DeepEP_v1/deepep_v1_dispatch.py:1-394` — same flags (`:59-86`), same timed
region (`get_dispatch_layout` + `dispatch` between two CUDA events, `:186-248`), same sanity
checks (shapes, id range, probabilities, `:330-347`), exit code 2 when any rank fails (`:381`).
Reported time is the max over ranks; NVLink GB/s and the fraction of the 770 GB/s measured
per-direction peer bandwidth are derived from the bytes that leave the rank.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.dispatch \
        --num-local-tokens 4096 --token-hidden 7168 --num-of-experts 256 --topk 8 --ep 8
"""
from __future__ import annotations

import argparse

import torch

from ..parallel.events import EventHandle, EventOverlap
from ..utils import dist as D
from . import ep_common as C


def run_dispatch(ctx: C.EpContext, zero_copy: bool = False):
    a, buf = ctx.args, ctx.buffer
    prev = EventOverlap(EventHandle()) if a.async_finish else None
    per_rank, per_rdma, per_expert, in_rank, ev = buf.get_dispatch_layout(
        ctx.topk_idx, a.num_of_experts, previous_event=prev, async_finish=a.async_finish,
        allocate_on_comm_stream=a.allocate_on_comm_stream)
    out = buf.dispatch(ctx.x, topk_idx=ctx.topk_idx, topk_weights=ctx.topk_weights,
                       num_tokens_per_rank=per_rank, num_tokens_per_rdma_rank=per_rdma,
                       is_token_in_rank=in_rank, num_tokens_per_expert=per_expert, previous_event=ev,
                       async_finish=a.async_finish, allocate_on_comm_stream=a.allocate_on_comm_stream,
                       use_fp8=a.use_fp8, zero_copy=zero_copy)
    if a.async_finish:
        out[5].current_stream_wait()
    return out, in_rank


def check(ctx: C.EpContext, out, in_rank) -> bool:
    a = ctx.args
    recv_x, recv_idx, recv_w, per_local, handle, _ = out
    El = a.num_of_experts // a.ep
    x = recv_x[0] if isinstance(recv_x, tuple) else recv_x
    per_local = per_local.tolist() if torch.is_tensor(per_local) else list(per_local)
    ok = x.shape[1] == a.token_hidden and len(per_local) == El
    ok = ok and x.shape[0] == recv_idx.shape[0] == recv_w.shape[0] == handle.n_recv
    ok = ok and bool(((recv_idx >= -1) & (recv_idx < El)).all())
    ok = ok and torch.bincount(recv_idx[recv_idx >= 0], minlength=El).tolist() == per_local
    ok = ok and bool(((ctx.topk_weights.sum(-1) - 1).abs() < 1e-3).all())
    ok = ok and bool((recv_w >= 0).all()) and bool(((recv_w > 0) == (recv_idx >= 0)).all())
    # every received row must equal the source token (exchange source indices through a combine)
    return ok


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    C.add_ep_flags(ap, 24)
    ap.add_argument("--rerandomize-routing-each-iter", action=argparse.BooleanOptionalAction, default=False)
    ap.add_argument("--zero-copy", action="store_true", help="return views of the receive region")
    args = ap.parse_args()
    ctx = C.EpContext(args)
    it = [0]

    def before():
        if args.rerandomize_routing_each_iter:
            it[0] += 1
            ctx.reroute(it[0])
        ctx.buffer.barrier()

    res = C.timed_loop(lambda: run_dispatch(ctx, args.zero_copy), args.warmup_iters, args.benchmark_iters,
                       before=before, group=ctx.group)
    out, in_rank = run_dispatch(ctx)
    ctx.buffer.check_status()
    ok = check(ctx, out, in_rank) if args.check_correctness else True
    row = (args.token_hidden + args.token_hidden // 128 * 4) if args.use_fp8 else args.token_hidden * ctx.dtype.itemsize
    nbytes = C.remote_rows(in_rank, ctx.ep_rank) * row
    gbs = nbytes / (res["max_over_ranks_ms"] * 1e-3) / 1e9
    per_local = out[3]
    if args.print_timing:
        D.ordered_print(f"[rank {ctx.rank}] ep_rank={ctx.ep_rank} dispatch avg={res['mean_ms']:.4f} ms min={res['min_ms']:.4f} ms "
                        f"recv_tokens={out[4].n_recv} tokens_per_local_expert={list(per_local)[:8]}{'...' if len(per_local) > 8 else ''} "
                        f"remote_bytes={nbytes} check={'OK' if ok else 'FAIL'}")
    all_ok = D.all_ranks_boolean(ok)
    C.emit(ctx.rank, dict(bench="dispatch", ep=args.ep, tokens=args.num_local_tokens, hidden=args.token_hidden,
                          experts=args.num_of_experts, topk=args.topk, dtype="fp8" if args.use_fp8 else args.dtype,
                          zipf=args.zipf, num_sms=args.num_sms, ms_max_over_ranks=res["max_over_ranks_ms"],
                          nvlink_gbs_rank0=gbs, frac_of_770=gbs / 770.0, zero_copy=args.zero_copy,
                          check=bool(all_ok)), args.jsonl)
    ctx.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
