"""EP combine benchmark: one set-up dispatch, then `combine` timed on its own.

Capability parity: `DeepEP_v1/deepep_v1_combine.py:1-385` (flags `:59-90`, set-up dispatch
`:190-226`, timed combine `:229-251`, `--fake-expert-output identity|random`, identity check
`combined / ranks_per_token == input` within 5e-3 for 16-bit types and 1e-5 for fp32, `:329-342`).

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.combine \
        --num-local-tokens 4096 --token-hidden 7168 --num-of-experts 256 --topk 8 --ep 8
"""
from __future__ import annotations

import argparse

import torch

from ..parallel.events import EventHandle, EventOverlap
from ..utils import dist as D
from . import ep_common as C
from .dispatch import run_dispatch


def run_combine(ctx: C.EpContext, y, handle):
    a = ctx.args
    prev = EventOverlap(EventHandle()) if a.async_finish else None
    out, _, ev = ctx.buffer.combine(y, handle, previous_event=prev, async_finish=a.async_finish,
                                    allocate_on_comm_stream=a.allocate_on_comm_stream)
    if a.async_finish:
        ev.current_stream_wait()
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    C.add_ep_flags(ap, 24)
    ap.add_argument("--fake-expert-output", choices=("identity", "random"), default="identity")
    args = ap.parse_args()
    if args.use_fp8:
        raise ValueError("combine takes bf16/fp16/fp32 rows; --use-fp8 applies to dispatch only")
    ctx = C.EpContext(args)
    (recv_x, _, _, _, handle, _), in_rank = run_dispatch(ctx)
    y = recv_x if args.fake_expert_output == "identity" else torch.randn_like(recv_x)
    res = C.timed_loop(lambda: run_combine(ctx, y, handle), args.warmup_iters, args.benchmark_iters,
                       before=ctx.buffer.barrier, group=ctx.group)
    out = run_combine(ctx, y, handle)
    ctx.buffer.check_status()
    ok = out.shape == ctx.x.shape and bool(torch.isfinite(out.float()).all())
    if args.check_correctness and args.fake_expert_output == "identity":
        n = in_rank.sum(1, keepdim=True).clamp_min(1).float()
        tol = 1e-5 if ctx.dtype == torch.float32 else 5e-3
        ok = ok and torch.allclose(out.float() / n, ctx.x.float(), atol=tol * 4, rtol=tol * 2)
    nbytes = C.remote_rows(in_rank, ctx.ep_rank) * args.token_hidden * ctx.dtype.itemsize
    gbs = nbytes / (res["max_over_ranks_ms"] * 1e-3) / 1e9
    if args.print_timing:
        D.ordered_print(f"[rank {ctx.rank}] ep_rank={ctx.ep_rank} combine avg={res['mean_ms']:.4f} ms min={res['min_ms']:.4f} ms "
                        f"rows_in={handle.n_recv} tokens_out={out.shape[0]} check={'OK' if ok else 'FAIL'}")
    all_ok = D.all_ranks_boolean(ok)
    C.emit(ctx.rank, dict(bench="combine", ep=args.ep, tokens=args.num_local_tokens, hidden=args.token_hidden,
                          experts=args.num_of_experts, topk=args.topk, dtype=args.dtype, zipf=args.zipf,
                          num_sms=args.num_sms, ms_max_over_ranks=res["max_over_ranks_ms"], nvlink_gbs_rank0=gbs,
                          frac_of_770=gbs / 770.0, fake_expert_output=args.fake_expert_output, check=bool(all_ok)),
           args.jsonl)
    ctx.close()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
