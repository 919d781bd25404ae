"""Measured comparator: MoE dispatch + combine through NCCL `all_to_all_single`
(`AllToAllTokenDispatcher`, standard "alltoall" token-dispatcher semantics) on the same inputs
as `bench.py` / `bench.dispatch` / `bench.combine`. The reference contains no such script (its
NCCL use is control traffic only, `Copy_Engine/nvlink_copy_engine_test.py:392-410`); this is the
same-box baseline that the library's own kernels are compared with.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.nccl_baseline \
        --num-local-tokens 4096 --token-hidden 7168 --num-of-experts 256 --topk 8 --ep 8
"""
from __future__ import annotations

import argparse

import torch

from ..ref.cpu_oracle import AllToAllTokenDispatcher, make_routing
from ..utils import dist as D
from ..utils.timing import L2Flusher
from . import ep_common as C


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    C.add_ep_flags(ap, 24)
    args = ap.parse_args()
    rank, world, _ = D.init_distributed()
    C.validate_args(args, world)
    if not D.is_dist():
        raise ValueError("the NCCL baseline needs a torchrun launch")
    group, ep_rank, _ = D.create_ep_group(args.ep)
    dev = torch.device("cuda", torch.cuda.current_device())
    T, H, E, K = args.num_local_tokens, args.token_hidden, args.num_of_experts, args.topk
    dtype = C.DTYPES[args.dtype]
    g = torch.Generator().manual_seed(args.seed + rank)
    x = torch.randn(T, H, generator=g).to(dtype).to(dev)
    idx, w = make_routing(T, E, K, seed=args.seed * 7 + rank, zipf_s=args.zipf)
    idx, w = idx.to(dev), w.to(dev)
    disp = AllToAllTokenDispatcher(group, E)
    flush = L2Flusher(dev)
    times = {"dispatch": [], "combine": [], "total": []}
    for it in range(args.warmup_iters + args.benchmark_iters):
        flush()
        D.barrier(group)
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        rows, probs, per_expert = disp.dispatch(x, idx, w)
        e1.record()
        out = disp.combine(rows, weights=w)
        e2.record()
        torch.cuda.synchronize()
        if it >= args.warmup_iters:
            times["dispatch"].append(e0.elapsed_time(e1))
            times["combine"].append(e1.elapsed_time(e2))
            times["total"].append(e0.elapsed_time(e2))
    ok = torch.allclose(out.float(), x.float() * w.sum(-1, keepdim=True), atol=5e-2, rtol=2e-2)
    mean = {k: sum(v) / len(v) for k, v in times.items()}
    mx = {k: D.all_reduce_scalar(v, "max", group) for k, v in mean.items()}
    D.ordered_print(f"[rank {rank}] nccl all_to_all_single dispatch={mean['dispatch']:.4f} ms combine={mean['combine']:.4f} ms "
                    f"total={mean['total']:.4f} ms rows={rows.shape[0]} check={'OK' if ok else 'FAIL'}")
    all_ok = D.all_ranks_boolean(ok)
    C.emit(rank, dict(bench="nccl_baseline", ep=args.ep, tokens=T, hidden=H, experts=E, topk=K, dtype=args.dtype,
                      zipf=args.zipf, dispatch_ms_max=mx["dispatch"], combine_ms_max=mx["combine"],
                      total_ms_max=mx["total"], rows_per_token="one per (token, expert)", check=bool(all_ok)), args.jsonl)
    D.shutdown()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
