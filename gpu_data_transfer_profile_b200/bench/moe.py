"""Megatron-style MoE loop: dispatch -> grouped expert MLP -> combine, timed per phase.

Capability parity: `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:631-963` (flags `:631-661`,
per-iteration phases with four CUDA events `:766-815`, sanity checks `:889-911`, per-rank averages
`:913-939`). Added here: `--dispatcher-mode fused|deepep`, `--expert-backend tcgen05`,
`--fuse-combine` (fc2 epilogue performs the combine send; forward only), `--backward` (runs the
backward pass too: dispatch and combine are each other's backward).

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.moe --num-local-tokens 8192 \
        --token-hidden 4096 --moe-ffn-hidden-size 14336 --num-of-experts 8 --topk 2 --ep 8
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass

import torch

from ..models import fused_a2a as A
from ..models.experts import ACTIVATIONS, build_experts
from ..models.token_dispatcher import B200TokenDispatcher
from ..utils import dist as D
from . import ep_common as C


@dataclass
class IterationResult:
    dispatch_ms: float
    expert_ms: float
    combine_ms: float
    total_ms: float
    output: torch.Tensor
    tokens_per_expert: torch.Tensor
    fwd_bwd_ms: float = 0.0


def run_one_iteration(ctx, manager, experts, args, x, fused: bool) -> IterationResult:
    e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    e0.record()
    fp8 = getattr(args, "fp8", False) and not args.backward
    if fp8:
        rows, tpe, probs = manager.dispatch_fp8(x, ctx.topk_idx, ctx.topk_weights)
    else:
        rows, tpe, probs = manager.dispatch(x, ctx.topk_idx, ctx.topk_weights)
    e1.record()
    if fp8:
        El = experts.num_local_experts
        y = experts.forward_fp8(rows, tpe, probs, expert_off=manager.handle.meta[2 + El: 2 + El + El + 1])
        e2.record()
        out = manager.combine(y)
    elif fused:
        buf = A.get_buffer(manager.group, A.get_hidden_bytes(x), manager.world)
        handle, manager.handle = manager.handle, None
        if args.backward:
            out = experts.forward_fused_combine_train(rows, tpe, probs, buf, handle)
        else:
            out = experts.forward_fused_combine(rows, probs, buf, handle)
        e2.record()
    else:
        y = experts(rows, tpe, probs)
        e2.record()
        out = manager.combine(y)
    e3.record()
    e4 = torch.cuda.Event(enable_timing=True)
    if args.backward:
        out.float().mean().backward()
    e4.record()
    torch.cuda.synchronize()
    r = IterationResult(e0.elapsed_time(e1), e1.elapsed_time(e2), e2.elapsed_time(e3), e0.elapsed_time(e3), out, tpe)
    r.fwd_bwd_ms = e0.elapsed_time(e4)
    return r


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    C.add_ep_flags(ap, 20)
    ap.add_argument("--moe-ffn-hidden-size", type=int, required=True)
    ap.add_argument("--activation", choices=ACTIVATIONS, default="swiglu")
    ap.add_argument("--expert-backend", choices=("auto", "te", "tcgen05", "torch"), default="auto")
    ap.add_argument("--dispatcher-mode", choices=("fused", "deepep"), default="fused")
    ap.add_argument("--fuse-combine", action="store_true")
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--fp8", action="store_true",
                    help="forward only: e4m3 dispatch (1x128 scales) feeding the block-scaled fp8 fc1 on the tensor cores")
    args = ap.parse_args()
    rank, world, _ = D.init_distributed()
    C.validate_args(args, world)
    group, ep_rank, _ = D.create_ep_group(args.ep)
    dev = torch.device("cuda", torch.cuda.current_device())
    from ..parallel.buffer import Buffer
    from ..parallel.symm import LocalWorld
    Buffer.set_num_sms(args.num_sms)
    T, H, E, K, F = args.num_local_tokens, args.token_hidden, args.num_of_experts, args.topk, args.moe_ffn_hidden_size
    El = E // args.ep
    A.configure_buffer(num_max_tokens_per_rank=T, num_topk=K, num_experts=E, group_by_expert=args.dispatcher_mode == "fused")
    lworld = None if D.is_dist() else LocalWorld.make(1, dev)[0]
    manager = B200TokenDispatcher(group, El, E, ep_rank * El, args.async_finish, args.allocate_on_comm_stream,
                                  mode=args.dispatcher_mode, world=lworld)
    dtype = C.DTYPES[args.dtype]
    experts, backend = build_experts(args.expert_backend, El, H, F, dtype, args.activation, dev, use_fp8=args.fp8)
    if args.fp8 and not getattr(experts, "use_fp8", False):
        raise ValueError("--fp8 needs the tcgen05 expert backend (hidden and ffn sizes multiples of 128)")

    class Ctx:
        pass
    ctx = Ctx()
    ctx.args = args
    g = torch.Generator().manual_seed(args.seed + rank)
    x = torch.randn(T, H, generator=g).to(dtype).to(dev).requires_grad_(args.backward)
    from ..ref.cpu_oracle import make_routing
    idx, w = make_routing(T, E, K, seed=args.seed * 7 + rank, zipf_s=args.zipf)
    ctx.topk_idx, ctx.topk_weights = idx.to(dev), w.to(dev)
    fused = args.fuse_combine and hasattr(experts, "forward_fused_combine") and args.dispatcher_mode == "fused"

    def one():
        if args.backward:
            return run_one_iteration(ctx, manager, experts, args, x, fused and args.activation == "swiglu")
        with torch.no_grad():
            return run_one_iteration(ctx, manager, experts, args, x, fused)

    for _ in range(args.warmup_iters):
        one()
    D.barrier(group)
    acc = [0.0, 0.0, 0.0, 0.0, 0.0]
    last = None
    for _ in range(args.benchmark_iters):
        last = one()
        for i, v in enumerate((last.dispatch_ms, last.expert_ms, last.combine_ms, last.total_ms, last.fwd_bwd_ms)):
            acc[i] += v / args.benchmark_iters
    D.barrier(group)
    ok = last.output.shape == (T, H) and bool(torch.isfinite(last.output.float()).all())
    ok = ok and last.tokens_per_expert.numel() == El
    A.get_buffer(group, A.get_hidden_bytes(x), lworld).check_status()
    tot_max = D.all_reduce_scalar(acc[3], "max", group)
    if args.print_timing:
        D.ordered_print(f"[rank {rank}] backend={backend} mode={args.dispatcher_mode} fused_combine={fused} "
                        f"dispatch={acc[0]:.4f} ms expert={acc[1]:.4f} ms combine={acc[2]:.4f} ms total={acc[3]:.4f} ms fwd+bwd={acc[4]:.4f} ms "
                        f"tokens_per_expert={last.tokens_per_expert.tolist()[:8]} check={'OK' if ok else 'FAIL'}")
    all_ok = D.all_ranks_boolean(ok)
    flops = 2.0 * int(last.tokens_per_expert.sum()) * H * F * (3 if args.activation == "swiglu" else 2)
    C.emit(rank, dict(bench="moe", ep=args.ep, tokens=T, hidden=H, ffn=F, experts=E, topk=K, backend=backend,
                      mode=args.dispatcher_mode, fused_combine=fused, backward=args.backward, fp8=args.fp8,
                      dispatch_ms=acc[0], expert_ms=acc[1], combine_ms=acc[2], total_ms_rank0=acc[3],
                      total_ms_max_over_ranks=tot_max,
                      fwd_bwd_ms_max_over_ranks=D.all_reduce_scalar(acc[4], "max", group) if args.backward else None, expert_tflops_rank0=flops / (acc[1] * 1e-3) / 1e12 if acc[1] else 0,
                      check=bool(all_ok)), args.jsonl)
    A.release_buffers()
    D.shutdown()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
