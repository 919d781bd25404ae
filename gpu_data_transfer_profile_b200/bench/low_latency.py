"""Low-latency (decode) dispatch + combine: latency per call, eager and under a CUDA graph.

Config of record: 128 tokens/rank, hidden 7168, 256 experts, top-8, fp8 e4m3 dispatch with
1x128 scales, bf16 combine, seeded uniform top-8 selection. The reference has no low-latency
path; the call shapes follow upstream DeepEP's `low_latency_dispatch` / `low_latency_combine`.

    torchrun --nproc-per-node 8 -m gpu_data_transfer_profile_b200.bench.low_latency --ep 8
"""
from __future__ import annotations

import argparse

import torch

from ..parallel.buffer import Buffer
from ..parallel.symm import LocalWorld
from ..ref.cpu_oracle import make_routing
from ..utils import dist as D
from . import ep_common as C


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--num-local-tokens", type=int, default=128)
    ap.add_argument("--token-hidden", type=int, default=7168)
    ap.add_argument("--num-of-experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--ep", type=int, required=True)
    ap.add_argument("--num-max-dispatch-tokens-per-rank", type=int, default=0)
    ap.add_argument("--no-fp8", action="store_true")
    ap.add_argument("--warmup-iters", type=int, default=10)
    ap.add_argument("--benchmark-iters", type=int, default=100)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--overlap-launches", action="store_true",
                    help="launch the kernels with programmatic stream serialisation (launch latencies overlap)")
    ap.add_argument("--signal-mode", type=int, choices=(0, 1), default=None,
                    help="0: every send CTA signals every peer; 1: the last CTA does; default: by group size")
    ap.add_argument("--combine", choices=("pull", "push"), default="pull",
                    help="pull: the expert output lies in the buffer's in-place combine input and is loaded by its "
                         "source ranks (one kernel); push: it is sent back to per-(token, k) slots (two kernels)")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--jsonl", default=None)
    a = ap.parse_args()
    rank, world, _ = D.init_distributed()
    group, ep_rank, _ = D.create_ep_group(a.ep)
    dev = torch.device("cuda", torch.cuda.current_device())
    T, H, E, K = a.num_local_tokens, a.token_hidden, a.num_of_experts, a.topk
    M = a.num_max_dispatch_tokens_per_rank or T
    fp8 = not a.no_fp8
    Buffer.set_num_sms(a.num_sms)
    Buffer.ll_signal_mode = a.signal_mode
    Buffer.ll_overlap_launches = a.overlap_launches
    lw = None if D.is_dist() else LocalWorld.make(1, dev)[0]
    buf = Buffer(group, Buffer.get_low_latency_nvl_size_hint(M, H, a.ep, E, K), 0, low_latency_mode=True, world=lw)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(a.seed + rank)).to(torch.bfloat16).to(dev)
    idx, w = make_routing(T, E, K, seed=a.seed * 7 + rank)
    idx, w = idx.to(dev), w.to(dev)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    El = E // a.ep

    state = {}

    def dispatch_only():
        state["recv"], state["count"], state["handle"], _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=fp8)

    def dequant():
        """bf16 stand-in for the expert output of the CURRENT dispatch (valid rows only)."""
        if not fp8:
            return state["recv"]
        q, sc = state["recv"]
        y = torch.zeros((El, a.ep * M, H), dtype=torch.bfloat16, device=dev)
        for e, n in enumerate(state["count"].tolist()):
            y[e, :n] = (q[e, :n].float().view(n, H // 128, 128) * sc[e, :n, :, None]).view(n, H).to(torch.bfloat16)
        return y

    dispatch_only()
    pull = a.combine == "pull"
    y_static = dequant().clone()     # timing input for combine (row order of this first dispatch)
    if pull:
        # the experts write their output in place: outside the timed region, as the expert GEMM's epilogue would
        y_in = buf.get_next_low_latency_combine_buffer(state["handle"])
        y_in.copy_(y_static)

    def combine_only():
        if pull:
            buf.low_latency_combine(y_in, idx, w, state["handle"], out=out)
        else:
            buf.low_latency_combine(y_static if fp8 else state["recv"], idx, w, state["handle"], out=out)

    def step():
        dispatch_only()
        combine_only()

    eager = C.timed_loop(step, a.warmup_iters, a.benchmark_iters, before=buf.barrier, group=group)
    d_only = C.timed_loop(dispatch_only, a.warmup_iters, a.benchmark_iters, before=buf.barrier, group=group)
    c_only = C.timed_loop(combine_only, a.warmup_iters, a.benchmark_iters, before=buf.barrier, group=group)
    # the same step captured once and replayed: no host work per call
    torch.cuda.synchronize()
    D.barrier(group)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    graphed = C.timed_loop(graph.replay, a.warmup_iters, a.benchmark_iters, before=buf.barrier, group=group)
    # correctness: one more round whose expert input is built from THAT dispatch (the slot order
    # inside a (local expert, source) block is not fixed between calls)
    dispatch_only()
    if pull:
        y_in.copy_(dequant())
        buf.low_latency_combine(y_in, idx, w, state["handle"], out=out)
    else:
        buf.low_latency_combine(dequant(), idx, w, state["handle"], out=out)
    buf.check_status()
    tol = 0.6 if fp8 else 0.08
    ok = torch.allclose(out.float(), x.float() * w.sum(1, keepdim=True), atol=tol, rtol=0.08)
    send_d = T * K * ((H + H // 128 * 4) if fp8 else H * 2)
    send_c = T * K * H * 2
    D.ordered_print(f"[rank {rank}] low-latency dispatch+combine eager={eager['mean_ms'] * 1e3:.1f} us "
                    f"dispatch={d_only['mean_ms'] * 1e3:.1f} us combine={c_only['mean_ms'] * 1e3:.1f} us "
                    f"graph={graphed['mean_ms'] * 1e3:.1f} us (min {graphed['min_ms'] * 1e3:.1f} us) combine={a.combine} "
                    f"check={'OK' if ok else 'FAIL'}")
    all_ok = D.all_ranks_boolean(ok)
    C.emit(rank, dict(bench="low_latency", combine=a.combine, ep=a.ep, tokens=T, hidden=H, experts=E, topk=K, fp8=fp8,
                      eager_us_max_over_ranks=eager["max_over_ranks_ms"] * 1e3,
                      graph_us_max_over_ranks=graphed["max_over_ranks_ms"] * 1e3,
                      dispatch_us_max_over_ranks=d_only["max_over_ranks_ms"] * 1e3,
                      combine_us_max_over_ranks=c_only["max_over_ranks_ms"] * 1e3,
                      bytes_dispatch=send_d, bytes_combine=send_c,
                      check=bool(all_ok)), a.jsonl)
    buf.destroy()
    D.shutdown()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
