"""Multi-GPU self-check: this library's dispatch/combine against the NCCL `all_to_all_single`
dispatcher on identical inputs. Exit code 0 when every rank agrees, 2 otherwise
(reduction of the per-rank verdict as in `DeepEP_v1/deepep_v1_dispatch.py:259-262,381`).

    torchrun --nproc-per-node 2 -m gpu_data_transfer_profile_b200.bench.moe_check --ep 2
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..parallel.buffer import Buffer
from ..ref.cpu_oracle import AllToAllTokenDispatcher, make_routing
from ..utils import dist as D


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ep", type=int, required=True)
    ap.add_argument("--num-local-tokens", type=int, default=512)
    ap.add_argument("--token-hidden", type=int, default=1024)
    ap.add_argument("--num-of-experts", type=int, default=32)
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--rounds", type=int, default=3)
    args = ap.parse_args()
    rank, world, _ = D.init_distributed()
    group, ep_rank, _ = D.create_ep_group(args.ep)
    dev = torch.device("cuda", torch.cuda.current_device())
    T, H, E, K = args.num_local_tokens + 16 * ep_rank, args.token_hidden, args.num_of_experts, args.topk
    cfg = Buffer.get_dispatch_config(args.ep, args.num_local_tokens + 16 * args.ep, K, E,
                                     group_by_expert=True)  # same on every rank
    buf = Buffer(group, cfg.get_nvl_buffer_size_hint(H * 2, args.ep), 0, timeout_s=10.0)
    oracle = AllToAllTokenDispatcher(group, E)
    ok = True
    msgs = []
    for rnd in range(args.rounds):
        g = torch.Generator().manual_seed(17 * rnd + rank)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        idx, w = make_routing(T, E, K, seed=1000 * rnd + rank, zipf_s=1.2 if rnd % 2 else 0.0)
        idx, w = idx.to(dev), w.to(dev)
        rows_ref, probs_ref, cnt_ref = oracle.dispatch(x, idx, w)
        out_ref = oracle.combine((rows_ref.float() * probs_ref[:, None]).to(torch.bfloat16))
        # expert-grouped mode: must equal the oracle row for row
        rx, _, _, cnt, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, group_by_expert=True,
                                          num_experts=E)
        e1 = cnt == cnt_ref and torch.equal(rx, rows_ref) and torch.equal(h.recv_prob, probs_ref)
        y = (rx.float() * h.recv_prob[:, None]).to(torch.bfloat16)
        out, _, _ = buf.combine(y, h)
        e2 = torch.allclose(out.float(), out_ref.float(), atol=3e-2, rtol=2e-2)
        # rank mode: identity expert returns x * (#destination ranks); counts equal the oracle's
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        rx2, ridx, rw, cnt2, h2, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=pr,
                                                 is_token_in_rank=inr, num_tokens_per_expert=pe)
        e3 = cnt2 == cnt_ref and rx2.shape[0] == h2.n_recv
        El = E // args.ep
        e3 = e3 and bool(((ridx >= -1) & (ridx < El)).all()) and \
            torch.bincount(ridx[ridx >= 0], minlength=El).tolist() == cnt_ref
        out2, _, _ = buf.combine(rx2, h2)
        e4 = torch.allclose(out2.float(), x.float() * inr.sum(1, keepdim=True).float(), atol=0.13, rtol=2e-2)
        # cached dispatch + fp8
        rx3, *_ = buf.dispatch(x * 2, handle=h2)
        e5 = torch.equal(rx3, rx2 * 2)
        (q, s), *_ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=pr,
                                  is_token_in_rank=inr, num_tokens_per_expert=pe, use_fp8=True)
        deq = (q.float().view(q.shape[0], H // 128, 128) * s[..., None]).view(q.shape[0], H)
        e6 = torch.allclose(deq, rx2.float(), atol=0.3, rtol=0.07)
        buf.check_status()
        good = all((e1, e2, e3, e4, e5, e6))
        ok = ok and good
        msgs.append(f"[rank {rank}] round {rnd}: expert_rows={e1} expert_combine={e2} rank_counts={e3} "
                    f"rank_combine={e4} cached={e5} fp8={e6} n_recv={h2.n_recv}")
    D.ordered_print("\n".join(msgs))
    all_ok = D.all_ranks_boolean(ok)
    if rank == 0:
        print("ALL OK" if all_ok else "CHECK FAILED", flush=True)
    buf.destroy()
    D.shutdown()
    return 0 if all_ok else 2


if __name__ == "__main__":
    D.run_main(main)
