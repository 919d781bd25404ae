"""fp32 PyTorch oracles for the EP kernels. No CUDA, no native code.

Two forms:
* list-based, single process: every argument is a list with one entry per rank. Used to
  check the GPU kernels (whole tensors, exact for bf16 payload copies).
* `AllToAllTokenDispatcher`: a real multi-process dispatcher built on
  `torch.distributed.all_to_all_single` (gloo on CPU, NCCL on GPU). It is the correctness
  oracle of the world_size=2 CPU test and, on GPUs, the measured NCCL comparator
  (standard "alltoall" MoE token-dispatcher semantics: sort by expert, exchange counts,
  exchange rows, regroup by local expert).

Row orders are the ones the kernels produce:
  rank mode   : rows sorted by (source rank, token index)
  expert mode : rows sorted by (local expert, source rank, token index, k)
Semantics being reproduced: `DeepEP_v1/deepep_v1_dispatch.py:199-230` (dispatch outputs),
`DeepEP_v1/deepep_v1_combine.py:335-342` (combine = unweighted sum over destination ranks),
`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:276-403` (permute / unpermute).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def make_routing(num_tokens: int, num_experts: int, topk: int, seed: int,
                 zipf_s: float = 0.0, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """Seeded router stand-in: top-k of softmax(N(0,1) logits [+ Zipf(s) expert bias]).
    Returns (topk_idx int64 [T,K], topk_weights f32 [T,K], rows normalised to 1)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    logits = torch.randn(num_tokens, num_experts, generator=g)
    if zipf_s > 0:
        ranks = torch.arange(1, num_experts + 1, dtype=torch.float32)
        perm = torch.randperm(num_experts, generator=torch.Generator().manual_seed(seed // 7 + 3))
        bias = torch.empty(num_experts)
        bias[perm] = -zipf_s * torch.log(ranks)
        gumbel = -torch.log(-torch.log(torch.rand(num_tokens, num_experts, generator=g).clamp_min(1e-9)))
        logits = bias[None, :] + gumbel       # top-k of this = sampling w/o replacement ~ Zipf(s)
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, topk, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).to(torch.float32)
    return idx.to(torch.int64).to(device), w.to(device)


def layout_ref(topk_idx: torch.Tensor, num_experts: int, num_ranks: int):
    """(num_tokens_per_rank[R], num_tokens_per_expert[E], is_token_in_rank[T,R])."""
    T, K = topk_idx.shape
    El = num_experts // num_ranks
    valid = topk_idx >= 0
    per_expert = torch.bincount(topk_idx[valid].flatten(), minlength=num_experts).to(torch.int32)
    in_rank = torch.zeros(T, num_ranks, dtype=torch.bool)
    r = torch.where(valid, topk_idx // El, torch.zeros_like(topk_idx))
    for k in range(K):
        in_rank[torch.arange(T)[valid[:, k]], r[valid[:, k], k]] = True
    per_rank = in_rank.sum(0).to(torch.int32)
    return per_rank, per_expert, in_rank


def dispatch_rank_mode_ref(xs: Sequence[torch.Tensor], idxs: Sequence[torch.Tensor],
                           ws: Sequence[torch.Tensor], num_experts: int):
    """Per destination rank: (recv_x, recv_topk_idx(local, -1 elsewhere), recv_topk_w, src_rank,
    src_token, per-local-expert counts)."""
    R = len(xs)
    El = num_experts // R
    out = []
    for d in range(R):
        rx, ri, rw, sr, stok = [], [], [], [], []
        for s in range(R):
            idx, w = idxs[s], ws[s]
            hit = ((idx >= d * El) & (idx < (d + 1) * El))
            sel = hit.any(1).nonzero().flatten()
            rx.append(xs[s][sel])
            li = torch.where(hit[sel], idx[sel] - d * El, torch.full_like(idx[sel], -1))
            ri.append(li)
            rw.append(torch.where(hit[sel], w[sel], torch.zeros_like(w[sel])))
            sr.append(torch.full((sel.numel(),), s, dtype=torch.int64))
            stok.append(sel)
        ri_c = torch.cat(ri)
        cnt = torch.bincount(ri_c[ri_c >= 0].flatten(), minlength=El).tolist()
        out.append((torch.cat(rx), ri_c, torch.cat(rw), torch.cat(sr), torch.cat(stok), cnt))
    return out


def dispatch_expert_mode_ref(xs, idxs, ws, num_experts: int):
    """Per destination rank: (recv_x, recv_prob, src_rank, src_token, src_k, counts per local expert);
    rows sorted by (local expert, source rank, token, k)."""
    R = len(xs)
    El = num_experts // R
    out = []
    for d in range(R):
        rx, rp, sr, stok, sk, cnt = [], [], [], [], [], []
        for e in range(d * El, (d + 1) * El):
            n_e = 0
            for s in range(R):
                t, k = (idxs[s] == e).nonzero(as_tuple=True)   # row-major order = (token, k)
                rx.append(xs[s][t])
                rp.append(ws[s][t, k])
                sr.append(torch.full((t.numel(),), s, dtype=torch.int64))
                stok.append(t)
                sk.append(k)
                n_e += t.numel()
            cnt.append(n_e)
        out.append((torch.cat(rx), torch.cat(rp), torch.cat(sr), torch.cat(stok), torch.cat(sk), cnt))
    return out


def combine_ref(ys: Sequence[torch.Tensor], src_rank: Sequence[torch.Tensor],
                src_token: Sequence[torch.Tensor], num_tokens: Sequence[int],
                row_weight: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
    """ys[d] are the rows held by rank d (same order as the dispatch oracle's output); returns
    for every source rank the fp32 sum of its returned rows (optionally weighted per row)."""
    R = len(ys)
    H = ys[0].shape[1]
    outs = [torch.zeros(num_tokens[s], H, dtype=torch.float32) for s in range(R)]
    for d in range(R):
        y = ys[d].to(torch.float32)
        if row_weight is not None:
            y = y * row_weight[d].to(torch.float32)[:, None]
        for s in range(R):
            m = src_rank[d] == s
            outs[s].index_add_(0, src_token[d][m], y[m])
    return outs


def fp8_block_quant_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """1x128 block scaling to e4m3: returns (q fp8 [T,H], scales f32 [T,H/128])."""
    T, H = x.shape
    xf = x.to(torch.float32).view(T, H // 128, 128)
    amax = xf.abs().amax(-1).clamp_min(1e-4)
    q = (xf * (448.0 / amax)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(T, H)
    return q, amax / 448.0


def fp8_block_dequant_ref(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    T, H = q.shape
    return (q.to(torch.float32).view(T, H // 128, 128) * scales[..., None]).view(T, H)


class AllToAllTokenDispatcher:
    """MoE token dispatcher over `all_to_all_single` (works on gloo/CPU and NCCL/GPU).

    dispatch(x[T,H], topk_idx[T,K], topk_w[T,K]) ->
        rows[N,H] grouped by local expert, probs[N], tokens_per_local_expert (list[int])
    combine(y[N,H]) -> out[T,H] = sum over the token's (expert) rows (weights already applied
    by the caller, as in the Megatron path, or pass weighted=True to apply them here).
    """

    def __init__(self, group, num_experts: int):
        self.group = group
        self.R = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E = num_experts
        self.El = num_experts // self.R

    def dispatch(self, x, topk_idx, topk_w):
        T, K = topk_idx.shape
        R, El = self.R, self.El
        flat_e = topk_idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)              # (expert, token, k)
        self._order, self._T, self._K = order, T, K
        tok = order // K
        send = x[tok].contiguous()
        send_p = topk_w.reshape(-1)[order].contiguous()
        cnt_e = torch.bincount(flat_e, minlength=self.E)        # tokens per global expert
        recv_cnt_e = torch.empty_like(cnt_e)
        dist.all_to_all_single(recv_cnt_e, cnt_e, group=self.group)   # [R, El] from every source
        self._in_split = cnt_e.view(R, El).sum(1).tolist()
        self._out_split = recv_cnt_e.view(R, El).sum(1).tolist()
        recv = x.new_empty((sum(self._out_split), x.shape[1]))
        recv_p = send_p.new_empty(sum(self._out_split))
        dist.all_to_all_single(recv, send, self._out_split, self._in_split, group=self.group)
        dist.all_to_all_single(recv_p, send_p, self._out_split, self._in_split, group=self.group)
        # received order is (source, local expert, ...); regroup to (local expert, source, ...)
        per = recv_cnt_e.view(R, El)
        seg_expert = torch.arange(El, device=x.device).repeat(R)
        seg_len = per.reshape(-1)
        row_expert = torch.repeat_interleave(seg_expert, seg_len)
        regroup = torch.argsort(row_expert, stable=True)
        self._regroup = regroup
        return recv[regroup], recv_p[regroup], per.sum(0).tolist()

    def combine(self, y, weights: Optional[torch.Tensor] = None):
        inv = torch.empty_like(self._regroup)
        inv[self._regroup] = torch.arange(self._regroup.numel(), device=y.device)
        back_src = y[inv].contiguous()
        back = y.new_empty((sum(self._in_split), y.shape[1]))
        dist.all_to_all_single(back, back_src, self._in_split, self._out_split, group=self.group)
        out = torch.zeros((self._T, y.shape[1]), dtype=torch.float32, device=y.device)
        tok = self._order // self._K
        contrib = back.to(torch.float32)
        if weights is not None:
            contrib = contrib * weights.reshape(-1)[self._order].to(torch.float32)[:, None]
        out.index_add_(0, tok, contrib)
        return out.to(y.dtype)
