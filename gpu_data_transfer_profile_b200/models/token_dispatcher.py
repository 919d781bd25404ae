"""Megatron-style MoE token dispatcher hooks on top of `Buffer`.

Parity: `DeepepDispatchCombineManager` of
`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:252-453`:
`dispatch(hidden, token_indices, token_probs) -> (rows grouped by local expert,
tokens_per_expert, one probability per row)` and `combine(rows) -> hidden`.

Two flavours share that interface:
  * `mode="fused"` (default): the expert-grouped dispatch kernel delivers rows already
    sorted by local expert, and combine returns them from that order; there is no
    multihot, permute or unpermute step and no extra host synchronisation.
  * `mode="deepep"`: rank-mode dispatch (one row per token and rank) followed by the
    reference's local glue, restated with sort-based PyTorch ops: multihot
    (`:276-338`), permute (`:340-388`), unpermute via index_add_ (`:390-403`). Kept as the
    behavioural twin of the reference path and as a cross-check of the fused one.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import fused_a2a as A


class B200TokenDispatcher:
    def __init__(self, group, num_local_experts: int, num_experts: int, local_expert_start: int,
                 async_finish: bool = False, allocate_on_comm_stream: bool = False,
                 mode: str = "fused", world=None):
        if mode not in ("fused", "deepep"):
            raise ValueError("mode must be 'fused' or 'deepep'")
        self.group, self.world = group, world
        self.num_local_experts = num_local_experts
        self.num_experts = num_experts
        self.local_expert_start = local_expert_start
        self.async_finish = async_finish
        self.allocate_on_comm_stream = allocate_on_comm_stream
        self.mode = mode
        self.handle = None
        self.dispatched_probs: Optional[torch.Tensor] = None
        self.tokens_per_expert: Optional[torch.Tensor] = None
        self._n_before_permute: Optional[int] = None
        self._reverse_map: Optional[torch.Tensor] = None

    # ---- reference-style local glue (mode="deepep") -----------------------------------
    def _indices_to_multihot(self, indices: torch.Tensor, probs: torch.Tensor,
                             expected: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """[N,K] ids + probs -> bool/f32 maps [N, E_local]. Accepts local ids (-1 elsewhere) or
        global ids and keeps the convention whose column counts equal `expected`."""
        if indices.dim() == 1:
            indices, probs = indices[:, None], probs[:, None]
        n, El = indices.shape[0], self.num_local_experts
        lo = self.local_expert_start
        exp = expected.to(torch.int64).cpu()

        def build(local, valid):
            rmap = torch.zeros((n, El), dtype=torch.bool, device=indices.device)
            pmap = torch.zeros((n, El), dtype=torch.float32, device=indices.device)
            rows = torch.arange(n, device=indices.device)[:, None].expand_as(local)
            rmap[rows[valid], local[valid]] = True
            pmap[rows[valid], local[valid]] = probs.float()[valid]
            return rmap, pmap

        cands = [(indices, (indices >= 0) & (indices < El)),
                 (indices - lo, (indices >= lo) & (indices < lo + El))]
        for local, valid in cands:
            rmap, pmap = build(local.clamp(0, El - 1), valid)
            if torch.equal(rmap.sum(0).cpu(), exp):
                return rmap, pmap
        raise RuntimeError("dispatched expert ids match neither the local nor the global convention")

    def _permute_to_local_experts(self, hidden, indices, probs, tokens_per_expert):
        rmap, pmap = self._indices_to_multihot(indices, probs, tokens_per_expert)
        # rows of expert 0 first, then expert 1, ...; token order inside an expert
        e_idx, t_idx = rmap.t().nonzero(as_tuple=True)
        self._n_before_permute = hidden.shape[0]
        self._reverse_map = t_idx
        counts = rmap.sum(0).to(torch.int64).cpu()
        if int(counts.sum()) != t_idx.numel():
            raise RuntimeError("inconsistent expert counts after permutation")
        return hidden.index_select(0, t_idx), counts, pmap.t()[e_idx, t_idx]

    def _unpermute_from_local_experts(self, hidden):
        out = torch.zeros((self._n_before_permute, hidden.shape[1]), dtype=hidden.dtype, device=hidden.device)
        out.index_add_(0, self._reverse_map, hidden)
        self._n_before_permute = self._reverse_map = None
        return out

    # ---- hooks ------------------------------------------------------------------------
    def dispatch(self, hidden_states, token_indices, token_probs):
        if self.mode == "fused":
            rows, row_probs, tpe, handle = A.FusedDispatchGrouped.apply(
                hidden_states.contiguous(), token_indices.contiguous(), token_probs.contiguous().float(),
                self.num_experts, self.group, self.world)
        else:
            rows, d_idx, d_probs, tpe, handle = A.fused_dispatch(
                hidden_states, token_indices, token_probs, self.num_experts, self.group,
                self.async_finish, self.allocate_on_comm_stream, self.world)
            if tpe.numel() != self.num_local_experts:
                raise RuntimeError(f"tokens_per_expert has length {tpe.numel()}, expected {self.num_local_experts}")
            rows, tpe, row_probs = self._permute_to_local_experts(rows, d_idx, d_probs, tpe)
        if tpe.numel() != self.num_local_experts:
            raise RuntimeError(f"tokens_per_expert has length {tpe.numel()}, expected {self.num_local_experts}")
        self.handle, self.tokens_per_expert, self.dispatched_probs = handle, tpe, row_probs
        return rows, tpe, row_probs

    @torch.no_grad()
    def dispatch_fp8(self, hidden_states, token_indices, token_probs):
        """Forward-only, fused mode: the dispatch kernel casts every row to e4m3 with one f32 scale
        per 128 channels on its way out. Returns ((rows e4m3 [N,H], scales f32 [N,H/128]),
        tokens_per_expert, one probability per row); `combine` then takes the experts' bf16 output."""
        if self.mode != "fused":
            raise ValueError("fp8 dispatch is offered by the fused (expert-grouped) dispatcher")
        buf = A.get_buffer(self.group, A.get_hidden_bytes(hidden_states), self.world)
        rows, _, _, per_local, handle, _ = buf.dispatch(
            hidden_states.contiguous(), topk_idx=token_indices.contiguous(), topk_weights=token_probs.contiguous().float(),
            group_by_expert=True, num_experts=self.num_experts, use_fp8=True)
        tpe = torch.tensor(per_local, dtype=torch.int64)
        self.handle, self.tokens_per_expert, self.dispatched_probs = handle, tpe, handle.recv_prob
        return rows, tpe, handle.recv_prob

    def combine(self, hidden_states):
        if self.handle is None:
            raise RuntimeError("combine() called before dispatch()")
        if self.mode == "fused":
            out = A.FusedCombineGrouped.apply(hidden_states.contiguous(), self.group, self.handle, self.world)
        else:
            hidden_states = self._unpermute_from_local_experts(hidden_states)
            out, _ = A.fused_combine(hidden_states, self.group, self.handle, self.async_finish,
                                     self.allocate_on_comm_stream, self.world)
        self.handle = self.dispatched_probs = self.tokens_per_expert = None
        return out


DeepepDispatchCombineManager = B200TokenDispatcher
