"""A Megatron-style MoE layer: router -> dispatch -> grouped experts -> combine.

The reference's "model" is exactly this loop with a random router stand-in
(`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:731-742,766-815`); here it is an
`nn.Module` with a learnable router so that forward AND backward run (dispatch and combine
are each other's backward, expert GEMMs have dgrad/wgrad).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .experts import build_experts
from .token_dispatcher import B200TokenDispatcher


def topk_softmax_router(logits: torch.Tensor, topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(indices int64 [T,K], probabilities f32 [T,K] renormalised over the chosen experts)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, topk, dim=-1)
    return idx, w / w.sum(-1, keepdim=True)


class MoELayer(torch.nn.Module):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, num_experts: int, topk: int, group=None, *,
                 ep_size: int = 1, ep_rank: int = 0, dtype=torch.bfloat16, activation: str = "swiglu",
                 expert_backend: str = "auto", dispatcher_mode: str = "fused", world=None, device="cuda",
                 fuse_combine: bool = True, use_fp8: bool = False):
        super().__init__()
        if num_experts % ep_size:
            raise ValueError("num_experts must be divisible by the EP size")
        self.hidden_size, self.num_experts, self.topk = hidden_size, num_experts, topk
        self.fuse_combine = fuse_combine
        self.num_local_experts = num_experts // ep_size
        self.router = torch.nn.Linear(hidden_size, num_experts, bias=False, dtype=torch.float32, device=device)
        torch.nn.init.normal_(self.router.weight, std=0.02)
        self.experts, self.expert_backend = build_experts(expert_backend, self.num_local_experts, hidden_size,
                                                          ffn_hidden_size, dtype, activation, device, use_fp8=use_fp8)
        # fp8 inference path: e4m3 rows with 1x128 scales leave the dispatch kernel and feed the
        # block-scaled fp8 fc1 directly (no dequantisation pass); training stays bf16
        self.use_fp8 = bool(use_fp8) and getattr(self.experts, "use_fp8", False)
        self.dispatcher = B200TokenDispatcher(group, self.num_local_experts, num_experts,
                                              ep_rank * self.num_local_experts, mode=dispatcher_mode, world=world)

    def forward(self, hidden_states: torch.Tensor, router_logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """hidden_states [T,H]; router_logits [T,E] override the learnable router when given."""
        if router_logits is None:
            router_logits = self.router(hidden_states.float())
        idx, probs = topk_softmax_router(router_logits, self.topk)
        if self.use_fp8 and not torch.is_grad_enabled() and self.dispatcher.mode == "fused":
            rows, tokens_per_expert, row_probs = self.dispatcher.dispatch_fp8(hidden_states, idx, probs)
            El = self.num_local_experts
            off = self.dispatcher.handle.meta[2 + El: 2 + El + El + 1]
            return self.dispatcher.combine(self.experts.forward_fp8(rows, tokens_per_expert, row_probs, expert_off=off))
        rows, tokens_per_expert, row_probs = self.dispatcher.dispatch(hidden_states, idx, probs)
        if (self.fuse_combine and self.dispatcher.mode == "fused" and hasattr(self.experts, "forward_fused_combine")
                and (not torch.is_grad_enabled() or self.experts.activation == "swiglu")):
            # the fc2 epilogue stores straight into the source ranks' slots (no combine-send kernel)
            from . import fused_a2a as A
            buf = A.get_buffer(self.dispatcher.group, A.get_hidden_bytes(hidden_states), self.dispatcher.world)
            handle = self.dispatcher.handle
            self.dispatcher.handle = None
            if torch.is_grad_enabled():
                return self.experts.forward_fused_combine_train(rows, tokens_per_expert, row_probs, buf, handle)
            return self.experts.forward_fused_combine(rows, row_probs, buf, handle)
        out_rows = self.experts(rows, tokens_per_expert, row_probs)
        return self.dispatcher.combine(out_rows)
