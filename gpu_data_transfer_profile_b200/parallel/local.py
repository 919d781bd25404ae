"""Lock-step driver for several virtual ranks on ONE GPU (`LocalWorld`).

A kernel that waits for a peer must not run concurrently with, or before, the kernel it waits
for when both share a GPU. The driver therefore runs phase k of every virtual rank before
phase k+1 of any rank, on one stream, so every wait finds its flag already set.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .buffer import Buffer
from .symm import LocalWorld


class LocalGroup:
    def __init__(self, size: int, num_nvl_bytes: int, device: Optional[torch.device] = None,
                 timeout_s: float = 2.0):
        self.size = size
        worlds = LocalWorld.make(size, device)
        self.buffers: List[Buffer] = [Buffer(None, num_nvl_bytes, world=w, timeout_s=timeout_s)
                                      for w in worlds]

    def get_dispatch_layout(self, topk_idx: Sequence[torch.Tensor], num_experts: int):
        return [b.get_dispatch_layout(t, num_experts) for b, t in zip(self.buffers, topk_idx)]

    def dispatch(self, xs, *, handles=None, layouts=None, topk_idx=None, topk_weights=None,
                 use_fp8=False, group_by_expert=False, zero_copy=False, num_experts=0):
        n = self.size
        sts = []
        for r, b in enumerate(self.buffers):
            lay = layouts[r] if layouts is not None else (None, None, None, None, None)
            sts.append(b._dispatch_p1(
                xs[r], handles[r] if handles is not None else None, lay[3], lay[2],
                topk_idx[r] if topk_idx is not None else None,
                topk_weights[r] if topk_weights is not None else None,
                use_fp8, group_by_expert, num_experts))
        for r, b in enumerate(self.buffers):
            b._dispatch_p2(sts[r])
        return [b._dispatch_p3(sts[r], zero_copy) for r, b in enumerate(self.buffers)]

    def combine(self, ys, handles, topk_weights=None, item_weights=None):
        tw = lambda r: topk_weights[r] if topk_weights is not None else None
        if all(b._use_pull(ys[r], tw(r)) for r, b in enumerate(self.buffers)):
            # rows stay in their producers' regions: every rank announces, then every rank pulls
            for r, b in enumerate(self.buffers):
                b._combine_pull(1, ys[r], handles[r], tw(r))
            return [b._combine_pull(2, ys[r], handles[r], tw(r),
                                    item_weights[r] if item_weights is not None else None)
                    for r, b in enumerate(self.buffers)]
        sts = [b._combine_p1(ys[r], handles[r], topk_weights[r] if topk_weights is not None else None)
               for r, b in enumerate(self.buffers)]
        return [b._combine_p2(sts[r], handles[r], item_weights[r] if item_weights is not None else None)
                for r, b in enumerate(self.buffers)]

    def fused_fc2_combine(self, acts, w2s, handles, item_weights=None):
        """fc2 GEMMs whose epilogues store into the other virtual ranks' slots (all ranks first),
        then every rank's reduction."""
        sts = [b._fused_fc2_send(acts[r], w2s[r], handles[r]) for r, b in enumerate(self.buffers)]
        return [b._combine_p2(sts[r], handles[r], item_weights[r] if item_weights is not None else None)[0]
                for r, b in enumerate(self.buffers)]

    def low_latency_dispatch(self, xs, topk_idx, num_max_tokens: int, num_experts: int, use_fp8=True):
        for r, b in enumerate(self.buffers):     # every virtual rank prepares its regions before anyone sends
            b._ll_state(num_experts, topk_idx[r].shape[1], xs[r].shape[1], num_max_tokens)
        ds = [b._ll_dispatch_send(xs[r], topk_idx[r], num_max_tokens, num_experts, use_fp8)
              for r, b in enumerate(self.buffers)]
        return [b._ll_dispatch_recv(ds[r]) for r, b in enumerate(self.buffers)]

    def low_latency_combine(self, ys, topk_idx, topk_weights, handles):
        if all(b._ll_is_combine_buffer(ys[r], handles[r]) for r, b in enumerate(self.buffers)):
            for r, b in enumerate(self.buffers):            # every rank announces, then every rank pulls
                b._ll_combine_pull(1, topk_idx[r], topk_weights[r], handles[r])
            return [b._ll_combine_pull(2, topk_idx[r], topk_weights[r], handles[r])
                    for r, b in enumerate(self.buffers)]
        cs = [b._ll_combine_send(ys[r], handles[r]) for r, b in enumerate(self.buffers)]
        return [b._ll_combine_recv(cs[r], topk_idx[r], topk_weights[r]) for r, b in enumerate(self.buffers)]

    def check_status(self):
        for b in self.buffers:
            b.check_status()

    def check_canaries(self):
        for b in self.buffers:
            b.check_canaries()

    def destroy(self):
        for b in self.buffers:
            b.destroy()
