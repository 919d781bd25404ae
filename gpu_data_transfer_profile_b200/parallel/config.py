"""Sizing hints and tuning knobs (`Buffer.get_dispatch_config` / `get_combine_config`).

Parity: the reference sizes its buffer as the max over the dispatch and combine configs of
`get_nvl_buffer_size_hint(hidden_bytes, group_size)` / `get_rdma_buffer_size_hint(...)`
(`DeepEP_v1/deepep_v1_dispatch.py:35-56`). This library stores every token directly in its
final row of the receiver's region, so the region is sized for the worst case
(every token of every rank lands on one rank) instead of for a ring of chunks; the
config therefore also carries the token bound that the hint is computed for.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..utils.sizes import align_up

FIXED_BYTES = 1 << 20          # flags + count matrices + low-latency control words
REGION_ALIGN = 1024


@dataclass
class Config:
    num_sms: int = 24
    num_max_tokens_per_rank: int = 4096
    num_topk: int = 8
    num_experts: int = 256
    combine_elem_bytes: int = 2
    group_by_expert: bool = False   # size for one row per (token, expert) instead of per (token, rank)
    # Optional bound on the rows one rank can RECEIVE per dispatch (0 = worst case: every token of
    # every rank lands here). A routing that exceeds the bound ends in status 6 (receive overflow),
    # never in an out-of-range store. Pass the same value to `Buffer(num_max_recv_tokens=...)`.
    num_max_recv_tokens: int = 0
    # False: reserve no combine slots. Combine is then only possible in its pull form (rows read in
    # place from the producers' receive regions), which needs no slots; the region is about half
    # the size. Pass the same value to `Buffer(combine_slots=...)`.
    combine_slots: bool = True

    def per_row_bytes(self, hidden_bytes: int) -> int:
        """Bytes that one receive row plus one combine slot occupy (all side arrays)."""
        k = self.num_topk
        hidden_elems = max(hidden_bytes // 2, 1)
        scales = ((hidden_elems + 127) // 128) * 4
        recv = hidden_bytes + scales + k * 8 + k * 4 + 8 + 4
        comb = (hidden_elems * max(self.combine_elem_bytes, 2) + k * 4) if self.combine_slots else 0
        return align_up(recv, 16) + align_up(comb, 16) + 64

    def get_nvl_buffer_size_hint(self, hidden_bytes: int, group_size: int) -> int:
        rows = group_size * self.num_max_tokens_per_rank
        if self.group_by_expert:
            # worst case: every token of every rank picks min(top-k, local experts) experts here
            rows *= max(1, min(self.num_topk, max(self.num_experts // group_size, 1)))
        if self.num_max_recv_tokens > 0:
            rows = min(rows, self.num_max_recv_tokens)
        body = 2 * rows * self.per_row_bytes(hidden_bytes)  # two epoch parities
        return FIXED_BYTES + align_up(body, REGION_ALIGN) + 16 * REGION_ALIGN * 2

    def get_rdma_buffer_size_hint(self, hidden_bytes: int, group_size: int) -> int:
        """Inter-node transport is outside a single NVLink domain: accepted, always 0."""
        return 0
