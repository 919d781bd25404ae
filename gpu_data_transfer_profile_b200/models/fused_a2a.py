"""Autograd wrappers that make dispatch and combine each other's backward.

Parity: `FusedDispatch` / `FusedCombine` / `fused_dispatch()` / `fused_combine()` /
`get_deepep_buffer` of `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:57-249`
(forward of dispatch = layout + dispatch, its backward = combine that also reduces the
routing-weight gradients, `:146-168`; forward of combine = combine, its backward = dispatch
with the cached handle, `:195-209`). The reference defines these but never runs a backward
pass; here both directions are exercised by tests.

`FusedDispatchGrouped` / `FusedCombineGrouped` are the expert-grouped forms: rows arrive
already sorted by local expert, so the multihot/permute/unpermute glue of the reference
(`:276-403`) has no counterpart.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..parallel.buffer import Buffer
from ..parallel.events import EventHandle, EventOverlap

_BUFFERS: Dict[Tuple[int, int], Buffer] = {}
_DEFAULTS = dict(num_max_tokens_per_rank=4096, num_topk=8, num_experts=256, group_by_expert=False)


def configure_buffer(**kw) -> None:
    """Bounds used to size the shared buffer (tokens per rank, top-k, experts, grouping)."""
    _DEFAULTS.update(kw)


def get_hidden_bytes(x: torch.Tensor) -> int:
    return x.shape[1] * max(x.element_size(), 2)


def get_buffer(group, hidden_bytes: int, world=None) -> Buffer:
    """One cached `Buffer` per (group, world); re-created when a larger one is needed."""
    key = (id(group), id(world))
    size = world.size if world is not None else torch.distributed.get_world_size(group)
    need = 0
    for cfg in (Buffer.get_dispatch_config(size, **_DEFAULTS), Buffer.get_combine_config(size, **_DEFAULTS)):
        need = max(need, cfg.get_nvl_buffer_size_hint(hidden_bytes, size))
    buf = _BUFFERS.get(key)
    if buf is None or buf.num_nvl_bytes < need:
        if buf is not None:
            buf.destroy()
        buf = Buffer(group, need, 0, world=world)
        _BUFFERS[key] = buf
    return buf


def set_buffer(group, buf: Buffer, world=None) -> None:
    _BUFFERS[(id(group), id(world))] = buf


def release_buffers() -> None:
    for b in _BUFFERS.values():
        b.destroy()
    _BUFFERS.clear()


get_deepep_buffer = get_buffer


def _seed(async_finish: bool) -> Optional[EventOverlap]:
    return EventOverlap(EventHandle()) if async_finish else None


class FusedDispatch(torch.autograd.Function):
    """Rank-mode dispatch (DeepEP layout). Returns
    (recv_x, recv_token_indices, recv_token_probs, tokens_per_expert[int64 cpu], handle)."""

    @staticmethod
    def forward(ctx, x, token_indices, token_probs, num_experts, group, async_finish=False,
                allocate_on_comm_stream=False, world=None):
        buf = get_buffer(group, get_hidden_bytes(x), world)
        prev = _seed(async_finish)
        per_rank, per_rdma, per_expert, in_rank, ev = buf.get_dispatch_layout(
            token_indices, num_experts, previous_event=prev, async_finish=async_finish,
            allocate_on_comm_stream=allocate_on_comm_stream)
        recv_x, recv_idx, recv_probs, per_local, handle, after = buf.dispatch(
            x, topk_idx=token_indices, topk_weights=token_probs, num_tokens_per_rank=per_rank,
            num_tokens_per_rdma_rank=per_rdma, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
            previous_event=ev, async_finish=async_finish, allocate_on_comm_stream=allocate_on_comm_stream)
        if async_finish:
            after.current_stream_wait()
        ctx.buf, ctx.handle = buf, handle
        ctx.async_finish, ctx.alloc = async_finish, allocate_on_comm_stream
        tokens_per_expert = (per_local.detach().cpu().to(torch.int64) if torch.is_tensor(per_local)
                             else torch.tensor(per_local, dtype=torch.int64))
        ctx.mark_non_differentiable(recv_idx, tokens_per_expert)
        return recv_x, recv_idx, recv_probs, tokens_per_expert, handle

    @staticmethod
    def backward(ctx, grad_x, _gi, grad_probs, _gt, _gh):
        tw = grad_probs.float().contiguous() if grad_probs is not None else None
        gx, gw, after = ctx.buf.combine(grad_x.contiguous(), ctx.handle, topk_weights=tw,
                                        previous_event=_seed(ctx.async_finish), async_finish=ctx.async_finish,
                                        allocate_on_comm_stream=ctx.alloc)
        if ctx.async_finish:
            after.current_stream_wait()
        return gx, None, gw, None, None, None, None, None


class FusedCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, handle, async_finish=False, allocate_on_comm_stream=False, world=None):
        buf = get_buffer(group, get_hidden_bytes(x), world)
        out, _, after = buf.combine(x, handle, previous_event=_seed(async_finish), async_finish=async_finish,
                                    allocate_on_comm_stream=allocate_on_comm_stream)
        if async_finish:
            after.current_stream_wait()
        ctx.buf, ctx.handle = buf, handle
        ctx.async_finish, ctx.alloc = async_finish, allocate_on_comm_stream
        return out

    @staticmethod
    def backward(ctx, grad_out):
        gx, *_rest, after = ctx.buf.dispatch(grad_out.contiguous(), handle=ctx.handle,
                                             previous_event=_seed(ctx.async_finish),
                                             async_finish=ctx.async_finish, allocate_on_comm_stream=ctx.alloc)
        if ctx.async_finish:
            after.current_stream_wait()
        return gx, None, None, None, None, None


def fused_dispatch(x, token_indices, token_probs, num_experts, group, async_finish=False,
                   allocate_on_comm_stream=False, world=None):
    return FusedDispatch.apply(x.contiguous(), token_indices.contiguous(), token_probs.contiguous().float(),
                               num_experts, group, async_finish, allocate_on_comm_stream, world)


def fused_combine(x, group, handle, async_finish=False, allocate_on_comm_stream=False, world=None):
    return FusedCombine.apply(x.contiguous(), group, handle, async_finish, allocate_on_comm_stream, world), None


class FusedDispatchGrouped(torch.autograd.Function):
    """Expert-grouped dispatch: (rows[N,H] sorted by local expert, row_probs[N],
    tokens_per_expert[int64 cpu], handle)."""

    @staticmethod
    def forward(ctx, x, token_indices, token_probs, num_experts, group, world=None):
        buf = get_buffer(group, get_hidden_bytes(x), world)
        rows, _, _, per_local, handle, _ = buf.dispatch(
            x, topk_idx=token_indices, topk_weights=token_probs, group_by_expert=True, num_experts=num_experts)
        ctx.buf, ctx.handle = buf, handle
        tpe = torch.tensor(per_local, dtype=torch.int64)
        ctx.mark_non_differentiable(tpe)
        return rows, handle.recv_prob, tpe, handle

    @staticmethod
    def backward(ctx, grad_rows, grad_row_probs, _gt, _gh):
        side = grad_row_probs.float().contiguous() if grad_row_probs is not None else None
        gx, gw, _ = ctx.buf.combine(grad_rows.contiguous(), ctx.handle, topk_weights=side)
        return gx, None, gw, None, None, None


class FusedCombineGrouped(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, group, handle, world=None):
        buf = get_buffer(group, get_hidden_bytes(rows), world)
        out, _, _ = buf.combine(rows, handle)
        ctx.buf, ctx.handle = buf, handle
        return out

    @staticmethod
    def backward(ctx, grad_out):
        g_rows, *_ = ctx.buf.dispatch(grad_out.contiguous(), handle=ctx.handle)
        return g_rows, None, None, None
