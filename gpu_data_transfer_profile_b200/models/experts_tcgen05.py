"""Grouped expert MLP on this library's tcgen05 kernels.

Forward: fc1 with SwiGLU x probability fused into its epilogue (one kernel), fc2 either as a
plain grouped GEMM or with the combine send fused into its epilogue (`forward_fused_combine`).
Tile scheduling reads the per-expert row offsets on the device. Backward (SwiGLU path): the two
data gradients run on the same grouped GEMM reading the forward weights in place as an N-major
operand, the two weight gradients on the ragged-reduction kernel (`ops.gemm.grouped_wgrad`), the
element-wise part on the fused SwiGLU backward kernel; no library GEMM and no host-side split.
gelu / silu / relu (`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:516-526`) take the same
route with the ungated activation kernels of csrc/gemm/swiglu.cu.
"""
from __future__ import annotations

import torch

from ..ops import gemm as G
from .experts import GroupedExpertsBase


def _wgrad(dy, a, counts, out_shape, expert_off=None):
    """dW[e] = dy_e^T @ a_e per local expert on the tcgen05 ragged-reduction kernel (dW rows and
    columns multiples of 8, which the constructor guarantees); a library GEMM per expert only when
    no device-side offsets were given or there are no rows at all."""
    if expert_off is not None and out_shape[1] % 8 == 0 and out_shape[2] % 8 == 0 and dy.shape[0] > 0:
        return G.grouped_wgrad(dy.contiguous(), a.contiguous(), expert_off)
    dw = torch.zeros(out_shape, dtype=dy.dtype, device=dy.device)
    r = 0
    for e, c in enumerate(counts):
        if c:
            torch.mm(dy[r:r + c].t(), a[r:r + c], out=dw[e])
        r += c
    return dw


class _GroupedMLP(torch.autograd.Function):
    """Training path. SwiGLU: fc1 (tcgen05; the epilogue applies SwiGLU x prob AND stores the
    pre-activation h for backward) -> fc2 (tcgen05). Backward: fused swiglu backward kernel, both dgrads on
    the tcgen05 grouped GEMM (weights read in place, N-major), both wgrads on the tcgen05
    ragged-reduction kernel."""

    @staticmethod
    def forward(ctx, x, w1, w2, probs, expert_off, counts, activation):
        ctx.counts, ctx.activation = counts, activation
        ctx.off = expert_off
        if activation == "swiglu":
            # one kernel: fc1, SwiGLU x prob in the epilogue, and the pre-activation kept for backward
            h = torch.empty((x.shape[0], w1.shape[1]), dtype=x.dtype, device=x.device)
            act = G.grouped_gemm_swiglu(x, w1, expert_off, probs, pre_out=h)
            y = G.grouped_gemm(act, w2, expert_off)
            ctx.save_for_backward(x, w1, w2, probs, h, act)
            return y
        h = G.grouped_gemm(x, w1, expert_off)
        act = G.act_fwd(h, probs, activation)
        ctx.save_for_backward(x, w1, w2, probs, h, act)
        return G.grouped_gemm(act, w2, expert_off)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        x, w1, w2, probs, h, act = ctx.saved_tensors
        rows = sum(ctx.counts)
        dact = G.grouped_gemm(dy, w2, ctx.off, w_kn=True)                             # [rows, F]
        if ctx.activation == "swiglu":
            dh, dp = G.swiglu_bwd(h, probs, dact)
        else:
            dh, dp = G.act_bwd(h, probs, dact, ctx.activation)
        dx = G.grouped_gemm(dh, w1, ctx.off, w_kn=True)                               # [rows, H]
        dw2 = _wgrad(dy[:rows], act[:rows], ctx.counts, w2.shape, ctx.off)
        dw1 = _wgrad(dh[:rows], x[:rows], ctx.counts, w1.shape, ctx.off)
        return dx, dw1, dw2, dp, None, None, None


class _GroupedMLPFusedCombine(torch.autograd.Function):
    """Training path with the combine send fused into the fc2 GEMM epilogue: the forward returns
    the COMBINED [T, H] tensor of this rank's tokens; the backward first dispatches the output
    gradient with the cached handle (dispatch is combine's backward) and then runs the expert MLP
    backward on the received rows."""

    @staticmethod
    def forward(ctx, x, w1, w2, probs, expert_off, counts, buffer, handle):
        h = torch.empty((x.shape[0], w1.shape[1]), dtype=x.dtype, device=x.device)
        act = G.grouped_gemm_swiglu(x, w1, expert_off, probs, pre_out=h)
        out = buffer.fused_fc2_combine(act, w2, handle)
        ctx.save_for_backward(x, w1, w2, probs, h, act)
        ctx.counts, ctx.off, ctx.buffer, ctx.handle = counts, expert_off, buffer, handle
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, w1, w2, probs, h, act = ctx.saved_tensors
        dy, *_ = ctx.buffer.dispatch(grad_out.contiguous(), handle=ctx.handle)
        rows = sum(ctx.counts)
        dact = G.grouped_gemm(dy, w2, ctx.off, w_kn=True)
        dh, dp = G.swiglu_bwd(h, probs, dact)
        dx = G.grouped_gemm(dh, w1, ctx.off, w_kn=True)
        dw2 = _wgrad(dy[:rows], act[:rows], ctx.counts, w2.shape, ctx.off)
        dw1 = _wgrad(dh[:rows], x[:rows], ctx.counts, w1.shape, ctx.off)
        return dx, dw1, dw2, dp, None, None, None, None


class Tcgen05GroupedExperts(GroupedExpertsBase):
    """`use_fp8=True` adds an inference path for inputs that arrive as (e4m3 rows, 1x128 f32 scales),
    i.e. the output of an fp8 dispatch: fc1 runs on the block-scaled fp8 tensor-core kernel against
    fp8 copies of the fc1 weights (one scale per 128 x 128 block, refreshed by `refresh_fp8_weights`),
    SwiGLU x prob in its epilogue; fc2 stays bf16. Parameters and training stay bf16."""

    def __init__(self, num_local_experts, hidden_size, ffn_hidden_size, dtype=torch.bfloat16,
                 activation="swiglu", device="cuda", init_std: float = 0.02, use_fp8: bool = False):
        if dtype != torch.bfloat16:
            raise ValueError("the tcgen05 grouped GEMM takes bf16 parameters (fp8 inputs: use_fp8=True)")
        if hidden_size % 8 or ffn_hidden_size % 8 or (activation == "swiglu" and ffn_hidden_size % 128):
            raise ValueError("hidden/ffn sizes must be multiples of 8 (ffn of 128 with swiglu)")
        if use_fp8 and (hidden_size % 128 or ffn_hidden_size % 128):
            raise ValueError("the fp8 path needs hidden and ffn sizes that are multiples of 128")
        super().__init__(num_local_experts, hidden_size, ffn_hidden_size, dtype, activation, device, init_std)
        self.use_fp8 = bool(use_fp8)
        self._w1_fp8 = None

    @torch.no_grad()
    def refresh_fp8_weights(self) -> None:
        """Re-quantise the fc1 weights (call after the bf16 parameters changed)."""
        self._w1_fp8 = G.quantize_weights_128x128(self.weight1)

    @torch.no_grad()
    def forward_fp8(self, hidden_states, tokens_per_expert, routed_probs, expert_off=None):
        """hidden_states = (e4m3 [rows, H], f32 [rows, H/128]) as delivered by an fp8 dispatch.
        Forward only. Returns bf16 [rows, H]."""
        if not self.use_fp8:
            raise ValueError("construct the experts with use_fp8=True")
        x_q, x_s = hidden_states
        if self._w1_fp8 is None:
            self.refresh_fp8_weights()
        w_q, w_s = self._w1_fp8
        counts, off = self._offsets(tokens_per_expert, x_q.device, expert_off)
        probs = routed_probs.float().contiguous()
        if self.activation == "swiglu":
            act = G.grouped_gemm_fp8(x_q, x_s, w_q, w_s, off, swiglu=True, row_prob=probs)
        else:
            act = G.act_fwd(G.grouped_gemm_fp8(x_q, x_s, w_q, w_s, off), probs, self.activation)
        return G.grouped_gemm(act, self.weight2, off)

    @staticmethod
    def _offsets(tokens_per_expert, device, expert_off=None):
        counts = [int(v) for v in (tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else tokens_per_expert)]
        if expert_off is None:
            expert_off = G.offsets_from_counts(counts, device)
        return counts, expert_off

    def forward(self, hidden_states, tokens_per_expert, routed_probs, expert_off=None):
        if isinstance(hidden_states, tuple):
            return self.forward_fp8(hidden_states, tokens_per_expert, routed_probs, expert_off)
        counts, off = self._offsets(tokens_per_expert, hidden_states.device, expert_off)
        return _GroupedMLP.apply(hidden_states.contiguous(), self.weight1, self.weight2,
                                 routed_probs.float().contiguous(), off, counts, self.activation)

    def forward_fused_combine_train(self, hidden_states, tokens_per_expert, routed_probs, buffer, handle):
        """Differentiable twin of `forward_fused_combine` (SwiGLU only)."""
        if self.activation != "swiglu":
            raise ValueError("the fused training path supports swiglu")
        El = self.num_local_experts
        counts = [int(v) for v in (tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else tokens_per_expert)]
        off = handle.meta[2 + El: 2 + El + El + 1]
        return _GroupedMLPFusedCombine.apply(hidden_states.contiguous(), self.weight1, self.weight2,
                                             routed_probs.float().contiguous(), off, counts, buffer, handle)

    @torch.no_grad()
    def forward_fused_combine(self, hidden_states, routed_probs, buffer, handle):
        """Inference/forward-only fast path: fc1(+SwiGLU x prob) then fc2 with the combine send in
        its epilogue; returns the combined [T, H] tensor of THIS rank's tokens."""
        El = self.num_local_experts
        off = handle.meta[2 + El: 2 + El + El + 1]
        x = hidden_states.contiguous()
        if self.activation == "swiglu":
            act = G.grouped_gemm_swiglu(x, self.weight1, off, routed_probs.float().contiguous())
        else:
            act = G.act_fwd(G.grouped_gemm(x, self.weight1, off), routed_probs.float().contiguous(), self.activation)
        return buffer.fused_fc2_combine(act, self.weight2, handle)
