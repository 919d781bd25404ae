"""Python front-end of the tcgen05 grouped GEMM (csrc/gemm/grouped_gemm.cu).

`expert_off` is a DEVICE int32 tensor [E_local+1] (exclusive prefix of rows per local expert),
so no host synchronisation is needed to schedule tiles; the reference reads the split sizes
back to the host for every call (`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:536,586`).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _ext

PLAIN, SWIGLU, COMBINE = 0, 1, 2

# Default form of the kernel: True = a CTA pair (cluster of two SMs, `cta_group::2`) per
# 256 x 256 tile, False = one CTA per 128 x 256 tile. The pair form measured 10-17 % faster on
# every shape tried (it fetches each weight tile once per pair and halves the shared-memory
# reads of B per flop). Every entry point takes `pair=` to override the default.
PAIR_DEFAULT = os.environ.get("B200EP_GEMM_PAIR", "1") == "1"

# Tile order: bytes of activation rows per band that stays in L2 while every weight tile passes
# over it (the band height in rows follows from the reduction length).
BAND_BYTES = int(os.environ.get("B200EP_GEMM_BAND_BYTES", str(24 << 20)))


def _band_rows(k: int, band_bytes: Optional[int] = None) -> int:
    return max(256, (band_bytes or BAND_BYTES) // (2 * k) // 256 * 256)


def _pair(pair: Optional[bool]) -> bool:
    return PAIR_DEFAULT if pair is None else bool(pair)


def _ctas(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def offsets_from_counts(tokens_per_expert, device) -> torch.Tensor:
    t = torch.as_tensor(tokens_per_expert, dtype=torch.int64)
    off = torch.zeros(t.numel() + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(t, 0).to(torch.int32)
    return off.to(device, non_blocking=True)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, expert_off: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                 ctas: int = 0, pair: Optional[bool] = None, band_bytes: Optional[int] = None,
                 w_kn: bool = False) -> torch.Tensor:
    """out[r] = a[r] @ w[e(r)].T   (a bf16 [rows,K], w bf16 [E,N,K]) -> bf16 [rows,N].
    w_kn=True: w is stored [E,K,N] and out[r] = a[r] @ w[e(r)] (the data gradient of a layer whose
    forward weight is [E,K,N]-shaped, read in place without a transposed copy)."""
    if out is None:
        out = torch.empty((a.shape[0], w.shape[2] if w_kn else w.shape[1]), dtype=torch.bfloat16, device=a.device)
    _ext.load().grouped_gemm(a, w, expert_off, PLAIN, out, None, None, [], 0, 0, 0, -1, 0, None, 0,
                             ctas or _ctas(a.device), _pair(pair), _band_rows(a.shape[1], band_bytes), w_kn, None)
    return out


def grouped_gemm_swiglu(a: torch.Tensor, w: torch.Tensor, expert_off: torch.Tensor, row_prob: Optional[torch.Tensor],
                        *, out: Optional[torch.Tensor] = None, ctas: int = 0,
                        pair: Optional[bool] = None, band_bytes: Optional[int] = None,
                        pre_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """w bf16 [E, 2F, K] (gate rows first): out[r] = silu(a[r] @ Wg.T) * (a[r] @ Wl.T) * row_prob[r] -> bf16 [rows,F].
    pre_out (bf16 [rows, 2F]): if given, the same kernel also stores the pre-activation a[r] @ W.T
    there (what the backward pass needs), so the training forward needs no separate activation kernel."""
    F = w.shape[1] // 2
    if out is None:
        out = torch.empty((a.shape[0], F), dtype=torch.bfloat16, device=a.device)
    _ext.load().grouped_gemm(a, w, expert_off, SWIGLU, out, row_prob, None, [], 0, 0, 0, -1, 0, None, 0,
                             ctas or _ctas(a.device), _pair(pair), _band_rows(a.shape[1], band_bytes), False, pre_out)
    return out


def grouped_gemm_combine(a: torch.Tensor, w: torch.Tensor, expert_off: torch.Tensor, recv_meta: torch.Tensor,
                         peers, comb_off: int, slot_cap: int, rank: int, *, signal_flag_off: int = -1,
                         epoch: int = 0, counter: Optional[torch.Tensor] = None, status_ptr: int = 0,
                         ctas: int = 0, pair: Optional[bool] = None, band_bytes: Optional[int] = None) -> None:
    """fc2 with the combine send fused into the epilogue: row r of a @ w[e].T is stored into slot
    recv_meta[r,0] of rank recv_meta[r,1]'s combine region (peer LSU stores)."""
    _ext.load().grouped_gemm(a, w, expert_off, COMBINE, None, None, recv_meta, list(peers), comb_off, slot_cap,
                             rank, signal_flag_off, epoch, counter, status_ptr, ctas or _ctas(a.device), _pair(pair), _band_rows(a.shape[1], band_bytes), False, None)


def grouped_wgrad(g: torch.Tensor, x: torch.Tensor, expert_off: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                  ctas: int = 0, pair: Optional[bool] = None) -> torch.Tensor:
    """dW[e] = g_e.T @ x_e over the rows of local expert e (g bf16 [rows,M], x bf16 [rows,N]) -> bf16 [E,M,N].
    Both operands are read as stored; an expert without rows gets zeros. M % 8 == 0 (the pair form
    needs M % 256 == 0 and is skipped otherwise), N % 8 == 0."""
    E = expert_off.numel() - 1
    if out is None:
        out = torch.empty((E, g.shape[1], x.shape[1]), dtype=torch.bfloat16, device=g.device)
    use_pair = _pair(pair) and g.shape[1] % 256 == 0
    _ext.load().grouped_wgrad(g, x, expert_off, out, 0, ctas or _ctas(g.device), use_pair)
    return out


def swiglu_fwd(h: torch.Tensor, row_prob: Optional[torch.Tensor]) -> torch.Tensor:
    """act = silu(h[:, :F]) * h[:, F:] * row_prob[:, None]  (bf16 in, bf16 out)."""
    act = torch.empty((h.shape[0], h.shape[1] // 2), dtype=torch.bfloat16, device=h.device)
    _ext.load().swiglu_fwd(h, row_prob, act)
    return act


def swiglu_bwd(h: torch.Tensor, row_prob: Optional[torch.Tensor], dact: torch.Tensor):
    """-> (dh bf16 [rows, 2F], dprob f32 [rows]) for act = swiglu(h) * prob."""
    dh = torch.empty_like(h)
    dp = torch.empty(h.shape[0], dtype=torch.float32, device=h.device)
    _ext.load().swiglu_bwd(h, row_prob, dact.contiguous(), dh, dp)
    return dh, dp


ACT_KIND = {"gelu": 0, "silu": 1, "relu": 2}


def act_fwd(h: torch.Tensor, row_prob: Optional[torch.Tensor], activation: str) -> torch.Tensor:
    """act = f(h) * row_prob[:, None] for f in gelu (erf form) / silu / relu (bf16 in, bf16 out)."""
    act = torch.empty_like(h)
    _ext.load().act_fwd(h, row_prob, act, ACT_KIND[activation])
    return act


def act_bwd(h: torch.Tensor, row_prob: Optional[torch.Tensor], dact: torch.Tensor, activation: str):
    """-> (dh bf16 [rows, F], dprob f32 [rows]) for act = f(h) * prob."""
    dh = torch.empty_like(h)
    dp = torch.empty(h.shape[0], dtype=torch.float32, device=h.device)
    _ext.load().act_bwd(h, row_prob, dact.contiguous(), dh, dp, ACT_KIND[activation])
    return dh, dp


# ---- block-scaled fp8 (e4m3) forward path ---------------------------------------------------------
def quantize_rows_1x128(x: torch.Tensor):
    """bf16/f32 [rows, K] -> (e4m3 [rows, K], f32 scales [rows, K/128]); scale = max(amax, 1e-4) / 448
    per row and 128 channels: the same rule as the cast inside the fp8 dispatch kernel."""
    rows, K = x.shape
    xf = x.float().view(rows, K // 128, 128)
    amax = xf.abs().amax(-1).clamp_min(1e-4)
    q = (xf * (448.0 / amax)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(rows, K)
    return q, (amax / 448.0).contiguous()


def quantize_weights_128x128(w: torch.Tensor):
    """[E, N, K] -> (e4m3 [E, N, K], f32 scales [E, N/128, K/128]), one scale per 128 x 128 block."""
    E, N, K = w.shape
    wf = w.float().view(E, N // 128, 128, K // 128, 128)
    amax = wf.abs().amax(dim=(2, 4)).clamp_min(1e-6)
    q = (wf * (448.0 / amax)[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(E, N, K)
    return q.contiguous(), (amax / 448.0).contiguous()


def dequantize_weights_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    E, N, K = q.shape
    return (q.float().view(E, N // 128, 128, K // 128, 128) * s[:, :, None, :, None]).view(E, N, K)


def grouped_gemm_fp8(a_q: torch.Tensor, a_s: torch.Tensor, w_q: torch.Tensor, w_s: torch.Tensor,
                     expert_off: torch.Tensor, *, swiglu: bool = False, row_prob: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None, ctas: int = 0, band_bytes: Optional[int] = None) -> torch.Tensor:
    """Block-scaled fp8 grouped GEMM on the tensor cores (`tcgen05.mma kind::f8f6f4`, partial sums
    promoted to f32 per 128-wide reduction block with the product of both scales).
    a_q e4m3 [rows, K] + a_s f32 [rows, K/128] (what the fp8 dispatch delivers), w_q e4m3 [E, Nw, K]
    + w_s f32 [E, Nw/128, K/128]. Plain: out[r] = a[r] @ w[e(r)].T -> bf16 [rows, Nw]. swiglu: Nw = 2F
    (gate rows first), out = silu(gate) * linear * row_prob -> bf16 [rows, F]."""
    n_out = w_q.shape[1] // 2 if swiglu else w_q.shape[1]
    if out is None:
        out = torch.empty((a_q.shape[0], n_out), dtype=torch.bfloat16, device=a_q.device)
    _ext.load().grouped_gemm_fp8(a_q, a_s, w_q, w_s, expert_off, SWIGLU if swiglu else PLAIN, out, row_prob, 0,
                                 ctas or _ctas(a_q.device), max(256, (band_bytes or BAND_BYTES) // a_q.shape[1] // 256 * 256))
    return out
