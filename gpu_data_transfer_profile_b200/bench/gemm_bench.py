"""Grouped expert GEMM throughput: this library's tcgen05 kernels vs the per-expert library
GEMM loop (the reference's torch fallback, `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:590-600`).

All variants are timed round-robin inside one loop (variant 1, variant 2, ..., variant 1, ...), so
they see the same clocks and temperature; the figure of a variant is the median over its samples.

    python -m gpu_data_transfer_profile_b200.bench.gemm_bench --rows 16384 --hidden 4096 --ffn 14336 --experts 1
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import gemm as G
from ..utils.timing import L2Flusher


def _time_round_robin(fns, iters, warmup, flush):
    """fns: {name: callable}. Returns {name: (median ms, best ms)}."""
    for _ in range(warmup):
        for fn in fns.values():
            fn()
    torch.cuda.synchronize()
    ms = {k: [] for k in fns}
    for _ in range(iters):
        for name, fn in fns.items():
            flush()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            ms[name].append(a.elapsed_time(b))
    out = {}
    for k, v in ms.items():
        v.sort()
        out[k] = (v[len(v) // 2], v[0])
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--skip-torch", action="store_true")
    ap.add_argument("--wgrad", action="store_true", help="also time the two weight-gradient GEMMs (ragged reduction)")
    ap.add_argument("--form", choices=["cta", "pair", "both"], default="both",
                    help="cta: one CTA per 128x256 tile; pair: a CTA pair (cta_group::2) per 256x256 tile")
    ap.add_argument("--peaks", default=None, help="JSON file with {bf16_tflops: measured library GEMM rate}")
    ap.add_argument("--fp8", action="store_true",
                    help="also time the block-scaled fp8 fc1 (e4m3 rows with 1x128 scales, e4m3 weights with 128x128 scales)")
    ap.add_argument("--band-mb", type=str, default="",
                    help="comma-separated L2 band sizes (MiB) of the tile order to compare; empty = the default")
    args = ap.parse_args()
    dev = torch.device("cuda")
    E, H, F, rows = args.experts, args.hidden, args.ffn, args.rows
    counts = [rows // E] * E
    counts[-1] += rows - sum(counts)
    off = G.offsets_from_counts(counts, dev)
    x = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * F, H, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, F, device=dev) * 0.02).to(torch.bfloat16)
    prob = torch.rand(rows, device=dev)
    act = torch.empty(rows, F, dtype=torch.bfloat16, device=dev)
    out = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
    flush = L2Flusher(dev)
    peaks = {}
    if args.peaks and os.path.exists(args.peaks):
        peaks = json.load(open(args.peaks))
    # fraction denominator: the measured library bf16 GEMM rate of this machine when a peaks file is
    # given, else 1590 TFLOP/s (an earlier measurement on the same kind of GPU); fp8 rows use it too
    peak = peaks.get("bf16_tflops", 1590.0)
    f1 = 2.0 * rows * H * 2 * F
    f2 = 2.0 * rows * F * H
    bands = [int(float(b) * (1 << 20)) for b in args.band_mb.split(",") if b] or [None]
    fns, flops = {}, {}
    for form in (["cta", "pair"] if args.form == "both" else [args.form]):
        pair = form == "pair"
        for band in bands:
            tag = ("_pair" if pair else "") + (f"_band{band >> 20}" if band else "")
            fns["fc1_swiglu_tcgen05" + tag] = (
                lambda pair=pair, band=band: G.grouped_gemm_swiglu(x, w1, off, prob, out=act, pair=pair, band_bytes=band))
            fns["fc2_tcgen05" + tag] = (
                lambda pair=pair, band=band: G.grouped_gemm(act, w2, off, out=out, pair=pair, band_bytes=band))
            flops["fc1_swiglu_tcgen05" + tag], flops["fc2_tcgen05" + tag] = f1, f2
    if args.fp8:
        xq, xs = G.quantize_rows_1x128(x)
        wq, ws = G.quantize_weights_128x128(w1)
        fns["fc1_swiglu_fp8_tcgen05"] = lambda: G.grouped_gemm_fp8(xq, xs, wq, ws, off, swiglu=True, row_prob=prob, out=act)
        flops["fc1_swiglu_fp8_tcgen05"] = f1
        hpl = torch.empty(rows, 2 * F, dtype=torch.bfloat16, device=dev)
        fns["fc1_plain_fp8_tcgen05"] = lambda: G.grouped_gemm_fp8(xq, xs, wq, ws, off, out=hpl)
        flops["fc1_plain_fp8_tcgen05"] = f1
    if args.wgrad:
        dh = torch.randn(rows, 2 * F, device=dev).to(torch.bfloat16)
        dy = torch.randn(rows, H, device=dev).to(torch.bfloat16)
        dw1, dw2 = torch.empty_like(w1), torch.empty_like(w2)
        dact = torch.empty(rows, F, dtype=torch.bfloat16, device=dev)
        for form in (["cta", "pair"] if args.form == "both" else [args.form]):
            pair = form == "pair"
            tag = "_pair" if pair else ""
            fns["wgrad1_tcgen05" + tag] = lambda pair=pair: G.grouped_wgrad(dh, x, off, out=dw1, pair=pair)
            fns["wgrad2_tcgen05" + tag] = lambda pair=pair: G.grouped_wgrad(dy, act, off, out=dw2, pair=pair)
            flops["wgrad1_tcgen05" + tag], flops["wgrad2_tcgen05" + tag] = f1, f2
            # data gradients: the forward weights read in place as an N-major operand
            fns["dgrad1_tcgen05" + tag] = lambda pair=pair: G.grouped_gemm(dh, w1, off, out=out, pair=pair, w_kn=True)
            fns["dgrad2_tcgen05" + tag] = lambda pair=pair: G.grouped_gemm(dy, w2, off, out=dact, pair=pair, w_kn=True)
            flops["dgrad1_tcgen05" + tag], flops["dgrad2_tcgen05" + tag] = f1, f2
        # training forward of fc1: one kernel that also stores the pre-activation, vs plain fc1 + SwiGLU kernel
        hpre = torch.empty(rows, 2 * F, dtype=torch.bfloat16, device=dev)

        def fc1_train_separate():
            G.grouped_gemm(x, w1, off, out=hpre)
            return G.swiglu_fwd(hpre, prob)
        fns["fc1_train_fused_tcgen05"] = lambda: G.grouped_gemm_swiglu(x, w1, off, prob, out=act, pre_out=hpre)
        fns["fc1_train_separate_tcgen05"] = fc1_train_separate
        flops["fc1_train_fused_tcgen05"] = flops["fc1_train_separate_tcgen05"] = f1
        if not args.skip_torch:
            def torch_wgrad(gg, xx, dw):
                r = 0
                for e, c in enumerate(counts):
                    torch.mm(gg[r:r + c].t(), xx[r:r + c], out=dw[e])
                    r += c
            fns["wgrad1_torch"] = lambda: torch_wgrad(dh, x, dw1)
            fns["wgrad2_torch"] = lambda: torch_wgrad(dy, act, dw2)
            flops["wgrad1_torch"], flops["wgrad2_torch"] = f1, f2
    if not args.skip_torch:
        def torch_fc1():
            r = 0
            for e, c in enumerate(counts):
                h = torch.nn.functional.linear(x[r:r + c], w1[e])
                g, l = h.chunk(2, -1)
                act[r:r + c] = (torch.nn.functional.silu(g) * l * prob[r:r + c, None]).to(torch.bfloat16)
                r += c

        def torch_fc2():
            r = 0
            for e, c in enumerate(counts):
                out[r:r + c] = torch.nn.functional.linear(act[r:r + c], w2[e])
                r += c
        fns["fc1_swiglu_torch"], fns["fc2_torch"] = torch_fc1, torch_fc2
        flops["fc1_swiglu_torch"], flops["fc2_torch"] = f1, f2
    res = {}
    for name, (med, best) in _time_round_robin(fns, args.iters, args.warmup, flush).items():
        res[name] = dict(ms=med, best_ms=best, tflops=flops[name] / med / 1e9)
        if "torch" not in name:
            res[name]["frac_of_measured_peak"] = flops[name] / med / 1e9 / peak
    print(json.dumps(dict(bench="gemm", rows=rows, hidden=H, ffn=F, experts=E, peak_tflops_measured=peak, **res)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
