"""Grouped expert GEMM throughput: this library's tcgen05 kernels vs the per-expert library
GEMM loop (the reference's torch fallback, `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:590-600`).

    python -m gpu_data_transfer_profile_b200.bench.gemm_bench --rows 16384 --hidden 4096 --ffn 14336 --experts 1
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import gemm as G
from ..utils.timing import L2Flusher


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(iters):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b))
    ms.sort()
    return ms[len(ms) // 2], ms[0]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--skip-torch", action="store_true")
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
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    peak = peaks.get("bf16_tflops", 1590.0)
    res = {}
    f1 = 2.0 * rows * H * 2 * F
    f2 = 2.0 * rows * F * H
    med, best = _time(lambda: G.grouped_gemm_swiglu(x, w1, off, prob, out=act), args.iters, args.warmup, flush)
    res["fc1_swiglu_tcgen05"] = dict(ms=med, best_ms=best, tflops=f1 / med / 1e9, frac_of_measured_peak=f1 / med / 1e9 / peak)
    med, best = _time(lambda: G.grouped_gemm(act, w2, off, out=out), args.iters, args.warmup, flush)
    res["fc2_tcgen05"] = dict(ms=med, best_ms=best, tflops=f2 / med / 1e9, frac_of_measured_peak=f2 / med / 1e9 / peak)
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
        med, best = _time(torch_fc1, args.iters, args.warmup, flush)
        res["fc1_swiglu_torch"] = dict(ms=med, best_ms=best, tflops=f1 / med / 1e9)
        med, best = _time(torch_fc2, args.iters, args.warmup, flush)
        res["fc2_torch"] = dict(ms=med, best_ms=best, tflops=f2 / med / 1e9)
    print(json.dumps(dict(bench="gemm", rows=rows, hidden=H, ffn=F, experts=E, peak_tflops_measured=peak, **res)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
