"""Turns `ncu -i REPORT --page raw --csv` output into the short text summary kept under
profiles/: duration, DRAM bytes and throughput, tensor-pipe activity, warps, registers, and the
achieved fraction of the measured roofline.

    ncu -i prof.ncu-rep --page raw --csv > raw.csv
    python -m gpu_data_transfer_profile_b200.prof.ncu_summary raw.csv --kernel grouped_gemm --flops 2.4e12
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys
from typing import Dict, List

WANTED = ("gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
          "dram__cycles_active.avg", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
          "sm__pipe_tensor_op_hmma_cycles_active.avg.pct_of_peak_sustained_active", "sm__warps_active.avg.pct_of_peak_sustained_active",
          "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio", "launch__registers_per_thread",
          "launch__grid_size", "launch__block_size", "sm__throughput.avg.pct_of_peak_sustained_elapsed",
          "lts__t_bytes.sum", "l1tex__t_bytes.sum", "launch__shared_mem_per_block_dynamic")


_UNIT_SCALE = {"ns": 1.0, "us": 1e3, "ms": 1e6, "s": 1e9,                       # times -> ns
               "byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}  # sizes -> bytes


def read_raw(path: str) -> List[Dict[str, str]]:
    """Rows of the raw page: one dict per profiled launch. The page's second row gives each
    column's unit (ncu picks us/ms and Kbyte/Mbyte per column); times are rescaled to ns and
    sizes to bytes, so every consumer sees one unit."""
    with open(path, newline="") as f:
        lines = [l for l in f if l.startswith('"')]
    rows = list(csv.DictReader(lines))
    units = next((r for r in rows if not r.get("ID", "").strip().isdigit()), {})
    out = []
    for r in rows:
        if not r.get("ID", "").strip().isdigit():
            continue
        for k, u in units.items():
            scale = _UNIT_SCALE.get((u or "").strip())
            v = _num(r.get(k))
            if scale is not None and scale != 1.0 and v is not None:
                r[k] = repr(v * scale)
        out.append(r)
    return out


def _num(v: str):
    try:
        return float(v.replace(",", ""))
    except (ValueError, AttributeError):
        return None


def summarize(rows: List[Dict[str, str]], kernel: str = "", flops: float = 0.0, bytes_algo: float = 0.0,
              peaks: Dict[str, float] = None) -> List[Dict[str, object]]:
    out = []
    for r in rows:
        name = r.get("Kernel Name", "")
        if kernel and kernel not in name:
            continue
        d = {"kernel": name[:100], "id": r.get("ID")}
        for k in r:
            for w in WANTED:
                if k.startswith(w):
                    d[w] = _num(r[k])
        dur_ns = d.get("gpu__time_duration.sum")
        rd, wr = d.get("dram__bytes_read.sum") or 0.0, d.get("dram__bytes_write.sum") or 0.0
        if dur_ns:
            d["dram_gb_s"] = (rd + wr) / dur_ns
            if flops:
                d["tflops"] = flops / dur_ns / 1e3
            if peaks:
                if flops and peaks.get("bf16_tflops"):
                    d["frac_of_measured_bf16_peak"] = d["tflops"] / peaks["bf16_tflops"]
                if bytes_algo and peaks.get("hbm_gbs"):
                    d["frac_of_measured_hbm_peak"] = bytes_algo / dur_ns / peaks["hbm_gbs"]
        out.append(d)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("raw_csv")
    ap.add_argument("--kernel", default="")
    ap.add_argument("--flops", type=float, default=0.0, help="algorithmic FLOPs per launch")
    ap.add_argument("--bytes", type=float, default=0.0, help="algorithmic bytes per launch")
    ap.add_argument("--peaks", default=None,
                    help="JSON file with measured peaks {hbm_gbs, bf16_tflops}; without it no fraction is printed")
    a = ap.parse_args(argv)
    peaks = json.load(open(a.peaks)) if a.peaks and os.path.exists(a.peaks) else None
    for d in summarize(read_raw(a.raw_csv), a.kernel, a.flops, a.bytes, peaks):
        print(json.dumps(d))
    return 0


if __name__ == "__main__":
    sys.exit(main())
