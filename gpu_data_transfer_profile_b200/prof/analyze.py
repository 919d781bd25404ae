"""Command-line analyzers for stored Nsight Systems reports of the copy benchmarks.

    python -m gpu_data_transfer_profile_b200.prof.analyze copy    REPORT [--json]
    python -m gpu_data_transfer_profile_b200.prof.analyze a2a     REPORT --timed-iterations 100
    python -m gpu_data_transfer_profile_b200.prof.analyze layout  REPORT --warmup-iterations 10 --timed-iterations 100
    python -m gpu_data_transfer_profile_b200.prof.analyze msrc    REPORT
    python -m gpu_data_transfer_profile_b200.prof.analyze kernel  REPORT --kernel-name lsu_copy_kernel --csv out.csv

Parity (flags and metrics): copy = `Copy_Engine/Results/nvlink_copy_engine_test/analyze_nvlink_copy_engine_report.py:57-104,371`;
a2a = `.../nvlink_all_to_all_copy_engine_test/analyze_nvlink_all_to_all_copy_engine_report.py:60-122,226-244,327-363,488`;
layout = `.../nvlink_batch_address_layout_test/analyze_nvlink_batch_address_layout_report.py:97-114`;
msrc = `.../nvlink_multi_source_all_to_all_batch_test/analyze_nvlink_multi_source_all_to_all_batch_report.py:132-256,356`;
kernel = `LSU_TMA/Results/analyze_nvlink_lsu_tma_report.py:35-40,231-304,391,476-524`.
Every analyzer returns a plain dict (`build_*_summary`) so plotters and tests can import it.
"""
from __future__ import annotations

import argparse
import csv
import json
import sys
from pathlib import Path
from typing import Any, Dict, List, Optional

from . import nsys_sqlite as N

KERNEL_CANDIDATES = ("lsu_rr_copy_kernel", "tma_staged_push_kernel", "tma_staged_pull_kernel", "lsu_copy_kernel",
                     "batched_copy_kernel", "dispatch_send_kernel", "combine_kernel", "combine_pull_kernel", "grouped_gemm_kernel",
                     "grouped_gemm_fp8_kernel",
                     "lsu_round_robin_copy_kernel", "tma_round_robin_copy_kernel", "tma_copy_kernel")


def _window(events):
    return (events[0].start_ns, events[-1].end_ns) if events else (None, None)


def _copy_summary(conn, events: List[N.CopyEvent], peak: Optional[float], include_protocol: bool) -> Dict[str, Any]:
    t0, t1 = _window(events)
    return {
        "event_count": len(events),
        "throughput": N.summarize_throughput(events),
        "gap": N.summarize_gaps(events),
        "duration": N.summarize_durations(events),
        "api_to_copy_wait": N.summarize_waits(events),
        "nvlink": N.summarize_nvlink(conn, t0, t1, peak, include_protocol),
        "window_ns": [t0, t1],
    }


def build_copy_summary(conn, bus_id: str = N.DEFAULT_BUS_ID, peak_gb_s: Optional[float] = None,
                       skip_warmup_copies: int = 0, include_protocol: bool = False) -> Dict[str, Any]:
    """Pairwise copy-engine report: events whose source is the GPU at `bus_id`."""
    if skip_warmup_copies < 0:
        raise ValueError("--skip-warmup-copies must be non-negative")
    gpu = N.find_gpu(conn, bus_id)
    events = N.load_copy_events(conn, gpu["id"])
    kept = N.trim_warmup(events, skip_events=skip_warmup_copies)
    out = _copy_summary(conn, kept, peak_gb_s, include_protocol)
    out.update(gpu={"name": gpu["name"], "bus": gpu["busLocation"], "device": gpu["cuDevice"]},
               total_events=len(events), skipped_warmup_events=len(events) - len(kept))
    return out


def build_a2a_summary(conn, bus_id: str = N.DEFAULT_BUS_ID, peak_gb_s: Optional[float] = None,
                      copy_mode: Optional[str] = None, report_name: str = "", skip_warmup_iterations: int = 0,
                      copies_per_iteration: int = 0, batch_calls_per_iteration: int = 1,
                      timed_iterations: int = 0, include_protocol: bool = False) -> Dict[str, Any]:
    """Fan-out report. Warm-up is trimmed by iterations: in separate mode an iteration is
    `copies_per_iteration` events, in batch mode `batch_calls_per_iteration` submissions."""
    gpu = N.find_gpu(conn, bus_id)
    mode = copy_mode or N.detect_copy_mode(conn, report_name)
    events = N.load_copy_events(conn, gpu["id"])
    if timed_iterations > 0 and skip_warmup_iterations == 0:
        groups = N.group_by_submission(events)
        per_iter = batch_calls_per_iteration if mode == "batch" else max(copies_per_iteration, 1)
        total_iters = len(groups) // max(per_iter, 1)
        skip_warmup_iterations = max(total_iters - timed_iterations, 0)
    if mode == "batch":
        kept = N.trim_warmup(events, skip_iterations=skip_warmup_iterations,
                             submissions_per_iteration=batch_calls_per_iteration)
    else:
        kept = N.trim_warmup(events, skip_events=skip_warmup_iterations * max(copies_per_iteration, 1))
    out = _copy_summary(conn, kept, peak_gb_s, include_protocol)
    groups = N.group_by_submission(kept)
    out.update(copy_mode=mode, total_events=len(events), skipped_warmup_iterations=skip_warmup_iterations,
               api_groups={"count": len(groups),
                           "events_per_group": (sum(len(g) for g in groups) / len(groups)) if groups else None},
               destinations=sorted({e.dst_device_id for e in kept if e.dst_device_id is not None}))
    return out


def build_layout_summary(conn, bus_id: str = N.DEFAULT_BUS_ID, peak_gb_s: Optional[float] = None,
                         warmup_iterations: int = 10, timed_iterations: int = 100,
                         include_protocol: bool = False) -> Dict[str, Any]:
    """Address-layout report: like `copy`, warm-up share inferred from the iteration counts."""
    gpu = N.find_gpu(conn, bus_id)
    n = len(N.load_copy_events(conn, gpu["id"]))
    skip = N.infer_warmup_skip(n, warmup_iterations, timed_iterations)
    out = build_copy_summary(conn, bus_id, peak_gb_s, skip, include_protocol)
    out["inferred_warmup_skip"] = skip
    return out


def build_msrc_summary(conn, bus_id: str = N.DEFAULT_BUS_ID, peak_gb_s: Optional[float] = None,
                       report_name: str = "", timed_iterations: int = 0, processes_per_report: int = 8,
                       include_protocol: bool = False) -> Dict[str, Any]:
    """Multi-source report: per-destination submission structure; falls back to timing the runtime
    calls (bytes taken from the file name) when the trace holds no peer memcpy activity."""
    gpu = N.find_gpu(conn, bus_id)
    events = N.load_copy_events(conn, gpu["id"])
    source = "memcpy_activity"
    if not events:
        sizes = N.sizes_in_name(report_name)
        per_call = sizes[0] if sizes else 0
        events = N.load_runtime_events(conn, N.BATCH_API, per_call) or N.load_runtime_events(conn, "cudaGraphLaunch%", per_call)
        source = "runtime_api_fallback"
    groups = N.group_by_submission(events)
    dsts = sorted({e.dst_device_id for e in events if e.dst_device_id is not None})
    calls_per_iter = max(len(dsts), 1)
    skip = 0
    if timed_iterations > 0 and groups:
        skip = max(len(groups) // calls_per_iter - timed_iterations, 0)
    kept = N.trim_warmup(events, skip_iterations=skip, submissions_per_iteration=calls_per_iter)
    out = _copy_summary(conn, kept, peak_gb_s, include_protocol)
    kg = N.group_by_submission(kept)
    out.update(event_source=source, batch_calls_per_iteration=calls_per_iter,
               entries_per_batch=(sum(len(g) for g in kg) / len(kg)) if kg else None,
               processes_per_report=processes_per_report, skipped_warmup_iterations=skip, destinations=dsts)
    return out


def build_kernel_summary(conn, bus_id: str = N.DEFAULT_BUS_ID, kernel_name: Optional[str] = None,
                         peak_gb_s: Optional[float] = None, skip_warmup_launches: int = 1,
                         bytes_per_launch: int = 0, include_protocol: bool = False) -> Dict[str, Any]:
    """SM copy kernels: duration per launch and NVLink RX/TX percent over each kernel's window."""
    gpu = N.find_gpu(conn, bus_id)
    name = kernel_name or N.detect_kernel_name(conn, KERNEL_CANDIDATES)
    if name is None:
        raise RuntimeError("no known copy kernel found; pass --kernel-name")
    ev = N.load_kernel_events(conn, gpu["id"], name)
    kept = ev[skip_warmup_launches:]
    per = []
    for k in kept:
        nv = N.summarize_nvlink(conn, k.start_ns, k.end_ns, peak_gb_s, include_protocol)
        per.append({"start_ns": k.start_ns, "duration_us": k.duration_ns / 1e3, "grid": list(k.grid), "block": list(k.block),
                    "nvlink_rx_percent": nv.get("rx", {}).get("average_percent_of_peak"),
                    "nvlink_tx_percent": nv.get("tx", {}).get("average_percent_of_peak"),
                    "gib_s": (bytes_per_launch / (k.duration_ns * 1e-9) / float(1 << 30)) if bytes_per_launch else None})

    def avg(key):
        v = [p[key] for p in per if p[key] is not None]
        return sum(v) / len(v) if v else None
    return {"kernel": name, "launches": len(ev), "skipped_warmup_launches": len(ev) - len(kept),
            "duration": N.summarize_durations(kept), "average_nvlink_rx_percent": avg("nvlink_rx_percent"),
            "average_nvlink_tx_percent": avg("nvlink_tx_percent"), "average_gib_s": avg("gib_s"), "per_launch": per}


# ---- output ---------------------------------------------------------------------------------
def format_text(kind: str, s: Dict[str, Any]) -> str:
    lines = [f"== {kind} summary =="]
    if "kernel" in s:
        d = s["duration"]
        lines += [f"kernel                : {s['kernel']}", f"launches (kept)       : {d['count']} (of {s['launches']})",
                  f"avg duration          : {d['average_us']} us",
                  f"avg NVLink RX / TX    : {s['average_nvlink_rx_percent']} % / {s['average_nvlink_tx_percent']} %"]
        return "\n".join(lines)
    t, g, d, w = s["throughput"], s["gap"], s["duration"], s["api_to_copy_wait"]
    lines += [f"events (kept)         : {s['event_count']}",
              f"avg throughput        : {t['average_gib_s']} GiB/s (per-event bytes/duration)",
              f"avg inter-copy gap    : {g['average_us']} us", f"avg copy duration     : {d['average_us']} us",
              f"avg API-end -> start  : {w['average_us']} us"]
    for dname, nv in s.get("nvlink", {}).items():
        lines.append(f"NVLink {dname.upper()} user data   : {nv['average_percent_of_peak']} % of peak ({nv['sample_count']} samples)")
    for k in ("copy_mode", "event_source", "batch_calls_per_iteration", "entries_per_batch", "inferred_warmup_skip"):
        if k in s:
            lines.append(f"{k:22s}: {s[k]}")
    return "\n".join(lines)


def write_csv(path: str, s: Dict[str, Any]) -> None:
    rows = s.get("per_launch")
    with open(path, "w", newline="") as f:
        if rows:
            wr = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
            wr.writeheader()
            for r in rows:
                wr.writerow(r)
        else:
            wr = csv.writer(f)
            wr.writerow(["metric", "value"])
            for sec in ("throughput", "gap", "duration", "api_to_copy_wait"):
                for k, v in s.get(sec, {}).items():
                    wr.writerow([f"{sec}.{k}", v])
            for d, nv in s.get("nvlink", {}).items():
                for k, v in nv.items():
                    wr.writerow([f"nvlink.{d}.{k}", v])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kind", choices=["copy", "a2a", "layout", "msrc", "kernel"])
    ap.add_argument("report", type=Path, help=".nsys-rep or .sqlite")
    ap.add_argument("--gpu-bus-id", default=N.DEFAULT_BUS_ID)
    ap.add_argument("--force-export", action="store_true")
    ap.add_argument("--nvlink-peak-gb-s", type=float, default=None)
    ap.add_argument("--include-protocol", action="store_true", help="count NVLink protocol bytes too")
    ap.add_argument("--skip-warmup-copies", type=int, default=0)
    ap.add_argument("--skip-warmup-iterations", type=int, default=0)
    ap.add_argument("--skip-warmup-launches", type=int, default=1)
    ap.add_argument("--warmup-iterations", type=int, default=10)
    ap.add_argument("--timed-iterations", type=int, default=0)
    ap.add_argument("--copy-mode", choices=["separate", "batch"], default=None)
    ap.add_argument("--copies-per-iteration", type=int, default=0)
    ap.add_argument("--batch-calls-per-iteration", type=int, default=1)
    ap.add_argument("--ptop-events-per-batch", type=int, default=0, help="accepted for compatibility; inferred")
    ap.add_argument("--processes-per-report", type=int, default=8)
    ap.add_argument("--kernel-name", default=None)
    ap.add_argument("--bytes-per-launch", type=int, default=0)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--csv", default=None)
    a = ap.parse_args(argv)
    conn = N.connect(N.resolve_sqlite(a.report, a.force_export))
    common = dict(bus_id=a.gpu_bus_id, peak_gb_s=a.nvlink_peak_gb_s, include_protocol=a.include_protocol)
    if a.kind == "copy":
        s = build_copy_summary(conn, skip_warmup_copies=a.skip_warmup_copies, **common)
    elif a.kind == "a2a":
        s = build_a2a_summary(conn, copy_mode=a.copy_mode, report_name=a.report.name,
                              skip_warmup_iterations=a.skip_warmup_iterations, copies_per_iteration=a.copies_per_iteration,
                              batch_calls_per_iteration=a.batch_calls_per_iteration, timed_iterations=a.timed_iterations,
                              **common)
    elif a.kind == "layout":
        s = build_layout_summary(conn, warmup_iterations=a.warmup_iterations, timed_iterations=a.timed_iterations or 100,
                                 **common)
    elif a.kind == "msrc":
        s = build_msrc_summary(conn, report_name=a.report.name, timed_iterations=a.timed_iterations,
                               processes_per_report=a.processes_per_report, **common)
    else:
        s = build_kernel_summary(conn, kernel_name=a.kernel_name, skip_warmup_launches=a.skip_warmup_launches,
                                 bytes_per_launch=a.bytes_per_launch, **common)
    if a.csv:
        write_csv(a.csv, s)
    print(json.dumps(s, indent=1) if a.json else format_text(a.kind, s))
    return 0


if __name__ == "__main__":
    sys.exit(main())
