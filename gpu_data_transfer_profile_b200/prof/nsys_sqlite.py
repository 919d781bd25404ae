"""Readers for Nsight Systems SQLite exports: copy-engine events, kernel events, NVLink metrics.

One module replaces the reference's five analyzers
(`Copy_Engine/Results/*/analyze_*.py`, `LSU_TMA/Results/analyze_nvlink_lsu_tma_report.py`) and
keeps their metrics: per-event throughput (bytes/duration, gaps excluded), inter-copy gap, copy
duration, API-end -> copy-start wait, and NVLink RX/TX user-data percent of peak averaged over
the copy/kernel window. Tables read: TARGET_INFO_GPU, ENUM_CUDA_MEMCPY_OPER,
CUPTI_ACTIVITY_KIND_MEMCPY, CUPTI_ACTIVITY_KIND_RUNTIME, CUPTI_ACTIVITY_KIND_KERNEL, StringIds,
PROCESSES, GPU_METRICS, TARGET_INFO_GPU_METRICS.

Parity, by function of `Copy_Engine/Results/nvlink_copy_engine_test/analyze_nvlink_copy_engine_report.py`:
report -> SQLite through `nsys export` (`:107-141`), peer-copy kind and GPU by PCI bus id
(`:156-189`), source copy events joined to their runtime calls (`:191-254`), gap / wait / duration
statistics (`:263-308`), NVLink RX/TX metrics averaged over the copy window (`:310-368`); kernel
events by name for the SM copies as `LSU_TMA/Results/analyze_nvlink_lsu_tma_report.py:216-305`
(name detection, launches with their durations) and `:328-389` (NVLink metrics over the kernel window).
"""
from __future__ import annotations

import re
import shutil
import sqlite3
import subprocess
from collections import defaultdict
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

DEFAULT_BUS_ID = "0000:03:00.0"
# runtime entry points that submit peer copies: one-per-copy, batched (any spelling), graph launch
PEER_API_PATTERNS = ("cudaMemcpyPeerAsync%", "cudaMemcpy%Batch%", "cudaGraphLaunch%", "cudaMemcpyAsync%")
SEPARATE_API, BATCH_API = "cudaMemcpyPeerAsync%", "cudaMemcpy%Batch%"


@dataclass
class CopyEvent:
    start_ns: int
    end_ns: int
    bytes: int
    dst_device_id: Optional[int] = None
    correlation_id: Optional[int] = None
    global_pid: Optional[int] = None
    api_start_ns: Optional[int] = None
    api_end_ns: Optional[int] = None
    api_name: Optional[str] = None

    @property
    def duration_ns(self) -> int:
        return self.end_ns - self.start_ns

    @property
    def throughput_gib_s(self) -> float:
        return self.bytes / (self.duration_ns * 1e-9) / float(1 << 30)


@dataclass
class KernelEvent:
    start_ns: int
    end_ns: int
    name: str
    grid: Tuple[int, int, int] = (0, 0, 0)
    block: Tuple[int, int, int] = (0, 0, 0)

    @property
    def duration_ns(self) -> int:
        return self.end_ns - self.start_ns


# ---- locating the database --------------------------------------------------------------
def resolve_sqlite(report: Path, force_export: bool = False) -> Path:
    """`x.sqlite` is used as is; for `x.nsys-rep` a sibling `x.sqlite` is reused, else exported
    with `nsys export --type sqlite` when the nsys CLI exists."""
    report = Path(report)
    if report.suffix == ".sqlite":
        if not report.exists():
            raise FileNotFoundError(report)
        return report
    sq = report.with_suffix(".sqlite")
    if sq.exists() and not force_export:
        return sq
    nsys = shutil.which("nsys")
    if nsys is None:
        raise RuntimeError(f"{sq} does not exist and the nsys CLI is not installed; export it where nsys is "
                           f"available: nsys export --type sqlite --output {sq} {report}")
    subprocess.run([nsys, "export", "--type", "sqlite", "--force-overwrite", "true", "--output", str(sq),
                    str(report)], check=True)
    return sq


def connect(path: Path) -> sqlite3.Connection:
    conn = sqlite3.connect(str(path))
    conn.row_factory = sqlite3.Row
    return conn


def has_table(conn, name: str) -> bool:
    return conn.execute("SELECT 1 FROM sqlite_master WHERE type='table' AND name=?", (name,)).fetchone() is not None


def find_gpu(conn, bus_id: str = DEFAULT_BUS_ID) -> sqlite3.Row:
    row = conn.execute("SELECT id, cuDevice, name, busLocation FROM TARGET_INFO_GPU WHERE lower(busLocation)=lower(?)",
                       (bus_id,)).fetchone()
    if row is None:
        known = [dict(r) for r in conn.execute("SELECT cuDevice, name, busLocation FROM TARGET_INFO_GPU ORDER BY cuDevice")]
        raise RuntimeError(f"GPU bus id {bus_id!r} not found; known GPUs: {known}")
    return row


def ptop_copy_kind(conn) -> int:
    if has_table(conn, "ENUM_CUDA_MEMCPY_OPER"):
        r = conn.execute("SELECT id FROM ENUM_CUDA_MEMCPY_OPER WHERE name='CUDA_MEMCPY_KIND_PTOP' "
                         "OR label='Peer-to-Peer' LIMIT 1").fetchone()
        if r is not None:
            return int(r[0])
    return 10


# ---- events -----------------------------------------------------------------------------
def load_copy_events(conn, src_device_id: int, api_patterns: Sequence[str] = PEER_API_PATTERNS) -> List[CopyEvent]:
    """Peer-to-peer memcpy activities whose source is `src_device_id`, joined with the runtime call
    that submitted them (same correlation id and process)."""
    if not has_table(conn, "CUPTI_ACTIVITY_KIND_MEMCPY"):
        return []
    like = " OR ".join("s.value LIKE ?" for _ in api_patterns)
    rows = conn.execute(
        f"""
        WITH api AS (
          SELECT r.start, r.end, r.correlationId, p.globalPid, s.value AS apiName
          FROM CUPTI_ACTIVITY_KIND_RUNTIME r JOIN StringIds s ON s.id = r.nameId
          JOIN PROCESSES p ON p.globalPid = r.globalTid - p.pid
          WHERE {like})
        SELECT m.start, m.end, m.bytes, m.dstDeviceId, m.correlationId, m.globalPid,
               api.start AS apiStart, api.end AS apiEnd, api.apiName
        FROM CUPTI_ACTIVITY_KIND_MEMCPY m
        LEFT JOIN api ON api.correlationId = m.correlationId AND api.globalPid = m.globalPid
        WHERE m.copyKind = ? AND m.srcDeviceId = ?
        ORDER BY m.start, m.end""", (*api_patterns, ptop_copy_kind(conn), src_device_id)).fetchall()
    return [CopyEvent(int(r["start"]), int(r["end"]), int(r["bytes"]), r["dstDeviceId"], r["correlationId"],
                      r["globalPid"], r["apiStart"], r["apiEnd"], r["apiName"])
            for r in rows if r["end"] > r["start"]]


def load_runtime_events(conn, api_pattern: str, bytes_per_call: int) -> List[CopyEvent]:
    """Fallback when no peer memcpy activity was recorded: time the runtime calls themselves and
    take the bytes per call from the caller (e.g. parsed from the report's file name)."""
    rows = conn.execute(
        """SELECT r.start, r.end, r.correlationId, s.value AS apiName
           FROM CUPTI_ACTIVITY_KIND_RUNTIME r JOIN StringIds s ON s.id = r.nameId
           WHERE s.value LIKE ? ORDER BY r.start""", (api_pattern,)).fetchall()
    return [CopyEvent(int(r["start"]), int(r["end"]), bytes_per_call, None, r["correlationId"], None,
                      int(r["start"]), int(r["end"]), r["apiName"]) for r in rows if r["end"] > r["start"]]


def count_api_calls(conn, api_pattern: str) -> int:
    return int(conn.execute("SELECT COUNT(*) FROM CUPTI_ACTIVITY_KIND_RUNTIME r JOIN StringIds s ON s.id=r.nameId "
                            "WHERE s.value LIKE ?", (api_pattern,)).fetchone()[0])


def load_kernel_events(conn, device_id: int, name_substr: str) -> List[KernelEvent]:
    if not has_table(conn, "CUPTI_ACTIVITY_KIND_KERNEL"):
        return []
    rows = conn.execute(
        """SELECT k.start, k.end, COALESCE(d.value, s.value) AS name, k.gridX, k.gridY, k.gridZ,
                  k.blockX, k.blockY, k.blockZ
           FROM CUPTI_ACTIVITY_KIND_KERNEL k
           LEFT JOIN StringIds s ON s.id = k.shortName LEFT JOIN StringIds d ON d.id = k.demangledName
           WHERE k.deviceId = ? AND (s.value LIKE ? OR d.value LIKE ?) ORDER BY k.start""",
        (device_id, f"%{name_substr}%", f"%{name_substr}%")).fetchall()
    return [KernelEvent(int(r["start"]), int(r["end"]), r["name"], (r["gridX"], r["gridY"], r["gridZ"]),
                        (r["blockX"], r["blockY"], r["blockZ"])) for r in rows if r["end"] > r["start"]]


def detect_kernel_name(conn, candidates: Sequence[str]) -> Optional[str]:
    for c in candidates:
        if conn.execute("SELECT 1 FROM CUPTI_ACTIVITY_KIND_KERNEL k LEFT JOIN StringIds s ON s.id=k.shortName "
                        "LEFT JOIN StringIds d ON d.id=k.demangledName WHERE s.value LIKE ? OR d.value LIKE ? LIMIT 1",
                        (f"%{c}%", f"%{c}%")).fetchone() is not None:
            return c
    return None


# ---- statistics ---------------------------------------------------------------------------
def _stats(values: Iterable[float], unit_div: float = 1000.0) -> Dict[str, Any]:
    v = [float(x) for x in values]
    if not v:
        return {"count": 0, "average_ns": None, "average_us": None, "min_ns": None, "max_ns": None}
    avg = sum(v) / len(v)
    return {"count": len(v), "average_ns": avg, "average_us": avg / unit_div, "min_ns": min(v), "max_ns": max(v)}


def summarize_gaps(events: Sequence) -> Dict[str, Any]:
    return _stats(events[i].start_ns - events[i - 1].end_ns for i in range(1, len(events)))


def summarize_durations(events: Sequence) -> Dict[str, Any]:
    return _stats(e.duration_ns for e in events)


def summarize_waits(events: Sequence[CopyEvent]) -> Dict[str, Any]:
    return _stats(e.start_ns - e.api_end_ns for e in events if e.api_end_ns is not None)


def summarize_throughput(events: Sequence[CopyEvent]) -> Dict[str, Any]:
    t = [e.throughput_gib_s for e in events]
    total = sum(e.bytes for e in events)
    return {"count": len(t), "average_gib_s": sum(t) / len(t) if t else None, "min_gib_s": min(t) if t else None,
            "max_gib_s": max(t) if t else None, "total_bytes": total}


def summarize_nvlink(conn, t0: Optional[int], t1: Optional[int], peak_gb_s: Optional[float] = None,
                     include_protocol: bool = False) -> Dict[str, Dict[str, Any]]:
    """Average NVLink RX/TX percent-of-peak metric over [t0, t1] (values of one timestamp summed)."""
    if t0 is None or t1 is None or not has_table(conn, "GPU_METRICS"):
        return {}
    flt = "" if include_protocol else "AND ti.metricName LIKE '%User Data%'"
    rows = conn.execute(
        f"""SELECT gm.timestamp AS ts,
                   CASE WHEN ti.metricName LIKE 'NVLink RX%' THEN 'rx' WHEN ti.metricName LIKE 'NVLink TX%' THEN 'tx' END AS dir,
                   SUM(gm.value) AS value
            FROM GPU_METRICS gm JOIN TARGET_INFO_GPU_METRICS ti ON ti.typeId = gm.typeId AND ti.metricId = gm.metricId
            WHERE gm.timestamp BETWEEN ? AND ? AND (ti.metricName LIKE 'NVLink RX%' OR ti.metricName LIKE 'NVLink TX%') {flt}
            GROUP BY gm.timestamp, dir HAVING dir IS NOT NULL ORDER BY gm.timestamp""", (t0, t1)).fetchall()
    vals: Dict[str, List[float]] = defaultdict(list)
    for r in rows:
        vals[r["dir"]].append(float(r["value"]))
    out = {}
    for d in ("rx", "tx"):
        v = vals.get(d, [])
        avg = sum(v) / len(v) if v else None
        out[d] = {"sample_count": len(v), "average_percent_of_peak": avg, "min_percent_of_peak": min(v) if v else None,
                  "max_percent_of_peak": max(v) if v else None}
        if avg is not None and peak_gb_s is not None:
            out[d]["average_gb_s"] = avg / 100.0 * peak_gb_s
    return out


# ---- warm-up trimming / grouping ------------------------------------------------------------
def infer_warmup_skip(n_events: int, warmup: int, timed: int) -> int:
    """Events belonging to warm-up iterations when the trace holds warmup+timed equal iterations."""
    if warmup <= 0 or warmup + timed <= 0:
        return 0
    return int(round(n_events * warmup / float(warmup + timed)))


def group_by_submission(events: Sequence[CopyEvent]) -> List[List[CopyEvent]]:
    """Copies submitted by one runtime call share (process, correlation id)."""
    groups: Dict[Tuple, List[CopyEvent]] = {}
    order: List[Tuple] = []
    for e in events:
        key = (e.global_pid, e.correlation_id)
        if key not in groups:
            groups[key] = []
            order.append(key)
        groups[key].append(e)
    return [groups[k] for k in order]


def trim_warmup(events: Sequence[CopyEvent], *, skip_events: int = 0, skip_iterations: int = 0,
                submissions_per_iteration: int = 1) -> List[CopyEvent]:
    """Drop the first `skip_events` events, or the events of the first `skip_iterations`
    iterations (an iteration = `submissions_per_iteration` runtime submissions)."""
    ev = list(events)
    if skip_iterations > 0:
        groups = group_by_submission(ev)
        keep = groups[skip_iterations * submissions_per_iteration:]
        return [e for g in keep for e in g]
    return ev[skip_events:]


def detect_copy_mode(conn, report_name: str = "") -> str:
    """'batch' or 'separate' from the report's file name, else from which API was called more."""
    n = report_name.lower()
    if "batch" in n and "separate" not in n:
        return "batch"
    if "separate" in n:
        return "separate"
    b, s = count_api_calls(conn, BATCH_API) + count_api_calls(conn, "cudaGraphLaunch%"), count_api_calls(conn, SEPARATE_API)
    return "batch" if b > s else "separate"


_SIZE_IN_NAME = re.compile(r"(\d+(?:\.\d+)?)\s*(k|m|g|kib|mib|gib|kb|mb|gb)(?![a-z])", re.I)


def sizes_in_name(name: str) -> List[int]:
    """All byte sizes that appear in a report file name ('..._4x2048K_...' -> [2097152])."""
    from ..utils.sizes import parse_nbytes
    return [parse_nbytes(m.group(1) + m.group(2)) for m in _SIZE_IN_NAME.finditer(name)]
