"""Tables and plots from a directory of analysed reports or from the benchmarks' JSONL records.

    python -m gpu_data_transfer_profile_b200.prof.plot copy   RESULTS_DIR --out OUT_DIR
    python -m gpu_data_transfer_profile_b200.prof.plot a2a | layout | copies-per-iter | msrc | msrc-dst-sizes | sm ...
    python -m gpu_data_transfer_profile_b200.prof.plot jsonl  sweep.jsonl --x nbytes --y aggregate_gib_s --series copy_mode

Parity: the seven plotters under `Copy_Engine/Results/*/plot_*.py` and
`LSU_TMA/Results/plot_nvlink_lsu_tma_sm_summary.py` (discover `.sqlite` files by name, call the
sibling analyzer, print the values table, write throughput / gap+duration / NVLink RX-TX
figures): size from the file name and report discovery as
`Copy_Engine/Results/nvlink_copy_engine_test/plot_nvlink_copy_engine_summary.py:90-128`, the three
figure kinds as `:130-273`, SM-count / method classification of the SM-copy reports as
`LSU_TMA/Results/plot_nvlink_lsu_tma_sm_summary.py:132-207` and its values table `:284-297`. The table (stdout + CSV + JSON) is always produced. Figures are PNG files when
matplotlib is installed (Agg backend, CPU rasterisation); without it the same line plots are
written as SVG files by a small built-in renderer, so a machine with nothing but Python still
gets its figures.
"""
from __future__ import annotations

import argparse
import csv
import json
import re
import sys
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence

from . import analyze as A
from . import nsys_sqlite as N

_SIZE = re.compile(r"(\d+(?:\.\d+)?)(k|m|g|kib|mib|gib)(?![a-z])", re.I)


def parse_report_name(name: str) -> Dict[str, Any]:
    """Pull the knobs that the sweep scripts encode in file names: size, copy mode, layout,
    copies per iteration, SM count, method."""
    low = name.lower()
    out: Dict[str, Any] = {"name": name}
    sizes = N.sizes_in_name(name)
    if sizes:
        out["nbytes"] = sizes[-1]
    out["copy_mode"] = "batch" if "batch" in low and "separate" not in low else ("separate" if "separate" in low else None)
    for lay in ("both-discontinuous", "src-discontinuous", "dst-discontinuous", "contiguous"):
        if lay in low or lay.replace("-", "_") in low:
            out["layout"] = lay
            break
    m = re.search(r"(\d+)\s*(?:copies|x)(?![a-z0-9])", low)
    if m:
        out["copies"] = int(m.group(1))
    m = re.search(r"(\d+)\s*sms?(?![a-z])", low)
    if m:
        out["sms"] = int(m.group(1))
    out["method"] = "tma" if "tma" in low else ("lsu" if "lsu" in low else None)
    out["round_robin"] = "rr" in re.split(r"[_\-.]", low) or "round" in low
    return out


def _have_matplotlib():
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt  # noqa: F401
        return True
    except Exception:
        return False


_COLOURS = ("#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf")


def _curves(rows, x, ys, series):
    """[(label, [(x, y), ...])] in the order both renderers draw them."""
    out = []
    keys = sorted({r.get(series) for r in rows}, key=str) if series else [None]
    for k in keys:
        sel = sorted((r for r in rows if (not series or r.get(series) == k) and r.get(x) is not None), key=lambda r: r[x])
        for y in ys:
            pts = [(float(r[x]), float(r[y])) for r in sel if r.get(y) is not None]
            if pts:
                label = " ".join(str(v) for v in (k, y if len(ys) > 1 else None) if v is not None) or y
                out.append((label, pts))
    return out


def _fmt_tick(v: float, is_bytes: bool) -> str:
    if is_bytes:
        for unit, sz in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
            if v >= sz:
                return f"{v / sz:g}{unit}"
    return f"{v:g}"


def svg_line_plot(rows: List[Dict[str, Any]], x: str, ys: Sequence[str], series: Optional[str], title: str,
                  ylabel: str, path: Path, logx: bool = True) -> bool:
    """Dependency-free renderer: one polyline with markers and value labels per curve, log2 or
    linear x axis, linear y axis from 0, legend on the right. Returns False when nothing is
    plottable."""
    import math
    from xml.sax.saxutils import escape
    curves = _curves(rows, x, ys, series)
    if not curves:
        return False
    xs = [p[0] for _, pts in curves for p in pts]
    ymax = max(p[1] for _, pts in curves for p in pts) or 1.0
    use_log = logx and min(xs) > 0
    fx = (lambda v: math.log2(v)) if use_log else (lambda v: v)
    x0, x1 = fx(min(xs)), fx(max(xs))
    if x1 == x0:
        x0, x1 = x0 - 1, x1 + 1
    W, H, L, R, T, B = 960, 540, 70, 220, 40, 60
    px = lambda v: L + (fx(v) - x0) / (x1 - x0) * (W - L - R)
    py = lambda v: H - B - v / (ymax * 1.08) * (H - T - B)
    el = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="11">',
          f'<rect width="{W}" height="{H}" fill="white"/>',
          f'<text x="{(L + W - R) / 2}" y="22" text-anchor="middle" font-size="15">{escape(title)}</text>',
          f'<text x="{(L + W - R) / 2}" y="{H - 14}" text-anchor="middle">{escape(x)}</text>',
          f'<text transform="translate(16,{(T + H - B) / 2}) rotate(-90)" text-anchor="middle">{escape(ylabel)}</text>']
    step = 10 ** math.floor(math.log10(ymax * 1.08 / 4)) if ymax > 0 else 1.0
    step = next(m * step for m in (1, 2, 5, 10) if ymax * 1.08 / (m * step) <= 8)
    v = 0.0
    while v <= ymax * 1.08:
        el.append(f'<line x1="{L}" y1="{py(v):.1f}" x2="{W - R}" y2="{py(v):.1f}" stroke="#ddd"/>')
        el.append(f'<text x="{L - 6}" y="{py(v) + 4:.1f}" text-anchor="end">{v:g}</text>')
        v += step
    ticks = sorted(set(xs))
    if len(ticks) > 14:
        ticks = ticks[::math.ceil(len(ticks) / 14)]
    for t in ticks:
        el.append(f'<line x1="{px(t):.1f}" y1="{H - B}" x2="{px(t):.1f}" y2="{H - B + 5}" stroke="black"/>')
        el.append(f'<text x="{px(t):.1f}" y="{H - B + 18}" text-anchor="middle">{_fmt_tick(t, x in ("nbytes", "bytes"))}</text>')
    el.append(f'<rect x="{L}" y="{T}" width="{W - L - R}" height="{H - T - B}" fill="none" stroke="black"/>')
    for i, (label, pts) in enumerate(curves):
        c = _COLOURS[i % len(_COLOURS)]
        el.append(f'<polyline fill="none" stroke="{c}" stroke-width="1.6" points="' +
                  " ".join(f"{px(a):.1f},{py(b):.1f}" for a, b in pts) + '"/>')
        for a, b in pts:
            el.append(f'<circle cx="{px(a):.1f}" cy="{py(b):.1f}" r="2.6" fill="{c}"/>')
            el.append(f'<text x="{px(a):.1f}" y="{py(b) - 6:.1f}" text-anchor="middle" font-size="8">{b:.3g}</text>')
        ly = T + 14 + 16 * i
        el.append(f'<line x1="{W - R + 12}" y1="{ly - 4}" x2="{W - R + 36}" y2="{ly - 4}" stroke="{c}" stroke-width="2"/>')
        el.append(f'<text x="{W - R + 42}" y="{ly}">{escape(label)}</text>')
    el.append("</svg>")
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text("\n".join(el))
    return True


def line_plot(rows: List[Dict[str, Any]], x: str, ys: Sequence[str], series: Optional[str], title: str,
              ylabel: str, path: Path, logx: bool = True) -> bool:
    """PNG through matplotlib when it is installed, else the same figure as `<path>.svg`."""
    if not _have_matplotlib():
        return svg_line_plot(rows, x, ys, series, title, ylabel, path.with_suffix(".svg"), logx)
    import matplotlib.pyplot as plt
    fig, ax = plt.subplots(figsize=(8, 4.5))
    keys = sorted({r.get(series) for r in rows}, key=str) if series else [None]
    for k in keys:
        sel = sorted((r for r in rows if (not series or r.get(series) == k) and r.get(x) is not None), key=lambda r: r[x])
        for y in ys:
            pts = [(r[x], r[y]) for r in sel if r.get(y) is not None]
            if pts:
                label = " ".join(str(v) for v in (k, y if len(ys) > 1 else None) if v is not None) or y
                ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", label=label)
                for px, py in pts:
                    ax.annotate(f"{py:.3g}", (px, py), textcoords="offset points", xytext=(0, 5), fontsize=7, ha="center")
    if logx:
        ax.set_xscale("log", base=2)
    ax.set_xlabel(x)
    ax.set_ylabel(ylabel)
    ax.set_title(title)
    ax.grid(True, alpha=0.3)
    ax.legend(fontsize=8)
    fig.tight_layout()
    fig.savefig(path, dpi=130)
    plt.close(fig)
    return True


def write_table(rows: List[Dict[str, Any]], out: Path, stem: str) -> None:
    out.mkdir(parents=True, exist_ok=True)
    cols: List[str] = []
    for r in rows:
        for k in r:
            if k not in cols:
                cols.append(k)
    with open(out / f"{stem}.csv", "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=cols)
        w.writeheader()
        for r in rows:
            w.writerow(r)
    (out / f"{stem}.json").write_text(json.dumps(rows, indent=1))
    print(" | ".join(cols))
    for r in rows:
        print(" | ".join("" if r.get(c) is None else (f"{r[c]:.4g}" if isinstance(r[c], float) else str(r[c])) for c in cols))


def _flatten(meta: Dict[str, Any], s: Dict[str, Any]) -> Dict[str, Any]:
    row = dict(meta)
    if "kernel" in s:
        row.update(kernel=s["kernel"], duration_us=s["duration"]["average_us"], nvlink_rx=s["average_nvlink_rx_percent"],
                   nvlink_tx=s["average_nvlink_tx_percent"], gib_s=s["average_gib_s"])
        return row
    row.update(throughput_gib_s=s["throughput"]["average_gib_s"], gap_us=s["gap"]["average_us"],
               duration_us=s["duration"]["average_us"], wait_us=s["api_to_copy_wait"]["average_us"],
               nvlink_rx=s.get("nvlink", {}).get("rx", {}).get("average_percent_of_peak"),
               nvlink_tx=s.get("nvlink", {}).get("tx", {}).get("average_percent_of_peak"))
    if "copy_mode" in s and not row.get("copy_mode"):
        row["copy_mode"] = s["copy_mode"]
    return row


def collect(results_dir: Path, builder: Callable[..., Dict[str, Any]], **kw) -> List[Dict[str, Any]]:
    rows = []
    for sq in sorted(Path(results_dir).glob("*.sqlite")):
        conn = N.connect(sq)
        try:
            extra = {"report_name": sq.name} if "report_name" in builder.__code__.co_varnames else {}
            rows.append(_flatten(parse_report_name(sq.stem), builder(conn, **extra, **kw)))
        except Exception as e:  # one bad report should not hide the others
            print(f"[skip] {sq.name}: {e}", file=sys.stderr)
        finally:
            conn.close()
    return rows


KINDS = {
    "copy": (A.build_copy_summary, "nbytes", None, "copy-engine ring copy"),
    "a2a": (A.build_a2a_summary, "nbytes", "copy_mode", "fan-out copy-engine copy"),
    "layout": (A.build_layout_summary, "nbytes", "layout", "batch address layout"),
    "copies-per-iter": (A.build_layout_summary, "nbytes", "copies", "equal total bytes, different copies per iteration"),
    "msrc": (A.build_msrc_summary, "nbytes", "copy_mode", "multi-source all-to-all batched copy"),
    "msrc-dst-sizes": (A.build_msrc_summary, "name", None, "multi-source, destination-indexed sizes"),
    "sm": (A.build_kernel_summary, "sms", "method", "SM copy kernels vs SM count"),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kind", choices=list(KINDS) + ["jsonl"])
    ap.add_argument("path", type=Path)
    ap.add_argument("--out", type=Path, default=None)
    ap.add_argument("--gpu-bus-id", default=N.DEFAULT_BUS_ID)
    ap.add_argument("--nvlink-peak-gb-s", type=float, default=None)
    ap.add_argument("--x", default="nbytes")
    ap.add_argument("--y", default="aggregate_gib_s")
    ap.add_argument("--series", default=None)
    a = ap.parse_args(argv)
    out = a.out or (a.path if a.path.is_dir() else a.path.parent)
    if a.kind == "jsonl":
        rows = [json.loads(l) for l in a.path.read_text().splitlines() if l.strip()]
        write_table(rows, out, a.path.stem + "_table")
        ok = line_plot(rows, a.x, [a.y], a.series, a.path.stem, a.y, out / f"{a.path.stem}_{a.y}.png",
                       logx=a.x in ("nbytes", "bytes"))
        print(f"[plot] {'figure written' if ok else 'no plottable rows'}" + ("" if _have_matplotlib() else " (SVG: matplotlib not installed)"))
        return 0
    builder, x, series, title = KINDS[a.kind]
    rows = collect(a.path, builder, bus_id=a.gpu_bus_id, peak_gb_s=a.nvlink_peak_gb_s)
    if not rows:
        print("no .sqlite reports found", file=sys.stderr)
        return 1
    write_table(rows, out, f"{a.kind}_summary")
    logx = x == "nbytes"
    made = [
        line_plot(rows, x, ["gib_s" if a.kind == "sm" else "throughput_gib_s"], series, f"{title}: throughput", "GiB/s",
                  out / f"{a.kind}_throughput.png", logx),
        line_plot(rows, x, ["duration_us"] if a.kind == "sm" else ["gap_us", "duration_us"], series,
                  f"{title}: gap and duration", "microseconds", out / f"{a.kind}_timing.png", logx),
        line_plot(rows, x, ["nvlink_rx", "nvlink_tx"], series, f"{title}: NVLink RX/TX", "% of peak",
                  out / f"{a.kind}_nvlink.png", logx),
    ]
    print(f"[plot] {sum(made)} figure(s) written" + ("" if _have_matplotlib() else " as SVG (matplotlib not installed)"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
