"""Profiling driver: runs the two sweeps of the reference's `Copy_Engine/sample_run.sh:4-32`
(fan-out copy 1-10 MiB; address layouts 8K-2048K) and wraps every run in Nsight Systems with the
reference's options (`-s none --cpuctxsw=none --trace=cuda,nvtx --gpu-metrics-devices=0
--gpu-metrics-frequency=10000`) when the `nsys` CLI exists (`--tool nsys`, the default when it is
found). `--tool ncu` is the path for machines that only have Nsight Compute: every run is wrapped
in a ONE-PASS launch list (`ncu --metrics gpu__time_duration.sum --clock-control none --csv`),
which is only done for single-process runs (`--gpus 1`; a multi-rank command is never put under
ncu), and the launch list is reduced to per-kernel count / total / mean microseconds in
`<out>/<name>.kernels.json`. `--tool none` just runs the sweeps and appends their JSONL records.

    python -m gpu_data_transfer_profile_b200.bench.profile_sweep --gpus 8 --out results/
    python -m gpu_data_transfer_profile_b200.bench.profile_sweep --gpus 1 --tool ncu --only a2a_batch_1M --out results/
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import shutil
import subprocess
import sys


def summarize_launch_list(path: str) -> dict:
    """`ncu --csv --metrics gpu__time_duration.sum` log -> {kernel: {launches, total_us, mean_us}}."""
    with open(path, newline="") as f:
        lines = [l for l in f if l.startswith('"')]
    out = {}
    for r in csv.DictReader(lines):
        if r.get("Metric Name") != "gpu__time_duration.sum":
            continue
        try:
            ns = float(r["Metric Value"].replace(",", ""))
        except (KeyError, ValueError):
            continue
        unit = r.get("Metric Unit", "ns")
        us = ns * {"ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6}.get(unit, 1e-3)
        name = r.get("Kernel Name", "?").split("(")[0]
        d = out.setdefault(name, dict(launches=0, total_us=0.0))
        d["launches"] += 1
        d["total_us"] += us
    for d in out.values():
        d["mean_us"] = d["total_us"] / d["launches"]
    return out


def commands(gpus: int, out: str, iters: int, warmup: int, batch_impl: str = "graph"):
    tr = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
          "--master-addr", "127.0.0.1", "--master-port", "29577"]
    pk = "gpu_data_transfer_profile_b200.bench."
    common = ["--iters", str(iters), "--warmup", str(warmup), "--check"]
    for mib in range(1, 11 if gpus >= 2 else 0):           # the fan-out needs a peer: skipped on one GPU
        for mode in ("separate", "batch"):
            yield (f"a2a_{mode}_{mib}M", tr + ["-m", pk + "a2a_copy", "--nbytes", f"{mib}M", "--copy-mode", mode,
                                                "--jsonl", os.path.join(out, "a2a.jsonl")] + common)
    for kib in (8, 16, 32, 64, 128, 256, 512, 1024, 2048):
        for layout in ("contiguous", "src-discontinuous", "dst-discontinuous", "both-discontinuous"):
            for mode in ("separate", "batch"):
                yield (f"layout_{layout}_{mode}_4x{kib}K",
                       tr + ["-m", pk + "layout_copy", "--nbytes", f"{kib}K", "--copies-per-iter", "4", "--layout", layout,
                             "--copy-mode", mode, "--batch-impl", batch_impl,
                             "--jsonl", os.path.join(out, "layout.jsonl")] + common)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--out", default="results")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--gpu-metrics-set", default=None, help="e.g. gb100; omitted when not given")
    ap.add_argument("--tool", choices=("auto", "nsys", "ncu", "none"), default="auto",
                    help="auto: nsys when installed, else none")
    ap.add_argument("--dry-run", action="store_true", help="print the command lines only")
    ap.add_argument("--only", default="", help="substring filter on the run name")
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    nsys = shutil.which("nsys") if a.tool in ("auto", "nsys") else None
    if a.tool == "nsys" and not nsys:
        print("nsys is not installed; use --tool ncu or --tool none", file=sys.stderr)
        return 2
    ncu = shutil.which("ncu") if a.tool == "ncu" else None
    if a.tool == "ncu" and (not ncu or a.gpus != 1):
        print("--tool ncu needs the ncu CLI and --gpus 1 (a multi-rank command is never put under ncu)", file=sys.stderr)
        return 2
    rc = 0
    # under ncu only kernels are listed: a batch is then submitted as ONE SM-kernel launch over a
    # descriptor table instead of a graph of memcpy nodes, so the launch list shows the batch
    for name, cmd in commands(a.gpus, a.out, a.iters, a.warmup, "kernel" if ncu else "graph"):
        if a.only and a.only not in name:
            continue
        if ncu:
            # single rank: run the module directly (no launcher process between ncu and the kernels)
            cmd = [sys.executable] + cmd[cmd.index("-m", 2):]
            log = os.path.join(a.out, name + ".launches.csv")
            print(("[dry-run] " if a.dry_run else "[run] ") + " ".join(cmd), flush=True)
            if not a.dry_run:
                plain = subprocess.run(cmd).returncode          # must succeed without the profiler first
                rc |= plain
                if plain == 0:
                    prof = [ncu, "--metrics", "gpu__time_duration.sum", "--clock-control", "none", "--csv", "--log-file", log]
                    rc |= subprocess.run(prof + cmd).returncode
                    if os.path.exists(log):
                        with open(os.path.join(a.out, name + ".kernels.json"), "w") as f:
                            json.dump(summarize_launch_list(log), f, indent=1)
            continue
        if nsys:
            prof = [nsys, "profile", "-s", "none", "--cpuctxsw=none", "--trace=cuda,nvtx", "--gpu-metrics-devices=0",
                    "--gpu-metrics-frequency=10000", "--force-overwrite", "true", "-o", os.path.join(a.out, name)]
            if a.gpu_metrics_set:
                prof.append(f"--gpu-metrics-set={a.gpu_metrics_set}")
            cmd = prof + cmd
        print(("[dry-run] " if a.dry_run else "[run] ") + " ".join(cmd), flush=True)
        if not a.dry_run:
            rc |= subprocess.run(cmd).returncode
    return rc


if __name__ == "__main__":
    sys.exit(main())
