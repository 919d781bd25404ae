"""Profiling driver: runs the two sweeps of the reference's `Copy_Engine/sample_run.sh:4-32`
(fan-out copy 1-10 MiB; address layouts 8K-2048K) and wraps every run in Nsight Systems with the
reference's options (`-s none --cpuctxsw=none --trace=cuda,nvtx --gpu-metrics-devices=0
--gpu-metrics-frequency=10000`) when the `nsys` CLI exists. Without nsys the runs still execute
and append their JSONL records, so the sweep is usable on machines that only have `ncu`.

    python -m gpu_data_transfer_profile_b200.bench.profile_sweep --gpus 8 --out results/
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys


def commands(gpus: int, out: str, iters: int, warmup: int):
    tr = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
          "--master-addr", "127.0.0.1", "--master-port", "29577"]
    pk = "gpu_data_transfer_profile_b200.bench."
    common = ["--iters", str(iters), "--warmup", str(warmup), "--check"]
    for mib in range(1, 11):
        for mode in ("separate", "batch"):
            yield (f"a2a_{mode}_{mib}M", tr + ["-m", pk + "a2a_copy", "--nbytes", f"{mib}M", "--copy-mode", mode,
                                                "--jsonl", os.path.join(out, "a2a.jsonl")] + common)
    for kib in (8, 16, 32, 64, 128, 256, 512, 1024, 2048):
        for layout in ("contiguous", "src-discontinuous", "dst-discontinuous", "both-discontinuous"):
            for mode in ("separate", "batch"):
                yield (f"layout_{layout}_{mode}_4x{kib}K",
                       tr + ["-m", pk + "layout_copy", "--nbytes", f"{kib}K", "--copies-per-iter", "4", "--layout", layout,
                             "--copy-mode", mode, "--jsonl", os.path.join(out, "layout.jsonl")] + common)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--out", default="results")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--gpu-metrics-set", default=None, help="e.g. gb100; omitted when not given")
    ap.add_argument("--dry-run", action="store_true", help="print the command lines only")
    ap.add_argument("--only", default="", help="substring filter on the run name")
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    nsys = shutil.which("nsys")
    rc = 0
    for name, cmd in commands(a.gpus, a.out, a.iters, a.warmup):
        if a.only and a.only not in name:
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
