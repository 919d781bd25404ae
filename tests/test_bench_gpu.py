"""bench.py on one GPU: every flag combination prints ONE JSON line with the contract's keys and
passes its own identity check; the reference arm answers `unavailable` without touching a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches")


def _run(extra):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, "bench.py"] + extra, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--fp8"], ["--zipf", "1.2"], ["--host-count"]])
def test_bench_one_gpu_flags(extra):
    d = _run(["--steps", "3", "--warmup", "3", "--tokens", "1024"] + extra)
    assert all(k in d for k in KEYS), sorted(set(KEYS) - set(d))
    assert d["check"] == "ok" and d["n_gpus"] == 1 and d["steps"] == 3 and d["value"] > 0
    assert d["gpu_launches"] == 12 and d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["value"] > 0
    assert d["higher_is_better"] is False and d["vs_baseline"] is not None


def test_bench_reference_arm_is_unavailable():
    d = _run(["--impl", "reference"])
    assert d["impl"] == "reference" and "unavailable" in d


def test_bench_reference_arm_prints_once_per_job():
    """Launched as several ranks (as the driver does for N > 1), only rank 0 prints the line."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--gpus", "2"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""
