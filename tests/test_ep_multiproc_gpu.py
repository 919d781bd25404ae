"""Multi-process, multi-GPU checks (one process per GPU, NCCL bootstrap, CUDA-IPC symmetric
memory). Skipped when fewer than 2 GPUs are visible."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(n, script_args, timeout=300, env_extra=None):
    env = dict(os.environ)
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port())] + script_args
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_dispatch_combine_cli_two_or_more_gpus():
    n = min(_ngpu(), 8)
    n -= n % 2
    r = _torchrun(n, ["-m", "gpu_data_transfer_profile_b200.bench.moe_check", "--ep", str(n)])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ALL OK" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_bench_two_gpus():
    r = _torchrun(2, ["bench.py", "--gpus", "2", "--steps", "3", "--warmup", "3"])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert '"check": "ok"' in r.stdout
