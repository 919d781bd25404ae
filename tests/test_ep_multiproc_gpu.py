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


EP_ARGS = ["--num-local-tokens", "512", "--token-hidden", "1024", "--num-of-experts", "16", "--topk", "4",
           "--warmup-iters", "2", "--benchmark-iters", "3"]


@pytest.mark.parametrize("mod,extra", [
    ("dispatch", []), ("dispatch", ["--use-fp8", "--zipf", "1.2", "--no-async-finish", "--no-allocate-on-comm-stream"]),
    ("combine", []), ("combine", ["--dtype", "fp32", "--fake-expert-output", "random"]),
    ("moe", ["--moe-ffn-hidden-size", "512", "--expert-backend", "torch", "--dispatcher-mode", "deepep"]),
    ("moe", ["--moe-ffn-hidden-size", "512", "--expert-backend", "tcgen05", "--fuse-combine"]),
    ("moe", ["--moe-ffn-hidden-size", "512", "--expert-backend", "tcgen05", "--backward"]),
])
def test_ep_clis_single_gpu(mod, extra):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, "-m", f"gpu_data_transfer_profile_b200.bench.{mod}", "--ep", "1"] + EP_ARGS + extra,
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "check=OK" in r.stdout and '"check": true' in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("mod,extra", [
    ("dispatch", []), ("combine", []), ("nccl_baseline", []),
    ("moe", ["--moe-ffn-hidden-size", "512", "--expert-backend", "tcgen05", "--fuse-combine"]),
    ("moe", ["--moe-ffn-hidden-size", "512", "--expert-backend", "tcgen05", "--backward"]),
])
def test_ep_clis_two_gpus(mod, extra):
    r = _torchrun(2, ["-m", f"gpu_data_transfer_profile_b200.bench.{mod}", "--ep", "2"] + EP_ARGS + extra)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert '"check": true' in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("mod,extra", [
    ("copy_engine", ["--nbytes", "1M", "--copies-per-iter", "4", "--copy-mode", "batch"]),
    ("a2a_copy", ["--nbytes", "256K", "--rotate-destination-order"]),
    ("layout_copy", ["--nbytes", "64K", "--layout", "both-discontinuous"]),
    ("msrc_copy", ["--nbytes", "128K", "--num-source-buffers", "3"]),
    ("sm_copy", ["--nbytes", "1M", "--method", "tma", "--executor", "src", "--num-sms", "4", "--persistent-kernel"]),
    ("sm_copy", ["--nbytes", "1M", "--method", "lsu", "--executor", "dst", "--num-sms", "4"]),
    ("rr_copy", ["--nbytes", "1M", "--method", "tma", "--num-sms", "4", "--tma-tile-bytes", "32K"]),
    ("rr_copy", ["--nbytes", "1M", "--method", "lsu", "--num-sms", "4", "--persistent-kernel"]),
])
def test_copy_clis_two_gpus(mod, extra):
    r = _torchrun(2, ["-m", f"gpu_data_transfer_profile_b200.bench.{mod}", "--iters", "5", "--warmup", "2", "--check"] + extra)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "check=OK" in r.stdout and "check=FAIL" not in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_multimem_fanout_two_gpus():
    """Switch-multicast broadcast: exit code 3 = the platform offers no multicast mapping (not a failure)."""
    r = _torchrun(2, ["-m", "gpu_data_transfer_profile_b200.bench.a2a_copy", "--copy-mode", "multimem", "--nbytes", "1M",
                      "--iters", "5", "--warmup", "2", "--check"])
    assert r.returncode in (0, 3), r.stdout[-3000:] + r.stderr[-3000:]
    if r.returncode == 0:
        assert "check=OK" in r.stdout and "check=FAIL" not in r.stdout
    else:
        assert "multimem unavailable" in r.stdout
