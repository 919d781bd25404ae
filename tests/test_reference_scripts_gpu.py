"""API parity: the reference's own DeepEP scripts, UNMODIFIED, import this library through the
`deep_ep` compatibility module and must run to their own "completed successfully" line.

The scripts are not part of this repository. Point `B200EP_REFERENCE_SCRIPTS` at a directory that
holds `DeepEP_v1/deepep_v1_dispatch.py`, `DeepEP_v1/deepep_v1_combine.py` and
`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py` (default: `baseline/_ref` under the repository
root, which is not tracked); the tests are skipped when they are absent. A run of these scripts goes
through THIS library's kernels: it checks the call shapes, it is never a reference measurement.
"""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("B200EP_REFERENCE_SCRIPTS", os.path.join(ROOT, "baseline", "_ref"))
SCRIPTS = {
    "dispatch": os.path.join(REF, "DeepEP_v1", "deepep_v1_dispatch.py"),
    "combine": os.path.join(REF, "DeepEP_v1", "deepep_v1_combine.py"),
    "megatron": os.path.join(REF, "DeepEP_Megatron", "test_deepep_moe_dispatch_combine.py"),
}
SHAPE = ["--num-local-tokens", "256", "--token-hidden", "1024", "--num-of-experts", "16", "--topk", "4", "--ep", "2",
         "--warmup-iters", "2", "--benchmark-iters", "3"]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(script, extra):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "deep_ep_compat"), ROOT, env.get("PYTHONPATH", "")])
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), script] + SHAPE + extra
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("which,extra", [
    ("dispatch", []),
    ("dispatch", ["--no-async-finish", "--no-allocate-on-comm-stream", "--rerandomize-routing-each-iter"]),
    ("combine", []),
    ("combine", ["--dtype", "fp32", "--fake-expert-output", "random"]),
    ("megatron", ["--moe-ffn-hidden-size", "512", "--expert-backend", "torch"]),
    ("megatron", ["--moe-ffn-hidden-size", "512", "--expert-backend", "torch", "--activation", "gelu"]),
])
def test_unmodified_reference_script_runs_on_this_library(which, extra):
    script = SCRIPTS[which]
    if not os.path.exists(script):
        pytest.skip(f"reference script not present: {script}")
    r = _run(script, extra)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "All distributed ranks completed successfully." in r.stdout
    assert "sanity_ok=True" in r.stdout and "sanity_ok=False" not in r.stdout
