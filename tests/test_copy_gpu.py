"""Single-GPU checks of the copy kernels and the copy-engine submission engine: every result
is compared byte for byte with the source (full-buffer compare, position-dependent data)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _pattern(n, seed=0):
    i = torch.arange(n, device="cuda", dtype=torch.int64)
    return ((i * 131 + seed * 7919 + (i >> 11) * 17) % 251).to(torch.uint8)


@pytest.mark.parametrize("n,vec,off", [(1 << 20, 16, 0), (1 << 20, 32, 0), (12345, 16, 0), (4096 + 48, 32, 16),
                                       (70001, 16, 3)])
def test_lsu_copy(n, vec, off):
    from gpu_data_transfer_profile_b200.ops import copy as K
    src = _pattern(n + 64, 1)[off:off + n]
    base = torch.full((n + 128,), 253, dtype=torch.uint8, device="cuda")
    dst = base[off:off + n]
    K.lsu_copy(dst, src, n, ctas=8, threads=256, iters=2, vec_bytes=vec)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    assert bool((base[off + n:] == 253).all()) and bool((base[:off] == 253).all())


@pytest.mark.parametrize("pull", [False, True])
@pytest.mark.parametrize("n,tile,piece,stages,ctas", [(1 << 20, 32768, 32768, 4, 4), (1 << 20, 65536, 8192, 3, 5),
                                                      (160 * 1024 + 48, 16384, 16384, 2, 3), (4096, 8192, 4096, 2, 2)])
def test_tma_staged_copy(pull, n, tile, piece, stages, ctas):
    from gpu_data_transfer_profile_b200.ops import copy as K
    src = _pattern(n, 2)
    base = torch.full((n + 256,), 253, dtype=torch.uint8, device="cuda")
    st = K.StagedStatus(torch.device("cuda"))
    K.tma_staged_copy([base[:n]], src, n, pull=pull, tile=tile, piece=piece, stages=stages, ctas=ctas,
                      threads=160, iters=3, status=st)
    torch.cuda.synchronize()
    st.check()
    assert torch.equal(base[:n], src)
    assert bool((base[n:] == 253).all())


@pytest.mark.parametrize("method", ["lsu", "tma"])
@pytest.mark.parametrize("n,rr,ndst", [(1 << 20, 8192, 7), (300 * 1024, 4096, 3), (64 * 1024 + 16, 16, 2)])
def test_round_robin_copy(method, n, rr, ndst):
    from gpu_data_transfer_profile_b200.ops import copy as K
    src = _pattern(n, 3)
    dsts = [torch.full((n,), 200 + i, dtype=torch.uint8, device="cuda") for i in range(ndst)]
    if method == "lsu":
        K.lsu_rr_copy(dsts, src, n, rr, ctas=6, threads=256, iters=2)
    else:
        st = K.StagedStatus(torch.device("cuda"))
        K.tma_staged_copy(dsts, src, n, rr_bytes=rr, tile=32768, stages=3, ctas=5, threads=160, iters=2, status=st)
        torch.cuda.synchronize()
        st.check()
    torch.cuda.synchronize()
    off = torch.arange(n, device="cuda")
    for i, d in enumerate(dsts):
        own = ((off // rr) % ndst) == i
        assert torch.equal(d[own], src[own])
        assert bool((d[~own] == 200 + i).all())


def test_staged_rejects_bad_arguments():
    from gpu_data_transfer_profile_b200.ops import copy as K
    src = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    dst = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        K.tma_staged_copy([dst], src, 4090)
    with pytest.raises(ValueError):
        K.tma_staged_copy([dst], src, 4096, tile=4096, piece=8192)
    with pytest.raises(ValueError):
        K.tma_staged_copy([dst], src, 4096, tile=65536, stages=8)
    with pytest.raises(ValueError):
        K.lsu_copy(dst, src, 8192)


@pytest.mark.parametrize("mode", ["separate", "graph", "kernel"])
@pytest.mark.parametrize("proxy", [True, False])
def test_copy_engine_modes(mode, proxy):
    from gpu_data_transfer_profile_b200.ops.copy import CopyEngine
    sizes = [4096, 65536, 100000, 16]
    src = _pattern(sum(sizes) + 3 * 64, 4)
    dst = torch.full((sum(sizes) + 3 * 64,), 253, dtype=torch.uint8, device="cuda")
    copies, o = [], 0
    for s in sizes:
        copies.append((dst.data_ptr() + o, 0, src.data_ptr() + o, 0, s))
        o += s + 64
    eng = CopyEngine(copies, mode, stream_device=0, use_proxy=proxy)
    r = eng.run(5)
    assert r["wall_seconds"] > 0 and eng.bytes_per_iter == sum(sizes)
    o = 0
    for s in sizes:
        assert torch.equal(dst[o:o + s], src[o:o + s])
        assert bool((dst[o + s:o + s + 64] == 253).all()) or o + s + 64 > dst.numel()
        o += s + 64


def test_copy_engine_python_thread_comparator():
    """One runtime call per copy from the Python thread (the reference's submission path):
    same bytes land, gaps stay untouched, a bad index is an error code and not a crash."""
    from gpu_data_transfer_profile_b200.ops.copy import CopyEngine
    sizes = [4096, 100000, 16]
    src = _pattern(sum(sizes) + 3 * 64, 9)
    dst = torch.full((sum(sizes) + 3 * 64,), 253, dtype=torch.uint8, device="cuda")
    copies, o = [], 0
    for s in sizes:
        copies.append((dst.data_ptr() + o, 0, src.data_ptr() + o, 0, s))
        o += s + 64
    eng = CopyEngine(copies, "separate", stream_device=0, use_proxy=False)
    assert eng.run_from_python(3) > 0
    o = 0
    for s in sizes:
        assert torch.equal(dst[o:o + s], src[o:o + s]) and bool((dst[o + s:o + s + 64] == 253).all())
        o += s + 64
    assert eng._eng.enqueue_copy(len(sizes)) != 0 and eng._eng.enqueue_copy(-1) != 0


@pytest.mark.parametrize("mod,extra", [
    ("copy_engine", ["--nbytes", "1M", "--copies-per-iter", "4", "--copy-mode", "batch"]),
    ("copy_engine", ["--nbytes", "256K", "--copies-per-iter", "3", "--non-uniform-copy-size", "--mode", "reverse-ring"]),
    ("layout_copy", ["--nbytes", "64K", "--layout", "both-discontinuous", "--copy-mode", "batch", "--batch-impl", "kernel"]),
    ("layout_copy", ["--nbytes", "64K", "--layout", "dst-discontinuous", "--copy-mode", "separate"]),
    ("sm_copy", ["--nbytes", "1M", "--method", "lsu", "--num-sms", "4", "--persistent-kernel", "--executor", "src"]),
    ("sm_copy", ["--nbytes", "1M", "--method", "tma", "--num-sms", "4", "--executor", "dst", "--tma-tile-bytes", "32K"]),
    ("sm_copy", ["--nbytes", "1M", "--method", "tma", "--num-sms", "3", "--executor", "src", "--copies-per-iter", "2"]),
])
def test_copy_clis_single_process(mod, extra):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, "-m", f"gpu_data_transfer_profile_b200.bench.{mod}", "--iters", "5",
                        "--warmup", "2", "--check"] + extra, cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "check=OK" in r.stdout and "[aggregate]" in r.stdout


def test_lsu_copy_overlapping_launches():
    from gpu_data_transfer_profile_b200.ops import copy as K
    n = 1 << 20
    src = _pattern(n, 9)
    dst = torch.zeros(n, dtype=torch.uint8, device="cuda")
    K.lsu_copy(dst, src, n, ctas=16, threads=512, launches=5, overlap_launches=True)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs in one process")
def test_nvlink_packet_probe_single_process_two_gpus():
    """The probe that is profiled with the NVLink counters: one process pushes from GPU 0 to GPU 1."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "gpu_data_transfer_profile_b200.bench.nvlink_packet_probe", "--nbytes", "4M"],
                       cwd=root, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["check"] and rec["lsu16_gbs"] > 0 and rec["copy_engine_gbs"] > 0
