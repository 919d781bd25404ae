"""Analyzer unit tests on a synthetic Nsight Systems SQLite export (no GPU, no nsys)."""
import json
import sqlite3

import pytest

from gpu_data_transfer_profile_b200.prof import analyze as A
from gpu_data_transfer_profile_b200.prof import ncu_summary, nsys_sqlite as N, plot as P

BUS = "0000:03:00.0"


def _make_db(path, *, copies, api="cudaMemcpyPeerAsync_v8000", kernels=(), metrics=()):
    c = sqlite3.connect(path)
    c.executescript("""
    CREATE TABLE TARGET_INFO_GPU (id INT, cuDevice INT, name TEXT, busLocation TEXT, uuid TEXT);
    CREATE TABLE ENUM_CUDA_MEMCPY_OPER (id INT, name TEXT, label TEXT);
    CREATE TABLE StringIds (id INT, value TEXT);
    CREATE TABLE PROCESSES (globalPid INT, pid INT, name TEXT);
    CREATE TABLE CUPTI_ACTIVITY_KIND_RUNTIME (start INT, end INT, nameId INT, correlationId INT, globalTid INT);
    CREATE TABLE CUPTI_ACTIVITY_KIND_MEMCPY (start INT, end INT, bytes INT, copyKind INT, srcDeviceId INT,
                                             dstDeviceId INT, correlationId INT, globalPid INT);
    CREATE TABLE CUPTI_ACTIVITY_KIND_KERNEL (start INT, end INT, deviceId INT, shortName INT, demangledName INT,
                                             gridX INT, gridY INT, gridZ INT, blockX INT, blockY INT, blockZ INT);
    CREATE TABLE TARGET_INFO_GPU_METRICS (typeId INT, metricId INT, metricName TEXT);
    CREATE TABLE GPU_METRICS (timestamp INT, typeId INT, metricId INT, value REAL);
    """)
    c.execute("INSERT INTO TARGET_INFO_GPU VALUES (0, 0, 'GPU', ?, 'u')", (BUS,))
    c.execute("INSERT INTO TARGET_INFO_GPU VALUES (1, 1, 'GPU', '0000:04:00.0', 'v')")
    c.execute("INSERT INTO ENUM_CUDA_MEMCPY_OPER VALUES (10, 'CUDA_MEMCPY_KIND_PTOP', 'Peer-to-Peer')")
    c.execute("INSERT INTO StringIds VALUES (1, ?)", (api,))
    c.execute("INSERT INTO StringIds VALUES (2, 'lsu_copy_kernel')")
    c.execute("INSERT INTO PROCESSES VALUES (1000, 7, 'python')")
    for i, (corr, start, end, nbytes, dst, src) in enumerate(copies):
        c.execute("INSERT INTO CUPTI_ACTIVITY_KIND_MEMCPY VALUES (?,?,?,10,?,?,?,1000)", (start, end, nbytes, src, dst, corr))
    for corr in sorted({cp[0] for cp in copies}):
        first = min(cp[1] for cp in copies if cp[0] == corr)
        c.execute("INSERT INTO CUPTI_ACTIVITY_KIND_RUNTIME VALUES (?,?,1,?,1007)", (first - 3000, first - 1000, corr))
    for start, end in kernels:
        c.execute("INSERT INTO CUPTI_ACTIVITY_KIND_KERNEL VALUES (?,?,0,2,2,4,1,1,256,1,1)", (start, end))
    c.execute("INSERT INTO TARGET_INFO_GPU_METRICS VALUES (1, 1, 'NVLink RX Responses User Data [Throughput %]')")
    c.execute("INSERT INTO TARGET_INFO_GPU_METRICS VALUES (1, 2, 'NVLink TX Requests User Data [Throughput %]')")
    c.execute("INSERT INTO TARGET_INFO_GPU_METRICS VALUES (1, 3, 'NVLink TX Requests Protocol Data [Throughput %]')")
    for ts, rx, tx in metrics:
        c.execute("INSERT INTO GPU_METRICS VALUES (?,1,1,?)", (ts, rx))
        c.execute("INSERT INTO GPU_METRICS VALUES (?,1,2,?)", (ts, tx))
        c.execute("INSERT INTO GPU_METRICS VALUES (?,1,3,?)", (ts, 1.0))
    c.commit()
    c.close()


def test_copy_summary_metrics(tmp_path):
    # 4 copies of 1 MiB, 10 us long, 5 us apart, from GPU0; one copy from GPU1 must be ignored
    copies = [(i + 1, 100_000 + i * 15_000, 110_000 + i * 15_000, 1 << 20, 1, 0) for i in range(4)]
    copies.append((99, 100_000, 200_000, 1 << 20, 0, 1))
    db = tmp_path / "ring_1M.sqlite"
    _make_db(db, copies=copies, metrics=[(105_000, 40.0, 42.0), (130_000, 60.0, 58.0), (900_000, 1.0, 1.0)])
    s = A.build_copy_summary(N.connect(db), BUS, peak_gb_s=450.0, skip_warmup_copies=1)
    assert s["total_events"] == 4 and s["event_count"] == 3
    assert s["duration"]["average_us"] == pytest.approx(10.0)
    assert s["gap"]["average_us"] == pytest.approx(5.0)
    assert s["api_to_copy_wait"]["average_us"] == pytest.approx(1.0)
    assert s["throughput"]["average_gib_s"] == pytest.approx((1 << 20) / 10e-6 / (1 << 30))
    assert s["nvlink"]["rx"]["average_percent_of_peak"] == pytest.approx(60.0)   # only the sample inside the window
    assert s["nvlink"]["tx"]["average_gb_s"] == pytest.approx(0.58 * 450.0)
    with pytest.raises(RuntimeError):
        A.build_copy_summary(N.connect(db), "0000:ff:00.0")


def test_a2a_batch_grouping_and_warmup_by_iterations(tmp_path):
    # 3 iterations; each iteration = one batched submission that fans out to 2 peers
    copies = []
    for it in range(3):
        for d in (1, 2):
            s0 = 1_000_000 * (it + 1) + d * 20_000
            copies.append((it + 1, s0, s0 + 8_000, 65536, d, 0))
    db = tmp_path / "a2a_batch_64K.sqlite"
    _make_db(db, copies=copies, api="cudaMemcpy" + "Batched_v1")
    conn = N.connect(db)
    assert N.detect_copy_mode(conn, db.name) == "batch"
    s = A.build_a2a_summary(conn, BUS, report_name=db.name, timed_iterations=2)
    assert s["copy_mode"] == "batch" and s["skipped_warmup_iterations"] == 1
    assert s["event_count"] == 4 and s["api_groups"] == {"count": 2, "events_per_group": 2.0}
    assert s["destinations"] == [1, 2]


def test_layout_infers_warmup_and_msrc_fallback(tmp_path):
    copies = [(i + 1, 10_000 * (i + 1), 10_000 * (i + 1) + 2_000, 8192, 1, 0) for i in range(22)]
    db = tmp_path / "layout_8K.sqlite"
    _make_db(db, copies=copies)
    s = A.build_layout_summary(N.connect(db), BUS, warmup_iterations=10, timed_iterations=100)
    assert s["inferred_warmup_skip"] == 2 and s["event_count"] == 20
    assert N.infer_warmup_skip(110, 10, 100) == 10
    db2 = tmp_path / "msrc_4x128K_batch.sqlite"
    _make_db(db2, copies=[], api="cudaGraphLaunch_v10000")
    c = sqlite3.connect(db2)
    for i in range(5):
        c.execute("INSERT INTO CUPTI_ACTIVITY_KIND_RUNTIME VALUES (?,?,1,?,1007)", (1000 * i, 1000 * i + 400, 500 + i))
    c.commit()
    c.close()
    s2 = A.build_msrc_summary(N.connect(db2), BUS, report_name=db2.name)
    assert s2["event_source"] == "runtime_api_fallback" and s2["event_count"] == 5
    assert s2["throughput"]["total_bytes"] == 5 * 128 * 1024


def test_kernel_summary_and_outputs(tmp_path, capsys):
    db = tmp_path / "lsu_4sms_1M.sqlite"
    _make_db(db, copies=[], kernels=[(1000, 5000), (10_000, 12_000), (20_000, 22_000)],
             metrics=[(11_000, 20.0, 21.0), (21_000, 22.0, 23.0)])
    s = A.build_kernel_summary(N.connect(db), BUS, bytes_per_launch=1 << 20)
    assert s["kernel"] == "lsu_copy_kernel" and s["launches"] == 3 and s["duration"]["count"] == 2
    assert s["average_nvlink_rx_percent"] == pytest.approx(21.0)
    assert s["average_gib_s"] == pytest.approx((1 << 20) / 2e-6 / (1 << 30))
    A.write_csv(str(tmp_path / "k.csv"), s)
    assert "duration_us" in (tmp_path / "k.csv").read_text()
    assert A.main(["kernel", str(db), "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["launches"] == 3
    assert "avg duration" in A.format_text("kernel", s)
    # plot front-end: table always, figures only with matplotlib
    assert P.main(["sm", str(tmp_path), "--out", str(tmp_path / "o")]) == 0
    rows = json.loads((tmp_path / "o" / "sm_summary.json").read_text())
    assert rows and rows[0]["sms"] == 4 and rows[0]["method"] == "lsu"
    # figures are always produced: PNG with matplotlib, else SVG from the built-in renderer
    figs = list((tmp_path / "o").glob("sm_timing.*"))
    assert figs and figs[0].suffix in (".png", ".svg") and figs[0].stat().st_size > 500


def test_svg_renderer_draws_one_polyline_per_curve(tmp_path):
    import xml.dom.minidom as minidom
    rows = [dict(nbytes=1 << (10 + i), gbs=10.0 * (i + 1) * (2 if v == "b" else 1), variant=v) for i in range(5) for v in "ab"]
    out = tmp_path / "f.svg"
    assert P.svg_line_plot(rows, "nbytes", ["gbs"], "variant", "t <&>", "GB/s", out)
    doc = minidom.parse(str(out))
    lines = doc.getElementsByTagName("polyline")
    assert len(lines) == 2 and all(len(l.getAttribute("points").split()) == 5 for l in lines)
    # the highest value sits above the lowest one (y grows downwards in SVG)
    ys = [float(p.split(",")[1]) for p in lines[1].getAttribute("points").split()]
    assert ys[-1] < ys[0]
    assert not P.svg_line_plot([], "nbytes", ["gbs"], None, "t", "y", tmp_path / "e.svg")


def test_report_name_parsing_and_sqlite_resolution(tmp_path):
    m = P.parse_report_name("layout_both-discontinuous_batch_4copies_2048K")
    assert m["nbytes"] == 2048 * 1024 and m["copy_mode"] == "batch" and m["layout"] == "both-discontinuous" and m["copies"] == 4
    assert N.sizes_in_name("x_10M_y_8KiB") == [10 << 20, 8192]
    with pytest.raises((RuntimeError, FileNotFoundError)):
        N.resolve_sqlite(tmp_path / "missing.nsys-rep")


def test_ncu_raw_summary(tmp_path):
    p = tmp_path / "raw.csv"
    p.write_text('==PROF== noise\n"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum","launch__registers_per_thread"\n'
                 '"","","ns","byte","byte","register/thread"\n'
                 '"0","grouped_gemm_kernel<1>","2000000","1000000000","500000000","146"\n')
    rows = ncu_summary.summarize(ncu_summary.read_raw(str(p)), "grouped_gemm", flops=2.4e12, peaks={"bf16_tflops": 1600.0, "hbm_gbs": 6500.0})
    assert len(rows) == 1 and rows[0]["tflops"] == pytest.approx(1200.0)
    assert rows[0]["dram_gb_s"] == pytest.approx(750.0) and rows[0]["frac_of_measured_bf16_peak"] == pytest.approx(0.75)
    # ncu chooses the unit per column: the same launch reported in ms and Mbyte reads the same
    p.write_text('"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum"\n'
                 '"","","ms","Gbyte","Mbyte"\n"0","grouped_gemm_kernel<1>","2.0","1.0","500"\n')
    rows = ncu_summary.summarize(ncu_summary.read_raw(str(p)), "grouped_gemm", flops=2.4e12)
    assert rows[0]["tflops"] == pytest.approx(1200.0) and rows[0]["dram_gb_s"] == pytest.approx(750.0)


def test_profile_sweep_reduces_an_ncu_launch_list(tmp_path):
    """The ncu path of the profiling driver: a one-pass launch list becomes per-kernel totals."""
    from gpu_data_transfer_profile_b200.bench.profile_sweep import summarize_launch_list
    log = tmp_path / "run.launches.csv"
    log.write_text(
        '==PROF== Connected to process 1\n'
        '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
        '"0","1","python","h","b200ep::batched_copy_kernel(const CopyDesc *, int)","1","7","(256, 1, 1)","(8, 7, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","12,000"\n'
        '"1","1","python","h","b200ep::batched_copy_kernel(const CopyDesc *, int)","1","7","(256, 1, 1)","(8, 7, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","8,000"\n'
        '"2","1","python","h","void at::fill_kernel<int>(int)","1","7","(256, 1, 1)","(8, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","3.5"\n')
    res = summarize_launch_list(str(log))
    k = res["b200ep::batched_copy_kernel"]
    assert k["launches"] == 2 and abs(k["total_us"] - 20.0) < 1e-9 and abs(k["mean_us"] - 10.0) < 1e-9
    assert abs(res["void at::fill_kernel<int>"]["total_us"] - 3.5) < 1e-9


def test_profile_sweep_dry_run_with_ncu_tool_refuses_multi_rank(capsys):
    import sys
    from gpu_data_transfer_profile_b200.bench import profile_sweep as P
    argv = sys.argv
    try:
        sys.argv = ["profile_sweep", "--gpus", "8", "--tool", "ncu", "--dry-run", "--out", "/tmp/_ps_out"]
        assert P.main() == 2
    finally:
        sys.argv = argv


def test_profile_sweep_command_lists():
    """Eight GPUs: the reference's two sweeps (fan-out 1-10 MiB x 2 modes, 9 sizes x 4 layouts x 2
    modes). One GPU: no fan-out runs (they need a peer); under ncu a batch is one SM-kernel launch."""
    from gpu_data_transfer_profile_b200.bench.profile_sweep import commands
    full = list(commands(8, "out", 100, 10))
    assert len(full) == 10 * 2 + 9 * 4 * 2
    assert sum(n.startswith("a2a_") for n, _ in full) == 20 and "--nproc-per-node=8" in full[0][1]
    one = list(commands(1, "out", 5, 2, "kernel"))
    assert len(one) == 72 and all(n.startswith("layout_") for n, _ in one)
    name, cmd = one[1]
    assert name == "layout_contiguous_batch_4x8K"
    assert cmd[cmd.index("--batch-impl") + 1] == "kernel" and cmd[cmd.index("--copy-mode") + 1] == "batch"
    assert cmd[cmd.index("--iters") + 1] == "5" and "--check" in cmd
