"""CPU tests of size parsing and traffic-pattern arithmetic."""
import argparse

import pytest

from gpu_data_transfer_profile_b200.utils import patterns as P
from gpu_data_transfer_profile_b200.utils import sizes as S


def test_parse_nbytes_units():
    assert S.parse_nbytes("64K") == 65536
    assert S.parse_nbytes("1M") == 1 << 20
    assert S.parse_nbytes("1G") == 1 << 30
    assert S.parse_nbytes("1.5MiB") == 1572864
    assert S.parse_nbytes("2MB") == 2_000_000
    assert S.parse_nbytes("8kib") == 8192
    assert S.parse_nbytes("4096") == 4096
    assert S.parse_nbytes(123) == 123
    with pytest.raises(ValueError):
        S.parse_nbytes("12Q")
    with pytest.raises(ValueError):
        S.parse_nbytes("abc")


def test_fmt_bytes():
    assert S.fmt_bytes(1024) == "1.00 KiB"
    assert S.fmt_bytes(1536 * 1024) == "1.50 MiB"
    assert S.fmt_bytes(10) == "10.00 B"


def test_size_list_and_offsets():
    assert S.parse_size_list("64K,128K,1M") == (65536, 131072, 1 << 20)
    with pytest.raises(argparse.ArgumentTypeError):
        S.parse_size_list("64K,,1M")
    assert S.contiguous_offsets((10, 20, 30)) == (0, 10, 30)
    sz = S.default_nonuniform_sizes(1 << 20, 4)
    assert len(sz) == 4 and sum(sz) == 1 << 20 and len(set(sz)) == 4
    assert all(s % 16 == 0 for s in sz)
    assert S.pow2_sweep(4096, 65536) == (4096, 8192, 16384, 32768, 65536)
    assert S.parse_gpu_ids("0,2,2,5", 8) == (0, 2, 5)
    with pytest.raises(ValueError):
        S.parse_gpu_ids("9", 8)


def test_choose_pair():
    assert P.choose_pair(3, 8, "ring") == (3, 4)
    assert P.choose_pair(7, 8, "ring") == (7, 0)
    assert P.choose_pair(0, 8, "reverse-ring") == (0, 7)
    assert P.choose_pair(2, 8, "pair") == (2, 3)
    assert P.choose_pair(3, 8, "pair") == (3, 2)
    with pytest.raises(ValueError):
        P.choose_pair(0, 3, "pair")
    with pytest.raises(ValueError):
        P.choose_pair(0, 4, "star")


def test_destination_orders():
    assert P.destination_order(2, 4, rotate=True) == (3, 0, 1)
    assert P.destination_order(2, 4, rotate=False) == (0, 1, 3)
    assert P.rr_destinations(1, 4, "ring") == (2, 3, 0)
    assert P.rr_destinations(1, 4, "reverse-ring") == (0, 3, 2)
    with pytest.raises(ValueError):
        P.rr_destinations(0, 4, "pair")


def test_round_robin_chunks_cover_range_once():
    chunks = P.rr_chunks(100_000, 8192, 7)
    assert sum(c[2] for c in chunks) == 100_000
    assert [c[0] for c in chunks[:9]] == [0, 1, 2, 3, 4, 5, 6, 0, 1]
    assert chunks[-1][1] + chunks[-1][2] == 100_000
    assert P.rr_owner(8192 * 7 + 5, 8192, 7) == 0


@pytest.mark.parametrize("layout", P.LAYOUTS)
def test_gap_layout(layout):
    lay = P.build_layout(layout, (100, 200, 300), gap=64)
    sg = "src" in layout or "both" in layout
    dg = "dst" in layout or "both" in layout
    assert lay.src_offsets == ((0, 164, 428) if sg else (0, 100, 300))
    assert lay.dst_offsets == ((0, 164, 428) if dg else (0, 100, 300))
    assert lay.src_bytes == (728 if sg else 600)
    assert lay.dst_gaps() == ([(100, 64), (364, 64)] if dg else [])


def test_multi_source_plan():
    sizes = P.msrc_sizes(4, 2, 1000)
    plan = P.build_multi_source_plan(1, 4, sizes, source_gap=64)
    assert plan.src_bytes == 2 * 3000 + 64
    assert plan.dst_bytes == (2000, 2000, 2000)
    assert [plan.peer(k) for k in range(3)] == [2, 3, 0]
    b = list(plan.batches())
    assert b[0][2] == [(0, 0, 1000), (3064, 1000, 1000)]
    sizes = P.msrc_sizes(4, 2, 0, destination_sizes=(16, 32, 48))
    assert sizes == ((16, 32, 48), (16, 32, 48))
    sizes = P.msrc_sizes(4, 2, 0, source_sizes=(16, 32))
    assert sizes == ((16, 16, 16), (32, 32, 32))
    with pytest.raises(ValueError):
        P.msrc_sizes(4, 2, 0, source_sizes=(1,))


def test_fill_values_stay_below_sentinels():
    for r in range(16):
        for c in range(40):
            assert P.layout_chunk_value(r, c) < P.SRC_GAP_SENTINEL
            assert P.msrc_chunk_value(r, c, c % 7) < P.SRC_GAP_SENTINEL
    assert P.pair_fill_value(3) != P.pair_prefill_value(3)


def test_variant_selector_uses_nearest_measured_size():
    from gpu_data_transfer_profile_b200.ops import variants as V
    table = {"one-to-one": [{"nbytes": 4096, "variant": "lsu16"}, {"nbytes": 1 << 20, "variant": "tma_staged"},
                            {"nbytes": 1 << 30, "variant": "ce"}]}
    assert V.select("one-to-one", 8192, table) == "lsu16"
    assert V.select("one-to-one", 3 << 20, table) == "tma_staged"
    assert V.select("one-to-one", 1 << 29, table) == "ce"
    with pytest.raises(KeyError):
        V.select("ring-of-fire", 1, table)
    assert V.select("round-robin", 1 << 20) in ("lsu_rr", "tma_rr", "ce_graph")


def test_deep_ep_compat_module_exposes_the_api_the_reference_imports():
    import importlib
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "deep_ep_compat"))
    try:
        deep_ep = importlib.import_module("deep_ep")
        utils = importlib.import_module("deep_ep.utils")
        import torch
        assert deep_ep.topk_idx_t == torch.int64
        for name in ("set_num_sms", "get_dispatch_config", "get_combine_config", "get_dispatch_layout", "dispatch",
                     "combine", "low_latency_dispatch", "low_latency_combine"):
            assert hasattr(deep_ep.Buffer, name)
        cfg = deep_ep.Buffer.get_dispatch_config(8)
        assert cfg.get_nvl_buffer_size_hint(7168 * 2, 8) > 0 and cfg.get_rdma_buffer_size_hint(7168 * 2, 8) == 0
        assert utils.EventOverlap(utils.EventHandle()) is not None
        deep_ep.Buffer.set_num_sms(24)
        with pytest.raises(ValueError):
            deep_ep.Buffer.set_num_sms(0)
    finally:
        sys.path.pop(0)
        sys.modules.pop("deep_ep", None)
        sys.modules.pop("deep_ep.utils", None)


def test_parse_cpulist_and_binding_is_a_no_op_without_a_gpu():
    from gpu_data_transfer_profile_b200.utils import dist as D
    assert D.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert D.parse_cpulist("") == []
    assert D.parse_cpulist("5") == [5]
    import os
    before = os.sched_getaffinity(0)
    assert D.gpu_local_cpus(0) == []            # no GPU here: nothing is known, nothing changes
    assert D.bind_to_gpu_cpus(0) == []
    assert os.sched_getaffinity(0) == before


def test_low_latency_regions_are_aligned_disjoint_and_inside_the_size_hint():
    from gpu_data_transfer_profile_b200.parallel.buffer import _LLCarve
    from gpu_data_transfer_profile_b200.parallel.config import FIXED_BYTES, REGION_ALIGN
    for R, E, M, H, K in [(1, 4, 16, 256, 2), (2, 8, 64, 512, 2), (8, 256, 128, 7168, 8), (4, 16, 48, 1024, 4)]:
        need = _LLCarve.required_bytes(R, E, M, H, K)
        c = _LLCarve(need, R, E, M, H, K)
        sizes = _LLCarve._sizes(R, E, M, H, K)
        spans = []
        for name, sz in sizes.items():
            for p in range(2):
                off = getattr(c, name)[p]
                assert off % REGION_ALIGN == 0 and off >= FIXED_BYTES
                spans.append((off, off + sz))
        spans.sort()
        for (a0, a1), (b0, _) in zip(spans, spans[1:]):
            assert a1 <= b0                                  # no two regions (either parity) overlap
        assert spans[-1][1] <= need
        assert c.count[0] < c.count[1] < FIXED_BYTES          # per-parity count rows live in the control area
        import pytest
        with pytest.raises(ValueError):
            _LLCarve(need - REGION_ALIGN - 1, R, E, M, H, K)


def test_gemm_band_height_follows_the_reduction_length():
    from gpu_data_transfer_profile_b200.ops import gemm as G
    assert G._band_rows(4096, 32 << 20) == 4096               # 32 MiB of 8 KiB rows
    assert G._band_rows(14336, 32 << 20) == 1024              # rounded down to a multiple of 256 rows
    assert G._band_rows(1 << 20, 32 << 20) == 256             # never below one 256-row tile
    assert G._band_rows(4096) == G._band_rows(4096, G.BAND_BYTES)


def test_cumulative_counter_comparison_survives_the_32_bit_wrap():
    """The low-latency arrival counters grow for the life of a buffer; the wait compares modulo
    2^32, so it must stay correct when the target passes 0x7fffffff -> 0x80000000 and 2^32 -> 0."""
    from gpu_data_transfer_profile_b200 import _ext
    reached = _ext.load().counter_reached
    assert reached(5, 5) and reached(6, 5) and not reached(4, 5)
    # target just past the sign bit, counter still just below it: not reached (a signed `>=` says it is)
    assert not reached(0x7FFFFFF0, 0x80000010)
    assert reached(0x80000010, 0x80000010) and reached(0x80000090, 0x80000010)
    assert not reached(0x7FFFFFFF, 0x80000000) and reached(0x80000000, 0x7FFFFFFF)
    # across the unsigned wrap
    assert not reached(0xFFFFFFF0, 0x00000010) and reached(0x00000010, 0xFFFFFFF0)
    assert reached(0x00000010, 0x00000010)


def test_control_area_blocks_have_shape_independent_positions():
    """Flag words are epochs that are never reset, so their offsets must not move when the expert
    count (and with it the size of the count matrices) changes."""
    from gpu_data_transfer_profile_b200.parallel.buffer import _Carve
    a = _Carve(64 << 20, 8, 256, 8, 1024, 2048, 2048)
    b = _Carve(64 << 20, 2, 8, 2, 512, 1024, 1024)
    assert (a.flags, a.pull_info) == (b.flags, b.pull_info)
    assert a.pull_info < a.counts[0] and a.counts[1] < a.ll_ctrl
    assert _Carve(64 << 20, 8, 256, 8, 1024, 2048, 2048, max_recv_rows=100).cap == 100


def test_guard_bands_separate_every_region_and_fit_the_size_hint():
    """Each receive / combine region ends in a guard band of >= 256 bytes that starts exactly at
    the region's last byte + 1, touches nothing else, and the whole layout fits the size hint."""
    from gpu_data_transfer_profile_b200.parallel.buffer import GUARD_BYTES, _Carve
    from gpu_data_transfer_profile_b200.parallel.config import FIXED_BYTES, Config
    for slots, bound in ((True, 0), (False, 0), (False, 3000)):
        cfg = Config(24, num_max_tokens_per_rank=512, num_topk=8, num_experts=64,
                     num_max_recv_tokens=bound, combine_slots=slots)
        nbytes = cfg.get_nvl_buffer_size_hint(2048 * 2, 8)
        c = _Carve(nbytes, 8, 64, 8, 2048, 4096, 4096, max_recv_rows=bound, combine_slots=slots)
        assert c.cap >= (bound or 8 * 512) and c.bytes_used <= nbytes
        spans = []
        for par, d in enumerate(c.regions):
            for name, off in d.items():
                spans.append((off, name, par))
        spans.sort()
        assert len(c.guards) == len(spans) == 16 and spans[0][0] == FIXED_BYTES
        guards = {(name, par): (g0, n) for name, par, g0, n in c.guards}
        for i, (off, name, par) in enumerate(spans):
            g0, n = guards[(name, par)]
            nxt = spans[i + 1][0] if i + 1 < len(spans) else c.bytes_used
            assert off <= g0 and n >= GUARD_BYTES and g0 + n == nxt     # band = [end of region, next region)


def test_fp8_block_quantisation_round_trips_within_e4m3_precision():
    """1x128 row scales and 128x128 weight scales: scale = amax / 448, the quantised block uses the
    full e4m3 range, and dequantisation returns every value within e4m3's relative step (2^-3 of
    the value, plus half the smallest subnormal step of the block)."""
    import torch
    from gpu_data_transfer_profile_b200.ops import gemm as G
    g = torch.Generator().manual_seed(3)
    x = torch.randn(20, 384, generator=g) * torch.logspace(-2, 2, 20)[:, None]
    x[3] = 0                                           # an all-zero row keeps a finite, positive scale
    q, s = G.quantize_rows_1x128(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (20, 3) and bool((s > 0).all())
    back = q.float().view(20, 3, 128) * s[..., None]
    err = (back - x.view(20, 3, 128)).abs()
    bound = x.view(20, 3, 128).abs() * 0.0625 + s[..., None] * 2.0 ** -9
    assert bool((err <= bound * 1.001).all())
    nz = [r for r in range(20) if r != 3]
    assert bool((q.float().view(20, 3, 128)[nz].abs().amax(-1) == 448).all())   # amax maps onto the top code
    w = torch.randn(2, 256, 384, generator=g)
    wq, ws = G.quantize_weights_128x128(w)
    assert ws.shape == (2, 2, 3)
    wb = G.dequantize_weights_128x128(wq, ws)
    assert bool(((wb - w).abs() <= w.abs() * 0.0625 + ws.max() * 2.0 ** -9).all())


def test_ep_cli_argument_validation_names_the_flag():
    import argparse
    from gpu_data_transfer_profile_b200.bench import ep_common as C
    ap = argparse.ArgumentParser()
    C.add_ep_flags(ap)
    base = ["--num-local-tokens", "64", "--token-hidden", "256", "--num-of-experts", "8", "--topk", "2", "--ep", "2"]
    C.validate_args(ap.parse_args(base), 2)
    C.validate_args(ap.parse_args(base), 4)            # EP groups of 2 inside a world of 4
    for edit, world, word in ((["--ep", "3"], 2, "--ep"), (["--topk", "9"], 2, "--topk"),
                              (["--num-of-experts", "7"], 2, "--num-of-experts"),
                              (["--token-hidden", "12"], 2, "16 bytes"),
                              (["--no-async-finish", "--allocate-on-comm-stream"], 2, "--async-finish"),
                              (["--benchmark-iters", "0"], 2, "--benchmark-iters")):
        with pytest.raises(ValueError, match=word):
            C.validate_args(ap.parse_args(base + edit), world)


def test_clock_sample_summary_takes_the_loaded_half_and_names_reasons():
    from gpu_data_transfer_profile_b200.utils.clocks import parse_clock_csv
    head = "index, clocks.sm [MHz], clocks.max.sm [MHz], power.draw [W], active, hw, hwt, swt, swp\n"
    idle = "0, 345, 1965, 180.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"
    busy = "0, 1950, 1965, 900.0, 0x4, Not Active, Not Active, Not Active, Active\n"
    d = parse_clock_csv(head + idle * 3 + busy * 5)
    assert d["sm_mhz"] == 1950 and d["sm_max_mhz"] == 1965 and d["reasons"] == ["sw_power_cap"] and d["samples"] == 8
    hot = "0, 1200, 1965, 950.0, 0x40, Not Active, Active, Not Active, Not Active\n"
    assert "hw_thermal_slowdown" in parse_clock_csv(busy + hot)["reasons"]
    assert parse_clock_csv("garbage\n")["sm_mhz"] is None
