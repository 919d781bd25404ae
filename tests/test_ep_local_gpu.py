"""Single-GPU checks of the EP data path with several virtual ranks (one kernel set per rank,
phases run in lock step). Every kernel result is compared with the fp32 PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_data_transfer_profile_b200.ref import cpu_oracle as O


def _mk(R, T, H, E, K, dtype=torch.bfloat16, seed=0, zipf=0.0, uneven=False):
    xs, idxs, ws = [], [], []
    for r in range(R):
        t = T + (7 * r if uneven else 0)
        g = torch.Generator().manual_seed(seed * 100 + r)
        xs.append(torch.randn(t, H, generator=g).to(dtype))
        i, w = O.make_routing(t, E, K, seed * 100 + r, zipf)
        idxs.append(i)
        ws.append(w)
    return xs, idxs, ws


def _group(R, nbytes=256 << 20):
    from gpu_data_transfer_profile_b200.parallel.local import LocalGroup
    return LocalGroup(R, nbytes, timeout_s=2.0)


@pytest.mark.parametrize("R,T,H,E,K", [(1, 64, 256, 8, 2), (2, 128, 256, 8, 2), (4, 200, 512, 32, 4),
                                       (8, 96, 1024, 64, 8)])
def test_layout_matches_oracle(R, T, H, E, K):
    xs, idxs, ws = _mk(R, T, H, E, K)
    g = _group(R, 64 << 20)
    try:
        lays = g.get_dispatch_layout([i.cuda() for i in idxs], E)
        for r in range(R):
            pr, pe, inr = O.layout_ref(idxs[r], E, R)
            assert torch.equal(lays[r][0].cpu(), pr)
            assert lays[r][1] is None
            assert torch.equal(lays[r][2].cpu(), pe)
            assert torch.equal(lays[r][3].cpu(), inr)
        g.check_status()
    finally:
        g.destroy()


@pytest.mark.parametrize("R,T,H,E,K,dtype", [
    (1, 64, 256, 8, 2, torch.bfloat16), (2, 128, 256, 8, 2, torch.bfloat16),
    (4, 200, 512, 32, 4, torch.bfloat16), (8, 96, 1024, 64, 8, torch.bfloat16),
    (2, 128, 256, 8, 2, torch.float32), (4, 33, 384, 16, 3, torch.float16)])
def test_dispatch_combine_rank_mode(R, T, H, E, K, dtype):
    xs, idxs, ws = _mk(R, T, H, E, K, dtype, uneven=True)
    g = _group(R)
    try:
        cx = [x.cuda() for x in xs]
        ci = [i.cuda() for i in idxs]
        cw = [w.cuda() for w in ws]
        lays = g.get_dispatch_layout(ci, E)
        outs = g.dispatch(cx, layouts=lays, topk_idx=ci, topk_weights=cw)
        ref = O.dispatch_rank_mode_ref(xs, idxs, ws, E)
        for d in range(R):
            rx, ri, rw, cnt, h = outs[d]
            ex, ei, ew, sr, stok, ecnt = ref[d]
            assert rx.shape == ex.shape
            assert torch.equal(rx.cpu(), ex)
            assert torch.equal(ri.cpu(), ei)
            assert torch.equal(rw.cpu(), ew)
            assert cnt == ecnt
            assert h.n_recv == ex.shape[0]
        # combine with an "expert" that scales by (1 + rank): checks routing of every row
        ys = [(outs[d][0].float() * (1 + d)).to(dtype) for d in range(R)]
        comb = g.combine(ys, [o[4] for o in outs], topk_weights=[o[2] for o in outs])
        cref = O.combine_ref([y.cpu() for y in ys], [r[3] for r in ref], [r[4] for r in ref],
                             [x.shape[0] for x in xs])
        wref = O.combine_ref([r[2] for r in ref], [r[3] for r in ref], [r[4] for r in ref],
                             [x.shape[0] for x in xs])
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for s in range(R):
            got, got_w = comb[s]
            torch.testing.assert_close(got.cpu().float(), cref[s], atol=tol * 8, rtol=tol)
            torch.testing.assert_close(got_w.cpu(), wref[s], atol=1e-6, rtol=1e-6)
        g.check_status()
        g.check_canaries()
    finally:
        g.destroy()


@pytest.mark.parametrize("R,T,H,E,K", [(1, 64, 256, 8, 2), (2, 128, 256, 8, 2), (4, 100, 512, 32, 4),
                                       (8, 64, 1024, 8, 2)])
def test_dispatch_combine_expert_mode(R, T, H, E, K):
    xs, idxs, ws = _mk(R, T, H, E, K, zipf=1.2)
    g = _group(R)
    try:
        cx = [x.cuda() for x in xs]
        ci = [i.cuda() for i in idxs]
        cw = [w.cuda() for w in ws]
        outs = g.dispatch(cx, topk_idx=ci, topk_weights=cw, group_by_expert=True, num_experts=E)
        ref = O.dispatch_expert_mode_ref(xs, idxs, ws, E)
        for d in range(R):
            rx, _, _, cnt, h = outs[d]
            ex, ep, sr, stok, sk, ecnt = ref[d]
            assert cnt == ecnt
            assert torch.equal(rx.cpu(), ex)
            assert torch.equal(h.recv_prob.cpu(), ep)
        # weighted combine: out[t] = sum_k w[t,k] * x[t]  == x[t] (weights sum to 1)
        comb = g.combine([o[0] for o in outs], [o[4] for o in outs], item_weights=cw)
        for s in range(R):
            torch.testing.assert_close(comb[s][0].cpu().float(), xs[s].float(), atol=3e-2, rtol=2e-2)
        g.check_status()
        g.check_canaries()
    finally:
        g.destroy()


def test_dispatch_fp8_and_cached():
    R, T, H, E, K = 4, 96, 1024, 32, 4
    xs, idxs, ws = _mk(R, T, H, E, K)
    g = _group(R)
    try:
        cx = [x.cuda() for x in xs]
        ci = [i.cuda() for i in idxs]
        cw = [w.cuda() for w in ws]
        lays = g.get_dispatch_layout(ci, E)
        outs = g.dispatch(cx, layouts=lays, topk_idx=ci, topk_weights=cw, use_fp8=True)
        ref = O.dispatch_rank_mode_ref(xs, idxs, ws, E)
        for d in range(R):
            (q, s), _, _, _, h = outs[d]
            eq, es = O.fp8_block_quant_ref(ref[d][0])
            torch.testing.assert_close(s.cpu(), es, rtol=1e-6, atol=0)
            deq = O.fp8_block_dequant_ref(q.cpu(), s.cpu())
            torch.testing.assert_close(deq, ref[d][0].float(), atol=0.3, rtol=0.07)
            assert (q.cpu().view(torch.uint8) != eq.view(torch.uint8)).float().mean() < 0.01
        # cached-handle dispatch of new data reuses the layout
        x2 = [torch.randn_like(x) for x in cx]
        outs2 = g.dispatch(x2, handles=[o[4] for o in outs])
        ref2 = O.dispatch_rank_mode_ref([x.cpu() for x in x2], idxs, ws, E)
        for d in range(R):
            assert torch.equal(outs2[d][0].cpu(), ref2[d][0])
        g.check_status()
    finally:
        g.destroy()


def test_lost_peer_is_an_error_not_a_hang():
    g = _group(1, 8 << 20)
    try:
        assert g.buffers[0].probe_timeout(0.05) == 8
        g.check_status()
    finally:
        g.destroy()


def test_recorded_fault_is_raised_by_the_next_op_without_check_status():
    """A time-out leaves its code in the status word AND in a mapped host word; the next public
    op on the buffer raises it even though nobody called check_status()."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer, EpTimeoutError
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    T, H, E, K = 64, 256, 8, 2
    buf = Buffer(None, 32 << 20, world=LocalWorld.make(1)[0], timeout_s=2.0)
    try:
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 3)
        idx, w = idx.cuda(), w.cuda()
        assert buf.probe_timeout(0.05, clear=False) == 8
        with pytest.raises(EpTimeoutError):
            buf.get_dispatch_layout(idx, E)
        # the fault was consumed: the buffer works again
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        rx, _, _, _, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, is_token_in_rank=inr,
                                         num_tokens_per_expert=pe)
        assert torch.equal(rx, x)
        buf.check_status()
    finally:
        buf.destroy()


def test_cached_dispatch_refuses_a_handle_made_for_another_layout():
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    T, H, E, K = 64, 256, 8, 2
    buf = Buffer(None, 32 << 20, world=LocalWorld.make(1)[0], timeout_s=2.0)
    try:
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 3)
        idx, w = idx.cuda(), w.cuda()
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        _, _, _, _, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, is_token_in_rank=inr,
                                        num_tokens_per_expert=pe)
        y, _, _, _, _, _ = buf.dispatch(x * 2, handle=h)          # same width: fine
        assert torch.equal(y, x * 2)
        with pytest.raises(ValueError):
            buf.dispatch(x.float(), handle=h)                      # wider rows: other layout, smaller capacity
        buf.check_status()
    finally:
        buf.destroy()


def test_receive_bound_overflow_is_a_status_not_a_fault():
    """`num_max_recv_tokens` caps the receive region; a routing that needs more rows ends in
    status 6 and every out-of-range row is skipped."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer, EpStatusError
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    T, H, E, K = 96, 256, 8, 2
    buf = Buffer(None, 32 << 20, world=LocalWorld.make(1)[0], timeout_s=2.0, num_max_recv_tokens=64)
    try:
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 3)
        idx, w = idx.cuda(), w.cuda()
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        with pytest.raises(EpStatusError):
            buf.dispatch(x, topk_idx=idx, topk_weights=w, is_token_in_rank=inr, num_tokens_per_expert=pe)
            buf.check_status()
        torch.cuda.synchronize()
        try:
            buf.check_status()
        except EpStatusError:
            pass
        # a smaller batch fits
        x2, idx2, w2 = x[:48].contiguous(), idx[:48].contiguous(), w[:48].contiguous()
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx2, E)
        rx, _, _, _, h, _ = buf.dispatch(x2, topk_idx=idx2, topk_weights=w2, is_token_in_rank=inr,
                                         num_tokens_per_expert=pe)
        assert torch.equal(rx, x2)
        buf.check_status()
        buf.check_canaries()        # the skipped rows of the overflowing call touched no guard band
    finally:
        buf.destroy()


def test_guard_bands_are_checked_and_a_stray_store_is_named():
    """Every region of the carve ends in a painted guard band; `check_canaries` passes after real
    traffic (receive region filled to its last row) and names the region behind which a byte changed."""
    from gpu_data_transfer_profile_b200.parallel.buffer import CANARY, Buffer, EpStatusError
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    T, H, E, K = 64, 256, 8, 2
    buf = Buffer(None, 32 << 20, world=LocalWorld.make(1)[0], timeout_s=2.0, num_max_recv_tokens=T)
    try:
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 5)
        idx, w = idx.cuda(), w.cuda()
        for _ in range(3):          # both epoch parities; T rows = exactly the capacity
            pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
            rx, _, _, _, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, is_token_in_rank=inr,
                                             num_tokens_per_expert=pe)
            out, _, _ = buf.combine(rx, h)
            assert rx.shape[0] == T == buf._carve.cap
        buf.check_status()
        buf.check_canaries()
        name, parity, off, n = buf._carve.guards[0]
        band = buf.region.view(off, (n,), "uint8")
        assert bool((band == CANARY).all())
        band[7] = 0                 # what a store one row past the region would do
        with pytest.raises(EpStatusError, match=name):
            buf.check_canaries()
        band[7] = CANARY
        buf.check_canaries()
    finally:
        buf.destroy()


@pytest.mark.parametrize("R,T,H,E,K,dtype", [(1, 70, 256, 8, 2, torch.bfloat16), (4, 150, 1024, 32, 4, torch.bfloat16),
                                             (8, 64, 7168, 64, 8, torch.bfloat16), (2, 100, 384, 8, 2, torch.float32)])
def test_pull_combine_reads_rows_in_place_and_matches_the_oracle(R, T, H, E, K, dtype):
    """Zero-copy dispatch output, modified in place by the 'expert', combined by the pull form
    (no slot region): result and reduced side values equal the oracle. Three rounds with
    different data, so a stale cached row from an earlier round would be seen."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    xs, idxs, ws = _mk(R, T, H, E, K, dtype, uneven=True, seed=7)
    g = _group(R)
    try:
        ci, cw = [i.cuda() for i in idxs], [w.cuda() for w in ws]
        for rep in range(3):
            cx = [(x.float() * (1 + rep)).to(dtype).cuda() for x in xs]
            ref = O.dispatch_rank_mode_ref([c.cpu() for c in cx], idxs, ws, E)
            lays = g.get_dispatch_layout(ci, E)
            outs = g.dispatch(cx, layouts=lays, topk_idx=ci, topk_weights=cw, zero_copy=True)
            for d in range(R):
                assert g.buffers[d]._use_pull(outs[d][0], outs[d][2])
                outs[d][0].mul_(1 + d)                       # the "expert": in place, inside the region
            ys = [o[0] for o in outs]
            comb = g.combine(ys, [o[4] for o in outs], topk_weights=[o[2] for o in outs])
            cref = O.combine_ref([(r[0].float() * (1 + d)).to(dtype) for d, r in enumerate(ref)],
                                 [r[3] for r in ref], [r[4] for r in ref], [x.shape[0] for x in xs])
            wref = O.combine_ref([r[2] for r in ref], [r[3] for r in ref], [r[4] for r in ref],
                                 [x.shape[0] for x in xs])
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            for s in range(R):
                got, got_w = comb[s]
                torch.testing.assert_close(got.cpu().float(), cref[s], atol=tol * 16 * (1 + rep), rtol=tol)
                torch.testing.assert_close(got_w.cpu(), wref[s], atol=1e-6, rtol=1e-6)
        # forcing the push form on the same tensors gives the same numbers
        old = Buffer.combine_transport
        Buffer.combine_transport = "push"
        try:
            comb2 = g.combine(ys, [o[4] for o in outs], topk_weights=[o[2] for o in outs])
        finally:
            Buffer.combine_transport = old
        for s in range(R):
            assert torch.equal(comb2[s][0], comb[s][0])
        g.check_status()
    finally:
        g.destroy()


def test_pull_combine_expert_mode_with_item_weights():
    R, T, H, E, K = 4, 100, 512, 32, 4
    xs, idxs, ws = _mk(R, T, H, E, K, zipf=1.2)
    g = _group(R)
    try:
        cx, ci, cw = [x.cuda() for x in xs], [i.cuda() for i in idxs], [w.cuda() for w in ws]
        outs = g.dispatch(cx, topk_idx=ci, topk_weights=cw, group_by_expert=True, num_experts=E, zero_copy=True)
        assert all(g.buffers[d]._use_pull(outs[d][0], None) for d in range(R))
        comb = g.combine([o[0] for o in outs], [o[4] for o in outs], item_weights=cw)
        for s in range(R):
            torch.testing.assert_close(comb[s][0].cpu().float(), xs[s].float(), atol=3e-2, rtol=2e-2)
        g.check_status()
        g.check_canaries()
    finally:
        g.destroy()


def test_dispatch_without_host_sync_num_worst_tokens():
    """num_worst_tokens: outputs sized by the caller's bound, true count only on the device."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    T, H, E, K = 100, 256, 8, 2
    buf = Buffer(None, 32 << 20, world=LocalWorld.make(1)[0], timeout_s=2.0)
    try:
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 3)
        idx, w = idx.cuda(), w.cuda()
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        rx, ri, rw, cnt, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=pr, is_token_in_rank=inr,
                                            num_tokens_per_expert=pe, num_worst_tokens=256, zero_copy=True)
        assert rx.shape == (256, H) and cnt == [] and h.n_recv == 256
        assert int(h.n_recv_dev.item()) == T
        assert torch.equal(rx[:T], x)
        out, _, _ = buf.combine(rx, h)
        torch.testing.assert_close(out.float(), x.float())
        with pytest.raises(ValueError):
            buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=pr, is_token_in_rank=inr,
                         num_tokens_per_expert=pe, num_worst_tokens=1 << 30)
        buf.check_status()
    finally:
        buf.destroy()


def test_dispatch_accepts_caller_quantised_fp8_tuple():
    R, T, H, E, K = 2, 64, 512, 8, 2
    xs, idxs, ws = _mk(R, T, H, E, K)
    g = _group(R, 64 << 20)
    try:
        qs = [O.fp8_block_quant_ref(x) for x in xs]
        ci, cw = [i.cuda() for i in idxs], [w.cuda() for w in ws]
        lays = g.get_dispatch_layout(ci, E)
        outs = g.dispatch([(q.cuda(), s.cuda()) for q, s in qs], layouts=lays, topk_idx=ci, topk_weights=cw)
        ref_q = O.dispatch_rank_mode_ref([q.view(torch.uint8) for q, _ in qs], idxs, ws, E)
        ref_s = O.dispatch_rank_mode_ref([s for _, s in qs], idxs, ws, E)
        for d in range(R):
            (rq, rs), _, _, _, h = outs[d]
            assert rq.dtype == torch.float8_e4m3fn and h.fp8
            assert torch.equal(rq.cpu().view(torch.uint8), ref_q[d][0])
            assert torch.equal(rs.cpu(), ref_s[d][0])
        g.check_status()
    finally:
        g.destroy()


@pytest.mark.parametrize("num_sms", [1, 3, 24, 148])
def test_round_trip_is_independent_of_the_cta_knob(num_sms):
    """Same routing, different numbers of CTAs in the send/reduce kernels: the received rows and the
    combined result must not depend on how the work is cut (shakes out ordering assumptions)."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    R, T, H, E, K = 4, 150, 512, 32, 4
    xs, idxs, ws = _mk(R, T, H, E, K, uneven=True, seed=3)
    old = Buffer.num_sms
    Buffer.set_num_sms(num_sms)
    g = _group(R)
    try:
        cx, ci, cw = [x.cuda() for x in xs], [i.cuda() for i in idxs], [w.cuda() for w in ws]
        ref = O.dispatch_rank_mode_ref(xs, idxs, ws, E)
        for rep in range(2):
            lays = g.get_dispatch_layout(ci, E)
            outs = g.dispatch(cx, layouts=lays, topk_idx=ci, topk_weights=cw)
            for d in range(R):
                assert torch.equal(outs[d][0].cpu(), ref[d][0])
                assert torch.equal(outs[d][1].cpu(), ref[d][1])
            comb = g.combine([o[0] for o in outs], [o[4] for o in outs])
            cref = O.combine_ref([r[0] for r in ref], [r[3] for r in ref], [r[4] for r in ref],
                                 [x.shape[0] for x in xs])
            for s in range(R):
                got = comb[s][0] if isinstance(comb[s], tuple) else comb[s]
                torch.testing.assert_close(got.cpu().float(), cref[s], atol=0.16, rtol=2e-2)
        g.check_status()
    finally:
        g.destroy()
        Buffer.set_num_sms(old)


@pytest.mark.parametrize("R", [2, 4])
def test_fc2_epilogue_combine_addresses_every_virtual_rank(R):
    """The fc2 grouped GEMM's combine epilogue stores each output row into its token's slot on the
    SOURCE rank; with several virtual ranks the slots live in different regions, so the peer
    addressing of the epilogue is exercised on one GPU. Oracle: per-expert fp32 matmul of the
    dispatched rows, summed per token by the list-based combine oracle."""
    T, H, F, E, K = 120, 256, 256, 8, 2
    xs, idxs, ws = _mk(R, T, H, E, K, seed=9)
    El = E // R
    g = _group(R)
    try:
        cx, ci, cw = [x.cuda() for x in xs], [i.cuda() for i in idxs], [w.cuda() for w in ws]
        outs = g.dispatch(cx, topk_idx=ci, topk_weights=cw, group_by_expert=True, num_experts=E)
        ref = O.dispatch_expert_mode_ref(xs, idxs, ws, E)
        torch.manual_seed(1)
        w2s = [(torch.randn(El, H, H, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(R)]
        acts = [o[0] for o in outs]                     # stand-in for the fc1 output: F == H here
        comb = g.fused_fc2_combine(acts, w2s, [o[4] for o in outs])
        ys = []
        for d in range(R):
            ex, ep, sr, stok, sk, ecnt = ref[d]
            rows, r0 = [], 0
            for e, c in enumerate(ecnt):
                rows.append(ex[r0:r0 + c].float() @ w2s[d][e].float().cpu().t())
                r0 += c
            ys.append(torch.cat(rows) if rows else torch.zeros(0, H))
        cref = O.combine_ref(ys, [r[2] for r in ref], [r[3] for r in ref], [x.shape[0] for x in xs])
        for s in range(R):
            torch.testing.assert_close(comb[s].cpu().float(), cref[s], atol=6e-2, rtol=3e-2)
        g.check_status()
    finally:
        g.destroy()


def test_buffer_without_combine_slots_pulls_and_refuses_to_push():
    """`combine_slots=False` halves the region: the zero-copy rows are combined by the pull form,
    a tensor outside the region cannot be combined at all, and the size hint shrinks accordingly."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    T, H, E, K = 100, 512, 8, 2
    full = Buffer.get_dispatch_config(1, T, K, E).get_nvl_buffer_size_hint(H * 2, 1)
    half = Buffer.get_dispatch_config(1, T, K, E, combine_slots=False).get_nvl_buffer_size_hint(H * 2, 1)
    from gpu_data_transfer_profile_b200.parallel.config import FIXED_BYTES
    assert (half - FIXED_BYTES) < 0.6 * (full - FIXED_BYTES)          # the fixed control area aside
    buf = Buffer(None, half, world=LocalWorld.make(1)[0], timeout_s=2.0, combine_slots=False)
    try:
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 3)
        idx, w = idx.cuda(), w.cuda()
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        rx, _, _, _, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, is_token_in_rank=inr,
                                         num_tokens_per_expert=pe, zero_copy=True)
        out, _, _ = buf.combine(rx, h)
        torch.testing.assert_close(out.float(), x.float())
        with pytest.raises(ValueError):
            buf.combine(rx.clone(), h)
        buf.check_status()
    finally:
        buf.destroy()
