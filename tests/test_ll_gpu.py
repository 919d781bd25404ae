"""Low-latency dispatch/combine on one GPU with virtual ranks, against the PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_data_transfer_profile_b200.ref import cpu_oracle as O


def _inputs(R, T, H, E, K, seed=0):
    xs, idxs, ws = [], [], []
    for r in range(R):
        g = torch.Generator().manual_seed(seed * 100 + r)
        xs.append(torch.randn(T - r, H, generator=g).to(torch.bfloat16))
        i, w = O.make_routing(T - r, E, K, seed * 100 + r)
        i[0, 0] = -1          # a masked choice must be skipped
        idxs.append(i)
        ws.append(w)
    return xs, idxs, ws


def _unpack(src):
    return (src >> 24) & 0xff, (src & 0xffffff) >> 5, src & 31


# signal_mode: 0 = every send CTA adds 1 on every peer's arrival counter, 1 = the last CTA adds the grid size
@pytest.mark.parametrize("signal_mode", [0, 1])
@pytest.mark.parametrize("R,T,H,E,K,fp8", [(1, 16, 256, 4, 2, False), (2, 32, 512, 8, 2, True),
                                           (4, 48, 1024, 16, 4, True), (8, 24, 512, 32, 8, False)])
def test_low_latency_round_trip(R, T, H, E, K, fp8, signal_mode, monkeypatch):
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.local import LocalGroup
    monkeypatch.setattr(Buffer, "ll_signal_mode", signal_mode)
    M = 64
    g = LocalGroup(R, Buffer.get_low_latency_nvl_size_hint(M, H, R, E, K), timeout_s=2.0)
    try:
        xs, idxs, ws = _inputs(R, T, H, E, K)
        cx, ci, cw = [x.cuda() for x in xs], [i.cuda() for i in idxs], [w.cuda() for w in ws]
        El = E // R
        for rep in range(3):     # repeated calls exercise both epoch parities
            outs = g.low_latency_dispatch(cx, ci, M, E, use_fp8=fp8)
            ys = []
            for d in range(R):
                recv, count, handle = outs[d]
                cnt = count.cpu().tolist()
                want = [sum(int((idxs[s] == d * El + e).sum()) for s in range(R)) for e in range(El)]
                assert cnt == want
                src = handle[0].cpu()
                if fp8:
                    q, sc = recv
                    val = (q.float().view(El, R * M, H // 128, 128) * sc[..., None]).view(El, R * M, H).cpu()
                else:
                    val = recv.float().cpu()
                # every (source, token, k) that chose a local expert appears exactly once among its rows
                for e in range(El):
                    keys = src[e, :cnt[e]].tolist()
                    assert len(set(keys)) == len(keys)
                for e in range(El):
                    s_r, s_t, s_k = _unpack(src[e, :cnt[e]])
                    for j in range(cnt[e]):
                        r_, t_, k_ = int(s_r[j]), int(s_t[j]), int(s_k[j])
                        assert int(idxs[r_][t_, k_]) == d * El + e
                        torch.testing.assert_close(val[e, j], xs[r_][t_].float(),
                                                   atol=0.3 if fp8 else 0, rtol=0.07 if fp8 else 0)
                y = torch.zeros((El, R * M, H), dtype=torch.bfloat16, device="cuda")
                for e in range(El):    # "expert" = scale by (1 + global expert id)
                    y[e, :cnt[e]] = (val[e, :cnt[e]] * (1 + d * El + e)).to(torch.bfloat16).cuda()
                ys.append(y)
            comb = g.low_latency_combine(ys, ci, cw, [o[2] for o in outs])
            for s in range(R):
                scale = (torch.where(idxs[s] >= 0, (1 + idxs[s]).float() * ws[s], torch.zeros_like(ws[s]))).sum(1)
                want = xs[s].float() * scale[:, None]
                torch.testing.assert_close(comb[s].float().cpu(), want, atol=0.6 if fp8 else 0.15,
                                           rtol=0.08 if fp8 else 0.03)
        g.check_status()
    finally:
        g.destroy()


# overlap: the kernels are launched with programmatic stream serialisation (captured as such in the graph)
@pytest.mark.parametrize("overlap", [False, True])
def test_low_latency_cuda_graph_replay(overlap, monkeypatch):
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.local import LocalGroup
    monkeypatch.setattr(Buffer, "ll_overlap_launches", overlap)
    R, T, H, E, K, M = 1, 32, 512, 8, 4, 32
    g = LocalGroup(R, Buffer.get_low_latency_nvl_size_hint(M, H, R, E, K), timeout_s=2.0)
    try:
        b = g.buffers[0]
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 5)
        idx, w = idx.cuda(), w.cuda()
        out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")

        def step():
            recv, count, handle, _, _ = b.low_latency_dispatch(x, idx, M, E, use_fp8=False)
            b.low_latency_combine(recv, idx, w, handle, out=out)

        step()                      # warm-up outside capture (allocations, module load)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for rep in range(4):
            x.copy_(torch.randn(T, H, device="cuda").to(torch.bfloat16))
            out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            torch.testing.assert_close(out.float(), x.float() * w.sum(1, keepdim=True), atol=0.06, rtol=0.03)
        g.check_status()
    finally:
        g.destroy()


@pytest.mark.parametrize("R,T,H,E,K,fp8", [(1, 16, 256, 4, 2, False), (2, 32, 512, 8, 2, True),
                                           (4, 48, 7168, 16, 4, True), (8, 24, 1024, 32, 8, False)])
def test_low_latency_combine_pulls_expert_output_in_place(R, T, H, E, K, fp8):
    """The experts write into the buffer's in-place combine input; combine then loads and reduces
    the K rows of every token straight from the peers' regions. Three rounds with different
    expert scales (both announcement parities, no stale rows)."""
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.local import LocalGroup
    M = 64
    g = LocalGroup(R, Buffer.get_low_latency_nvl_size_hint(M, H, R, E, K), timeout_s=2.0)
    try:
        xs, idxs, ws = _inputs(R, T, H, E, K, seed=3)
        cx, ci, cw = [x.cuda() for x in xs], [i.cuda() for i in idxs], [w.cuda() for w in ws]
        El = E // R
        for rep in range(3):
            outs = g.low_latency_dispatch(cx, ci, M, E, use_fp8=fp8)
            ys = []
            for d in range(R):
                recv, count, handle = outs[d]
                cnt = count.cpu().tolist()
                if fp8:
                    q, sc = recv
                    val = (q.float().view(El, R * M, H // 128, 128) * sc[..., None]).view(El, R * M, H)
                else:
                    val = recv.float()
                y = g.buffers[d].get_next_low_latency_combine_buffer(handle)
                assert g.buffers[d]._ll_is_combine_buffer(y, handle)
                y.fill_(float("nan"))                 # rows that nobody owns must never be read
                for e in range(El):
                    y[e, :cnt[e]] = (val[e, :cnt[e]] * (1 + rep + d * El + e)).to(torch.bfloat16)
                ys.append(y)
            comb = g.low_latency_combine(ys, ci, cw, [o[2] for o in outs])
            for s in range(R):
                scale = (torch.where(idxs[s] >= 0, (1 + rep + idxs[s]).float() * ws[s], torch.zeros_like(ws[s]))).sum(1)
                want = xs[s].float() * scale[:, None]
                torch.testing.assert_close(comb[s].float().cpu(), want, atol=0.8 if fp8 else 0.2,
                                           rtol=0.08 if fp8 else 0.03)
        g.check_status()
    finally:
        g.destroy()


def test_low_latency_pull_combine_under_cuda_graph_replay():
    from gpu_data_transfer_profile_b200.parallel.buffer import Buffer
    from gpu_data_transfer_profile_b200.parallel.local import LocalGroup
    R, T, H, E, K, M = 1, 32, 512, 8, 4, 32
    g = LocalGroup(R, Buffer.get_low_latency_nvl_size_hint(M, H, R, E, K), timeout_s=2.0)
    try:
        b = g.buffers[0]
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = O.make_routing(T, E, K, 5)
        idx, w = idx.cuda(), w.cuda()
        out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")

        def step():
            recv, count, handle, _, _ = b.low_latency_dispatch(x, idx, M, E, use_fp8=False)
            y = b.get_next_low_latency_combine_buffer(handle)
            y.copy_(recv)                                  # identity "expert" writing in place
            b.low_latency_combine(y, idx, w, handle, out=out)

        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for rep in range(4):
            x.copy_(torch.randn(T, H, device="cuda").to(torch.bfloat16))
            out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            torch.testing.assert_close(out.float(), x.float() * w.sum(1, keepdim=True), atol=0.06, rtol=0.03)
        g.check_status()
    finally:
        g.destroy()
