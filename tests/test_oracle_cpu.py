"""CPU tests of the oracle itself and of the gloo world_size=2 dispatch -> identity expert ->
combine round trip (fp32, 128 tokens/rank, hidden 256, 8 experts, top-2 softmax routing)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gpu_data_transfer_profile_b200.ref import cpu_oracle as O


def test_routing_is_seeded_and_normalised():
    i1, w1 = O.make_routing(64, 16, 4, seed=7)
    i2, w2 = O.make_routing(64, 16, 4, seed=7)
    assert torch.equal(i1, i2) and torch.equal(w1, w2)
    assert i1.shape == (64, 4) and i1.dtype == torch.int64
    torch.testing.assert_close(w1.sum(-1), torch.ones(64))
    assert all(len(set(r.tolist())) == 4 for r in i1)
    iz, _ = O.make_routing(4096, 64, 4, seed=1, zipf_s=1.2)
    cnt = torch.bincount(iz.flatten(), minlength=64).sort(descending=True).values
    assert cnt[0] > 4 * cnt[32]          # skewed


def test_layout_ref_small():
    idx = torch.tensor([[0, 5], [4, 7], [1, -1]])
    pr, pe, inr = O.layout_ref(idx, 8, 2)
    assert pr.tolist() == [2, 2]
    assert pe.tolist() == [1, 1, 0, 0, 1, 1, 0, 1]
    assert inr.tolist() == [[True, True], [False, True], [True, False]]


def test_list_oracle_round_trip_equals_topk_weighted_sum():
    R, T, H, E, K = 2, 128, 256, 8, 2
    xs = [torch.randn(T, H, generator=torch.Generator().manual_seed(r)) for r in range(R)]
    rt = [O.make_routing(T, E, K, 10 + r) for r in range(R)]
    idxs, ws = [a for a, _ in rt], [b for _, b in rt]
    ref = O.dispatch_expert_mode_ref(xs, idxs, ws, E)
    outs = O.combine_ref([r[0] for r in ref], [r[2] for r in ref], [r[3] for r in ref], [T] * R,
                         row_weight=[r[1] for r in ref])
    for s in range(R):
        torch.testing.assert_close(outs[s], xs[s] * ws[s].sum(-1, keepdim=True))
    rk = O.dispatch_rank_mode_ref(xs, idxs, ws, E)
    outs = O.combine_ref([r[0] for r in rk], [r[3] for r in rk], [r[4] for r in rk], [T] * R)
    for s in range(R):
        n_ranks = O.layout_ref(idxs[s], E, R)[2].sum(1, keepdim=True)
        torch.testing.assert_close(outs[s], xs[s] * n_ranks)


def test_fp8_ref_round_trip():
    x = torch.randn(16, 512)
    q, s = O.fp8_block_quant_ref(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (16, 4)
    torch.testing.assert_close(O.fp8_block_dequant_ref(q, s), x, atol=0.3, rtol=0.07)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, H, E, K = 128, 256, 8, 2
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(100 + rank))
        idx, w = O.make_routing(T, E, K, seed=200 + rank)
        d = AllToAll = O.AllToAllTokenDispatcher(dist.group.WORLD, E)
        rows, probs, per_expert = d.dispatch(x, idx, w)
        assert rows.shape[0] == sum(per_expert) and len(per_expert) == E // world
        # every rank must have received exactly the tokens routed to its experts
        all_idx = [torch.empty_like(idx) for _ in range(world)]
        dist.all_gather(all_idx, idx)
        want = [sum(int((i == e).sum()) for i in all_idx) for e in range(rank * 4, rank * 4 + 4)]
        assert per_expert == want
        y = rows * probs[:, None]                      # identity expert, weight applied before combine
        out = d.combine(y)
        torch.testing.assert_close(out, x * w.sum(-1, keepdim=True), atol=1e-5, rtol=1e-5)
        out2 = d.combine(rows, weights=w)              # weighted reduction applied on arrival
        torch.testing.assert_close(out2, out, atol=1e-5, rtol=1e-5)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_gloo_world2_round_trip():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
