"""Host-side failure detection with gloo ranks on CPU: a rank that leaves before a collective
must surface as an error on its peer within the process-group timeout, not as a hang."""
import datetime
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _say(q, msg):
    q.put(msg)
    q.close()
    q.join_thread()          # flush before the process leaves without cleanup


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from gpu_data_transfer_profile_b200.ref.cpu_oracle import AllToAllTokenDispatcher, make_routing
    x = torch.randn(32, 64)
    idx, w = make_routing(32, 4, 2, seed=rank)
    d = AllToAllTokenDispatcher(dist.group.WORLD, 4)
    d.dispatch(x, idx, w)                      # one healthy round
    if rank == 1:
        _say(q, (rank, "left"))                # this rank "fails" between steps: it never joins the second collective
        os._exit(0)
    try:
        d.dispatch(x, idx, w)
        _say(q, (rank, "no error"))
    except Exception as e:
        _say(q, (rank, "error:" + type(e).__name__))
    os._exit(0)


def test_lost_rank_is_reported_within_the_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=90) for _ in procs)
    for p in procs:
        p.join(30)
    assert res[1] == "left"
    assert res[0].startswith("error:"), res
