"""Failure-detection check on real GPUs: one rank stops taking part BETWEEN steps (none of its
kernels in flight, its process and memory stay alive), the others' next dispatch must end with
`EpTimeoutError` after the buffer's short device-side wait limit - not hang. Exit code 0 when
every surviving rank saw the time-out and the GPU context is still usable afterwards.

The reference has no failure handling (a lost peer hangs inside DeepEP or a barrier,
`DeepEP_v1/deepep_v1_dispatch.py:384-394` only prints and re-raises host errors).

    NCCL_NVLS_ENABLE=0 torchrun --nproc-per-node 2 -m gpu_data_transfer_profile_b200.bench.lost_rank_check
"""
from __future__ import annotations

import argparse
import time

import torch
import torch.distributed as dist

from ..parallel.buffer import Buffer, EpTimeoutError
from ..ref.cpu_oracle import make_routing
from ..utils import dist as D


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--leaver", type=int, default=-1, help="rank that stops participating (-1 = last rank)")
    ap.add_argument("--timeout-s", type=float, default=1.0)
    a = ap.parse_args()
    rank, world, _ = D.init_distributed()
    if world < 2:
        raise ValueError("needs at least 2 ranks")
    leaver = a.leaver if a.leaver >= 0 else world - 1
    dev = torch.device("cuda", torch.cuda.current_device())
    T, H, E, K = 256, 512, 4 * world, 2
    cfg = Buffer.get_dispatch_config(world, T, K, E)
    buf = Buffer(dist.group.WORLD, cfg.get_nvl_buffer_size_hint(H * 2, world), 0, timeout_s=a.timeout_s)
    store = dist.distributed_c10d._get_default_store()
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    idx, w = make_routing(T, E, K, seed=rank)
    idx, w = idx.to(dev), w.to(dev)

    def step():
        pr, _, pe, inr, _ = buf.get_dispatch_layout(idx, E)
        rx, _, _, _, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=pr, is_token_in_rank=inr,
                                         num_tokens_per_expert=pe)
        out, _, _ = buf.combine(rx, h)
        return out

    for _ in range(2):                     # healthy steps with everybody
        step()
    torch.cuda.synchronize()
    dist.barrier()
    verdict = "n/a"
    if rank == leaver:
        # leave between steps: nothing of mine is in flight; stay alive so my memory stays mapped
        store.set(f"left_{rank}", "1")
        for r in range(world):
            if r != leaver:
                store.wait([f"done_{r}"])
    else:
        store.wait([f"left_{leaver}"])
        t0 = time.time()
        try:
            step()
            torch.cuda.synchronize()
            buf.check_status()
            verdict = "no error raised"
        except EpTimeoutError as e:
            verdict = f"EpTimeoutError after {time.time() - t0:.2f}s: {e}"
        torch.cuda.synchronize()
        # the context must still work after the time-out
        alive = float((torch.ones(8, device=dev) * 2).sum().item()) == 16.0
        verdict += f" | context usable={alive}"
        store.set(f"done_{rank}", verdict)
    ok = rank == leaver or (verdict.startswith("EpTimeoutError") and verdict.endswith("True"))
    print(f"[rank {rank}] {'left between steps' if rank == leaver else verdict}", flush=True)
    torch.cuda.synchronize()
    # no collective with the "lost" rank's kernels: plain host-side rendezvous, then tear down
    store.set(f"bye_{rank}", "1")
    store.wait([f"bye_{r}" for r in range(world)])
    buf.region.close()
    return 0 if ok else 2


if __name__ == "__main__":
    D.run_main(main)
