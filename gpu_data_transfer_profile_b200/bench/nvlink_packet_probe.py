"""One process, two GPUs: push a buffer from GPU 0 to GPU 1 with the LSU copy kernel (16- and
32-byte accesses) and, as the comparator, with one copy-engine peer memcpy. Prints GB/s per
variant. Meant to be run under `ncu` with the NVLink transmit counters, which split the bytes on
the wire into user data and protocol overhead for the SM kernels (the copy engine is not a kernel
and does not show up there):

    ncu --metrics nvltx__bytes_data_user.sum,nvltx__bytes_data_protocol.sum,nvltx__bytes.sum,gpu__time_duration.sum \
        --clock-control none -k regex:lsu_copy -c 4 python -m gpu_data_transfer_profile_b200.bench.nvlink_packet_probe --nbytes 64M

The reference reaches peer memory the same way (one process, `cudaDeviceEnablePeerAccess`,
`Copy_Engine/nvlink_copy_engine_test.py:495-518`).
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import copy as K
from ..utils.sizes import parse_nbytes


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--nbytes", type=parse_nbytes, default=parse_nbytes("64M"))
    ap.add_argument("--iters", type=int, default=2)
    a = ap.parse_args()
    if torch.cuda.device_count() < 2:
        print(json.dumps(dict(bench="nvlink_packet_probe", skipped="needs two visible GPUs in one process")))
        return 0
    K.enable_peer_access(0, 1)
    src = torch.empty(a.nbytes, dtype=torch.uint8, device="cuda:0").random_(0, 251)
    dst = torch.zeros(a.nbytes, dtype=torch.uint8, device="cuda:1")
    out = dict(bench="nvlink_packet_probe", nbytes=a.nbytes)
    torch.cuda.set_device(0)

    def timed(fn):
        fn()
        torch.cuda.synchronize(0)
        best = 1e9
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return a.nbytes / best / 1e6

    for vec in (16, 32):
        out[f"lsu{vec}_gbs"] = round(timed(lambda: K.lsu_copy(dst, src, a.nbytes, vec_bytes=vec, executor=torch.device("cuda", 0))), 1)
    out["copy_engine_gbs"] = round(timed(lambda: dst.copy_(src, non_blocking=True)), 1)
    torch.cuda.synchronize(1)
    out["check"] = bool(torch.equal(dst.cpu()[:4096], src.cpu()[:4096]) and torch.equal(dst.cpu()[-4096:], src.cpu()[-4096:]))
    print(json.dumps(out))
    return 0 if out["check"] else 2


if __name__ == "__main__":
    raise SystemExit(main())
