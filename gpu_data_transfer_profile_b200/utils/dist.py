"""Rank runtime shared by every CLI: bootstrap, EP sub-groups, scalar reductions, ordered print.

Parity: `get_rank_info/barrier/all_reduce_*` (`Copy_Engine/nvlink_copy_engine_test.py:384-410`),
`init_distributed/create_ep_group/ordered_print/all_ranks_boolean`
(`DeepEP_v1/deepep_v1_dispatch.py:124-154,251-262`). NCCL (or gloo on CPU) carries control
traffic only; payload moves through this library's own kernels.
"""
from __future__ import annotations

import os
import sys
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def env_rank_info() -> Tuple[int, int, int]:
    """(rank, world_size, local_rank) from the torchrun environment; (0, 1, LOCAL_RANK|0) without it."""
    if "RANK" not in os.environ:
        return 0, 1, int(os.environ.get("LOCAL_RANK", "0"))
    return int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))


def parse_cpulist(text: str) -> List[int]:
    """'0-3,8,10-11' (the kernel's cpulist format) -> [0, 1, 2, 3, 8, 10, 11]."""
    out: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.extend(range(int(lo), int(hi or lo) + 1))
    return out


def gpu_local_cpus(device_index: int) -> List[int]:
    """CPUs that the kernel reports as local to the GPU (its PCIe root's NUMA node); [] if unknown."""
    try:
        pr = torch.cuda.get_device_properties(device_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            return parse_cpulist(f.read())
    except Exception:
        return []


def bind_to_gpu_cpus(device_index: int) -> List[int]:
    """Restrict THIS process to the CPUs local to its GPU, so that the pinned host buffers it
    allocates afterwards (first touch) sit on the GPU's NUMA node and host<->device copies do
    not cross the socket interconnect. Only the calling process's CPU affinity changes. Returns
    the CPUs now allowed ([] = left as it was; B200EP_BIND_CPUS=0 switches this off)."""
    if os.environ.get("B200EP_BIND_CPUS", "1") == "0" or not hasattr(os, "sched_setaffinity"):
        return []
    try:
        allowed = set(os.sched_getaffinity(0))
        want = sorted(allowed & set(gpu_local_cpus(device_index)))
        if len(want) < 4 or len(want) == len(allowed):      # unknown, already bound, or too few cores to be worth it
            return []
        os.sched_setaffinity(0, want)
        return want
    except Exception:
        return []


def init_distributed(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Initialise torch.distributed when launched by torchrun; single process otherwise."""
    rank, world, local = env_rank_info()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local % max(torch.cuda.device_count(), 1))
        if world > 1:
            bind_to_gpu_cpus(torch.cuda.current_device())
    if "RANK" in os.environ and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if use_cuda:
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), **kw)
    return rank, world, local


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def barrier(group=None) -> None:
    if is_dist():
        dist.barrier(group=group)


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if (
        torch.cuda.is_available() and is_dist() and dist.get_backend() == "nccl") else torch.device("cpu")


def all_reduce_scalar(x: float, op: str = "max", group=None) -> float:
    if not is_dist():
        return float(x)
    t = torch.tensor([x], dtype=torch.float64, device=_dev())
    dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
                           "sum": dist.ReduceOp.SUM}[op], group=group)
    return float(t.item())


def all_reduce_max_float(x: float, group=None) -> float:
    return all_reduce_scalar(x, "max", group)


def all_reduce_sum_float(x: float, group=None) -> float:
    return all_reduce_scalar(x, "sum", group)


def all_ranks_boolean(ok: bool, group=None) -> bool:
    """True only if every rank passed (MIN-reduce of an int flag)."""
    return all_reduce_scalar(1.0 if ok else 0.0, "min", group) > 0.5


def create_ep_group(ep: int):
    """Contiguous EP groups of `ep` ranks; returns (group or None, ep_rank, group_index).
    Every rank must call this (new_group is collective for all groups)."""
    if not is_dist():
        if ep != 1:
            raise ValueError("--ep > 1 needs a torchrun launch")
        return None, 0, 0
    world, rank = dist.get_world_size(), dist.get_rank()
    if ep <= 0 or world % ep:
        raise ValueError(f"--ep {ep} must divide WORLD_SIZE {world}")
    mine = None
    for g in range(world // ep):
        ranks = list(range(g * ep, (g + 1) * ep))
        grp = dist.new_group(ranks)
        if rank in ranks:
            mine = grp
    return mine, rank % ep, rank // ep


def ordered_print(msg: str, group=None, file=sys.stdout) -> None:
    """Print one message per rank in rank order."""
    if not is_dist():
        print(msg, file=file, flush=True)
        return
    for r in range(dist.get_world_size()):
        if dist.get_rank() == r:
            print(msg, file=file, flush=True)
        dist.barrier()


def shutdown() -> None:
    if is_dist():
        dist.destroy_process_group()


def run_main(main) -> None:
    """Run a CLI `main() -> int` and leave through the interpreter's normal shut-down with its
    return value as the exit code. Only on an exception does the process leave at once (exit code
    1, after printing the traceback with the rank), so that the launcher tears the other ranks
    down instead of letting them wait inside a collective.
    Parity: the top-level handler of `DeepEP_v1/deepep_v1_dispatch.py:384-394`."""
    import traceback
    try:
        code = main()
    except SystemExit as e:
        code = e.code if isinstance(e.code, int) else (0 if e.code is None else 1)
    except BaseException:
        sys.stdout.flush()
        print(f"[rank {os.environ.get('RANK', '0')}] fatal:", file=sys.stderr)
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(1)
    sys.stdout.flush()
    sys.stderr.flush()
    try:
        shutdown()          # no-op when the CLI already destroyed its process group
    except Exception:
        pass
    sys.exit(int(code or 0))
