"""Symmetric memory: one region per rank, mapped into every rank of the group.

Two worlds share one interface:

* `ProcessWorld(group)` — one process per GPU (the deployment shape). The region is a plain
  device allocation exported with CUDA IPC; handles travel through `torch.distributed`
  (`all_gather_object`, so NCCL or gloo both work) and every peer is opened once.
  The reference instead lets one process own tensors on several GPUs and reaches them after
  `cudaDeviceEnablePeerAccess` (`Copy_Engine/nvlink_copy_engine_test.py:495-518`).
* `LocalWorld(n, device)` — n virtual ranks inside one process on one GPU. Peer pointers are
  ordinary device pointers. Used to exercise the multi-rank data path on a single GPU:
  kernels that wait for a peer are then launched only after the kernels they wait for
  (all ranks' send phases first, then all receive phases), never concurrently.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _ext


class SymmetricRegion:
    """`bytes` of zero-initialised device memory on this rank plus the mapped peers."""

    def __init__(self, world, nbytes: int):
        self.world = world
        self.nbytes = int(nbytes)
        self.C = _ext.load()
        self.device = world.device
        with torch.cuda.device(self.device):
            self.local_ptr = self.C.symm_alloc(self.nbytes)
        self._views = {}
        self.peer_ptrs: List[int] = world._map_peers(self)
        self._opened = [p for i, p in enumerate(self.peer_ptrs)
                        if world.is_remote(i) and p != self.local_ptr]

    def view(self, offset: int, shape, dtype: str) -> torch.Tensor:
        """Tensor over region bytes. Views are cached by (offset, shape, dtype): a steady-state loop
        asks for the same few views every step, and wrapping a pointer costs microseconds."""
        key = (int(offset), tuple(shape), dtype)
        t = self._views.get(key)
        if t is None:
            if len(self._views) > 256:
                self._views.clear()
            t = self.C.view_tensor(self.local_ptr + int(offset), list(shape), dtype, self.device.index)
            self._views[key] = t
        return t

    def close(self):
        """Unmap the peers, then free this rank's allocation. The CUDA runtime leaves it undefined
        what happens when an exported allocation is freed while another process still has it
        mapped, so every rank first closes its mappings of the peers, all ranks meet on the host,
        and only then does anyone free."""
        self._views = {}
        if self.local_ptr:
            for p in self._opened:
                self.C.ipc_close(p)
            if self._opened:
                self.world.host_barrier()       # every importer has closed before any exporter frees
            self._opened = []
            self.C.symm_free(self.local_ptr)
            self.local_ptr = 0


class ProcessWorld:
    """One rank per process; `group` is a torch.distributed process group (or None = WORLD)."""

    def __init__(self, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.local = False

    def is_remote(self, i: int) -> bool:
        return i != self.rank

    def _map_peers(self, region: SymmetricRegion) -> List[int]:
        handle = region.C.ipc_export(region.local_ptr)
        handles = [None] * self.size
        dist.all_gather_object(handles, (handle, region.nbytes), group=self.group)
        sizes = sorted({n for _, n in handles})
        if len(sizes) != 1:
            raise ValueError(f"symmetric region size differs across ranks: {sizes}; every rank must "
                             "pass the same num_nvl_bytes")
        handles = [h for h, _ in handles]
        out = []
        with torch.cuda.device(self.device):
            for i, h in enumerate(handles):
                out.append(region.local_ptr if i == self.rank else region.C.ipc_open(h))
        return out

    def host_barrier(self):
        dist.barrier(group=self.group)


class LocalWorld:
    """n virtual ranks in this process on one device. Create one per virtual rank with a
    shared `registry` list; regions are matched by creation order."""

    def __init__(self, rank: int, size: int, registry: list, device: Optional[torch.device] = None):
        self.rank, self.size = rank, size
        self.registry = registry            # list of per-region lists of pointers
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.group = None
        self.local = True
        self._n_regions = 0

    @staticmethod
    def make(size: int, device: Optional[torch.device] = None) -> List["LocalWorld"]:
        reg: list = []
        return [LocalWorld(r, size, reg, device) for r in range(size)]

    def is_remote(self, i: int) -> bool:
        return False

    def _map_peers(self, region: SymmetricRegion) -> List[int]:
        idx = self._n_regions
        self._n_regions += 1
        while len(self.registry) <= idx:
            self.registry.append([0] * self.size)
        slot = self.registry[idx]
        slot[self.rank] = region.local_ptr
        return slot  # shared list: complete once every virtual rank has allocated

    def host_barrier(self):
        pass
