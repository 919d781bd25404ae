"""Python front-ends of the copy kernels and of the copy-engine submission engine.

Launch contracts follow the reference's host launchers (uint8 contiguous CUDA tensors at
least `nbytes` long, threads <= 1024, iterations > 0: `LSU_TMA/nvlink_lsu_tma_copy_test.py:278-298`;
staged copies need 16-byte multiples and `tile >= piece`: `:336-376`;
round-robin: `LSU_TMA/nvlink_lsu_tma_round_robin_copy_test.py:548-657`).
All launches go to the current stream of the EXECUTOR device (the device that runs the kernel).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import _ext

MAX_SMEM_OPTIN = 227 * 1024
SEPARATE, GRAPH, KERNEL = 0, 1, 2
CE_MODES = {"separate": SEPARATE, "graph": GRAPH, "batch": GRAPH, "kernel": KERNEL}


def _check_u8(t: torch.Tensor, nbytes: int, name: str):
    if not (t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous()):
        raise ValueError(f"{name} must be a contiguous CUDA uint8 tensor")
    if t.numel() < nbytes:
        raise ValueError(f"{name} is smaller than nbytes")


def sm_count(device=None) -> int:
    return torch.cuda.get_device_properties(device or torch.cuda.current_device()).multi_processor_count


def resolve_num_ctas(num_sms: int, device=None) -> int:
    """0 = one CTA per SM of the executor; otherwise the requested count."""
    if num_sms < 0:
        raise ValueError("--num-sms must be >= 0")
    return sm_count(device) if num_sms == 0 else num_sms


def lsu_copy(dst: torch.Tensor, src: torch.Tensor, nbytes: int, *, ctas: int = 0, threads: int = 256,
             iters: int = 1, vec_bytes: int = 16, executor: Optional[torch.device] = None,
             launches: int = 1, overlap_launches: bool = False) -> None:
    """`iters` repeats the copy inside ONE launch (persistent mode); `launches` repeats the launch
    from a native loop; `overlap_launches` lets consecutive launches overlap (programmatic
    dependent launch) - only for copies that do not depend on each other."""
    _check_u8(dst, nbytes, "dst")
    _check_u8(src, nbytes, "src")
    ex = executor or src.device
    with torch.cuda.device(ex):
        _ext.load().lsu_copy(dst.data_ptr(), src.data_ptr(), nbytes, resolve_num_ctas(ctas, ex),
                             threads, iters, vec_bytes | (256 if overlap_launches else 0), launches)


def lsu_rr_copy(dsts: Sequence[torch.Tensor], src: torch.Tensor, nbytes: int, rr_bytes: int, *,
                ctas: int = 0, threads: int = 256, iters: int = 1, launches: int = 1) -> None:
    _check_u8(src, nbytes, "src")
    for i, d in enumerate(dsts):
        _check_u8(d, nbytes, f"dst[{i}]")
    if rr_bytes <= 0:
        raise ValueError("round-robin chunk size must be positive")
    with torch.cuda.device(src.device):
        _ext.load().lsu_rr_copy([d.data_ptr() for d in dsts], src.data_ptr(), nbytes, rr_bytes,
                                resolve_num_ctas(ctas, src.device), threads, iters, launches)


def check_staged_constraints(nbytes: int, tile: int, piece: int, stages: int, rr_bytes: int = 0,
                             ptrs: Sequence[int] = ()) -> None:
    """Raises ValueError with the violated rule (the bulk-copy engine moves 16-byte multiples
    between 16-byte aligned addresses; all stages must fit in opt-in shared memory)."""
    for name, v in (("nbytes", nbytes), ("tile bytes", tile), ("piece bytes", piece)):
        if v <= 0 or v % 16:
            raise ValueError(f"{name} must be a positive multiple of 16")
    if rr_bytes and rr_bytes % 16:
        raise ValueError("round-robin chunk size must be a multiple of 16")
    if piece > tile:
        raise ValueError("intra (stage) tile must be >= inter (store) tile")
    if not 1 <= stages <= 8:
        raise ValueError("stages must be in [1, 8]")
    if tile * stages > MAX_SMEM_OPTIN:
        raise ValueError(f"stages*tile = {tile * stages} exceeds the {MAX_SMEM_OPTIN}-byte opt-in limit")
    for p in ptrs:
        if p % 16:
            raise ValueError("pointers must be 16-byte aligned")


def pick_stages(tile: int, want: int = 4) -> int:
    return max(1, min(want, MAX_SMEM_OPTIN // tile, 8))


class StagedStatus:
    """Device word that the staged kernels set when one of their bounded waits runs out."""

    def __init__(self, device):
        self.t = torch.zeros(1, dtype=torch.int32, device=device)

    def check(self):
        code = int(self.t.item())
        if code:
            self.t.zero_()
            raise RuntimeError(f"staged copy kernel recorded status {code}")


def tma_staged_copy(dsts: Sequence[torch.Tensor], src: torch.Tensor, nbytes: int, *, pull: bool = False,
                    rr_bytes: int = 0, tile: int = 32768, piece: Optional[int] = None,
                    stages: Optional[int] = None, ctas: int = 0, threads: int = 160, iters: int = 1,
                    status: Optional[StagedStatus] = None, launches: int = 1) -> None:
    """Push (default): `src` local to the executor, `dsts` may be peers. Pull: `src` may be a
    peer, `dsts[0]` is local to the executor."""
    piece = piece or tile
    stages = stages or pick_stages(tile)
    _check_u8(src, nbytes, "src")
    for i, d in enumerate(dsts):
        _check_u8(d, nbytes, f"dst[{i}]")
    check_staged_constraints(nbytes, tile, piece, stages, rr_bytes,
                             [src.data_ptr()] + [d.data_ptr() for d in dsts])
    ex = dsts[0].device if pull else src.device
    with torch.cuda.device(ex):
        _ext.load().tma_staged_copy([d.data_ptr() for d in dsts], src.data_ptr(), nbytes, rr_bytes, pull,
                                    tile, piece, stages, resolve_num_ctas(ctas, ex), threads, iters,
                                    status.t.data_ptr() if status is not None else 0, launches)


class CopyEngine:
    """N copies per iteration submitted by a native loop (optionally on a proxy thread)."""

    def __init__(self, copies: Sequence[tuple], mode: str = "separate", stream_device: int = 0,
                 use_proxy: bool = True, kernel_ctas_per_copy: int = 8, kernel_threads: int = 512):
        """copies: (dst_ptr, dst_dev, src_ptr, src_dev, nbytes)"""
        if mode not in CE_MODES:
            raise ValueError(f"copy mode must be one of {sorted(CE_MODES)}")
        self.mode = mode
        self._eng = _ext.load().CeEngine([tuple(int(v) for v in c) for c in copies], CE_MODES[mode],
                                         stream_device, use_proxy, kernel_ctas_per_copy, kernel_threads)

    def run(self, iters: int) -> dict:
        r = self._eng.run(iters)
        if r["error"]:
            raise RuntimeError(f"{r['where']} failed: {r['error_string']} ({r['error']})")
        return r

    def run_from_python(self, iters: int) -> float:
        """The reference's submission path (`Copy_Engine/nvlink_copy_engine_test.py:551-560`): the
        Python thread makes ONE runtime call per copy, `iters` times over the list, then drains the
        stream once; returns wall seconds. The comparator that shows what the native loop and the
        proxy thread of `run()` buy."""
        import time
        eng, n = self._eng, self._eng.num_copies
        t0 = time.perf_counter()
        for _ in range(iters):
            for i in range(n):
                e = eng.enqueue_copy(i)
                if e:
                    raise RuntimeError(f"peer memcpy failed with CUDA error {e}")
        e = eng.synchronize()
        if e:
            raise RuntimeError(f"stream synchronize failed with CUDA error {e}")
        return time.perf_counter() - t0

    @property
    def bytes_per_iter(self) -> int:
        return self._eng.bytes_per_iter


def enable_peer_access(dev: int, peer: int) -> None:
    C = _ext.load()
    if dev == peer:
        return
    if not C.can_access_peer(dev, peer):
        raise RuntimeError(f"GPU {dev} cannot access GPU {peer}")
    rc = C.enable_peer_access(dev, peer)
    if rc:
        raise RuntimeError(f"cudaDeviceEnablePeerAccess({dev}->{peer}) failed with {rc}")


class MulticastBuffer:
    """A symmetric buffer with an NVSwitch multicast mapping (NVLS), obtained from PyTorch's
    symmetric-memory allocator. `available` is False when the platform offers no multicast
    (single GPU, no NVSwitch, or the allocator cannot exchange handles): callers then fall back
    to unicast variants. Collective: every rank of `group` must construct it."""

    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.available, self.why = False, ""
        self.nbytes = int(nbytes)
        try:
            grp = group if group is not None else dist.group.WORLD
            self.tensor = symm.empty(self.nbytes, dtype=torch.uint8, device=device or torch.device("cuda", torch.cuda.current_device()))
            self.handle = symm.rendezvous(self.tensor, grp)
            self.multicast_ptr = int(self.handle.multicast_ptr)
            self.available = self.multicast_ptr != 0
            if not self.available:
                self.why = "allocator reports no multicast support"
        except Exception as e:  # pragma: no cover - depends on the platform
            self.tensor, self.handle, self.multicast_ptr = None, None, 0
            self.why = f"{type(e).__name__}: {e}"

    def broadcast(self, src: torch.Tensor, nbytes: int, offset: int = 0, *, ctas: int = 0, threads: int = 512,
                  iters: int = 1, launches: int = 1) -> None:
        """Store src[0:nbytes] to [offset, offset+nbytes) of this buffer on EVERY rank."""
        if not self.available:
            raise RuntimeError(f"multicast unavailable: {self.why}")
        _check_u8(src, nbytes, "src")
        if offset % 16 or nbytes % 16 or offset + nbytes > self.nbytes:
            raise ValueError("offset and size must be multiples of 16 inside the buffer")
        _ext.load().multimem_bcast(self.multicast_ptr + offset, src.data_ptr(), nbytes,
                                   resolve_num_ctas(ctas, src.device), threads, iters, launches)

    def barrier(self):
        if self.handle is not None:
            self.handle.barrier()
