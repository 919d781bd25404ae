"""`Buffer`: the DeepEP-style expert-parallel communication object.

API parity (call shapes taken from the reference's call sites):
  `Buffer(group, num_nvl_bytes, num_rdma_bytes)`, `.group/.num_nvl_bytes/.num_rdma_bytes`
      `DeepEP_v1/deepep_v1_dispatch.py:35-56`
  `Buffer.set_num_sms`, `Buffer.get_dispatch_config`, `Buffer.get_combine_config`
      `DeepEP_v1/deepep_v1_dispatch.py:40-45,271`
  `get_dispatch_layout`, `dispatch` (fresh and cached-handle), `combine`
      `DeepEP_v1/deepep_v1_dispatch.py:199-230`, `DeepEP_v1/deepep_v1_combine.py:241-247`,
      `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:107-132,158-165,200-206`

How it works here (all data-path work is in the sm_100a kernels under csrc/ep):
  1. `notify_send`  counts + stable positions of every item, count vectors stored to all peers.
  2. `notify_wait`  bounded wait for the peers' counts, prefix sums -> exact destination rows;
                    N_recv goes to pinned host memory (no device synchronise).
  3. `dispatch_send` one pass over the local tokens: optional fp8 1x128 cast, 16-byte LSU
                    stores straight into the final row of each destination's receive region.
  4. bounded wait for the peers' done-flags; outputs are views (zero-copy) or clones.
  Combine pushes rows back into per-item slots on the source and reduces them there.
  Regions are double-buffered by epoch parity, flags are monotonically increasing epochs.

Each op is split into phases (`_dispatch_p1/_p2/_p3`, `_combine_p1/_p2`) so that several
virtual ranks living on ONE GPU (`LocalWorld`) can be driven phase by phase.
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .. import _ext
from ..utils.sizes import align_up
from .config import Config, FIXED_BYTES, REGION_ALIGN
from .events import EventHandle, EventOverlap
from .symm import LocalWorld, ProcessWorld, SymmetricRegion

STATUS_TEXT = {
    0: "ok", 1: "timeout waiting for peers' token counts (notify)",
    2: "timeout waiting for peers' dispatch-done flags", 3: "timeout waiting for peers' combine-done flags",
    4: "timeout waiting for low-latency counts", 5: "timeout in barrier",
    6: "receive region overflow (buffer too small for this routing)", 7: "expert index out of range",
    8: "self-test wait timed out (expected)", 9: "timeout on an in-kernel mbarrier",
    10: "combine slot overflow",
}


class EpTimeoutError(RuntimeError):
    pass


class EpStatusError(RuntimeError):
    pass


@dataclass
class DispatchHandle:
    """Everything combine / cached dispatch need. Opaque to callers."""
    mode: int                      # 0 rank mode, 1 expert mode
    T: int
    H: int
    K: int
    E: int
    n_recv: int
    send_row: torch.Tensor         # [T,J] int32 row at the destination (-1 = not sent)
    send_slot: torch.Tensor        # [T,J] int32 slot in my combine region (-1 = none)
    meta: torch.Tensor             # int32 device metadata (counts, prefixes, chunk boundaries)
    recv_meta: torch.Tensor        # [n_recv,2] int32 {slot at source, source rank}
    topk_idx: Optional[torch.Tensor]
    is_token_in_rank: Optional[torch.Tensor]
    num_recv_tokens_per_expert_list: List[int] = field(default_factory=list)
    fp8: bool = False
    recv_prob: Optional[torch.Tensor] = None
    carve_key: tuple = ()                  # region layout that the rows / slots refer to
    cap: int = 0                           # receive capacity (rows) of that layout

    @property
    def n_recv_dev(self) -> torch.Tensor:
        return self.meta[0:1]


class _Carve:
    """Byte offsets of every region for one (E, K, H, row bytes, combine row bytes) shape.

    The control area starts with the blocks whose position must never depend on the shape (flag
    words are epochs that only grow, so a word must not be reused for anything else): channel
    flags and the pull-combine announcements. The count matrices follow."""

    def __init__(self, nbytes: int, R: int, E: int, K: int, H: int, row_bytes: int, comb_row_bytes: int,
                 max_recv_rows: int = 0, combine_slots: bool = True):
        C = _ext.load()
        self.key = (E, K, H, row_bytes, comb_row_bytes)
        self.flags = 0
        off = align_up(C.NUM_CHANNELS * C.MAX_RANKS * 4, REGION_ALIGN)
        self.pull_info = off
        off = align_up(off + C.MAX_RANKS * 4 * 8, REGION_ALIGN)
        csz = align_up(R * (R + E) * 4, REGION_ALIGN)
        self.counts = (off, off + csz)
        off += 2 * csz
        self.ll_ctrl = off
        if off > FIXED_BYTES // 2:
            raise ValueError("too many experts/ranks for the fixed control area")
        self.scale_cols = max(H // 128, 1)
        sizes = dict(recv_x=row_bytes, recv_scales=self.scale_cols * 4, recv_topk_idx=K * 8,
                     recv_topk_w=K * 4, recv_meta=8, recv_prob=4,
                     comb_x=comb_row_bytes if combine_slots else 0, comb_w=K * 4 if combine_slots else 0)
        self.combine_slots = bool(combine_slots)
        per_row = sum(sizes.values())
        avail = nbytes - FIXED_BYTES - 2 * len(sizes) * (REGION_ALIGN + GUARD_BYTES)
        self.cap = max(avail // (2 * per_row), 0)
        if max_recv_rows > 0:
            self.cap = min(self.cap, int(max_recv_rows))
        # without slots the slot numbers that dispatch computes are never used as addresses
        self.slot_cap = self.cap if combine_slots else (1 << 30)
        self.regions = []  # per parity: dict name -> offset
        # Every region is followed by a guard band of at least GUARD_BYTES that no kernel may
        # write: (region name, parity, first byte, length). `Buffer.check_canaries` verifies them.
        self.guards = []
        off = FIXED_BYTES
        for parity in range(2):
            d = {}
            for name, sz in sizes.items():
                d[name] = off
                end = off + self.cap * sz
                off = align_up(end + GUARD_BYTES, REGION_ALIGN)
                self.guards.append((name, parity, end, off - end))
            self.regions.append(d)
        assert off <= nbytes or self.cap == 0
        self.bytes_used = off
        self._lists = {}

    def region_list(self, notify_parity: int, dispatch_parity: int, combine_parity: int):
        key = (notify_parity, dispatch_parity, combine_parity)
        out = self._lists.get(key)
        if out is None:
            d, c = self.regions[dispatch_parity], self.regions[combine_parity]
            out = [self.flags, self.counts[notify_parity], d["recv_x"], d["recv_scales"],
                   d["recv_topk_idx"], d["recv_topk_w"], d["recv_meta"], d["recv_prob"],
                   c["comb_x"], c["comb_w"], self.pull_info]
            self._lists[key] = out
        return out


GUARD_BYTES = 256              # canary band after every receive / combine region
CANARY = 0xA5
_NULL_CONTEXT = contextlib.nullcontext()
_ELEM_DTYPE = {torch.bfloat16: "bfloat16", torch.float16: "float16", torch.float32: "float32"}
_STATUS_MIRROR_SLOT = 4000     # int index inside the mapped host block that mirrors the status word


def _nvtx(name):
    """NVTX range around a public op so that profiler timelines show dispatch / combine blocks
    (the reference relies on a dedicated stream for readability, `Copy_Engine/nvlink_copy_engine_test.py:528-530`)."""
    def deco(fn):
        import functools

        @functools.wraps(fn)
        def wrapped(*a, **k):
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*a, **k)
            finally:
                torch.cuda.nvtx.range_pop()
        return wrapped
    return deco


class Buffer:
    num_sms: int = 24
    # How combine moves the rows. "push": every rank stores its rows into slots on the source,
    # which then reduces the slots. "pull": the rows stay where they are and the source LOADS and
    # reduces them in one pass; possible when the rows (and the side values, if any) lie inside
    # the symmetric region, e.g. the zero-copy output of dispatch or `combine_input()`.
    # "auto" pulls whenever that is the case. Every rank of the group must take the same path.
    combine_transport: str = "auto"

    # ---- static configuration --------------------------------------------------------
    @staticmethod
    def set_num_sms(n: int) -> None:
        if n <= 0:
            raise ValueError("num_sms must be positive")
        Buffer.num_sms = int(n)

    @staticmethod
    def get_dispatch_config(group_size: int, num_max_tokens_per_rank: int = 4096, num_topk: int = 8,
                            num_experts: int = 256, group_by_expert: bool = False,
                            num_max_recv_tokens: int = 0, combine_slots: bool = True) -> Config:
        return Config(Buffer.num_sms, num_max_tokens_per_rank, num_topk, num_experts,
                      group_by_expert=group_by_expert, num_max_recv_tokens=num_max_recv_tokens,
                      combine_slots=combine_slots)

    @staticmethod
    def get_combine_config(group_size: int, num_max_tokens_per_rank: int = 4096, num_topk: int = 8,
                           num_experts: int = 256, group_by_expert: bool = False,
                           num_max_recv_tokens: int = 0, combine_slots: bool = True) -> Config:
        return Config(Buffer.num_sms, num_max_tokens_per_rank, num_topk, num_experts,
                      group_by_expert=group_by_expert, num_max_recv_tokens=num_max_recv_tokens,
                      combine_slots=combine_slots)

    # ---- construction ----------------------------------------------------------------
    def __init__(self, group=None, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 low_latency_mode: bool = False, num_qps_per_rank: int = 1, *,
                 world=None, timeout_s: float = 20.0, blocks_per_sm: int = 2,
                 num_max_recv_tokens: int = 0, combine_slots: bool = True):
        self.C = _ext.load()
        self.world = world if world is not None else ProcessWorld(group)
        self.group = group
        self.rank, self.group_size = self.world.rank, self.world.size
        if self.group_size > self.C.MAX_RANKS:
            raise ValueError(f"group size {self.group_size} exceeds {self.C.MAX_RANKS}")
        self.num_nvl_bytes = int(num_nvl_bytes)
        self.num_rdma_bytes = int(num_rdma_bytes)   # accepted, unused inside one NVLink domain
        self.low_latency_mode = low_latency_mode
        self.device = self.world.device
        self.timeout_s = float(timeout_s)
        self.blocks_per_sm = blocks_per_sm
        self.num_max_recv_tokens = int(num_max_recv_tokens)
        self.combine_slots = bool(combine_slots)
        if self.num_nvl_bytes < FIXED_BYTES + REGION_ALIGN:
            raise ValueError("num_nvl_bytes too small; use Config.get_nvl_buffer_size_hint")
        self.region = SymmetricRegion(self.world, self.num_nvl_bytes)
        self.host_word = self.C.host_mapped_alloc(4 * 4096)
        with torch.cuda.device(self.device):
            # status block: [0] first fault code, [2..3] address of the host word that mirrors it
            self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
            self.status.view(torch.int64)[1] = self.host_word + 4 * _STATUS_MIRROR_SLOT
            self.counters = torch.zeros(8, dtype=torch.int32, device=self.device)
            self._ctr = [self.counters[i:i + 1] for i in range(8)]     # views made once, not per call
            self._side_stream = (torch.cuda.current_stream() if self.world.local
                                 else torch.cuda.Stream(device=self.device))
            self.comm_stream = None
        self._async_outstanding = False
        # One launch may both send and wait for peers only when no other rank shares this GPU.
        self._single_launch = (not self.world.local) or self.group_size == 1
        self._ws = {}
        self._layout_ws = None
        self._epoch = dict(notify=0, dispatch=0, combine=0, barrier=0, ll_dispatch=0, ll_combine=0)
        self._carve: Optional[_Carve] = None
        self._ll = None
        self._ll_words = None
        self.world.host_barrier()

    def destroy(self):
        if getattr(self, "region", None) is not None:
            torch.cuda.synchronize(self.device)
            self.world.host_barrier()
            self.region.close()
            self.region = None
            self.C.host_mapped_free(self.host_word)
            self.host_word = 0

    # ---- helpers ---------------------------------------------------------------------
    @property
    def peers(self) -> List[int]:
        return self.region.peer_ptrs

    @property
    def status_ptr(self) -> int:
        return self.status.data_ptr()

    @property
    def bytes_reserved(self) -> int:
        """Bytes of the symmetric region that the current shape actually uses (both parities)."""
        return self._carve.bytes_used if self._carve is not None else FIXED_BYTES

    def _timeout_ns(self) -> int:
        return int(self.timeout_s * 1e9)

    def _blocks(self) -> int:
        return max(1, Buffer.num_sms * self.blocks_per_sm)

    def _clear_status(self) -> None:
        self.status[0:2].zero_()
        self.counters.zero_()
        self.C.host_write_i32(self.host_word, _STATUS_MIRROR_SLOT, 0)

    @staticmethod
    def _raise_status(code: int):
        cls = EpTimeoutError if code in (1, 2, 3, 4, 5, 8, 9) else EpStatusError
        raise cls(f"b200ep status {code}: {STATUS_TEXT.get(code, 'unknown')}")

    def check_status(self) -> None:
        """Synchronising read of the device status word; raises on any recorded fault."""
        code = int(self.status[0].item())
        if code != 0:
            self._clear_status()
            self._raise_status(code)

    def _poll_status(self) -> None:
        """Non-synchronising check: a kernel that records a fault also copies the code to a mapped
        host word. Called on entry to every public op, so a time-out or overflow of an EARLIER op
        surfaces as an exception at the next call instead of as silently incomplete tensors."""
        code = self.C.host_read_i32(self.host_word, _STATUS_MIRROR_SLOT)
        if code != 0:
            torch.cuda.synchronize(self.device)
            self._clear_status()
            self._raise_status(code)

    def _get_carve(self, E: int, K: int, H: int, row_bytes: int, comb_row_bytes: int) -> _Carve:
        key = (E, K, H, row_bytes, comb_row_bytes)
        if self._carve is None or self._carve.key != key:
            if self._carve is not None or self._ll is not None:
                self.barrier()           # region reuse with another shape: drain every rank first
            self._ll = None
            self._carve = _Carve(self.num_nvl_bytes, self.group_size, E, K, H, row_bytes, comb_row_bytes,
                                 self.num_max_recv_tokens, self.combine_slots)
            # paint the guard bands of MY region; peers store into it only after they have seen
            # this rank's next count vector, which is stream-ordered after these fills
            for _, _, off, n in self._carve.guards:
                self.region.view(off, (n,), "uint8").fill_(CANARY)
        return self._carve

    def check_canaries(self) -> None:
        """Synchronising debug check: every guard band behind a receive / combine region of this
        rank still holds its fill pattern. A kernel (this rank's or a peer's) that stored past
        the end of a region would have hit one first. Raises `EpStatusError` naming the region."""
        carve = self._carve
        if carve is None:
            return
        bad = []
        for name, parity, off, n in carve.guards:
            v = self.region.view(off, (n,), "uint8")
            if bool((v != CANARY).any()):
                bad.append(f"{name}[parity {parity}] at byte {off}")
        if bad:
            raise EpStatusError("guard band overwritten behind " + ", ".join(bad))

    def _geom(self, *, E, K, T, mode, H, cap, slot_cap, epoch, epoch_wait=0, tail_wait=0) -> List[int]:
        R = self.group_size
        J, B = (R, R) if mode == 0 else (K, E)
        return [self.rank, R, E, E // R, K, T, mode, J, B, H, cap, slot_cap, epoch, epoch_wait, tail_wait,
                self._timeout_ns()]

    def _meta_ints(self, E: int, mode: int, K: int) -> int:
        R = self.group_size
        El = E // R
        B = R if mode == 0 else E
        return 2 + El + (El + 1) + (R + 1) + 2 * B

    def _enter(self, previous_event, allocate_on_comm_stream, async_finish):
        """Pick the stream for this op. Synchronous calls run on the caller's stream: no stream
        object is even looked up (`comm_stream` is None, and `torch.cuda.stream(None)` is a no-op
        context); `async_finish=True` or a `previous_event` uses the buffer's own communication
        stream."""
        if allocate_on_comm_stream and not async_finish:
            raise ValueError("allocate_on_comm_stream=True requires async_finish=True")
        self._poll_status()
        use_side = (async_finish or previous_event is not None) and not self.world.local
        if not use_side:
            self.comm_stream = None
            if self._async_outstanding:
                torch.cuda.current_stream(self.device).wait_stream(self._side_stream)   # earlier async work
                self._async_outstanding = False
            return None
        compute = torch.cuda.current_stream(self.device)
        self.comm_stream = self._side_stream
        ev = getattr(getattr(previous_event, "event", None), "event", None)
        if ev is not None:
            self.comm_stream.wait_event(ev)
        else:
            self.comm_stream.wait_stream(compute)
        return compute

    def _on_stream(self):
        """Context for the launches of one op: the communication stream when the op is
        asynchronous, nothing at all (no stream object, no device lookup) when it runs on the
        caller's stream."""
        return torch.cuda.stream(self.comm_stream) if self.comm_stream is not None else _NULL_CONTEXT

    def _exit(self, compute, async_finish, tensors) -> Optional[EventOverlap]:
        if compute is None:
            return EventOverlap(EventHandle()) if async_finish else None
        for t in tensors:
            if isinstance(t, torch.Tensor) and t.is_cuda:
                t.record_stream(compute)
        if async_finish:
            self._async_outstanding = True
            return EventOverlap(EventHandle(self.comm_stream), tuple(tensors))
        compute.wait_stream(self.comm_stream)
        return None

    def barrier(self) -> None:
        """Device-side barrier over the group on the communication stream."""
        self._epoch["barrier"] += 1
        self._enter(None, False, False)
        with self._on_stream():
            self.C.barrier(self.peers, 0, self.rank, self.group_size, self._epoch["barrier"],
                           self._timeout_ns(), self.status_ptr, not self.world.local)

    def probe_timeout(self, timeout_s: float = 0.2, clear: bool = True) -> int:
        """Wait on a flag that nothing sets, with a short limit; returns the status code that the
        kernel recorded (8). Shows that a lost peer ends in an error, not a hang. With
        `clear=False` the fault is left recorded, as after a real time-out: the next public op on
        this buffer raises it."""
        self._enter(None, False, False)
        with self._on_stream():
            self.C.wait_flags(self.region.local_ptr, 0, self.C.NUM_CHANNELS - 1, 1, 1 << 30,
                              int(timeout_s * 1e9), self.status_ptr, 8)
        code = int(self.status[0].item())
        if clear:
            self._clear_status()
        return code

    # ---- layout ----------------------------------------------------------------------
    @_nvtx("b200ep.layout")
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int,
                            previous_event=None, async_finish: bool = False,
                            allocate_on_comm_stream: bool = False):
        """-> (num_tokens_per_rank[R] i32, None, num_tokens_per_expert[E] i32,
               is_token_in_rank[T,R] bool, event)"""
        R = self.group_size
        if num_experts % R:
            raise ValueError("num_experts must be divisible by the group size")
        if topk_idx.dtype != torch.int64:
            topk_idx = topk_idx.to(torch.int64)
        topk_idx = topk_idx.contiguous()
        compute = self._enter(previous_event, allocate_on_comm_stream, async_finish)
        with self._on_stream():
            T = topk_idx.shape[0]
            need = self.C.layout_scratch_ints(T, num_experts, R)
            if self._layout_ws is None or self._layout_ws.numel() < need:
                self._layout_ws = torch.empty(need, dtype=torch.int32, device=self.device)
            counts = torch.empty(R + num_experts, dtype=torch.int32, device=self.device)
            per_rank, per_expert = counts[:R], counts[R:]
            in_rank = torch.empty((T, R), dtype=torch.bool, device=self.device)
            self.C.layout(topk_idx, num_experts, R, per_rank, per_expert, in_rank, self._layout_ws,
                          self._ctr[4], self.status_ptr)
        ev = self._exit(compute, async_finish, (per_rank, per_expert, in_rank, topk_idx))
        return per_rank, None, per_expert, in_rank, ev

    # ---- dispatch --------------------------------------------------------------------
    def _dispatch_p1(self, x, handle, is_token_in_rank, num_tokens_per_expert, topk_idx,
                     topk_weights, use_fp8, group_by_expert, num_experts):
        R = self.group_size
        scales_in = None
        if isinstance(x, tuple):
            # caller-quantised input (fp8 [T,H], f32 scales [T,H/128]): rows travel as raw bytes
            x, scales_in = x
            if x.dtype != torch.float8_e4m3fn or scales_in.dtype != torch.float32 or use_fp8:
                raise ValueError("tuple input must be (float8_e4m3fn [T,H], float32 [T,H/128]) with use_fp8=False")
            if x.shape[1] % 128 or tuple(scales_in.shape) != (x.shape[0], x.shape[1] // 128):
                raise ValueError("scales must have shape [num_tokens, hidden/128]")
            scales_in = scales_in.contiguous()
        if x.dim() != 2 or not x.is_contiguous():
            raise ValueError("x must be a contiguous [num_tokens, hidden] tensor")
        if x.dtype not in _ELEM_DTYPE and scales_in is None:
            raise ValueError(f"unsupported dtype {x.dtype}")
        T, H = x.shape
        st = dict(x=x.view(torch.uint8) if scales_in is not None else x, T=T, H=H, fp8=bool(use_fp8),
                  cached=handle is not None, scales_in=scales_in, fp8_out=bool(use_fp8) or scales_in is not None,
                  in_dtype=x.dtype)
        if handle is not None:
            if handle.T != T or handle.H != H:
                raise ValueError("cached handle does not match x")
            st.update(mode=handle.mode, K=handle.K, E=handle.E, handle=handle,
                      topk_idx=handle.topk_idx, topk_weights=None)
        else:
            mode = 1 if group_by_expert else 0
            if topk_idx is not None:
                topk_idx = topk_idx.to(torch.int64).contiguous()
            if topk_weights is not None:
                topk_weights = topk_weights.to(torch.float32).contiguous()
            if mode == 0 and is_token_in_rank is None:
                raise ValueError("rank-mode dispatch needs is_token_in_rank (get_dispatch_layout)")
            if mode == 1 and topk_idx is None:
                raise ValueError("expert-grouped dispatch needs topk_idx")
            if num_tokens_per_expert is not None:
                E = int(num_tokens_per_expert.numel())
            elif num_experts:
                E = int(num_experts)
            else:
                raise ValueError("num_tokens_per_expert (or num_experts) is required")
            K = int(topk_idx.shape[1]) if topk_idx is not None else 1
            st.update(mode=mode, K=K, E=E, topk_idx=topk_idx, topk_weights=topk_weights,
                      is_token_in_rank=is_token_in_rank, num_tokens_per_expert=num_tokens_per_expert)
        mode, K, E = st["mode"], st["K"], st["E"]
        if E % R:
            raise ValueError("num_experts must be divisible by the group size")
        row_bytes_out = H if st["fp8_out"] else H * x.element_size()
        elem = 2 if st["fp8_out"] else x.element_size()
        carve = self._get_carve(E, K, H, H * elem, H * elem)
        st["carve"] = carve
        if carve.cap <= 0:
            raise ValueError("num_nvl_bytes too small for this hidden size")
        J, B = (R, R) if mode == 0 else (K, E)
        st.update(J=J, B=B, row_bytes_out=row_bytes_out)
        if st["cached"]:
            # the handle's rows and slots index the region layout of ITS dispatch
            if handle.carve_key != carve.key or handle.cap > carve.cap:
                raise ValueError("cached dispatch: the handle was made for another region layout "
                                 f"(row bytes / capacity {handle.carve_key}, {handle.cap}) than this "
                                 f"input would use ({carve.key}, {carve.cap}); dispatch the same element "
                                 "width as the handle's own dispatch")
            st["meta"] = handle.meta
            st["send_row"], st["send_slot"] = handle.send_row, handle.send_slot
            return st
        self._epoch["notify"] += 1
        st["epoch_n"] = self._epoch["notify"]
        dev = self.device
        C_chunks = max((T + self.C.CHUNK_TOKENS - 1) // self.C.CHUNK_TOKENS, 1)
        key = (max(T, 1), J, C_chunks, B)
        ws = self._ws.get(key)
        if ws is None:      # scratch reused by every call of this shape (stream-ordered)
            ws = (torch.empty((max(T, 1), J), dtype=torch.int32, device=dev),
                  torch.empty((C_chunks, B), dtype=torch.int32, device=dev))
            self._ws = {key: ws}
        st["item_rank"], st["chunk_hist"] = ws
        n_meta = self._meta_ints(E, mode, K)
        n_tj = max(T, 1) * J
        owned = torch.empty(n_meta + 2 * n_tj, dtype=torch.int32, device=dev)   # handle-owned ints
        st["meta"] = owned[:n_meta]
        st["send_row"] = owned[n_meta:n_meta + n_tj].view(max(T, 1), J)
        st["send_slot"] = owned[n_meta + n_tj:].view(max(T, 1), J)
        regions = carve.region_list(st["epoch_n"] & 1, 0, 0)
        geom = self._geom(E=E, K=K, T=T, mode=mode, H=H, cap=carve.cap, slot_cap=carve.slot_cap,
                          epoch=st["epoch_n"])
        per_expert = st.get("num_tokens_per_expert")
        if per_expert is not None and per_expert.dtype != torch.int32:
            per_expert = per_expert.to(torch.int32)
        self.C.notify_send(geom, regions, self.peers,
                           st.get("is_token_in_rank") if mode == 0 else None,
                           st["topk_idx"] if mode == 1 else None,
                           per_expert if mode == 0 else None,
                           st["item_rank"], st["chunk_hist"], self._ctr[0], self.status_ptr)
        return st

    def _dispatch_p2(self, st):
        """The send kernel. One process per GPU: its last CTA also waits for the peers, so the
        receive region is complete when the kernel ends. Virtual ranks on one GPU: the wait is a
        separate launch (`_dispatch_p3`) issued after every rank's send."""
        carve = st["carve"]
        self._epoch["dispatch"] += 1
        st["epoch_d"] = self._epoch["dispatch"]
        pn = (st.get("epoch_n", 0)) & 1
        regions = carve.region_list(pn, st["epoch_d"] & 1, 0)
        st["regions"] = regions
        geom = self._geom(E=st["E"], K=st["K"], T=st["T"], mode=st["mode"], H=st["H"], cap=carve.cap,
                          slot_cap=carve.slot_cap, epoch=st["epoch_d"], epoch_wait=st.get("epoch_n", 0),
                          tail_wait=1 if self._single_launch else 0)
        st["geom"] = geom
        self.C.dispatch_send(geom, regions, self.peers, st["meta"], st["x"], st["fp8"], st["cached"],
                             st["topk_idx"], st.get("topk_weights"), st.get("item_rank"),
                             st.get("chunk_hist"), st["send_row"], st["send_slot"],
                             self._ctr[1], self.host_word, self.status_ptr, self._blocks(),
                             st.get("scales_in"))

    def _dispatch_p3(self, st, zero_copy: bool, num_worst_tokens: int = 0, expert_alignment: int = 1):
        R, E, K, H = self.group_size, st["E"], st["K"], st["H"]
        El = E // R
        carve = st["carve"]
        if not self._single_launch:
            self.C.wait_flags(self.region.local_ptr, 0, 1, R, st["epoch_d"], self._timeout_ns(),
                              self.status_ptr, 2)
        if st["cached"]:
            h = st["handle"]
            n_recv, per_expert_list = h.n_recv, h.num_recv_tokens_per_expert_list
        elif num_worst_tokens > 0:
            # No host synchronisation: outputs are sized for the caller's bound, the true count
            # stays on the device (handle.n_recv_dev) and rows beyond it are unspecified.
            if num_worst_tokens > carve.cap:
                raise ValueError(f"num_worst_tokens={num_worst_tokens} exceeds the buffer capacity {carve.cap}")
            n_recv, per_expert_list = int(num_worst_tokens), []
        else:
            if not self.C.host_wait_ge(self.host_word, 0, st["epoch_n"], self.timeout_s + 5.0):
                raise EpTimeoutError("host timed out waiting for the receive count")
            n_recv = self.C.host_read_i32(self.host_word, 1)
            if n_recv < 0:
                torch.cuda.synchronize(self.device)
                self._clear_status()
                raise EpTimeoutError("b200ep status 1: " + STATUS_TEXT[1])
            if n_recv > carve.cap:
                torch.cuda.synchronize(self.device)
                self._clear_status()
                raise EpStatusError(f"receive region overflow: {n_recv} rows > capacity {carve.cap}")
            per_expert_list = self.C.host_read_i32_list(self.host_word, 2, El)
            if expert_alignment > 1:
                per_expert_list = [align_up(c, expert_alignment) for c in per_expert_list]
            self._poll_status()       # the host already waited for the kernel's prologue: cheap to look
        reg = dict(zip(("flags", "counts", "recv_x", "recv_scales", "recv_topk_idx", "recv_topk_w",
                        "recv_meta", "recv_prob", "comb_x", "comb_w"), st["regions"]))
        keep = (lambda t: t) if zero_copy else (lambda t: t.clone())
        if st["fp8_out"]:
            rx = self.region.view(reg["recv_x"], (n_recv, H), "float8_e4m3fn")
            rs = self.region.view(reg["recv_scales"], (n_recv, H // 128), "float32")
            recv_x = (keep(rx), keep(rs))
        else:
            recv_x = keep(self.region.view(reg["recv_x"], (n_recv, H), _ELEM_DTYPE[st["in_dtype"]]))
        if st["cached"]:
            return recv_x, None, None, per_expert_list, st["handle"]
        recv_topk_idx = recv_topk_w = recv_prob = None
        if st["mode"] == 0 and st["topk_idx"] is not None:
            recv_topk_idx = keep(self.region.view(reg["recv_topk_idx"], (n_recv, K), "int64"))
            recv_topk_w = keep(self.region.view(reg["recv_topk_w"], (n_recv, K), "float32"))
        if st["mode"] == 1:
            recv_prob = keep(self.region.view(reg["recv_prob"], (n_recv,), "float32"))
        recv_meta = keep(self.region.view(reg["recv_meta"], (n_recv, 2), "int32"))
        handle = DispatchHandle(st["mode"], st["T"], H, K, E, n_recv, st["send_row"], st["send_slot"],
                                st["meta"], recv_meta, st["topk_idx"], st.get("is_token_in_rank"),
                                per_expert_list, st["fp8_out"], recv_prob, carve.key, carve.cap)
        return recv_x, recv_topk_idx, recv_topk_w, per_expert_list, handle

    @_nvtx("b200ep.dispatch")
    def dispatch(self, x, handle: Optional[DispatchHandle] = None, num_tokens_per_rank=None,
                 num_tokens_per_rdma_rank=None, is_token_in_rank=None, num_tokens_per_expert=None,
                 topk_idx=None, topk_weights=None, expert_alignment: int = 1, num_worst_tokens: int = 0,
                 config: Optional[Config] = None, previous_event=None, async_finish: bool = False,
                 allocate_on_comm_stream: bool = False, *, use_fp8: bool = False,
                 group_by_expert: bool = False, zero_copy: bool = False, num_experts: int = 0):
        """-> (recv_x | (recv_x_fp8, scales), recv_topk_idx, recv_topk_weights,
               num_recv_tokens_per_expert_list, handle, event)

        Rank mode (default): one row per (token, destination rank), rows ordered by source rank
        then token; `recv_topk_idx` holds LOCAL expert ids, -1 where the expert lives elsewhere.
        `group_by_expert=True`: one row per (token, expert), rows grouped by local expert;
        the per-row router probability is in `handle.recv_prob`.
        `zero_copy=True` returns views into the symmetric region (rows, routing side arrays and the
        handle's row table alike) that stay valid until the second next dispatch on this buffer.
        `num_worst_tokens > 0` removes the host read of the receive
        count: outputs have exactly that many rows (a bound chosen by the caller, e.g. group_size x
        tokens per rank), the per-expert list is empty and the true count is `handle.n_recv_dev`.
        `expert_alignment > 1` rounds every entry of the returned per-expert count list up to a
        multiple of it (the rows themselves are not padded)."""
        if expert_alignment < 1:
            raise ValueError("expert_alignment must be >= 1")
        compute = self._enter(previous_event, allocate_on_comm_stream, async_finish)
        with self._on_stream():
            st = self._dispatch_p1(x, handle, is_token_in_rank, num_tokens_per_expert, topk_idx,
                                   topk_weights, use_fp8, group_by_expert, num_experts)
            self._dispatch_p2(st)
            out = self._dispatch_p3(st, zero_copy, num_worst_tokens, expert_alignment)
        flat = []
        for o in out[:3]:
            flat.extend(o if isinstance(o, tuple) else (o,))
        ev = self._exit(compute, async_finish, [t for t in flat if t is not None] + [x])
        return (*out, ev)

    # ---- combine ---------------------------------------------------------------------
    def _combine_prepare(self, x, handle: DispatchHandle, topk_weights):
        if x.dim() != 2 or not x.is_contiguous() or x.shape[1] != handle.H:
            raise ValueError("x must be a contiguous [num_recv_tokens, hidden] tensor")
        if x.shape[0] < handle.n_recv:
            raise ValueError("x has fewer rows than the handle's receive count")
        if x.dtype not in _ELEM_DTYPE:
            raise ValueError(f"unsupported dtype {x.dtype}")
        carve = self._carve
        if carve is None or carve.key[:3] != (handle.E, handle.K, handle.H):
            raise ValueError("combine must follow a dispatch of the same shape on this buffer")
        if not carve.combine_slots:
            raise ValueError("this buffer has no combine slots: only the pull form of combine is available")
        if handle.H * x.element_size() > carve.key[4]:
            raise ValueError("combine dtype is wider than the region reserved at dispatch")
        self._epoch["combine"] += 1
        ep = self._epoch["combine"]
        regions = carve.region_list(0, 0, ep & 1)
        geom = self._geom(E=handle.E, K=handle.K, T=handle.T, mode=handle.mode, H=handle.H,
                          cap=handle.n_recv, slot_cap=carve.slot_cap, epoch=ep)
        if topk_weights is not None:
            topk_weights = topk_weights.to(torch.float32).contiguous()
        return dict(ep=ep, regions=regions, geom=geom, dtype=x.dtype, topk_w=topk_weights, x=x)

    def _combine_outputs(self, st, handle: DispatchHandle):
        out = torch.empty((handle.T, handle.H), dtype=st["dtype"], device=self.device)
        out_w = (torch.empty((handle.T, handle.K), dtype=torch.float32, device=self.device)
                 if st.get("topk_w") is not None else None)
        return out, out_w

    def _combine_p1(self, x, handle: DispatchHandle, topk_weights):
        """Push form, send half as its own launch (several virtual ranks on one GPU)."""
        st = self._combine_prepare(x, handle, topk_weights)
        self.C.combine(st["geom"], st["regions"], self.peers, 1, max(1, Buffer.num_sms), False,
                       handle.n_recv_dev, handle.recv_meta, x, st["topk_w"], self._ctr[2],
                       None, None, None, None, self.status_ptr)
        return st

    def _combine_p2(self, st, handle: DispatchHandle, weights=None):
        """Push form, reduce half as its own launch (waits for every rank's combine flag first)."""
        out, out_w = self._combine_outputs(st, handle)
        self.C.combine(st["geom"], st["regions"], self.peers, 2, max(1, Buffer.num_sms), True,
                       None, None, None, None, self._ctr[2],
                       handle.send_slot, weights, out, out_w, self.status_ptr)
        return out, out_w

    def _combine_fused(self, x, handle: DispatchHandle, topk_weights, weights=None):
        """Push form in ONE launch: every CTA sends its share of the rows, then waits for the peers'
        flags and reduces its share of the tokens."""
        st = self._combine_prepare(x, handle, topk_weights)
        out, out_w = self._combine_outputs(st, handle)
        self.C.combine(st["geom"], st["regions"], self.peers, 0, max(1, Buffer.num_sms), True,
                       handle.n_recv_dev, handle.recv_meta, x, st["topk_w"], self._ctr[2],
                       handle.send_slot, weights, out, out_w, self.status_ptr)
        return out, out_w

    def _region_offset(self, t: Optional[torch.Tensor]) -> int:
        """Byte offset of tensor `t` inside this rank's symmetric region, or -1 if it lies elsewhere."""
        if t is None or not t.is_cuda or not t.is_contiguous():
            return -1
        lo = self.region.local_ptr
        p = t.data_ptr()
        if p < lo or p + t.numel() * t.element_size() > lo + self.num_nvl_bytes:
            return -1
        return p - lo

    def _use_pull(self, x, topk_weights) -> bool:
        mode = Buffer.combine_transport
        if mode == "push":
            return False
        ok = self._region_offset(x) >= 0 and x.data_ptr() % 16 == 0 and (
            topk_weights is None or (topk_weights.dtype == torch.float32 and self._region_offset(topk_weights) >= 0))
        if (mode == "pull" or not self.combine_slots) and not ok:
            raise ValueError("this combine can only pull (combine_transport='pull' or a buffer without combine "
                             "slots): x (and topk_weights) must lie inside the symmetric region")
        return ok

    def _combine_pull(self, phase: int, x, handle: DispatchHandle, topk_weights, weights=None, out=None):
        """phase 0: announce + wait + reduce in one launch; 1: announce only; 2: wait + reduce."""
        carve = self._carve
        if carve is None or carve.key[:3] != (handle.E, handle.K, handle.H):
            raise ValueError("combine must follow a dispatch of the same shape on this buffer")
        if x.dim() != 2 or x.shape[1] != handle.H or x.dtype not in _ELEM_DTYPE:
            raise ValueError("x must be a [num_recv_tokens, hidden] bf16/fp16/fp32 tensor")
        if phase != 2:
            self._epoch["combine"] += 1
        ep = self._epoch["combine"]
        regions = carve.region_list(0, 0, ep & 1)
        geom = self._geom(E=handle.E, K=handle.K, T=handle.T, mode=handle.mode, H=handle.H,
                          cap=carve.cap, slot_cap=carve.slot_cap, epoch=ep)
        if out is None:
            out = torch.empty((handle.T, handle.H), dtype=x.dtype, device=self.device)
        out_w = (torch.empty((handle.T, handle.K), dtype=torch.float32, device=self.device)
                 if topk_weights is not None else None)
        self.C.combine_pull(geom, regions, self.peers, phase, max(1, Buffer.num_sms),
                            self._region_offset(x), self._region_offset(topk_weights), int(x.shape[0]),
                            handle.send_row, handle.topk_idx if handle.mode == 1 else None, weights, out, out_w,
                            self.status_ptr)
        return out, out_w

    def combine_input(self, num_rows: int, hidden: int, dtype=torch.bfloat16) -> torch.Tensor:
        """A [num_rows, hidden] tensor INSIDE the symmetric region for the expert computation to
        write its result into, so that combine can pull it without a copy. It aliases the combine
        slot area of the next combine's parity: valid until that combine returns, and only for
        callers that then combine this very tensor."""
        carve = self._carve
        if carve is None or not carve.combine_slots:
            raise ValueError("combine_input() must follow a dispatch on a buffer that has combine slots")
        es = torch.empty((), dtype=dtype).element_size()
        if num_rows * hidden * es > carve.slot_cap * carve.key[4]:
            raise ValueError("combine_input larger than the combine area of this buffer")
        off = carve.regions[(self._epoch["combine"] + 1) & 1]["comb_x"]
        return self.region.view(off, (num_rows, hidden), _ELEM_DTYPE[dtype])

    @_nvtx("b200ep.combine")
    def combine(self, x, handle: DispatchHandle, topk_weights=None, bias=None,
                config: Optional[Config] = None, previous_event=None, async_finish: bool = False,
                allocate_on_comm_stream: bool = False, *, item_weights=None):
        """-> (combined_x[T,H], combined_topk_weights | None, event).
        `topk_weights`: side values that travel back with the rows. Rank mode: [N_recv,K], summed
        over the destination ranks into [T,K] (the gradient of the routing weights when combine is
        dispatch's backward, `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:158-165`).
        Expert mode: [N_recv] (one value per row), returned as [T,K].
        Unweighted sum over the rows that each token was sent to (an identity expert returns
        x times the number of destinations, `DeepEP_v1/deepep_v1_combine.py:335-342`);
        `item_weights[T,J]` (J = ranks in rank mode, top-k in expert mode) turns it into a
        weighted reduction applied on arrival."""
        compute = self._enter(previous_event, allocate_on_comm_stream, async_finish)
        if topk_weights is not None and topk_weights.dtype != torch.float32:
            topk_weights = topk_weights.to(torch.float32)
        with self._on_stream():
            if self._use_pull(x, topk_weights):
                if self._single_launch:
                    out, out_w = self._combine_pull(0, x, handle, topk_weights, item_weights)
                else:
                    self._combine_pull(1, x, handle, topk_weights)
                    out, out_w = self._combine_pull(2, x, handle, topk_weights, item_weights)
            elif self._single_launch:
                out, out_w = self._combine_fused(x, handle, topk_weights, item_weights)
            else:
                st = self._combine_p1(x, handle, topk_weights)
                out, out_w = self._combine_p2(st, handle, item_weights)
            if bias is not None:
                out = out + (bias[0] if isinstance(bias, (tuple, list)) else bias)
        ev = self._exit(compute, async_finish, [out, x] + ([out_w] if out_w is not None else []))
        return out, out_w, ev

    # ---- low-latency mode -------------------------------------------------------------
    @staticmethod
    def get_low_latency_nvl_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int,
                                      num_experts: int, num_topk: int = 8) -> int:
        """Bytes of symmetric memory that low-latency mode needs for these bounds."""
        return _LLCarve.required_bytes(num_ranks, num_experts, num_max_dispatch_tokens_per_rank, hidden, num_topk)

    get_low_latency_rdma_size_hint = get_low_latency_nvl_size_hint   # upstream DeepEP's name

    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int = 0, hidden: int = 0,
                                 num_experts: int = 0) -> None:
        """Nothing to clean: flags are epochs and regions are double-buffered."""

    LL_SPLIT = 4          # combine-send CTAs per local expert
    # How a low-latency send kernel tells the peers that it is done: 0 = every CTA adds 1 to its
    # arrival counter on every peer, 1 = CTAs count themselves locally and the last one adds the
    # grid size on every peer. None = by group size (mode 0 measured faster with 2 ranks, where a
    # peer takes few remote atomics; mode 1 with 8). Must be the same on every rank.
    ll_signal_mode: Optional[int] = None
    # Launch the four low-latency kernels with programmatic stream serialisation: a kernel's CTAs
    # are placed while its predecessor still runs and wait in their first instruction until it has
    # completed, so launch latencies overlap (also inside a captured CUDA graph). Off by default:
    # with 2 ranks a graph replay went from 60.4 to 59.2 us, but eager calls got slower
    # (dispatch 45 -> 54 us).
    ll_overlap_launches: bool = False

    def _ll_state(self, E: int, K: int, H: int, M: int):
        key = (E, K, H, M)
        if self._ll is None or self._ll["key"] != key:
            reuse = self._ll is not None or self._carve is not None
            carve = _LLCarve(self.num_nvl_bytes, self.group_size, E, M, H, K)
            dev = self.device
            if reuse:
                # the region held other data: every rank drains, clears its per-expert row counters
                # (they must start at zero), and only then may anyone send again
                self.barrier()
                for off in carve.count:
                    self.region.view(off, (E // self.group_size,), "int32").zero_()
                self.barrier()
            self._ll_dispatch_pending = False
            if self._ll_words is None:
                # device-resident op state (epochs and arrival targets); lives as long as the buffer
                # because the peers' arrival counters are cumulative
                self._ll_words = torch.zeros(18, dtype=torch.int32, device=dev)
            self._ll = dict(key=key, carve=carve, words=self._ll_words,
                            send_cnt=torch.zeros(2 * E, dtype=torch.int32, device=dev),
                            send_slot=torch.full((M * K,), -1, dtype=torch.int32, device=dev))
            self._carve = None
        return self._ll

    def _ll_params(self, st, T: int, fp8: bool):
        E, K, H, M = st["key"]
        c = st["carve"]
        R = self.group_size
        El = E // R
        return [self.rank, R, E, El, K, H, M, T, int(fp8), 0, *c.count, *c.recv_x, *c.recv_scales,
                *c.recv_src, *c.comb_x, self._timeout_ns(), *c.recv_tag, min(M, 128), El * Buffer.LL_SPLIT,
                (1 if R >= 8 else 0) if Buffer.ll_signal_mode is None else int(Buffer.ll_signal_mode),
                int(bool(Buffer.ll_overlap_launches)), c.comb_in, *c.range_tab]

    def _ll_dispatch_send(self, x, topk_idx, M, E, use_fp8):
        if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
            raise ValueError("low-latency dispatch takes a contiguous bf16 [tokens, hidden] tensor")
        T, H = x.shape
        if T > M:
            raise ValueError(f"{T} tokens exceed num_max_dispatch_tokens_per_rank={M}")
        if E % self.group_size:
            raise ValueError("num_experts must be divisible by the group size")
        topk_idx = topk_idx.to(torch.int64).contiguous()
        K = topk_idx.shape[1]
        st = self._ll_state(E, K, H, M)
        if getattr(self, "_ll_dispatch_pending", False):
            # The receive region is single-buffered: a second dispatch may only overwrite it once every
            # peer has consumed the previous one. A combine in between proves that; without one, drain.
            self.barrier()
        self._ll_dispatch_pending = True
        pv = self._ll_params(st, T, use_fp8)
        self.C.ll_dispatch_send(pv, self.peers, x, topk_idx, st["send_cnt"], st["words"][0:6], self.status_ptr,
                                st["send_slot"])
        return dict(st=st, pv=pv, T=T, H=H, K=K, E=E, M=M, fp8=use_fp8, topk_idx=topk_idx, x=x)

    def _ll_dispatch_recv(self, d):
        """Count-only: the rows already lie packed per local expert in the receive region, which is
        what the returned tensors are views of (fixed addresses; valid until the next dispatch)."""
        R, El, M, H = self.group_size, d["E"] // self.group_size, d["M"], d["H"]
        c = d["st"]["carve"]
        rows = R * M
        out_count = torch.empty((El,), dtype=torch.int32, device=self.device)
        self.C.ll_dispatch_recv(d["pv"], self.region.local_ptr, out_count, d["st"]["words"][0:6], self.status_ptr)
        if d["fp8"]:
            out_x = (self.region.view(c.recv_x[0], (El, rows, H), "float8_e4m3fn"),
                     self.region.view(c.recv_scales[0], (El, rows, H // 128), "float32"))
        else:
            out_x = self.region.view(c.recv_x[0], (El, rows, H), "bfloat16")
        out_src = self.region.view(c.recv_src[0], (El, rows), "int32")
        handle = (out_src, None, M, H, d["E"], out_count, d["K"])
        return out_x, out_count, handle

    @_nvtx("b200ep.ll_dispatch")
    def low_latency_dispatch(self, x, topk_idx, num_max_dispatch_tokens_per_rank: int, num_experts: int,
                             use_fp8: bool = True, async_finish: bool = False,
                             return_recv_hook: bool = False):
        """-> (recv_x [E_local, R*M, H] | (fp8, scales), recv_count [E_local] i32, handle, event, hook).
        The first recv_count[e] rows of expert e are valid (in arrival order; `handle[0]` gives
        (source rank << 24 | token << 5 | k) per row). The tensors are views of the receive region:
        fixed addresses, valid until the next low_latency_dispatch on this buffer. No host
        synchronisation; may be captured in a CUDA graph. With return_recv_hook=True only the send half is launched and
        the returned hook launches the receive half (then fills the same tensors)."""
        compute = self._enter(None, False, False)
        with self._on_stream():
            d = self._ll_dispatch_send(x, topk_idx, num_max_dispatch_tokens_per_rank, num_experts, use_fp8)
            if return_recv_hook:
                box = {}

                def hook():
                    with self._on_stream():
                        box["out"] = self._ll_dispatch_recv(d)
                    return box["out"]
                ev = self._exit(compute, async_finish, [x])
                return None, None, None, ev, hook
            recv_x, count, handle = self._ll_dispatch_recv(d)
        flat = list(recv_x) if isinstance(recv_x, tuple) else [recv_x]
        ev = self._exit(compute, async_finish, flat + [count, x])
        return recv_x, count, handle, ev, None

    def get_next_low_latency_combine_buffer(self, handle) -> torch.Tensor:
        """bf16 [E_local, R*M, hidden] INSIDE the symmetric region, row (e, j) matching row (e, j) of
        the `recv_x` that `low_latency_dispatch` returned with this handle. Experts that write their
        output here let `low_latency_combine` pull the rows in place (one kernel, no send half).
        The tensor has a fixed address (usable under CUDA-graph replay) and may be rewritten once
        the next `low_latency_dispatch` on this buffer has returned."""
        _src, _range, M, H, E, _count, K = handle
        st = self._ll_state(E, K, H, M)
        El = E // self.group_size
        return self.region.view(st["carve"].comb_in, (El, self.group_size * M, H), "bfloat16")

    def _ll_combine_pull(self, phase: int, topk_idx, topk_weights, handle, out=None):
        _src, _rng, M, H, E, _count, K = handle
        if phase != 2:
            self._ll_dispatch_pending = False
        st = self._ll_state(E, K, H, M)
        topk_idx = topk_idx.to(torch.int64).contiguous()
        T = topk_idx.shape[0]
        pv = self._ll_params(st, T, False)
        if out is None:
            out = torch.empty((T, H), dtype=torch.bfloat16, device=self.device)
        w = topk_weights.to(torch.float32).contiguous() if topk_weights is not None else None
        self.C.ll_combine_pull(pv, self.peers, phase, st["send_slot"], topk_idx, w, out,
                               st["words"][12:18], self.status_ptr)
        return out

    def _ll_is_combine_buffer(self, x, handle) -> bool:
        if self._ll is None:
            return False
        return x.data_ptr() == self.region.local_ptr + self._ll["carve"].comb_in

    def _ll_combine_send(self, x, handle):
        src_info, _range, M, H, E, count, K = handle
        st = self._ll_state(E, K, H, M)
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("low-latency combine takes a contiguous bf16 [E_local, R*M, hidden] tensor")
        pv = self._ll_params(st, 0, False)
        self._ll_dispatch_pending = False
        self.C.ll_combine_send(pv, self.peers, x, src_info, count, st["words"][6:12], self.status_ptr)
        return dict(st=st, H=H)

    def _ll_combine_recv(self, c, topk_idx, topk_weights, out=None):
        topk_idx = topk_idx.to(torch.int64).contiguous()
        T = topk_idx.shape[0]
        pv = self._ll_params(c["st"], T, False)
        if out is None:
            out = torch.empty((T, c["H"]), dtype=torch.bfloat16, device=self.device)
        w = topk_weights.to(torch.float32).contiguous() if topk_weights is not None else None
        self.C.ll_combine_recv(pv, self.region.local_ptr, topk_idx, w, out, c["st"]["words"][6:12],
                               self.status_ptr, max(Buffer.num_sms * 4, 1))
        return out

    @_nvtx("b200ep.ll_combine")
    def low_latency_combine(self, x, topk_idx, topk_weights, handle, async_finish: bool = False,
                            return_recv_hook: bool = False, out: Optional[torch.Tensor] = None,
                            zero_copy: bool = False):
        """-> (combined_x [T,H] bf16 = sum_k topk_weights[t,k] * expert output of (t,k), event, hook).
        When `x` is the tensor from `get_next_low_latency_combine_buffer` (or `zero_copy=True`, which
        asserts that the expert output already lies there), the rows are pulled in place by one
        kernel; otherwise they are sent back to per-(token, k) slots and reduced there. Every rank
        of the group must use the same form."""
        compute = self._enter(None, False, False)
        if zero_copy or self._ll_is_combine_buffer(x, handle):
            with self._on_stream():
                res = self._ll_combine_pull(0 if self._single_launch else 1, topk_idx, topk_weights, handle, out)
                if not self._single_launch:
                    res = self._ll_combine_pull(2, topk_idx, topk_weights, handle, res)
            ev = self._exit(compute, async_finish, [res])
            return res, ev, ((lambda: res) if return_recv_hook else None)
        with self._on_stream():
            c = self._ll_combine_send(x, handle)
            if return_recv_hook:
                def hook():
                    with self._on_stream():
                        return self._ll_combine_recv(c, topk_idx, topk_weights, out)
                return None, self._exit(compute, async_finish, [x]), hook
            res = self._ll_combine_recv(c, topk_idx, topk_weights, out)
        return res, self._exit(compute, async_finish, [res, x]), None


class _LLCarve:
    """Region offsets of low-latency mode. Every region is laid out twice (index 0 / 1); the receive
    rows, scales and source words use copy 0 only (single-buffered, see csrc/ep/ll.cu), the
    push-combine slots alternate by epoch parity."""

    @staticmethod
    def _sizes(R, E, M, H, K):
        El = E // R
        rows = El * R * M
        return dict(recv_x=rows * H * 2, recv_scales=rows * max(H // 128, 1) * 4, recv_src=rows * 4,
                    recv_tag=rows * 4, comb_x=M * K * H * 2, range_tab=R * El * 4)

    @staticmethod
    def required_bytes(R, E, M, H, K) -> int:
        s = _LLCarve._sizes(R, E, M, H, K)
        comb_in = align_up((E // R) * R * M * H * 2, REGION_ALIGN)      # in-place expert output, one copy
        return FIXED_BYTES + 2 * sum(align_up(v, REGION_ALIGN) for v in s.values()) + comb_in + REGION_ALIGN

    def __init__(self, nbytes: int, R: int, E: int, M: int, H: int, K: int):
        need = self.required_bytes(R, E, M, H, K)
        if nbytes < need:
            raise ValueError(f"buffer of {nbytes} bytes is too small for low-latency mode: need {need} "
                             "(Buffer.get_low_latency_nvl_size_hint)")
        El = E // R
        csz = align_up(El * R * 4, REGION_ALIGN)
        base = FIXED_BYTES // 2
        if base + 2 * csz > FIXED_BYTES:
            raise ValueError("too many experts for the low-latency control area")
        self.count = (base, base + csz)
        off = FIXED_BYTES
        names = self._sizes(R, E, M, H, K)
        for name in names:
            setattr(self, name, [0, 0])
        for p in range(2):
            for name, sz in names.items():
                getattr(self, name)[p] = off
                off = align_up(off + sz, REGION_ALIGN)
        self.comb_in = off          # [El][R*M][H] bf16: where the experts write when combine pulls


def _fused_fc2_send(self: Buffer, act: torch.Tensor, w2: torch.Tensor, handle: DispatchHandle):
    """fc2 grouped GEMM whose epilogue IS the combine send: each output tile row is stored
    straight into its token's slot on the source rank (peer LSU stores from the tensor-core
    kernel) and the last CTA raises this rank's combine flag on every peer. Returns the state that
    `_combine_p2` (the reduce half) needs."""
    from ..ops import gemm as G
    if handle.mode != 1:
        raise ValueError("fused fc2+combine needs an expert-grouped dispatch handle")
    carve = self._carve
    if carve is None or carve.key[:3] != (handle.E, handle.K, handle.H):
        raise ValueError("fused combine must follow a dispatch of the same shape on this buffer")
    if not carve.combine_slots:
        raise ValueError("the fc2 epilogue stores into combine slots, which this buffer does not have")
    if w2.shape[1] != handle.H or act.dtype != torch.bfloat16:
        raise ValueError("w2 must be [E_local, hidden, ffn] and act bf16")
    self._epoch["combine"] += 1
    ep = self._epoch["combine"]
    regions = carve.region_list(0, 0, ep & 1)
    El = handle.E // self.group_size
    expert_off = handle.meta[2 + El: 2 + El + El + 1]
    flag_row = self.C.MAX_RANKS * 4 * 2          # byte offset of the combine channel's flag row
    G.grouped_gemm_combine(act, w2, expert_off, handle.recv_meta, self.peers, regions[8], carve.slot_cap,
                           self.rank, signal_flag_off=flag_row, epoch=ep, counter=self._ctr[3],
                           status_ptr=self.status_ptr)
    geom = self._geom(E=handle.E, K=handle.K, T=handle.T, mode=1, H=handle.H, cap=handle.n_recv,
                      slot_cap=carve.slot_cap, epoch=ep)
    return dict(ep=ep, regions=regions, geom=geom, dtype=torch.bfloat16, topk_w=None)


def _fused_fc2_combine(self: Buffer, act: torch.Tensor, w2: torch.Tensor, handle: DispatchHandle,
                       item_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fc2 with the combine send in its epilogue, then the reduction on arrival of this rank's own
    tokens. act: bf16 [N_recv, F] rows grouped by local expert (expert-mode handle), w2: bf16
    [E_local, H, F]. Returns combined [T, H] bf16."""
    compute = self._enter(None, False, False)
    with self._on_stream():
        st = _fused_fc2_send(self, act, w2, handle)
        out, _ = self._combine_p2(st, handle, item_weights)
    self._exit(compute, False, [out, act])
    return out


Buffer._fused_fc2_send = _fused_fc2_send
Buffer.fused_fc2_combine = _fused_fc2_combine
