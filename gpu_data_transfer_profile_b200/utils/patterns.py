"""Traffic patterns of the copy benchmarks: who sends what to whom, and where.

Everything here is pure integer arithmetic (no torch, no CUDA) so it is unit
tested on CPU and reused by the GPU CLIs and by the CPU copy oracle.

Behaviour parity with the reference scripts:
  pair topologies      `Copy_Engine/nvlink_copy_engine_test.py:413-427`
  fan-out order        `Copy_Engine/nvlink_all_to_all_copy_engine_test.py:66-71`
  gapped layouts       `Copy_Engine/nvlink_batch_address_layout_test.py:78-115`
  multi-source mapping `Copy_Engine/nvlink_multi_source_all_to_all_batch_test.py:66-102`
  round-robin mapping  `LSU_TMA/nvlink_lsu_tma_round_robin_copy_test.py:8-12,858-865`
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

PAIR_MODES = ("ring", "reverse-ring", "pair")
LAYOUTS = ("contiguous", "src-discontinuous", "dst-discontinuous", "both-discontinuous")
SRC_GAP_SENTINEL = 252
DST_GAP_SENTINEL = 253
_PRIME = 251  # fill values stay below the two sentinels


def choose_pair(rank: int, world: int, mode: str) -> Tuple[int, int]:
    """(source device, destination device) owned by `rank`."""
    if mode == "ring":
        return rank, (rank + 1) % world
    if mode == "reverse-ring":
        return rank, (rank - 1) % world
    if mode == "pair":
        if world % 2:
            raise ValueError("--mode pair requires an even number of ranks/GPUs")
        return rank, rank ^ 1
    raise ValueError(f"unknown mode {mode!r}; expected one of {PAIR_MODES}")


def destination_order(src: int, world: int, rotate: bool = True) -> Tuple[int, ...]:
    """All peers of `src`; rotated so that rank r starts at r+1 (spreads the
    first store of every rank over different switch ports) or plain ascending."""
    if rotate:
        return tuple((src + k) % world for k in range(1, world))
    return tuple(d for d in range(world) if d != src)


def rr_destinations(rank: int, world: int, mode: str) -> Tuple[int, ...]:
    """Peer order used by the chunk round-robin copy."""
    if mode == "ring":
        return tuple((rank + k) % world for k in range(1, world))
    if mode == "reverse-ring":
        return tuple((rank - k) % world for k in range(1, world))
    if mode == "pair":
        raise ValueError("--mode pair is not meaningful for all-peer round-robin copies")
    raise ValueError(f"unknown mode {mode!r}")


def rr_owner(byte_offset: int, rr_bytes: int, n_dst: int) -> int:
    """Index (into the destination table) that owns the chunk holding `byte_offset`."""
    return (byte_offset // rr_bytes) % n_dst


def rr_chunks(nbytes: int, rr_bytes: int, n_dst: int) -> List[Tuple[int, int, int]]:
    """[(dst_slot, offset, length)] for every chunk of a round-robin copy."""
    out = []
    off = 0
    while off < nbytes:
        ln = min(rr_bytes, nbytes - off)
        out.append((rr_owner(off, rr_bytes, n_dst), off, ln))
        off += ln
    return out


@dataclass(frozen=True)
class GapLayout:
    """Offsets of N chunks inside one source and one destination allocation."""
    src_offsets: Tuple[int, ...]
    dst_offsets: Tuple[int, ...]
    sizes: Tuple[int, ...]
    gap: int
    src_gapped: bool
    dst_gapped: bool

    @property
    def src_bytes(self) -> int:
        return self.src_offsets[-1] + self.sizes[-1]

    @property
    def dst_bytes(self) -> int:
        return self.dst_offsets[-1] + self.sizes[-1]

    def dst_gaps(self) -> List[Tuple[int, int]]:
        """(offset, length) of every untouched hole in the destination."""
        if not self.dst_gapped or self.gap == 0:
            return []
        return [(o + s, self.gap) for o, s in zip(self.dst_offsets[:-1], self.sizes[:-1])]


def build_layout(layout: str, sizes: Sequence[int], gap: int) -> GapLayout:
    if layout not in LAYOUTS:
        raise ValueError(f"unknown layout {layout!r}; expected one of {LAYOUTS}")
    sg = layout in ("src-discontinuous", "both-discontinuous")
    dg = layout in ("dst-discontinuous", "both-discontinuous")
    so, do = [], []
    s = d = 0
    for sz in sizes:
        so.append(s)
        do.append(d)
        s += sz + (gap if sg else 0)
        d += sz + (gap if dg else 0)
    return GapLayout(tuple(so), tuple(do), tuple(int(x) for x in sizes), gap, sg, dg)


def pair_fill_value(rank: int) -> int:
    return (rank + 17) % _PRIME


def pair_prefill_value(rank: int) -> int:
    return (rank + 18) % _PRIME


def layout_chunk_value(rank: int, chunk: int) -> int:
    return (rank * 17 + chunk) % _PRIME


def msrc_chunk_value(rank: int, source: int, dest_slot: int) -> int:
    return (rank * 37 + source * 19 + dest_slot * 7) % _PRIME


def source_buffer_name(i: int) -> str:
    return chr(ord("A") + i) if i < 26 else f"S{i}"


@dataclass(frozen=True)
class MultiSourcePlan:
    """N logical source buffers, each cut into world-1 sub-buffers; sub-buffer k of
    every source travels to peer (rank+k+1) % world, one batch per destination."""
    rank: int
    world: int
    sub_sizes: Tuple[Tuple[int, ...], ...]      # [source][dest_slot]
    src_offsets: Tuple[Tuple[int, ...], ...]    # [source][dest_slot], in the source allocation
    dst_offsets: Tuple[Tuple[int, ...], ...]    # [source][dest_slot], in that peer's allocation
    src_bytes: int
    dst_bytes: Tuple[int, ...]                  # [dest_slot]

    def peer(self, slot: int) -> int:
        return (self.rank + slot + 1) % self.world

    def batches(self):
        """Yield (dest_slot, peer, [(src_off, dst_off, nbytes) per source])."""
        for k in range(self.world - 1):
            yield k, self.peer(k), [
                (self.src_offsets[s][k], self.dst_offsets[s][k], self.sub_sizes[s][k])
                for s in range(len(self.sub_sizes))]


def build_multi_source_plan(rank: int, world: int, sub_sizes: Sequence[Sequence[int]],
                            source_gap: int) -> MultiSourcePlan:
    if world < 2:
        raise ValueError("multi-source all-to-all needs world_size >= 2")
    n_dst = world - 1
    for row in sub_sizes:
        if len(row) != n_dst:
            raise ValueError("every source needs one size per destination")
    src_off, cur = [], 0
    for row in sub_sizes:
        offs = []
        for sz in row:
            offs.append(cur)
            cur += sz
        src_off.append(tuple(offs))
        cur += source_gap
    src_bytes = cur - source_gap
    dst_off = [[0] * n_dst for _ in sub_sizes]
    dst_bytes = []
    for k in range(n_dst):
        acc = 0
        for s, row in enumerate(sub_sizes):
            dst_off[s][k] = acc
            acc += row[k]
        dst_bytes.append(acc)
    return MultiSourcePlan(rank, world, tuple(tuple(r) for r in sub_sizes), tuple(src_off),
                           tuple(tuple(r) for r in dst_off), src_bytes, tuple(dst_bytes))


def msrc_sizes(world: int, n_sources: int, nbytes: int,
               source_sizes: Sequence[int] = None,
               destination_sizes: Sequence[int] = None) -> Tuple[Tuple[int, ...], ...]:
    """Sub-buffer size table [source][dest_slot].
    source-indexed: one size per source, same for every destination;
    destination-indexed: one size per destination, same for every source."""
    n_dst = world - 1
    if source_sizes is not None and destination_sizes is not None:
        raise ValueError("give source-indexed or destination-indexed sizes, not both")
    if source_sizes is not None:
        if len(source_sizes) != n_sources:
            raise ValueError("--source-buffer-sizes needs one entry per source buffer")
        return tuple(tuple(int(s) for _ in range(n_dst)) for s in source_sizes)
    if destination_sizes is not None:
        if len(destination_sizes) != n_dst:
            raise ValueError("--destination-buffer-sizes needs world_size-1 entries")
        return tuple(tuple(int(d) for d in destination_sizes) for _ in range(n_sources))
    return tuple(tuple(nbytes for _ in range(n_dst)) for _ in range(n_sources))
