"""Byte-size parsing/formatting and chunk-offset helpers shared by every CLI.

Behaviour parity: `Copy_Engine/nvlink_copy_engine_test.py:334-381`
(`parse_nbytes`, `fmt_bytes`, `parse_copy_sizes`, `build_contiguous_offsets`).
Bare K/M/G and KiB/MiB/GiB are binary, KB/MB/GB are decimal.
"""
from __future__ import annotations

import argparse
import re
from typing import Iterable, List, Sequence, Tuple

_UNIT = {
    "": 1, "B": 1,
    "K": 1 << 10, "M": 1 << 20, "G": 1 << 30, "T": 1 << 40,
    "KIB": 1 << 10, "MIB": 1 << 20, "GIB": 1 << 30, "TIB": 1 << 40,
    "KB": 10 ** 3, "MB": 10 ** 6, "GB": 10 ** 9, "TB": 10 ** 12,
}
_SIZE_RE = re.compile(r"^\s*([0-9]*\.?[0-9]+(?:[eE][+-]?[0-9]+)?)\s*([A-Za-z]*)\s*$")


def parse_nbytes(text) -> int:
    """'64K' -> 65536, '1.5MiB' -> 1572864, '2MB' -> 2000000, 4096 -> 4096."""
    if isinstance(text, int):
        return text
    m = _SIZE_RE.match(str(text))
    if not m:
        raise ValueError(f"cannot parse byte size {text!r}")
    unit = m.group(2).upper()
    if unit not in _UNIT:
        raise ValueError(f"unknown size unit {m.group(2)!r} in {text!r}")
    return int(float(m.group(1)) * _UNIT[unit])


def fmt_bytes(n: float) -> str:
    """Binary-unit pretty printer with two decimals ('1.00 MiB')."""
    units = ("B", "KiB", "MiB", "GiB", "TiB", "PiB")
    v = float(n)
    for u in units[:-1]:
        if abs(v) < 1024.0:
            return f"{v:.2f} {u}"
        v /= 1024.0
    return f"{v:.2f} {units[-1]}"


def parse_size_list(spec: str) -> Tuple[int, ...]:
    """'64K,128K,1M' -> (65536, 131072, 1048576); argparse-friendly errors."""
    parts = [p.strip() for p in str(spec).split(",")]
    if not parts or any(p == "" for p in parts):
        raise argparse.ArgumentTypeError(
            "expected a comma-separated size list such as 64K,128K,1M")
    try:
        return tuple(parse_nbytes(p) for p in parts)
    except ValueError as e:
        raise argparse.ArgumentTypeError(str(e)) from e


parse_copy_sizes = parse_size_list  # reference flag name


def contiguous_offsets(sizes: Sequence[int]) -> Tuple[int, ...]:
    """Exclusive prefix sum: where each chunk starts when packed back to back."""
    out: List[int] = []
    acc = 0
    for s in sizes:
        out.append(acc)
        acc += int(s)
    return tuple(out)


build_contiguous_offsets = contiguous_offsets


def default_nonuniform_sizes(total: int, copies: int, align: int = 16) -> Tuple[int, ...]:
    """Split `total` bytes into `copies` unequal chunks (weights 1..copies),
    each a multiple of `align`; the last chunk absorbs the remainder."""
    if copies <= 0:
        raise ValueError("copies must be positive")
    wsum = copies * (copies + 1) // 2
    sizes = [max(align, (total * (i + 1) // wsum) // align * align) for i in range(copies)]
    sizes[-1] = max(align, total - sum(sizes[:-1]))
    return tuple(sizes)


def pow2_sweep(lo: int, hi: int) -> Tuple[int, ...]:
    """Powers of two from lo to hi inclusive (both rounded to powers of two)."""
    out = []
    v = 1
    while v < lo:
        v <<= 1
    while v <= hi:
        out.append(v)
        v <<= 1
    return tuple(out)


def parse_gpu_ids(spec, world_size: int) -> Tuple[int, ...]:
    """'0,2,5' -> (0, 2, 5), validated against world_size, deduplicated, sorted.
    Parity: `Copy_Engine/nvlink_all_to_all_copy_engine_test.py:149-170`."""
    if spec is None:
        return tuple(range(world_size))
    ids = sorted({int(p) for p in str(spec).split(",") if p.strip() != ""})
    if not ids:
        raise ValueError("empty GPU id list")
    for i in ids:
        if not 0 <= i < world_size:
            raise ValueError(f"GPU id {i} outside [0,{world_size})")
    return tuple(ids)


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def align_up(a: int, b: int) -> int:
    return ceil_div(a, b) * b
