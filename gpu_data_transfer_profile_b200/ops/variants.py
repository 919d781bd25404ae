"""Per-message-size choice of the peer-copy variant (copy engine / LSU / TMA-staged / batched),
taken from a MEASURED table produced by `bench/copy_sweep.py --table`. The reference compares the
variants by hand in its result READMEs; here the comparison is data that code can query.

`select(pattern, nbytes)` returns the variant that was fastest at the nearest measured size
(log scale). The packaged default table is `variant_table.json` beside this file; pass another
table (e.g. one measured on a different world size) with `load(path)`.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

_DEFAULT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "variant_table.json")
_FALLBACK = {"one-to-one": [{"nbytes": 4096, "variant": "lsu16"}, {"nbytes": 1 << 30, "variant": "ce"}],
             "all-to-all": [{"nbytes": 4096, "variant": "sm_batched"}, {"nbytes": 1 << 30, "variant": "ce"}],
             "round-robin": [{"nbytes": 8192, "variant": "lsu_rr"}]}
_table: Optional[Dict[str, List[dict]]] = None


def load(path: Optional[str] = None) -> Dict[str, List[dict]]:
    global _table
    p = path or _DEFAULT
    if os.path.exists(p):
        with open(p) as f:
            _table = json.load(f)["table"]
    else:
        _table = _FALLBACK
    return _table


def select(pattern: str, nbytes: int, table: Optional[Dict[str, List[dict]]] = None) -> str:
    t = table or _table or load()
    if pattern not in t or not t[pattern]:
        raise KeyError(f"no measurements for pattern {pattern!r}")
    n = max(int(nbytes), 1)
    best = min(t[pattern], key=lambda r: abs(math.log2(r["nbytes"]) - math.log2(n)))
    return best["variant"]
