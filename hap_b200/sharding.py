"""Ratio -> integer shard extents, through the C ABI (``hapx_sharding_round``).

Mirrors the planner's ``sharding_round`` (``hap.rs:3536-3559`` in the reference) and
its Python export ``hap.sharding_round(full_length, ratios)`` (``hap.rs:211-218``),
which overwrites the ratio list with the extents in place.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

from . import _native as N


def sharding_round(full_length: int, sharding_ratios: Sequence[float]) -> List[int]:
    """Return the integer extents for ``full_length`` split by ``sharding_ratios``."""
    w = len(sharding_ratios)
    ratios = (C.c_double * w)(*[float(x) for x in sharding_ratios])
    out = (C.c_int64 * w)()
    N.check(N.lib.hapx_sharding_round(int(full_length), ratios, w, out))
    return [int(v) for v in out]


def sharding_round_(full_length: int, sharding_ratios: list) -> None:
    """In-place form with the calling convention of the reference's ``hap.sharding_round``."""
    sharding_ratios[:] = sharding_round(full_length, sharding_ratios)
