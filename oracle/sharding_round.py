"""CPU restatement of the planner's ratio -> integer-extent rounding.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows ``hap.rs:3536-3559`` (``fn sharding_round``), exported to Python at
``hap.rs:211-218``:

* ``full_length == 1`` returns all ones (the broadcast hack, ``hap.rs:3538-3540``);
* every extent starts at ``trunc(ratio * full_length)`` computed in f64
  (Rust ``as usize`` truncates toward zero and saturates at 0 for negatives);
* while the extents sum to less than ``full_length`` the rank with the largest
  ``ratio - length / full_length`` gets one more element; Rust's
  ``Iterator::max_by_key`` returns the LAST maximal element, so ties go to the
  highest index.

Pinned by: the extents quoted for the benchmark configurations (computed from
the same Rust source by hand) in ``tests/test_sharding_round.py`` and by the
properties sum == full_length, each extent >= floor(ratio*full).
"""
from __future__ import annotations

from typing import List, Sequence


def sharding_round(full_length: int, sharding_ratios: Sequence[float]) -> List[int]:
    if full_length == 1:
        return [1] * len(sharding_ratios)
    lengths = []
    for ratio in sharding_ratios:
        v = float(ratio) * float(full_length)
        lengths.append(int(v) if v > 0.0 else 0)  # saturating truncation
    if sum(lengths) > full_length:
        raise AssertionError("ratios sum to more than 1")  # hap.rs:3543
    while sum(lengths) < full_length:
        best_i, best_key = -1, None
        for i, (ratio, length) in enumerate(zip(sharding_ratios, lengths)):
            key = float(ratio) - float(length) / float(full_length)
            if best_key is None or key >= best_key:  # ">=": last maximum wins
                best_i, best_key = i, key
        lengths[best_i] += 1
    return lengths
