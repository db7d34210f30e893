"""sharding_round: the oracle against the extents the benchmark configurations quote, and
the C ABI against the oracle (bit-exact: it fixes every shard extent of the program)."""
import math
import random

import pytest

import hap_b200
from oracle.sharding_round import sharding_round as oracle_round

R8 = [.22, .18, .15, .13, .11, .09, .07, .05]
R4 = [.3, .25, .2, .25]
R4x2 = [.15, .125, .1, .125] * 2

# Extents obtained by evaluating hap.rs:3536-3559 by hand for the benchmark configurations.
KNOWN = [
    (64, [.6, .4], [38, 26]),
    (1024, [.6, .4], [614, 410]),
    (4096, [.6, .4], [2458, 1638]),
    (256, R8, [56, 46, 39, 33, 28, 23, 18, 13]),
    (32, R8, [7, 6, 5, 4, 3, 3, 2, 2]),
    (768, R8, [169, 138, 115, 100, 85, 69, 54, 38]),
    (3072, R8, [676, 553, 461, 399, 338, 276, 215, 154]),
    (2304, R8, [507, 415, 346, 300, 253, 207, 161, 115]),
    (33280, R8, [7322, 5990, 4992, 4326, 3661, 2995, 2330, 1664]),
    (256, R4, [77, 64, 51, 64]),
    (768, R4, [230, 192, 154, 192]),
    (3072, R4, [922, 768, 614, 768]),
    (512, R4x2, [77, 64, 51, 64] * 2),
    (3072, R4x2, [461, 384, 307, 384] * 2),
    (256, [.55, .45], [141, 115]),
    (1, R8, [1] * 8),          # the broadcast hack, hap.rs:3538-3540
    (0, [.5, .5], [0, 0]),
]


@pytest.mark.parametrize("full,ratios,want", KNOWN)
def test_oracle_known_extents(full, ratios, want):
    assert oracle_round(full, ratios) == want


@pytest.mark.parametrize("full,ratios,want", KNOWN)
def test_native_known_extents(full, ratios, want):
    assert hap_b200.sharding_round(full, ratios) == want


def test_ties_go_to_the_last_index():
    # equal ratios, one element left over: Rust's max_by_key keeps the last maximum
    assert oracle_round(5, [.25, .25, .25, .25]) == [1, 1, 1, 2]
    assert hap_b200.sharding_round(5, [.25, .25, .25, .25]) == [1, 1, 1, 2]


def test_native_matches_oracle_fuzz():
    rng = random.Random(7)
    for _ in range(3000):
        w = rng.randint(1, 16)
        raw = [rng.random() ** rng.choice([1, 2, 4]) for _ in range(w)]
        if rng.random() < 0.2:
            raw[rng.randrange(w)] = 0.0
        tot = sum(raw) or 1.0
        ratios = [x / tot for x in raw]
        # keep the sum a hair under 1 so the reference's assert (sum of floors <= full) cannot trip on rounding
        ratios = [x * (1 - 1e-12) for x in ratios]
        full = rng.choice([0, 1, 2, 3, 7, 64, 255, 256, 1000, 4096, 33280, rng.randint(0, 10 ** 6)])
        want = oracle_round(full, ratios)
        got = hap_b200.sharding_round(full, ratios)
        assert got == want, (full, ratios)
        if full != 1:
            assert sum(got) == full
            assert all(g >= math.floor(r * full) for g, r in zip(got, ratios))


def test_in_place_form_matches_reference_export():
    lst = list(R8)
    hap_b200.sharding_round_(256, lst)          # hap.rs:211-218 overwrites the ratio list
    assert lst == [56, 46, 39, 33, 28, 23, 18, 13]


def test_ratios_over_one_are_rejected():
    from hap_b200._native import HapxError
    with pytest.raises(HapxError):
        hap_b200.sharding_round(10, [.9, .9])
    with pytest.raises(AssertionError):
        oracle_round(10, [.9, .9])
