"""Generate ``gating.pt`` in this directory from the reference's own top-2 gating.

Run once, on a machine that has the reference checkout (it is NOT needed to run the tests):

    python tests/golden/make_gating_golden.py --reference /path/to/hap --out tests/golden

The script imports the reference's ``models.py`` UNMODIFIED and calls ``_top_2_gating``
(``models.py:477-502``, the body behind the fx-wrapped ``top_2_gating``) on seeded float32
inputs.  Each case stores the inputs and, to keep the file small, the two results in sparse form:
the indices of the non-zero entries of the dispatch tensor, and the indices and values of the
non-zero entries of the combine tensor.  The cases
cover: every token kept, experts that overflow their capacity through first choices alone,
overflow caused only by the offset of the second choices (the reference adds the SUM of the
first-choice slot numbers of an expert, not their count, to its second-choice slots), and the
MoE configuration's expert count and capacity at a short sequence.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

# (name, batch, seq, d_model, n_expert, capacity, seed)
CASES = [
    ("roomy", 2, 16, 8, 4, 64, 11),
    ("tight", 2, 64, 8, 4, 20, 12),
    ("second_choice_offset", 3, 24, 16, 8, 6, 13),
    ("moe_config_short", 2, 96, 32, 32, 20, 14),
    ("one_token", 1, 1, 4, 2, 3, 15),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import models  # the reference's models.py, unmodified

    out = {}
    for name, b, s, d, e, c, seed in CASES:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(b, s, d, generator=g)
        w = torch.randn(d, e, generator=g) * d ** -0.5
        dispatch, combine = models._top_2_gating(x, e, c, w, train=True)
        assert set(dispatch.unique().tolist()) <= {0.0, 1.0}
        ci = combine.nonzero()
        out[name] = {"x": x, "gate_weight": w, "n_expert": e, "capacity": c, "shape": tuple(combine.shape),
                     "dispatch_nonzero": dispatch.nonzero().to(torch.int32), "combine_nonzero": ci.to(torch.int32),
                     "combine_values": combine[tuple(ci.t())].clone()}
        kept = int(dispatch.sum())
        print(f"{name}: b={b} s={s} e={e} c={c}: {kept} of {2 * b * s} assignments kept")
    torch.save(out, os.path.join(args.out, "gating.pt"))


if __name__ == "__main__":
    main()
