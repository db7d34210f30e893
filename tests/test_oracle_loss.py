"""The loss oracle is the reference's own two ops (models.py:116-117); this pins its conventions."""
import math

import torch

from oracle import loss_math


def test_summed_nll_of_uniform_logits_and_ignore_index():
    logits = torch.zeros(3, 4, 8)
    targets = torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7], [0, -100, 0, 0]])
    got = loss_math.nll_log_softmax_sum(logits, targets)
    assert abs(float(got) - 11 * math.log(8)) < 1e-5          # 12 rows, one ignored
    bf = loss_math.nll_log_softmax_sum(logits.to(torch.bfloat16), targets)
    assert bf.dtype == torch.float32 and abs(float(bf) - float(got)) < 1e-5
