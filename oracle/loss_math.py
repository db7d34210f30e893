"""CPU restatement of the models' loss (test infrastructure, never imported by the product).

The reference's language models end in ``torch.log_softmax(x, dim=-1)`` and
``NLLLoss(reduction='sum')`` (``models.py:116-117``), which the planner emits as two nodes
(``hap.rs:1808, 1858``).  Targets equal to torch's ``ignore_index`` (-100) contribute nothing.
"""
import torch
import torch.nn.functional as F


def nll_log_softmax_sum(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    V = logits.shape[-1]
    return F.nll_loss(F.log_softmax(logits.float(), dim=-1).reshape(-1, V), targets.reshape(-1), reduction="sum")
