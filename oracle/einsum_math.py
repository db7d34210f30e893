"""CPU restatement of the MoE einsums the planner emits (``hap.rs:2255-2276``; ``models.py:356-364``).

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  The reference calls ``torch.einsum`` with
these exact code strings; the oracle evaluates the same index expressions in float64, and autograd
of those expressions gives the reference's backward.
"""
import torch


def einsum(code: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.einsum(code, a.double(), b.double())
