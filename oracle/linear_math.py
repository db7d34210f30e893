"""CPU restatement of the sharded ``F.linear`` the planner emits, forward and backward.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

The reference program calls ``torch.nn.functional.linear(x, W, b)`` on per-rank shards
(emitted at ``hap.rs:1030-1037``; data-parallel and column-parallel variants at
``hap.rs:2787-2816``) and lets autograd produce ``dx = g W``, ``dW = g^T x``, ``db = sum_rows g``.
Here the same contractions are evaluated in float64 on the CPU from the (possibly bf16-rounded)
inputs, so the only difference to a bf16 tensor-core result is accumulation order and the final
rounding.  The arithmetic itself lives in a third-party library in the reference (cuBLAS via
ATen, torch 1.13.1 per ``environment.yml:153``), so parity is "unpinned" beyond the tolerance the
north star states: 1e-2 relative for bf16, 1e-5 for fp32.
"""
from __future__ import annotations

import math

import torch


def _act(v: torch.Tensor, name: str) -> torch.Tensor:
    if name == "none":
        return v
    if name == "relu":
        return torch.relu(v)
    if name == "gelu":
        return 0.5 * v * (1.0 + torch.erf(v / math.sqrt(2.0)))
    if name == "sigmoid":
        return torch.sigmoid(v)
    raise KeyError(name)


def linear_forward(x, w, b=None, act="none"):
    y = x.double() @ w.double().t()
    if b is not None:
        y = y + b.double()
    return _act(y, act)


def linear_backward(g, x, w):
    """(dx, dw, db) in float64."""
    g2, x2 = g.double().reshape(-1, g.shape[-1]), x.double().reshape(-1, x.shape[-1])
    return (g2 @ w.double()).reshape(x.shape), g2.t() @ x2, g2.sum(0)
