"""CPU restatement of the reference's step tail (test infrastructure, never imported by the product).

``worker.py:74`` clips with ``torch.nn.utils.clip_grad_norm_(params, 0.5)`` over the shards a rank
holds, ``worker.py:76`` steps ``torch.optim.Adam`` (created at ``worker.py:47`` with default betas,
eps and no weight decay).  This file restates both in float64/float32 tensor arithmetic so that the
fused GPU kernels can be compared with it; ``tests/test_optim_oracle.py`` pins it against the torch
functions themselves.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch


def clip_coefficient(grads: Sequence[torch.Tensor], max_norm: float):
    """(total 2-norm over all tensors, min(1, max_norm / (norm + 1e-6)))."""
    total = math.sqrt(sum(float(g.double().pow(2).sum()) for g in grads))
    return total, min(1.0, max_norm / (total + 1e-6))


def clip_adam_step(params: List[torch.Tensor], grads: List[torch.Tensor], exp_avg: List[torch.Tensor],
                   exp_avg_sq: List[torch.Tensor], step: int, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999,
                   eps: float = 1e-8, weight_decay: float = 0.0, max_norm: Optional[float] = None, compute=torch.float32):
    """One iteration, in place; ``step`` is the number of steps taken BEFORE this one.

    The arithmetic runs in ``compute`` precision and each result is rounded once to the tensor's dtype.
    Returns the gradient norm (0.0 without clipping).
    """
    norm, coef = (0.0, 1.0) if max_norm is None else clip_coefficient(grads, max_norm)
    t = step + 1
    bc1 = 1.0 - beta1 ** t
    bc2_sqrt = math.sqrt(1.0 - beta2 ** t)
    for p, g, m, v in zip(params, grads, exp_avg, exp_avg_sq):
        pf, gf, mf, vf = p.to(compute), g.to(compute) * coef, m.to(compute), v.to(compute)
        if weight_decay:
            gf = gf + weight_decay * pf
        mf = mf + (1.0 - beta1) * (gf - mf)
        vf = beta2 * vf + (1.0 - beta2) * gf * gf
        denom = vf.sqrt() / bc2_sqrt + eps
        pf = pf - (lr / bc1) * (mf / denom)
        p.copy_(pf.to(p.dtype)); m.copy_(mf.to(m.dtype)); v.copy_(vf.to(v.dtype))
    return norm
