"""CPU restatement of the self-attention the planner emits, in float64.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

The reference calls ``torch.nn.functional.multi_head_attention_forward`` with a packed
in-projection on (L, N, E) tensors (``hap.rs:1297-1329``); the language model adds the -inf
upper-triangular mask of ``models.py:72``.  Here: q, k, v = split(x W_in^T + b_in); per batch entry
and head softmax(q k^T / sqrt(d) + mask) v; heads concatenated; out-projection.  The arithmetic of
the reference lives in ATen (torch 1.13.1, ``environment.yml:153``); ``tests/test_oracle_attention.py``
pins this restatement against that function's CPU implementation in the installed torch.
"""
from __future__ import annotations

import math

import torch


def attention_core(qkv: torch.Tensor, num_heads: int, mask=None, keep=None, dropout_p: float = 0.0) -> torch.Tensor:
    """qkv (L, N, 3E) -> (L, N, E) in float64.  ``keep`` (N, H, L, L), 0/1: the dropout mask on the
    probabilities; kept entries are scaled by 1 / (1 - dropout_p) as ``F.dropout`` does inside
    ``multi_head_attention_forward``."""
    L, n, e3 = qkv.shape
    E = e3 // 3
    d = E // num_heads
    q, k, v = (t.double().reshape(L, n, num_heads, d).permute(1, 2, 0, 3) for t in qkv.split(E, dim=2))  # (N, H, L, d)
    s = q @ k.transpose(-1, -2) / math.sqrt(d)
    if mask is not None:
        s = s + mask.double()
    p = torch.softmax(s, dim=-1)
    if keep is not None:
        p = p * keep.double() / (1.0 - dropout_p)
    return (p @ v).permute(2, 0, 1, 3).reshape(L, n, E)


def multi_head_attention(x, in_w, in_b, out_w, out_b, num_heads, mask=None):
    qkv = x.double() @ in_w.double().t() + in_b.double()
    return attention_core(qkv, num_heads, mask) @ out_w.double().t() + out_b.double()


def causal_mask(L: int) -> torch.Tensor:
    return torch.full((L, L), float("-inf")).triu_(1)
