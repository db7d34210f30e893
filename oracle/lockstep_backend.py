"""CPU backend for ``hap_b200.spmd.LockstepWorld``: the list-in / list-out collectives computed
by ``collectives_math`` with autograd, so a whole synthesized SPMD program can be replayed on
the CPU for all ranks at once and compared with the CUDA path.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

``collectives_math`` is written with differentiable tensor ops, and differentiating the sum of
all ranks' losses through them yields exactly the backward duals of ``collectives.py:22-29,
80-84, 98-103, 161-166``.  Only ``replicate`` needs a custom backward (identity forward,
gradient all-reduce backward, ``collectives.py:171-180``).
"""
from __future__ import annotations

import torch

from . import collectives_math as cm


class _Replicate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, *tensors):
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        return tuple(cm.all_reduce(list(grads)))


class OracleCollectives:
    def all_gather(self, tensors, dim, lengths):
        return cm.all_gather(tensors, dim, lengths)

    all_gather_by_group_call = all_gather

    def reduce_scatter(self, tensors, dim, lengths):
        return cm.reduce_scatter(tensors, dim, lengths)

    reduce_scatter_by_group_call = reduce_scatter

    def all_reduce(self, tensors):
        return cm.all_reduce(tensors)

    def replicate(self, tensors):
        return list(_Replicate.apply(*tensors))

    def dynamic_slice(self, tensors, dim, lengths):
        return [cm.dynamic_slice(t, dim, lengths, r) for r, t in enumerate(tensors)]

    def all_to_all(self, tensors, split_dim, cat_dim, split_lengths, cat_lengths):
        return cm.all_to_all(tensors, split_dim, cat_dim, split_lengths, cat_lengths)
