"""The reference's collectives over a LOCAL communicator: ``world`` virtual ranks on one GPU.

Each function takes the list of all ranks' tensors and returns the list of all ranks'
results, with autograd.  Differentiating the sum of the ranks' losses gives every rank
exactly the gradient the distributed backward of ``collectives.py`` would give it, so the
reference's forward/backward checks (``collectives.py:187-324``) can be replayed on a single
device against the same kernels and flag protocol that run across GPUs.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from . import _native as N
from . import comm as _comm


class LocalCollectives:
    def __init__(self, comm: _comm.Comm):
        if comm.n_local != comm.world:
            raise ValueError("LocalCollectives needs a local communicator (hap_b200.comm.local_comm)")
        self.comm = comm
        self.world = comm.world

    # -- list-in / list-out, differentiable -----------------------------------------------
    def all_gather(self, shards, dim, sharding_lengths, mode=N.MODE_PADDING) -> List[torch.Tensor]:
        return list(_AllGatherL.apply(self.comm, dim, list(sharding_lengths), mode, *shards))

    def all_gather_by_group_call(self, shards, dim, sharding_lengths):
        return self.all_gather(shards, dim, sharding_lengths, N.MODE_GROUP_CALL)

    def reduce_scatter(self, tensors, dim, sharding_lengths, mode=N.MODE_PADDING) -> List[torch.Tensor]:
        return list(_ReduceScatterL.apply(self.comm, dim, list(sharding_lengths), mode, *tensors))

    def reduce_scatter_by_group_call(self, tensors, dim, sharding_lengths):
        return self.reduce_scatter(tensors, dim, sharding_lengths, N.MODE_GROUP_CALL)

    def all_reduce(self, tensors) -> List[torch.Tensor]:
        return list(_AllReduceL.apply(self.comm, *tensors))

    def replicate(self, tensors) -> List[torch.Tensor]:
        return list(_ReplicateL.apply(self.comm, *tensors))

    def all_to_all(self, tensors, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths) -> List[torch.Tensor]:
        return list(_AllToAllL.apply(self.comm, split_dim, cat_dim, list(split_sharding_lengths),
                                     list(cat_sharding_lengths), *tensors))

    def dynamic_slice(self, tensors, dim, sharding_lengths) -> List[torch.Tensor]:
        from .collectives import dynamic_slice
        return [dynamic_slice(t, dim, sharding_lengths, r) for r, t in enumerate(tensors)]


def _c(ts: Sequence[torch.Tensor]):
    return [t.contiguous() for t in ts]


class _AllGatherL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, dim, lengths, mode, *shards):
        ctx.meta = (comm, dim, lengths, mode)
        return tuple(comm.all_gather(_c(shards), dim, lengths, mode))

    @staticmethod
    def backward(ctx, *grads):
        comm, dim, lengths, mode = ctx.meta
        return (None, None, None, None, *comm.reduce_scatter(_c(grads), dim, lengths, mode))


class _ReduceScatterL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, dim, lengths, mode, *tensors):
        ctx.meta = (comm, dim, lengths, mode)
        return tuple(comm.reduce_scatter(_c(tensors), dim, lengths, mode))

    @staticmethod
    def backward(ctx, *grads):
        comm, dim, lengths, mode = ctx.meta
        return (None, None, None, None, *comm.all_gather(_c(grads), dim, lengths, mode))


class _AllReduceL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, *tensors):
        ctx.comm = comm
        return tuple(comm.all_reduce(_c(tensors)))

    @staticmethod
    def backward(ctx, *grads):
        return (None, *ctx.comm.all_reduce(_c(grads)))


class _ReplicateL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, *tensors):
        ctx.comm = comm
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        return (None, *ctx.comm.all_reduce(_c(grads)))


class _AllToAllL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, split_dim, cat_dim, split_lengths, cat_lengths, *tensors):
        ctx.meta = (comm, split_dim, cat_dim, split_lengths, cat_lengths)
        return tuple(comm.all_to_all(_c(tensors), split_dim, cat_dim, split_lengths, cat_lengths))

    @staticmethod
    def backward(ctx, *grads):
        comm, split_dim, cat_dim, split_lengths, cat_lengths = ctx.meta
        return (None, None, None, None, None, *comm.all_to_all(_c(grads), cat_dim, split_dim, cat_lengths, split_lengths))
