"""Single-process CPU restatement of what each uneven collective computes.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Every function takes the list of ALL ranks' input tensors (CPU) and returns the
list of all ranks' outputs, i.e. it states the value semantics of the
reference's ``collectives.py`` without any transport.  The padding the
reference adds around its NCCL calls (``collectives.py:9-12``) carries no
values into the result, so it has no counterpart here.

Reductions accumulate in float32 in rank order 0..W-1 and round once to the
output dtype; the reference's order is whatever its backend picks, so
reductions are compared with a tolerance (1e-5 relative for fp32, 1e-2 for
bf16), while gathers / re-sharding are compared bit-exactly.

Pinning: ``tests/golden/make_golden.py`` ran the reference's own
``collectives.py`` (imported unmodified) on gloo/CPU ranks and stored its
outputs; ``tests/test_oracle_golden.py`` checks these functions against those
files and against the known answers written in ``collectives.py:198-323``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def _acc_dtype(dtype: torch.dtype) -> torch.dtype:
    return torch.float64 if dtype == torch.float64 else torch.float32


def rank_sum(tensors: Sequence[torch.Tensor], scale: float = 1.0,
             out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Sum over ranks in rank order with a wide accumulator, then scale, then round."""
    acc_t = _acc_dtype(tensors[0].dtype)
    acc = tensors[0].to(acc_t).clone()
    for t in tensors[1:]:
        acc += t.to(acc_t)
    if scale != 1.0:
        acc = acc * scale
    return acc.to(out_dtype or tensors[0].dtype)


def all_gather(shards: Sequence[torch.Tensor], dim: int, sharding_lengths: Sequence[int]) -> List[torch.Tensor]:
    """``collectives.py:14-20`` (AllGather.forward) and ``:31-50`` (group-call forward).

    Rank r holds extent ``sharding_lengths[r]`` on ``dim``; every rank ends with
    the concatenation in rank order.
    """
    for r, (s, l) in enumerate(zip(shards, sharding_lengths)):
        assert s.shape[dim] == l, (r, tuple(s.shape), dim, l)
    full = torch.cat(list(shards), dim=dim)
    return [full.clone() for _ in shards]


def reduce_scatter(inputs: Sequence[torch.Tensor], dim: int, sharding_lengths: Sequence[int],
                   scale: float = 1.0, out_dtype: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """``collectives.py:88-96`` (ReduceScatter.forward) and ``:105-121`` (group-call forward).

    Every rank holds a full-shape partial; rank r ends with slice r (extent
    ``sharding_lengths[r]`` on ``dim``) of the elementwise sum.
    """
    total = rank_sum(inputs, scale, out_dtype)
    return [s.contiguous() for s in torch.split(total, list(sharding_lengths), dim=dim)]


def all_reduce(inputs: Sequence[torch.Tensor], scale: float = 1.0) -> List[torch.Tensor]:
    """``collectives.py:73-78`` (AllReduce.forward), ``:80-84`` and ``:176-180`` (backward of all_reduce / replicate)."""
    total = rank_sum(inputs, scale)
    return [total.clone() for _ in inputs]


def dynamic_slice(tensor: torch.Tensor, dim: int, sharding_lengths: Sequence[int], rank: int) -> torch.Tensor:
    """``collectives.py:146-148``."""
    return torch.split(tensor, list(sharding_lengths), dim=dim)[rank].contiguous()


def all_to_all(inputs: Sequence[torch.Tensor], split_dim: int, cat_dim: int,
               split_sharding_lengths: Sequence[int], cat_sharding_lengths: Sequence[int]) -> List[torch.Tensor]:
    """``collectives.py:152-159`` (AllToAll.forward).

    Rank p holds extent ``cat_sharding_lengths[p]`` on ``cat_dim`` and the full
    extent on ``split_dim``.  It cuts its tensor on ``split_dim`` and sends piece
    r to rank r; rank r concatenates what it received, in rank order, on
    ``cat_dim``.  Zero-length pieces are legal (``collectives.py:297-309``).
    """
    world = len(inputs)
    pieces = [torch.split(t, list(split_sharding_lengths), dim=split_dim) for t in inputs]
    outs = []
    for r in range(world):
        for p in range(world):
            assert pieces[p][r].shape[cat_dim] == cat_sharding_lengths[p]
        outs.append(torch.cat([pieces[p][r] for p in range(world)], dim=cat_dim).contiguous())
    return outs


# ----- backward duals (what the autograd.Functions return as input gradients) -----

def all_gather_backward(grad_outputs, dim, sharding_lengths):
    """``collectives.py:22-29`` / ``:52-66``: uneven reduce-scatter of the output gradients."""
    return reduce_scatter(grad_outputs, dim, sharding_lengths)


def reduce_scatter_backward(grad_outputs, dim, sharding_lengths):
    """``collectives.py:98-103`` / ``:123-140``: uneven all-gather of the output gradients."""
    return all_gather(grad_outputs, dim, sharding_lengths)


def all_to_all_backward(grad_outputs, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths):
    """``collectives.py:161-166``: the same exchange with the two dims swapped."""
    return all_to_all(grad_outputs, cat_dim, split_dim, cat_sharding_lengths, split_sharding_lengths)


def dynamic_slice_backward(grad_output, full_shape, dim, sharding_lengths, rank):
    """Autograd of split + getitem (``collectives.py:146-148``): zero outside the own slice."""
    g = torch.zeros(full_shape, dtype=grad_output.dtype)
    start = sum(sharding_lengths[:rank])
    g.narrow(dim, start, sharding_lengths[rank]).copy_(grad_output)
    return g
