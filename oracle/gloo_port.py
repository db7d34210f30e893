"""Multi-process CPU port of the reference's uneven collectives over ``torch.distributed``.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Used (a) to check the
single-process restatement in ``collectives_math.py`` through a real transport,
(b) as the timed CPU baseline of ``bench.py`` (``cpu_baseline.kind == "port"``),
because the reference tree itself does not travel to the GPU machine.

It keeps the reference's two strategies:

* padding mode (``collectives.py:14-29, 88-103``): pad every shard to
  ``max(sharding_lengths)``, run an equal-chunk list collective, strip the pads;
* group-call mode (``collectives.py:31-66, 105-140``): one rooted broadcast /
  reduce per shard with exact sizes.

Differences from the reference, all outside the arithmetic:

* every scratch buffer takes the input's dtype (the reference's ``torch.empty``
  calls at ``collectives.py:12,18,36,100,126,157,164`` omit it, so bf16 inputs
  fail there);
* pads are zero-filled instead of uninitialised (their values are discarded);
* the group-call variants issue their rooted collectives one after another
  instead of inside torch 1.13's private ``_coalescing_manager(None, reqs)``
  (``collectives.py:42,58,113,132``), whose signature changed in torch 2.x;
* ``all_to_all`` (``collectives.py:152-166``) uses ``all_to_all_single`` with
  uneven split sizes because gloo has no list all-to-all.

Pinned by ``tests/golden/make_golden.py``, which runs this port and the
unmodified reference side by side on gloo ranks and requires identical results.
"""
from __future__ import annotations


import torch
import torch.distributed as dist


def _with_extent(shape, dim, extent):
    shape = list(shape)
    shape[dim] = extent
    return shape


def _pad(t: torch.Tensor, dim: int, extent: int) -> torch.Tensor:
    """Grow ``t`` to ``extent`` on ``dim`` (``collectives.py:9-12``)."""
    short = extent - t.shape[dim]
    if short == 0:
        return t.contiguous()
    filler = torch.zeros(_with_extent(t.shape, dim, short), dtype=t.dtype, device=t.device)
    return torch.cat((t, filler), dim=dim).contiguous()


def _gather_padded(t, dim, lengths):
    """Equal-chunk all-gather of padded shards, pads stripped (``collectives.py:16-20, 100-102``)."""
    widest = max(lengths)
    recv = [torch.empty(_with_extent(t.shape, dim, widest), dtype=t.dtype, device=t.device) for _ in lengths]
    dist.all_gather(recv, _pad(t, dim, widest))
    return torch.cat([chunk.narrow(dim, 0, n) for chunk, n in zip(recv, lengths)], dim=dim)


def _scatter_sum_padded(t, dim, lengths, rank):
    """Equal-chunk reduce-scatter of padded slices, pad stripped (``collectives.py:24-28, 92-96``)."""
    widest = max(lengths)
    send = [_pad(piece, dim, widest) for piece in torch.split(t.contiguous(), list(lengths), dim=dim)]
    recv = torch.empty_like(send[0])
    dist.reduce_scatter(recv, send)
    return recv.narrow(dim, 0, lengths[rank]).contiguous()


def _gather_rooted(t, dim, lengths, rank):
    """One exact-size broadcast per shard (``collectives.py:35-50, 126-140``)."""
    parts = []
    for owner, n in enumerate(lengths):
        if owner == rank:
            buf = t.contiguous()
        else:
            buf = torch.empty(_with_extent(t.shape, dim, n), dtype=t.dtype, device=t.device)
        parts.append(buf)
    work = [dist.broadcast(buf, owner, async_op=True) for owner, buf in enumerate(parts)]
    for w in work:
        w.wait()
    return torch.cat(parts, dim=dim)


def _scatter_sum_rooted(t, dim, lengths, rank):
    """One exact-size rooted reduce per slice (``collectives.py:54-66, 109-121``)."""
    pieces = [p.contiguous().clone() for p in torch.split(t, list(lengths), dim=dim)]
    work = [dist.reduce(p, owner, async_op=True) for owner, p in enumerate(pieces)]
    for w in work:
        w.wait()
    return pieces[rank]


def _exchange(t, split_dim, cat_dim, split_lengths, cat_lengths, rank):
    """Uneven all-to-all (``collectives.py:154-159``)."""
    mine = torch.split(t.contiguous(), list(split_lengths), dim=split_dim)
    shape_of = lambda n: _with_extent(mine[rank].shape, cat_dim, n)
    send = torch.cat([p.contiguous().reshape(-1) for p in mine]) if len(mine) else t.reshape(-1)
    in_counts = [p.numel() for p in mine]
    out_counts = [int(torch.Size(shape_of(n)).numel()) for n in cat_lengths]
    recv = torch.empty(sum(out_counts), dtype=t.dtype, device=t.device)
    dist.all_to_all_single(recv, send, output_split_sizes=out_counts, input_split_sizes=in_counts)
    blocks = [b.reshape(shape_of(n)) for b, n in zip(torch.split(recv, out_counts), cat_lengths)]
    return torch.cat(blocks, dim=cat_dim)


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, dim, lengths, rank, rooted):
        ctx.meta = (dim, list(lengths), rank, rooted)
        return (_gather_rooted(t, dim, lengths, rank) if rooted else _gather_padded(t, dim, lengths))

    @staticmethod
    def backward(ctx, g):
        dim, lengths, rank, rooted = ctx.meta
        fn = _scatter_sum_rooted if rooted else _scatter_sum_padded
        return fn(g, dim, lengths, rank), None, None, None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, dim, lengths, rank, rooted):
        ctx.meta = (dim, list(lengths), rank, rooted)
        fn = _scatter_sum_rooted if rooted else _scatter_sum_padded
        return fn(t, dim, lengths, rank)

    @staticmethod
    def backward(ctx, g):
        dim, lengths, rank, rooted = ctx.meta
        out = _gather_rooted(g, dim, lengths, rank) if rooted else _gather_padded(g.contiguous(), dim, lengths)
        return out, None, None, None, None


class _AllReduce(torch.autograd.Function):
    """``collectives.py:73-84``: sum forward and backward (out of place here)."""

    @staticmethod
    def forward(ctx, t):
        out = t.contiguous().clone()
        dist.all_reduce(out)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.contiguous().clone()
        dist.all_reduce(out)
        return out


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, split_dim, cat_dim, split_lengths, cat_lengths, rank):
        ctx.meta = (split_dim, cat_dim, list(split_lengths), list(cat_lengths), rank)
        return _exchange(t, split_dim, cat_dim, split_lengths, cat_lengths, rank)

    @staticmethod
    def backward(ctx, g):
        split_dim, cat_dim, split_lengths, cat_lengths, rank = ctx.meta
        # the dual exchange: cut on cat_dim, concatenate on split_dim (collectives.py:161-166)
        return _exchange(g, cat_dim, split_dim, cat_lengths, split_lengths, rank), None, None, None, None, None


class _Replicate(torch.autograd.Function):
    """``collectives.py:171-180``: identity forward, gradient all-reduce backward."""

    @staticmethod
    def forward(ctx, t):
        return t

    @staticmethod
    def backward(ctx, g):
        out = g.contiguous().clone()
        dist.all_reduce(out)
        return out


def all_gather(tensor, dim, sharding_lengths, rank):
    return _AllGather.apply(tensor, dim, sharding_lengths, rank, False)


def all_gather_by_group_call(tensor, dim, sharding_lengths, rank):
    return _AllGather.apply(tensor, dim, sharding_lengths, rank, True)


def reduce_scatter(tensor, dim, sharding_lengths, rank):
    return _ReduceScatter.apply(tensor, dim, sharding_lengths, rank, False)


def reduce_scatter_by_group_call(tensor, dim, sharding_lengths, rank):
    return _ReduceScatter.apply(tensor, dim, sharding_lengths, rank, True)


def all_reduce(tensor):
    return _AllReduce.apply(tensor)


def dynamic_slice(tensor, dim, sharding_lengths, rank):
    return torch.split(tensor, list(sharding_lengths), dim=dim)[rank].contiguous()


def all_to_all(tensor, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths, rank):
    return _AllToAll.apply(tensor, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths, rank)


def replicate(tensor):
    return _Replicate.apply(tensor)
