"""Drop-in replacement for the reference's ``collectives.py`` (one process per GPU).

Same eight module-level functions, same positional signatures and the same autograd
duals as ``collectives.py:70,71,86,142,143,146,168,182`` of the reference, so the fx
program synthesized by the planner (``hap.rs:899-902`` resolves ``collectives.<name>``)
runs unchanged once this module is importable as ``collectives``
(see :func:`install_as_collectives`) or the node targets are rewritten
(:func:`retarget_fx_graph`).

Every function goes through the C ABI into the CUDA kernels; there is no fallback to
``torch.distributed`` collectives.  Differences from the reference, all documented
behaviour rather than arithmetic:

* inputs are never modified (the reference's ``all_reduce`` works in place on a
  contiguous input, ``collectives.py:76-78``, and ``reduce_scatter_by_group_call``
  overwrites its input through split views, ``collectives.py:109-121``);
* every buffer has the input's dtype (the reference allocates float32 receive buffers,
  ``collectives.py:12,18,36,100,126,157,164``, so its bf16 path fails);
* reductions accumulate in float32 in rank order and round once.
"""
from __future__ import annotations

import sys
from typing import Optional

import torch

from . import _native as N
from . import comm as _comm

_default: Optional[_comm.Comm] = None
_defer_replicate = False


def defer_replicate(on: bool) -> None:
    """While on, the backward of :func:`replicate` hands the gradient through unchanged.  The step
    driver turns this on when it reduces the gradients of all replicated parameters itself, as one
    all_reduce over a flat buffer, instead of one all_reduce per parameter (collectives.py:176-180)."""
    global _defer_replicate
    _defer_replicate = bool(on)


def set_default_comm(c: Optional[_comm.Comm]) -> None:
    global _default
    _default = c


def has_default_comm() -> bool:
    return _default is not None


def get_default_comm() -> _comm.Comm:
    """The process communicator; created from the default ``torch.distributed`` group on first use."""
    global _default
    if _default is None:
        _default = _comm.init_process_comm()
    if _default.n_local != 1:
        raise RuntimeError("hap_b200.collectives needs a one-rank-per-process communicator")
    return _default


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, dim, sharding_lengths, rank, mode):
        ctx.meta = (dim, list(sharding_lengths), mode)
        return get_default_comm().all_gather([tensor], dim, sharding_lengths, mode)[0]

    @staticmethod
    def backward(ctx, grad_output):
        dim, lengths, mode = ctx.meta
        return get_default_comm().reduce_scatter([grad_output], dim, lengths, mode)[0], None, None, None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, dim, sharding_lengths, rank, mode):
        ctx.meta = (dim, list(sharding_lengths), mode)
        return get_default_comm().reduce_scatter([tensor], dim, sharding_lengths, mode)[0]

    @staticmethod
    def backward(ctx, grad_output):
        dim, lengths, mode = ctx.meta
        return get_default_comm().all_gather([grad_output], dim, lengths, mode)[0], None, None, None, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor):
        return get_default_comm().all_reduce([tensor])[0]

    @staticmethod
    def backward(ctx, grad_output):
        return get_default_comm().all_reduce([grad_output])[0]


class _DynamicSlice(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, dim, sharding_lengths, rank):
        ctx.meta = (dim, list(sharding_lengths), rank)
        return _comm.dynamic_slice(tensor, dim, sharding_lengths, rank)

    @staticmethod
    def backward(ctx, grad_output):
        dim, lengths, rank = ctx.meta
        return _comm.dynamic_slice_backward(grad_output, dim, lengths, rank), None, None, None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths, rank):
        ctx.meta = (split_dim, cat_dim, list(split_sharding_lengths), list(cat_sharding_lengths))
        return get_default_comm().all_to_all([tensor], split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths)[0]

    @staticmethod
    def backward(ctx, grad_output):
        split_dim, cat_dim, split_lengths, cat_lengths = ctx.meta
        grad = get_default_comm().all_to_all([grad_output], cat_dim, split_dim, cat_lengths, split_lengths)[0]
        return grad, None, None, None, None, None


class _Replicate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor):
        return tensor

    @staticmethod
    def backward(ctx, grad_output):
        if _defer_replicate:
            return grad_output
        return get_default_comm().all_reduce([grad_output])[0]


# Plain module-level defs (not aliases): fx.Node.__repr__ needs __module__ (collectives.py:69).
def all_gather(tensor, dim, sharding_lengths, rank):
    return _AllGather.apply(tensor, dim, sharding_lengths, rank, N.MODE_PADDING)


def all_gather_by_group_call(tensor, dim, sharding_lengths, rank):
    return _AllGather.apply(tensor, dim, sharding_lengths, rank, N.MODE_GROUP_CALL)


def all_reduce(tensor):
    return _AllReduce.apply(tensor)


def reduce_scatter(tensor, dim, sharding_lengths, rank):
    return _ReduceScatter.apply(tensor, dim, sharding_lengths, rank, N.MODE_PADDING)


def reduce_scatter_by_group_call(tensor, dim, sharding_lengths, rank):
    return _ReduceScatter.apply(tensor, dim, sharding_lengths, rank, N.MODE_GROUP_CALL)


def dynamic_slice(tensor, dim, sharding_lengths, rank):
    return _DynamicSlice.apply(tensor, dim, sharding_lengths, rank)


def all_to_all(tensor, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths, rank):
    return _AllToAll.apply(tensor, split_dim, cat_dim, split_sharding_lengths, cat_sharding_lengths, rank)


def replicate(tensor):
    return _Replicate.apply(tensor)


class PendingGather:
    """An all_gather that was issued on the communicator's side stream: its result and the event
    that marks its completion.  :func:`all_gather_wait` turns it into the tensor."""

    __slots__ = ("tensor", "event")

    def __init__(self, tensor, event):
        self.tensor, self.event = tensor, event


def all_gather_start(tensor, dim, sharding_lengths, rank):
    """:func:`all_gather` issued on the communicator's side stream, so that it overlaps with whatever
    the current stream does next.  For gathers whose input is ready early - the ZeRO-style sharded
    parameters of a program (``hap.rs:2527-2555``), which only change in the optimizer step.  The
    backward pass (the uneven reduce_scatter of the gradient) then runs on that side stream as well,
    because autograd runs a node's backward on its forward's stream, and overlaps with the rest of
    the backward pass.  Returns a :class:`PendingGather`; :func:`all_gather_wait` makes the current
    stream wait for it.  Collectives stay ordered among themselves (one in flight per communicator)."""
    comm = get_default_comm()
    side = comm.side_stream()
    cur = torch.cuda.current_stream(tensor.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        out = _AllGather.apply(tensor, dim, sharding_lengths, rank, N.MODE_PADDING)
        event = torch.cuda.Event()
        event.record(side)
    return PendingGather(out, event)


def all_gather_wait(pending):
    """The gathered tensor of :func:`all_gather_start`, usable on the current stream."""
    cur = torch.cuda.current_stream(pending.tensor.device)
    cur.wait_event(pending.event)
    pending.tensor.record_stream(cur)
    return pending.tensor


NAMES = ("all_gather", "all_gather_by_group_call", "all_reduce", "reduce_scatter",
         "reduce_scatter_by_group_call", "dynamic_slice", "all_to_all", "replicate")


def install_as_collectives() -> None:
    """Make ``import collectives`` resolve to this module.  Call before ``import hap`` /
    ``hap.main`` so the planner's codegen picks these functions up (``hap.rs:25, 899-902``)."""
    sys.modules["collectives"] = sys.modules[__name__]


def retarget_fx_graph(graph) -> int:
    """Point every ``call_function`` node whose target is one of the reference's eight
    collectives (matched by ``__name__`` and a module called ``collectives``) at this module.
    Returns the number of nodes changed."""
    here = sys.modules[__name__]
    changed = 0
    for node in graph.nodes:
        if node.op != "call_function":
            continue
        target = node.target
        name = getattr(target, "__name__", None)
        module = getattr(target, "__module__", "") or ""
        if name in NAMES and module.split(".")[-1] == "collectives" and target is not getattr(here, name):
            node.target = getattr(here, name)
            changed += 1
    return changed
