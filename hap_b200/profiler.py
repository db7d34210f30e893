"""Cost-model constants for the planner, measured on this package's kernels.

The reference feeds its planner six collective bandwidths and a per-device flop rate
(``worker.py:24-36``: ``all_gather_bandwidth`` ... ``all_to_all_bandwidth``, ``device_flops``),
obtained by ``profiler.py``: for each collective the mean over 4/16/64/256 MiB of
``size / median time`` (``profiler.py:43-60``), with the tensor shapes of
``profiler.py:81-118`` ((256, size/1024) float32, split on dim 1 by ``[skewness, 1, 1, ...]``), and
the flop count of one training step divided by its time (``profiler.py:16-41``).

This module measures the same quantities with the same shapes on a :class:`hap_b200.comm.Comm`
(one process per GPU, or the single-GPU emulation), timed with CUDA events instead of the wall
clock, and returns them under the planner's key names so that the dict can be merged into the
``hap.main`` configuration unchanged.
"""
from __future__ import annotations

import statistics
from typing import Callable, Dict, List, Sequence

import torch

from . import _native as N
from .sharding import sharding_round

OPS = ("all_gather", "all_gather_by_group_call", "all_reduce", "reduce_scatter", "reduce_scatter_by_group_call", "all_to_all")
SIZES = (4 << 20, 16 << 20, 64 << 20, 256 << 20)


def case_lengths(op: str, size: int, world: int, skewness: float = 1.0):
    """(total columns, sharding lengths on dim 1, split lengths of the 256 rows) for one measurement:
    ``[skewness, 1, ..., 1]`` normalised and rounded like the planner rounds (``profiler.py:86-111``)."""
    total = size // 1024                       # (256, total) float32 holds `size` bytes
    raw = [float(skewness)] + [1.0] * (world - 1)
    ratios = [x / sum(raw) for x in raw]
    return total, sharding_round(total, ratios), sharding_round(256, ratios)


def _inputs(comm, op: str, size: int, skewness: float) -> List[torch.Tensor]:
    world = comm.world
    total, lengths, _ = case_lengths(op, size, world, skewness)
    outs = []
    for i, r in enumerate(comm.ranks()):
        cols = lengths[r] if op in ("all_gather", "all_gather_by_group_call", "all_to_all") else total
        t = comm.symm_empty((256, cols), torch.float32, local_index=i)
        t.uniform_()
        outs.append(t)
    return outs


def _call(comm, op: str, tensors, size: int, skewness: float):
    world = comm.world
    _, lengths, rows = case_lengths(op, size, world, skewness)
    if op == "all_reduce":
        return comm.all_reduce(tensors)
    if op == "all_gather":
        return comm.all_gather(tensors, 1, lengths, N.MODE_PADDING)
    if op == "all_gather_by_group_call":
        return comm.all_gather(tensors, 1, lengths, N.MODE_GROUP_CALL)
    if op == "reduce_scatter":
        return comm.reduce_scatter(tensors, 1, lengths, N.MODE_PADDING)
    if op == "reduce_scatter_by_group_call":
        return comm.reduce_scatter(tensors, 1, lengths, N.MODE_GROUP_CALL)
    if op == "all_to_all":
        return comm.all_to_all(tensors, 0, 1, rows, lengths)
    raise ValueError(op)


def measure_bandwidths(comm, skewness: float = 1.0, sizes: Sequence[int] = SIZES, reps: int = 5, warmup: int = 4,
                       barrier: Callable[[], None] = None) -> Dict[str, int]:
    """``{"<op>_bandwidth": bytes per second}`` for the six collectives, the planner's definition:
    the mean over ``sizes`` of ``size / median time`` (``profiler.py:55-57``).

    ``barrier`` (e.g. ``torch.distributed.barrier``) lines the ranks up before each timed call when
    every rank runs in its own process; every rank must call this function with the same arguments.
    The communicator's heap must hold the largest input (``max(sizes)`` bytes + slack).
    """
    out = {}
    dev = comm.device
    for op in OPS:
        est = []
        for size in sizes:
            comm.symm_reset()
            tensors = _inputs(comm, op, size, skewness)
            for _ in range(warmup):
                _call(comm, op, tensors, size, skewness)
            ts = []
            for _ in range(reps):
                torch.cuda.synchronize(dev)
                if barrier is not None:
                    barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                _call(comm, op, tensors, size, skewness)
                b.record()
                b.synchronize()
                ts.append(a.elapsed_time(b) * 1e-3)
            est.append(size / statistics.median(ts))
        out[op + "_bandwidth"] = int(sum(est) / len(est))
    comm.symm_reset()
    return out


def measure_device_flops(step: Callable[[], None], flops_per_step: float, warmup: int = 11, reps: int = 3) -> int:
    """Flop rate of one training step as the planner wants it (``profiler.py:19-41``): ``flops_per_step`` is
    the planner's own count for the model (``hap.stat``), ``step`` runs forward, backward and the update."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    return int(flops_per_step / statistics.median(ts))


def planner_config(bandwidths: Dict[str, int], device_flops: Sequence[int]) -> Dict[str, object]:
    """The fragment of ``hap.main``'s configuration these measurements fill (``worker.py:24-36``)."""
    cfg = {"device_flops": [int(f) for f in device_flops]}
    for op in OPS:
        cfg[op + "_bandwidth"] = int(bandwidths[op + "_bandwidth"])
    return cfg
