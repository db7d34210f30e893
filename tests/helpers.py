"""Shared helpers for the parity tests."""
import os

import torch

from oracle import collectives_math as cm

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(world):
    return torch.load(os.path.join(GOLDEN_DIR, f"collectives_w{world}.pt"), weights_only=False)


def oracle_forward(op, xs, args):
    """All ranks' outputs of `op` according to the single-process oracle."""
    world = len(xs)
    if op.startswith("all_gather"):
        return cm.all_gather(xs, *args)
    if op.startswith("reduce_scatter"):
        return cm.reduce_scatter(xs, *args)
    if op == "all_reduce":
        return cm.all_reduce(xs)
    if op == "replicate":
        return [x.clone() for x in xs]
    if op == "dynamic_slice":
        return [cm.dynamic_slice(xs[r], args[0], args[1], r) for r in range(world)]
    if op == "all_to_all":
        return cm.all_to_all(xs, *args)
    raise KeyError(op)


def oracle_backward(op, xs, ws, args):
    """Input gradients of loss_r = (out_r * w_r).sum() for every rank, per the backward duals."""
    world = len(xs)
    if op.startswith("all_gather"):
        return cm.all_gather_backward(ws, *args)
    if op.startswith("reduce_scatter"):
        return cm.reduce_scatter_backward(ws, *args)
    if op in ("all_reduce", "replicate"):
        return cm.all_reduce(ws)
    if op == "dynamic_slice":
        return [cm.dynamic_slice_backward(ws[r], xs[r].shape, args[0], args[1], r) for r in range(world)]
    if op == "all_to_all":
        return cm.all_to_all_backward(ws, *args)
    raise KeyError(op)


def exact_op(op):
    return op.startswith("all_gather") or op in ("dynamic_slice", "all_to_all", "replicate")
