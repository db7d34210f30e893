"""Emit the SPMD ``torch.fx`` programs the planner would synthesize, for a GIVEN plan.

The reference's planner (``hap.rs``, Rust) cannot be built where this package is developed, so
programs for the benchmark configurations are emitted here by following its code-generation
closures node for node:

* placeholders are cut with ``split`` + ``getitem`` (``hap.rs:2511-2515``);
* replicated parameters go through ``collectives.replicate`` (``hap.rs:2557-2578``), sharded
  parameters are cut IN PLACE on the module (``hap.rs:929-944``, ``2591-2593``) and read with
  ``get_attr``;
* re-sharding uses the collectives with ``sharding_round(extent, ratios)`` as lengths
  (``hap.rs:2631-2744``);
* data-parallel and column-parallel ``linear`` as in ``hap.rs:2787-2816``; the output must be a
  partial loss whose sum over ranks is the loss (``hap.rs:2602-2616``).

The emitter takes the callables it wires in (collectives module, linear function) as a
namespace, so the very same program can be bound to this package's CUDA path or to a CPU
implementation.
"""
from __future__ import annotations

import operator
from types import SimpleNamespace
from typing import Sequence

import torch
import torch.nn.functional as F

from .sharding import sharding_round


class MLP(torch.nn.Module):
    """The 2-layer MLP of the fp32 parity configuration: Linear(in, hidden), GELU, Linear(hidden, out),
    sum-reduced MSE against the targets.  Parameters use torch's default (Kaiming-uniform) init."""

    def __init__(self, in_features=1024, hidden=4096, out_features=1024):
        super().__init__()
        self.fc1 = torch.nn.Linear(in_features, hidden)
        self.fc2 = torch.nn.Linear(hidden, out_features)

    def forward(self, x, y):
        return F.mse_loss(self.fc2(F.gelu(self.fc1(x))), y, reduction="sum")


def default_namespace() -> SimpleNamespace:
    from . import collectives
    from .linear import linear
    return SimpleNamespace(collectives=collectives, linear=linear)


def shard_parameter_(module: torch.nn.Module, name: str, lengths: Sequence[int], dim: int, rank: int) -> None:
    """Replace parameter ``name`` by its shard, in place on the module (``hap.rs:36-47, 929-944``).
    Extent-1 dimensions are left alone (the broadcast hack of ``hap.rs:3538-3540``)."""
    owner = module
    *path, leaf = name.split(".")
    for p in path:
        owner = getattr(owner, p)
    param = getattr(owner, leaf)
    if param.shape[dim] == 1:
        return
    shard = torch.split(param.data, list(lengths), dim=dim)[rank].contiguous()
    setattr(owner, leaf, torch.nn.Parameter(shard, requires_grad=param.requires_grad))


def emit_mlp(model: MLP, plan: str, ratios: Sequence[float], rank: int, batch: int, ns=None) -> torch.fx.Graph:
    """fx graph of ``MLP.forward(x, y)`` for one rank under ``plan``:

    ``"dp"``  - batch-sharded inputs, replicated parameters (gradient all-reduce in backward);
    ``"tp"``  - both layers column-parallel: weights/biases sharded on dim 0, hidden activation
                all-gathered on dim 1 before the GELU (an activation's output is not
                communicatable, ``hap.rs:1102``), loss over the own output columns.
    The module's parameters are sharded in place for ``"tp"``.
    """
    ns = ns or default_namespace()
    col, linear = ns.collectives, ns.linear
    g = torch.fx.Graph()
    x, y = g.placeholder("x"), g.placeholder("y")
    hidden, out = model.fc1.out_features, model.fc2.out_features
    if plan == "dp":
        lb = sharding_round(batch, ratios)
        x_r = g.call_function(operator.getitem, (g.call_method("split", (x, lb, 0)), rank))
        y_r = g.call_function(operator.getitem, (g.call_method("split", (y, lb, 0)), rank))
        w1, b1, w2, b2 = (g.call_function(col.replicate, (g.get_attr(n),))
                          for n in ("fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"))
        z = g.call_function(linear, (x_r, w1, b1))
        h = g.call_function(F.gelu, (z,))
        o = g.call_function(linear, (h, w2, b2))
        loss = g.call_function(F.mse_loss, (o, y_r), {"reduction": "sum"})
    elif plan == "tp":
        lh, lo = sharding_round(hidden, ratios), sharding_round(out, ratios)
        shard_parameter_(model, "fc1.weight", lh, 0, rank)
        shard_parameter_(model, "fc1.bias", lh, 0, rank)
        shard_parameter_(model, "fc2.weight", lo, 0, rank)
        shard_parameter_(model, "fc2.bias", lo, 0, rank)
        w1, b1, w2, b2 = (g.get_attr(n) for n in ("fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"))
        z_r = g.call_function(linear, (x, w1, b1))
        z = g.call_function(col.all_gather, (z_r, 1, lh, rank))
        h = g.call_function(F.gelu, (z,))
        o_r = g.call_function(linear, (h, w2, b2))
        y_r = g.call_function(operator.getitem, (g.call_method("split", (y, lo, 1)), rank))
        loss = g.call_function(F.mse_loss, (o_r, y_r), {"reduction": "sum"})
    else:
        raise ValueError(f"unknown plan {plan!r}")
    g.output(loss)
    g.lint()
    return g
