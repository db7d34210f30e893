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


def _emb(ns):
    """embedding of the namespace (torch's forward, this package's backward kernel by default), else torch's."""
    return getattr(ns, "embedding", None) or F.embedding


def _ln(ns):
    """layer_norm of the namespace (this package's kernels by default), else torch's."""
    return getattr(ns, "layer_norm", None) or F.layer_norm


def _summed_nll(ns, call, method, logits, targets, classes):
    """The models' loss: ``log_softmax`` + ``nll_loss(reduction='sum')`` as the two nodes the planner
    emits (``hap.rs:1808, 1858``), or as the namespace's single fused op when it has one."""
    fused = getattr(ns, "nll", None)
    if fused is not None:
        return call(fused, logits, targets)
    logp = call(F.log_softmax, method(logits, "float"), -1)
    logp = method(logp, "reshape", -1, classes)
    return call(F.nll_loss, logp, method(targets, "reshape", -1), reduction="sum")


def default_namespace() -> SimpleNamespace:
    from . import collectives
    from .attention import multi_head_attention_forward
    from .dropout import dropout
    from .einsum import einsum
    from .embedding import embedding
    from .linear import linear
    from .loss import nll_log_softmax_sum
    from .norm import layer_norm
    return SimpleNamespace(collectives=collectives, linear=linear, mha=multi_head_attention_forward, einsum=einsum,
                           nll=nll_log_softmax_sum, layer_norm=layer_norm, dropout=dropout, embedding=embedding)


def _dropout_of(ns, call, p):
    """``x -> dropout(x, p)`` as the planner emits it (``torch.nn.functional.dropout(input, p)``,
    ``hap.rs:1446-1464``), or the identity for p == 0.  The sites are those of the reference's encoder
    layers (``torch.nn.TransformerEncoderLayer`` with ``dropout``, ``models.py:40, 74``): after the
    attention block, after the FFN activation and after the FFN."""
    if not p:
        return lambda x: x
    fn = getattr(ns, "dropout", None) or F.dropout
    return lambda x: call(fn, x, p)


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


# ---------------------------------------------------------------------------------------------
# Transformer language model (the bf16 throughput configuration)
# ---------------------------------------------------------------------------------------------
class TransformerLM(torch.nn.Module):
    """Parameters of a pre-LN Transformer language model in the (L, N, E) layout the planner's
    attention handler expects (``hap.rs:1284-1287``): token + positional embedding, ``nlayers`` blocks
    of x + MHA(LN(x)) and x + W2 relu(W1 LN(x)), final LN, tied-size decoder, summed NLL loss
    (``log_softmax`` + ``nll_loss``, the ops of ``hap.rs:1808, 1858``).  The vocabulary is padded to
    a multiple of 8 (the reference pads it to a multiple of the world size, ``config.py:116``)."""

    def __init__(self, vocab=33280, d_model=768, nheads=12, d_ffn=3072, nlayers=12, seqlen=256):
        super().__init__()
        self.vocab, self.d_model, self.nheads, self.nlayers, self.seqlen = vocab, d_model, nheads, nlayers, seqlen
        self.embed = torch.nn.Embedding(vocab, d_model)
        self.pos = torch.nn.Parameter(torch.randn(seqlen, 1, d_model) * 0.02)
        for i in range(nlayers):
            self.register_parameter(f"l{i}_ln1_w", torch.nn.Parameter(torch.ones(d_model)))
            self.register_parameter(f"l{i}_ln1_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_in_w", torch.nn.Parameter(torch.randn(3 * d_model, d_model) * d_model ** -0.5))
            self.register_parameter(f"l{i}_in_b", torch.nn.Parameter(torch.zeros(3 * d_model)))
            self.register_parameter(f"l{i}_out_w", torch.nn.Parameter(torch.randn(d_model, d_model) * d_model ** -0.5))
            self.register_parameter(f"l{i}_out_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_ln2_w", torch.nn.Parameter(torch.ones(d_model)))
            self.register_parameter(f"l{i}_ln2_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_w1", torch.nn.Parameter(torch.randn(d_ffn, d_model) * d_model ** -0.5))
            self.register_parameter(f"l{i}_b1", torch.nn.Parameter(torch.zeros(d_ffn)))
            self.register_parameter(f"l{i}_w2", torch.nn.Parameter(torch.randn(d_model, d_ffn) * d_ffn ** -0.5))
            self.register_parameter(f"l{i}_b2", torch.nn.Parameter(torch.zeros(d_model)))
        self.lnf_w = torch.nn.Parameter(torch.ones(d_model))
        self.lnf_b = torch.nn.Parameter(torch.zeros(d_model))
        self.dec_w = torch.nn.Parameter(torch.randn(vocab, d_model) * d_model ** -0.5)
        self.dec_b = torch.nn.Parameter(torch.zeros(vocab))

    def forward(self, tokens, targets):
        """Unsharded reference forward: tokens, targets (B, S) int64 -> summed NLL."""
        ns = SimpleNamespace(collectives=None, linear=F.linear, mha=F.multi_head_attention_forward)
        return _lm_forward(self, tokens, targets, ns, None, None, None, "none")


def _column_parallel_ffn(m, i, h, activation, emit, col, call, linear, param, drop, rank):
    """The FFN of layer ``i`` column-parallel (hap.rs:2807-2816): every rank multiplies the WHOLE batch by its
    rows of the weight, so the batch shards are gathered first (re-sharding batch -> replicated,
    hap.rs:2631-2653), the output columns are gathered on the last dimension before the activation (an
    activation's output is not communicatable, hap.rs:1102, 1432), and the own batch shard is cut out again
    at the end.  ``h`` is (L, B_r, E); so is the result."""
    lb, l_ffn, l_e = m._tp_lengths
    h = emit.call_function(col.all_gather, (h, 1, lb, rank))                                   # (L, B, E)
    z = call(linear, h, param(f"l{i}_w1"), param(f"l{i}_b1"))                                  # (L, B, ffn_r)
    z = emit.call_function(col.all_gather, (z, 2, l_ffn, rank))                                # (L, B, ffn)
    z = drop(call(activation, z))
    o = call(linear, z, param(f"l{i}_w2"), param(f"l{i}_b2"))                                  # (L, B, E_r)
    o = emit.call_function(col.all_gather, (o, 2, l_e, rank))                                  # (L, B, E)
    return emit.call_function(col.dynamic_slice, (o, 1, lb, rank))                             # (L, B_r, E)


def _shard_column_parallel_ffn_(model, ratios, rank, lb):
    """Cut the FFN weights and biases of every layer on dim 0 for good (plan ``"tp"``)."""
    d_ffn = model.l0_w1.shape[0]
    model._tp_lengths = (lb, sharding_round(d_ffn, ratios), sharding_round(model.d_model, ratios))
    for i in range(model.nlayers):
        for n, extent in ((f"l{i}_w1", d_ffn), (f"l{i}_b1", d_ffn), (f"l{i}_w2", model.d_model), (f"l{i}_b2", model.d_model)):
            shard_parameter_(model, n, sharding_round(extent, ratios), 0, rank)
            model._column_parallel.add(n)


def _lm_forward(m, tokens, targets, ns, emit, ratios, rank, plan, dropout_p=0.0):
    """The model's forward written once; `emit` (an fx graph) turns parameter reads and collectives
    into nodes, otherwise it runs eagerly on the unsharded module."""
    col, linear, mha = ns.collectives, ns.linear, ns.mha
    E, H = m.d_model, m.nheads

    def param(name, shardable=False):
        if emit is None:
            obj = m
            for part in name.split("."):
                obj = getattr(obj, part)
            return obj
        node = emit.get_attr(name)
        if name in getattr(m, "_column_parallel", ()):
            return node                  # column-parallel weight or bias: the in-place shard itself (hap.rs:2591-2593)
        if plan in ("dp_zero", "tp") and shardable and name in m._full_extent:
            # ZeRO-style: the parameter lives sharded on dim 0 and is gathered where it is used
            # (hap.rs:2527-2555); backward of the gather is the uneven reduce_scatter of its gradient
            full = m._full_extent[name]
            return emit.call_function(col.all_gather, (node, 0, sharding_round(full, ratios), rank))
        return emit.call_function(col.replicate, (node,))

    call = (lambda fn, *a, **k: fn(*a, **k)) if emit is None else (lambda fn, *a, **k: emit.call_function(fn, a, k))
    method = (lambda obj, name, *a: getattr(obj, name)(*a)) if emit is None else (lambda obj, name, *a: emit.call_method(name, (obj, *a)))

    drop = _dropout_of(ns, call, dropout_p)
    # look the tokens up in (S, B) order: the activations are then contiguous in the (L, N, E) layout the
    # attention handler wants (hap.rs:1284-1287) instead of a transposed view that every layer_norm copies
    x = call(_emb(ns), method(tokens, "transpose", 0, 1), param("embed.weight"))   # (S, B, E)
    x = call(operator.add, x, param("pos"))
    S = m.seqlen
    mask = call(torch.triu, call(torch.full, (S, S), float("-inf"), device=_device_of(m), dtype=m.pos.dtype), 1)
    for i in range(m.nlayers):
        h = call(_ln(ns), x, (E,), param(f"l{i}_ln1_w"), param(f"l{i}_ln1_b"))
        att = call(mha, query=h, key=h, value=h, embed_dim_to_check=E, num_heads=H,
                   in_proj_weight=param(f"l{i}_in_w", True), in_proj_bias=param(f"l{i}_in_b", True), bias_k=None, bias_v=None,
                   add_zero_attn=False, dropout_p=float(dropout_p), out_proj_weight=param(f"l{i}_out_w", True),
                   out_proj_bias=param(f"l{i}_out_b"), attn_mask=mask)
        x = call(operator.add, x, drop(call(operator.getitem, att, 0)))
        h = call(_ln(ns), x, (E,), param(f"l{i}_ln2_w"), param(f"l{i}_ln2_b"))
        if plan == "tp":
            h = _column_parallel_ffn(m, i, h, F.relu, emit, col, call, linear, param, drop, rank)
        else:
            h = call(linear, h, param(f"l{i}_w1", True), param(f"l{i}_b1", True))
            h = drop(call(F.relu, h))
            h = call(linear, h, param(f"l{i}_w2", True), param(f"l{i}_b2"))
        x = call(operator.add, x, drop(h))
    x = call(_ln(ns), x, (E,), param("lnf_w"), param("lnf_b"))
    logits = call(linear, x, param("dec_w", True), param("dec_b", True))  # (S, B, V)
    return _summed_nll(ns, call, method, logits, method(targets, "transpose", 0, 1), m.vocab)


def _device_of(m):
    return next(m.parameters()).device


def emit_lm(model: TransformerLM, plan: str, ratios: Sequence[float], rank: int, batch: int, ns=None,
            dropout_p: float = 0.0) -> torch.fx.Graph:
    """fx graph of the language model's training forward for one rank.

    ``"dp"``      - batch-sharded tokens/targets, every parameter replicated (gradient all-reduce);
    ``"dp_zero"`` - as above, but attention and FFN weights, the first FFN bias and the decoder live
                    sharded on dim 0 by ``ratios`` (cut in place on the module) and are all-gathered
                    at their use; their gradients come back through the uneven reduce_scatter.
    ``"tp"``      - hybrid: attention data parallel on the batch shards (the attention node is only ever batch-
                    sharded, ``hap.rs:2903-2926``) with ZeRO-style projection weights as in ``"dp_zero"``; the FFN
                    column-parallel (``hap.rs:2807-2816``): ``w1``/``b1``/``w2``/``b2`` sharded on dim 0 for good,
                    the batch gathered in front of it, the output columns gathered on the LAST dimension
                    (strided shards of 154 ... 676 columns under the r8 ratios) and the own batch shard cut out
                    afterwards; the decoder ZeRO-style.
    ``dropout_p`` > 0 adds the reference's dropout (``config.py:33``): on the attention probabilities
    (the attention node's ``dropout_p``, ``hap.rs:1257, 1307``) and as ``F.dropout`` nodes after the
    attention block, the FFN activation and the FFN.
    """
    ns = ns or default_namespace()
    if plan not in ("dp", "dp_zero", "tp"):
        raise ValueError(f"unknown plan {plan!r}")
    g = torch.fx.Graph()
    tokens, targets = g.placeholder("tokens"), g.placeholder("targets")
    lb = sharding_round(batch, ratios)
    tok_r = g.call_function(operator.getitem, (g.call_method("split", (tokens, lb, 0)), rank))
    tgt_r = g.call_function(operator.getitem, (g.call_method("split", (targets, lb, 0)), rank))
    model._full_extent = {}
    model._column_parallel = set()
    if plan == "tp":
        _shard_column_parallel_ffn_(model, ratios, rank, lb)
    if plan in ("dp_zero", "tp"):
        names = [n for i in range(model.nlayers) for n in (f"l{i}_in_w", f"l{i}_in_b", f"l{i}_out_w")]
        if plan == "dp_zero":
            names += [n for i in range(model.nlayers) for n in (f"l{i}_w1", f"l{i}_b1", f"l{i}_w2")]
        names += ["dec_w", "dec_b"]
        for n in names:
            full = getattr(model, n).shape[0]
            model._full_extent[n] = full
            shard_parameter_(model, n, sharding_round(full, ratios), 0, rank)
    loss = _lm_forward(model, tok_r, tgt_r, ns, g, list(ratios), rank, plan, dropout_p)
    g.output(loss)
    g.lint()
    return g


# ---------------------------------------------------------------------------------------------
# Vision Transformer (the image-classification configuration)
# ---------------------------------------------------------------------------------------------
class ViT(torch.nn.Module):
    """ViT in the shape of the reference's ``VTransformer`` (``models.py:147-177``): patch embedding,
    a class token in front, learned positions, ``nlayers`` encoder blocks without a mask, the class
    token's embedding through a linear head, ``log_softmax`` + summed ``nll_loss``.

    The patch embedding is a convolution whose kernel equals its stride, i.e. a linear map of each
    flattened patch: it is written as ``reshape`` / ``permute`` + ``linear`` so that it runs on the same
    tensor-core GEMM as every other projection.  Blocks are the pre-LN blocks of
    :class:`TransformerLM` with GELU in the MLP.  Defaults are ViT-B/16 on 224 x 224 images.
    """

    def __init__(self, image=224, patch=16, channels=3, d_model=768, nheads=12, d_ffn=3072, nlayers=12, nclasses=1000):
        super().__init__()
        if image % patch:
            raise ValueError("image size must be a multiple of the patch size")
        self.image, self.patch, self.channels = image, patch, channels
        self.d_model, self.nheads, self.nlayers, self.nclasses = d_model, nheads, nlayers, nclasses
        self.grid = image // patch
        self.seqlen = self.grid * self.grid + 1
        pdim = channels * patch * patch
        self.patch_w = torch.nn.Parameter(torch.randn(d_model, pdim) * pdim ** -0.5)
        self.patch_b = torch.nn.Parameter(torch.zeros(d_model))
        self.cls = torch.nn.Parameter(torch.randn(1, 1, d_model) * 0.02)
        self.pos = torch.nn.Parameter(torch.randn(self.seqlen, 1, d_model) * 0.02)
        for i in range(nlayers):
            self.register_parameter(f"l{i}_ln1_w", torch.nn.Parameter(torch.ones(d_model)))
            self.register_parameter(f"l{i}_ln1_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_in_w", torch.nn.Parameter(torch.randn(3 * d_model, d_model) * d_model ** -0.5))
            self.register_parameter(f"l{i}_in_b", torch.nn.Parameter(torch.zeros(3 * d_model)))
            self.register_parameter(f"l{i}_out_w", torch.nn.Parameter(torch.randn(d_model, d_model) * d_model ** -0.5))
            self.register_parameter(f"l{i}_out_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_ln2_w", torch.nn.Parameter(torch.ones(d_model)))
            self.register_parameter(f"l{i}_ln2_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_w1", torch.nn.Parameter(torch.randn(d_ffn, d_model) * d_model ** -0.5))
            self.register_parameter(f"l{i}_b1", torch.nn.Parameter(torch.zeros(d_ffn)))
            self.register_parameter(f"l{i}_w2", torch.nn.Parameter(torch.randn(d_model, d_ffn) * d_ffn ** -0.5))
            self.register_parameter(f"l{i}_b2", torch.nn.Parameter(torch.zeros(d_model)))
        self.lnf_w = torch.nn.Parameter(torch.ones(d_model))
        self.lnf_b = torch.nn.Parameter(torch.zeros(d_model))
        self.head_w = torch.nn.Parameter(torch.randn(nclasses, d_model) * d_model ** -0.5)
        self.head_b = torch.nn.Parameter(torch.zeros(nclasses))

    def forward(self, images, labels):
        """Unsharded reference forward: images (B, C, H, W), labels (B,) int64 -> summed NLL."""
        ns = SimpleNamespace(collectives=None, linear=F.linear, mha=F.multi_head_attention_forward)
        return _vit_forward(self, images, labels, ns, None, None, None, "none")


def _vit_forward(m, images, labels, ns, emit, ratios, rank, plan, dropout_p=0.0):
    col, linear, mha = ns.collectives, ns.linear, ns.mha
    E, H, G, P_, C_ = m.d_model, m.nheads, m.grid, m.patch, m.channels

    def param(name, shardable=False):
        if emit is None:
            return getattr(m, name)
        node = emit.get_attr(name)
        if name in m._column_parallel:
            return node                  # column-parallel weight or bias: the in-place shard itself
        if plan in ("dp_zero", "tp") and shardable and name in m._full_extent:
            return emit.call_function(col.all_gather, (node, 0, sharding_round(m._full_extent[name], ratios), rank))
        return emit.call_function(col.replicate, (node,))

    call = (lambda fn, *a, **k: fn(*a, **k)) if emit is None else (lambda fn, *a, **k: emit.call_function(fn, a, k))
    method = (lambda obj, name, *a: getattr(obj, name)(*a)) if emit is None else (lambda obj, name, *a: emit.call_method(name, (obj, *a)))

    drop = _dropout_of(ns, call, dropout_p)
    # (B, C, G*P, G*P) -> (B, G*G, C*P*P): one row per patch, elements in the order a conv kernel reads them
    x = method(images, "reshape", -1, C_, G, P_, G, P_)
    x = method(x, "permute", 0, 2, 4, 1, 3, 5)
    x = method(x, "reshape", -1, G * G, C_ * P_ * P_)
    x = call(linear, x, param("patch_w", True), param("patch_b"))          # (B, G*G, E)
    x = method(x, "transpose", 0, 1)                                        # (G*G, B, E)
    cls = method(param("cls"), "expand", -1, method(x, "size", 1), -1)      # (1, B, E)
    x = call(torch.cat, [cls, x], 0)                                        # (L, B, E): the (L, N, E) layout
    x = call(operator.add, x, param("pos"))
    for i in range(m.nlayers):
        h = call(_ln(ns), x, (E,), param(f"l{i}_ln1_w"), param(f"l{i}_ln1_b"))
        att = call(mha, query=h, key=h, value=h, embed_dim_to_check=E, num_heads=H,
                   in_proj_weight=param(f"l{i}_in_w", True), in_proj_bias=param(f"l{i}_in_b", True), bias_k=None, bias_v=None,
                   add_zero_attn=False, dropout_p=float(dropout_p), out_proj_weight=param(f"l{i}_out_w", True),
                   out_proj_bias=param(f"l{i}_out_b"), attn_mask=None)
        x = call(operator.add, x, drop(call(operator.getitem, att, 0)))
        h = call(_ln(ns), x, (E,), param(f"l{i}_ln2_w"), param(f"l{i}_ln2_b"))
        if plan == "tp":
            h = _column_parallel_ffn(m, i, h, F.gelu, emit, col, call, linear, param, drop, rank)
        else:
            h = call(linear, h, param(f"l{i}_w1", True), param(f"l{i}_b1", True))
            h = drop(call(F.gelu, h))
            h = call(linear, h, param(f"l{i}_w2", True), param(f"l{i}_b2"))
        x = call(operator.add, x, drop(h))
    x = call(operator.getitem, x, 0)                                        # the class token: (B, E)
    x = call(_ln(ns), x, (E,), param("lnf_w"), param("lnf_b"))
    logits = call(linear, x, param("head_w", True), param("head_b", True))
    return _summed_nll(ns, call, method, logits, labels, m.nclasses)


def emit_vit(model: ViT, plan: str, ratios: Sequence[float], rank: int, batch: int, ns=None,
             dropout_p: float = 0.0) -> torch.fx.Graph:
    """fx graph of the ViT training forward for one rank; plans as in :func:`emit_lm` (``"dp"``:
    images and labels batch-sharded by ``ratios``, parameters replicated; ``"dp_zero"``: projection
    weights additionally sharded on dim 0 and all-gathered at their use; ``"tp"``: the MLP of every block
    column-parallel, everything else as in ``"dp_zero"``)."""
    ns = ns or default_namespace()
    if plan not in ("dp", "dp_zero", "tp"):
        raise ValueError(f"unknown plan {plan!r}")
    g = torch.fx.Graph()
    images, labels = g.placeholder("images"), g.placeholder("labels")
    lb = sharding_round(batch, ratios)
    img_r = g.call_function(operator.getitem, (g.call_method("split", (images, lb, 0)), rank))
    lab_r = g.call_function(operator.getitem, (g.call_method("split", (labels, lb, 0)), rank))
    model._full_extent = {}
    model._column_parallel = set()
    if plan == "tp":
        _shard_column_parallel_ffn_(model, ratios, rank, lb)
    if plan in ("dp_zero", "tp"):
        names = [n for i in range(model.nlayers) for n in (f"l{i}_in_w", f"l{i}_in_b", f"l{i}_out_w")]
        if plan == "dp_zero":
            names += [n for i in range(model.nlayers) for n in (f"l{i}_w1", f"l{i}_b1", f"l{i}_w2")]
        names += ["patch_w", "head_w", "head_b"]
        for n in names:
            full = getattr(model, n).shape[0]
            model._full_extent[n] = full
            shard_parameter_(model, n, sharding_round(full, ratios), 0, rank)
    loss = _vit_forward(model, img_r, lab_r, ns, g, list(ratios), rank, plan, dropout_p)
    g.output(loss)
    g.lint()
    return g


# ---------------------------------------------------------------------------------------------
# MoE Transformer (expert-parallel configuration)
# ---------------------------------------------------------------------------------------------
_LOWER_ONES = {}


def _lower_ones(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    if key not in _LOWER_ONES:
        _LOWER_ONES[key] = torch.ones(n, n, dtype=torch.float32, device=device).tril()
    return _LOWER_ONES[key]


def top2_gating(x, gate_weight, n_expert: int, capacity: int):
    """Top-2 gating with a fixed per-expert capacity; reproduces the reference's fx-wrapped
    ``top_2_gating`` (``models.py:477-502``) entry for entry: softmax gate, two best experts per
    token, 1-based slot numbers handed out in sequence order per (choice, expert), and the
    second-choice slots of an expert shifted by the SUM of that expert's first-choice slot numbers
    (``models.py:482-484`` sums ``position_in_expert``, i.e. n(n+1)/2 for n first choices, not n).
    A slot number must stay below ``capacity`` (slot 0 is never used); combine weight = the raw gate
    probability.  Returns (dispatch, combine), both (batch, seq, n_expert, capacity) in x's dtype.
    Plain torch ops: the planner treats this function as an opaque leaf (``hap.rs:2169``)."""
    if not x.is_contiguous() and x.transpose(0, 1).is_contiguous():     # a (b, s, d) view of sequence-first memory:
        logits = torch.matmul(x.transpose(0, 1), gate_weight).transpose(0, 1)   # multiply in memory order, no copy of x
    else:
        logits = torch.matmul(x, gate_weight)
    gates = torch.softmax(logits.float(), dim=2)                                          # (b, s, e)
    top_p, top_i = torch.topk(gates, 2, dim=2)                                           # (b, s, 2)
    chosen = F.one_hot(top_i, n_expert).to(torch.float32)                                # (b, s, 2, e)
    first, second = chosen[:, :, 0, :], chosen[:, :, 1, :]
    # running counts along the sequence as a product with a lower-triangular matrix of ones: exact in float32
    # (counts stay below 2^24) and an order of magnitude faster on a GPU than an int64 scan over the middle dimension
    tri = _lower_ones(x.shape[1], x.device)
    counts = torch.matmul(tri, chosen.flatten(2))                                        # (b, s, 2 e): both choices in one product
    count1, count2 = counts[:, :, :n_expert], counts[:, :, n_expert:]
    slot1 = count1 * first                                                               # 1-based
    # the reference shifts an expert's second-choice slots by the SUM of its first-choice slot numbers; those are
    # 1 ... n for n first choices, i.e. n (n + 1) / 2 with n the last running count (exact in float32)
    n1 = count1[:, -1:, :]
    slot2 = (count2 + n1 * (n1 + 1.0) * 0.5) * second
    # Only the two chosen experts of a token can hold a non-zero entry, and they differ, so the (b, s, e, c) tensors
    # are written by scattering two values per token instead of by dense one-hot arithmetic over all e * c entries
    # (the reference's sums of `weight * one_hot(slot)` add zeros everywhere else).
    slots = torch.stack((slot1.gather(2, top_i[:, :, 0:1]), slot2.gather(2, top_i[:, :, 1:2])), dim=2).squeeze(3)   # (b, s, 2)
    keep = (slots > 0) & (slots < capacity)
    index = top_i * capacity + (slots * keep).clamp(max=capacity - 1).long()             # position in (e * c)
    weight32 = top_p * keep                                                              # (b, s, 2), zero where dropped
    weight = weight32.to(x.dtype)
    b, s = x.shape[0], x.shape[1]
    combine = torch.zeros(b, s, n_expert * capacity, dtype=x.dtype, device=x.device).scatter(2, index, weight)
    dispatch = torch.zeros(b, s, n_expert * capacity, dtype=x.dtype, device=x.device).scatter(2, index, (weight32 > 0).to(x.dtype))
    return dispatch.view(b, s, n_expert, capacity), combine.view(b, s, n_expert, capacity)

class MoETransformerLM(torch.nn.Module):
    """Post-LN MoE Transformer LM in the shape of the reference's ``Top2TransformerEncoderLayer``
    (``models.py:301-366``): x = LN(x + MHA(x)); x = LN(x + MoE(x)) with top-2 gating over
    ``n_expert`` expert FFNs (w1[e, d, h], relu, w2[e, h, d]); summed NLL loss."""

    def __init__(self, vocab=33280, d_model=1024, nheads=16, d_ffn=4096, nlayers=8, seqlen=512, n_expert=32, capacity=20):
        super().__init__()
        self.vocab, self.d_model, self.nheads, self.nlayers, self.seqlen = vocab, d_model, nheads, nlayers, seqlen
        self.n_expert, self.capacity = n_expert, capacity
        self.embed = torch.nn.Embedding(vocab, d_model)
        self.pos = torch.nn.Parameter((torch.randn(1, seqlen, d_model) * 0.02).transpose(0, 1).contiguous())   # (s, 1, d)
        P_ = lambda *shape, scale=1.0: torch.nn.Parameter(torch.randn(*shape) * scale)
        for i in range(nlayers):
            self.register_parameter(f"l{i}_in_w", P_(3 * d_model, d_model, scale=d_model ** -0.5))
            self.register_parameter(f"l{i}_in_b", torch.nn.Parameter(torch.zeros(3 * d_model)))
            self.register_parameter(f"l{i}_out_w", P_(d_model, d_model, scale=d_model ** -0.5))
            self.register_parameter(f"l{i}_out_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_ln1_w", torch.nn.Parameter(torch.ones(d_model)))
            self.register_parameter(f"l{i}_ln1_b", torch.nn.Parameter(torch.zeros(d_model)))
            self.register_parameter(f"l{i}_gate", P_(d_model, n_expert, scale=d_model ** -0.5))
            self.register_parameter(f"l{i}_w1", P_(n_expert, d_model, d_ffn, scale=d_model ** -0.5))
            self.register_parameter(f"l{i}_w2", P_(n_expert, d_ffn, d_model, scale=d_ffn ** -0.5))
            self.register_parameter(f"l{i}_ln2_w", torch.nn.Parameter(torch.ones(d_model)))
            self.register_parameter(f"l{i}_ln2_b", torch.nn.Parameter(torch.zeros(d_model)))
        self.dec_w = P_(vocab, d_model, scale=d_model ** -0.5)
        self.dec_b = torch.nn.Parameter(torch.zeros(vocab))

    def forward(self, tokens, targets):
        ns = SimpleNamespace(collectives=None, linear=F.linear, mha=F.multi_head_attention_forward, einsum=torch.einsum)
        return _moe_forward(self, tokens, targets, ns, None, None, None, None)


def _moe_forward(m, tokens, targets, ns, emit, ratios, rank, batch, dropout_p=0.0):
    col, linear, mha, einsum = ns.collectives, ns.linear, ns.mha, ns.einsum
    E, H, ne, cap = m.d_model, m.nheads, m.n_expert, m.capacity

    def param(name, sharded=False):
        if emit is None:
            return getattr(m, name) if "." not in name else m.get_parameter(name)
        node = emit.get_attr(name)
        return node if sharded else emit.call_function(col.replicate, (node,))   # expert weights: get_attr of the in-place shard (hap.rs:2591-2593)

    call = (lambda fn, *a, **k: fn(*a, **k)) if emit is None else (lambda fn, *a, **k: emit.call_function(fn, a, k))
    method = (lambda obj, name, *a: getattr(obj, name)(*a)) if emit is None else (lambda obj, name, *a: emit.call_method(name, (obj, *a)))

    drop = _dropout_of(ns, call, dropout_p)      # the Top-2 layer drops only after its attention block (models.py:346-351)
    # sequence-first activations (s, b, E), as in the language model: contiguous in the (L, N, E) layout the attention
    # handler wants (hap.rs:1284-1287); the gating function and the dispatch see the (b, s, E) view of the same memory
    x = call(operator.add, call(_emb(ns), method(tokens, "transpose", 0, 1), param("embed.weight")), param("pos"))
    for i in range(m.nlayers):
        att = call(mha, query=x, key=x, value=x, embed_dim_to_check=E, num_heads=H, in_proj_weight=param(f"l{i}_in_w"),
                   in_proj_bias=param(f"l{i}_in_b"), bias_k=None, bias_v=None, add_zero_attn=False, dropout_p=float(dropout_p),
                   out_proj_weight=param(f"l{i}_out_w"), out_proj_bias=param(f"l{i}_out_b"))
        a = drop(call(operator.getitem, att, 0))
        x = call(_ln(ns), call(operator.add, x, a), (E,), param(f"l{i}_ln1_w"), param(f"l{i}_ln1_b"))
        xb = method(x, "transpose", 0, 1)                                                              # (b_r, s, E)
        gated = call(top2_gating, xb, param(f"l{i}_gate"), ne, cap)
        dispatch, combine = call(operator.getitem, gated, 0), call(operator.getitem, gated, 1)
        ein = call(einsum, "bsd,bsec->becd", xb, dispatch)                                             # (b_r, e, c, d)
        if emit is not None:   # batch-sharded -> expert-sharded (hap.rs:2713-2744: all_to_all(x, split=j, cat=i, ...))
            le, lb = sharding_round(ne, ratios), sharding_round(batch, ratios)
            ein = emit.call_function(col.all_to_all, (ein, 1, 0, le, lb, rank))                       # (b, e_r, c, d)
        hid = call(F.relu, call(einsum, "edh,becd->bech", param(f"l{i}_w1", True), ein))
        eo = call(einsum, "ehd,bech->becd", param(f"l{i}_w2", True), hid)
        if emit is not None:
            eo = emit.call_function(col.all_to_all, (eo, 0, 1, lb, le, rank))                         # (b_r, e, c, d)
        y = method(call(einsum, "becd,bsec->bsd", eo, combine), "transpose", 0, 1)                     # (s, b_r, d)
        x = call(_ln(ns), call(operator.add, x, y), (E,), param(f"l{i}_ln2_w"), param(f"l{i}_ln2_b"))
    logits = call(linear, x, param("dec_w"), param("dec_b"))                                           # (s, b_r, V)
    return _summed_nll(ns, call, method, logits, method(targets, "transpose", 0, 1), m.vocab)


def emit_moe(model: MoETransformerLM, ratios: Sequence[float], rank: int, batch: int, ns=None,
             dropout_p: float = 0.0) -> torch.fx.Graph:
    """Expert-parallel program: tokens batch-sharded by ``ratios``; expert weights w1/w2 sharded on
    the expert dimension by ``sharding_round(n_expert, ratios)`` (cut in place); the dispatched
    tokens travel batch-sharded -> expert-sharded -> batch-sharded through two uneven all_to_all
    calls per layer; everything else replicated."""
    ns = ns or default_namespace()
    g = torch.fx.Graph()
    tokens, targets = g.placeholder("tokens"), g.placeholder("targets")
    lb = sharding_round(batch, ratios)
    tok_r = g.call_function(operator.getitem, (g.call_method("split", (tokens, lb, 0)), rank))
    tgt_r = g.call_function(operator.getitem, (g.call_method("split", (targets, lb, 0)), rank))
    le = sharding_round(model.n_expert, ratios)
    for i in range(model.nlayers):
        shard_parameter_(model, f"l{i}_w1", le, 0, rank)
        shard_parameter_(model, f"l{i}_w2", le, 0, rank)
    loss = _moe_forward(model, tok_r, tgt_r, ns, g, list(ratios), rank, batch, dropout_p)
    g.output(loss)
    g.lint()
    return g
