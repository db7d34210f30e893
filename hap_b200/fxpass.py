"""fx passes that point a planner-generated program at this package's kernels.

The planner stores function objects in its ``call_function`` nodes (``hap.rs:899-902``).  For the
collectives the replacement module is installed before the planner runs, or
:func:`hap_b200.collectives.retarget_fx_graph` is applied afterwards; for the tensor ops the
planner names torch functions directly (``torch.nn.functional.linear`` at ``hap.rs:995, 1032``,
``multi_head_attention_forward`` at ``hap.rs:1243, 1301``, ``torch.einsum`` at ``hap.rs:2240, 2273``,
``layer_norm`` at ``hap.rs:1637-1660``, ``log_softmax`` / ``nll_loss`` at ``hap.rs:1808, 1858``), so an
emitted graph is rewritten node by node here.  Every replacement takes the same arguments as the
function it replaces, so only ``node.target`` changes - except for the loss pair, which is folded
into one node.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F


def _is(target, *candidates) -> bool:
    return any(target is c for c in candidates)


def retarget_tensor_ops(graph: torch.fx.Graph, fold_loss: bool = True) -> Dict[str, int]:
    """Rewrite ``graph`` in place; returns how many nodes of each kind were changed.

    * ``F.linear`` -> :func:`hap_b200.linear`
    * ``F.multi_head_attention_forward`` -> :func:`hap_b200.attention.multi_head_attention_forward`
    * ``torch.einsum`` with one of the four MoE codes -> :func:`hap_b200.einsum`
    * ``F.layer_norm`` -> :func:`hap_b200.layer_norm`
    * ``F.dropout`` (``hap.rs:1446-1464``) -> :func:`hap_b200.dropout.dropout`
    * ``F.embedding`` -> :func:`hap_b200.embedding.embedding` (torch's forward, this package's backward kernel)
    * ``nll_loss(log_softmax(x[.float()], -1)[.reshape(-1, V)], y[.reshape(-1)], reduction='sum')``
      -> :func:`hap_b200.nll_log_softmax_sum` ``(x, y)`` when the intermediate nodes have no other user.
    """
    from .attention import multi_head_attention_forward
    from .dropout import dropout
    from .einsum import CODES as SUPPORTED_CODES, einsum
    from .embedding import embedding
    from .linear import linear
    from .loss import nll_log_softmax_sum
    from .norm import layer_norm

    changed = {"linear": 0, "multi_head_attention_forward": 0, "einsum": 0, "layer_norm": 0, "dropout": 0, "embedding": 0, "loss": 0}
    for node in list(graph.nodes):
        if node.op != "call_function":
            continue
        t = node.target
        if _is(t, F.linear, torch._C._nn.linear):
            node.target = linear
            changed["linear"] += 1
        elif _is(t, F.multi_head_attention_forward):
            node.target = multi_head_attention_forward
            changed["multi_head_attention_forward"] += 1
        elif _is(t, torch.einsum) and node.args and isinstance(node.args[0], str) and node.args[0].replace(" ", "") in SUPPORTED_CODES:
            node.target = einsum
            changed["einsum"] += 1
        elif _is(t, F.layer_norm):
            node.target = layer_norm
            changed["layer_norm"] += 1
        elif _is(t, F.dropout):
            node.target = dropout
            changed["dropout"] += 1
        elif _is(t, F.embedding):
            node.target = embedding
            changed["embedding"] += 1
        elif fold_loss and _is(t, F.nll_loss) and _fold_loss(graph, node, nll_log_softmax_sum):
            changed["loss"] += 1
    graph.lint()
    return changed


def prefetch_parameter_gathers(graph: torch.fx.Graph) -> int:
    """Issue the all_gathers of sharded PARAMETERS early and on the communicator's side stream.

    The planner gathers a ZeRO-style sharded parameter right where it is used (``hap.rs:2527-2555``), so a
    step pays one short, latency-bound collective in front of every projection.  A parameter does not
    change between the optimizer steps, so its gather can start at the top of the program: every node
    ``all_gather(get_attr(p), dim, L, rank)`` (either entry point) becomes
    ``collectives.all_gather_start(...)`` at the top of the graph plus ``collectives.all_gather_wait(...)``
    where the gather stood.  The gathers then run next to the layers before their use, and their backward
    reduce_scatters next to the remaining backward pass.  Values are unchanged; the gathered weights live
    from the top of the step instead of from their first use (autograd keeps them until backward anyway).
    Returns the number of gathers moved."""
    from . import collectives

    moved = 0
    anchor = None
    for node in graph.nodes:
        if node.op == "placeholder":
            anchor = node
    for node in list(graph.nodes):
        if node.op != "call_function" or getattr(node.target, "__name__", "") not in ("all_gather", "all_gather_by_group_call"):
            continue
        if (getattr(node.target, "__module__", "") or "").split(".")[-1] != "collectives":
            continue
        src = node.args[0]
        if not (isinstance(src, torch.fx.Node) and src.op == "get_attr"):
            continue
        if anchor is None:
            with graph.inserting_before(next(iter(graph.nodes))):
                attr = graph.get_attr(src.target)
        else:
            with graph.inserting_after(anchor):
                attr = graph.get_attr(src.target)
        with graph.inserting_after(attr):
            start = graph.call_function(collectives.all_gather_start, (attr,) + tuple(node.args[1:]))
        anchor = start
        with graph.inserting_before(node):
            done = graph.call_function(collectives.all_gather_wait, (start,))
        node.replace_all_uses_with(done)
        graph.erase_node(node)
        if not src.users:
            graph.erase_node(src)
        moved += 1
    graph.lint()
    return moved


GATING_FUNCTIONS = ("top2_gating", "top_2_gating", "_top_2_gating", "switch_gating", "_switch_gating")


def sparsify_moe(graph: torch.fx.Graph) -> int:
    """Replace the dense dispatch / combine einsums of the MoE layers by row gathers.

    ``einsum("bsd,bsec->becd", x, D)`` and ``einsum("becd,bsec->bsd", y, C)`` (``models.py:356, 364``; emitted at
    ``hap.rs:2266-2276``) are rewritten to :func:`hap_b200.einsum.sparse_dispatch` / ``sparse_combine`` when D / C
    is ``getitem(g, 0)`` / ``getitem(g, 1)`` of a call of one of the reference's gating functions
    (``models.py:441-502``, matched by name), whose outputs hold at most one token per slot and at most two
    slots per token.  Einsums fed by anything else are left on the dense kernels.  A dispatch whose rows feed
    the expert contractions directly (single-rank programs) writes them in the experts' memory layout.  Returns
    the number of nodes rewritten."""
    import operator
    from .einsum import einsum, sparse_combine, sparse_dispatch

    def from_gating(n, index):
        if not (isinstance(n, torch.fx.Node) and n.op == "call_function" and _is(n.target, operator.getitem)):
            return False
        src, idx = n.args
        return (idx == index and isinstance(src, torch.fx.Node) and src.op == "call_function"
                and getattr(src.target, "__name__", "") in GATING_FUNCTIONS)

    changed = 0
    for node in list(graph.nodes):
        if node.op != "call_function" or not _is(node.target, torch.einsum, einsum) or len(node.args) != 3:
            continue
        code = node.args[0].replace(" ", "") if isinstance(node.args[0], str) else None
        if code == "bsd,bsec->becd" and from_gating(node.args[2], 0):
            # the rows go straight into the expert GEMMs' layout unless a real all_to_all (more than one rank in
            # its length lists) stands between the gather and the experts
            def exchanges(u):
                return (u.op == "call_function" and getattr(u.target, "__name__", "") == "all_to_all"
                        and any(isinstance(a, (list, tuple)) and len(a) > 1 for a in u.args))
            expert_major = not any(exchanges(u) for u in node.users)
            node.target, node.args = sparse_dispatch, (node.args[1], node.args[2], expert_major)
            changed += 1
        elif code == "becd,bsec->bsd" and from_gating(node.args[2], 1):
            # a result that is only ever read through transpose(0, 1) is written in that memory order
            users = list(node.users)
            swapped = len(users) == 1 and users[0].op == "call_method" and users[0].target == "transpose" and \
                tuple(users[0].args[1:]) in ((0, 1), (1, 0))
            node.target, node.args = sparse_combine, (node.args[1], node.args[2], swapped)
            changed += 1
    graph.lint()
    return changed


def fuse_elementwise(graph: torch.fx.Graph) -> Dict[str, int]:
    """Fold the elementwise neighbours of the dropout sites into single-pass kernels; rewrites ``graph``
    in place and returns how many nodes of each kind were folded.

    * ``operator.add(a, dropout(b, p))`` (either order; the dropout feeds nothing else)
      -> :func:`hap_b200.dropout.dropout_add` ``(b, a, p)``
    * ``dropout(relu(x), p)`` / ``dropout(gelu(x), p)`` (the activation feeds nothing else)
      -> :func:`hap_b200.dropout.act_dropout` ``(x, act, p)``
    * a remaining ``relu(x)`` / ``gelu(x)`` (erf form) -> ``act_dropout(x, act, 0.0)``: the bare activation
      on the package's kernel, whose backward needs only the activation's output (relu).

    Run it after :func:`retarget_tensor_ops`; it recognises torch's ``F.dropout`` / ``F.relu`` /
    ``F.gelu`` as well as this package's ``dropout``.  The arithmetic is unchanged: each fused kernel
    rounds once where the separate kernels rounded after every op, and draws its mask from the same
    generator (the call ids of the remaining sites shift, as after any change of the program)."""
    import operator
    from .dropout import act_dropout, dropout, dropout_add

    def is_dropout(n):
        return isinstance(n, torch.fx.Node) and n.op == "call_function" and _is(n.target, F.dropout, dropout)

    def dropout_args(n):
        x = n.args[0] if n.args else n.kwargs["input"]
        p = n.args[1] if len(n.args) > 1 else n.kwargs.get("p", 0.5)
        training = n.args[2] if len(n.args) > 2 else n.kwargs.get("training", True)
        return x, p, training

    def act_of(n):
        if not (isinstance(n, torch.fx.Node) and n.op == "call_function"):
            return None
        if _is(n.target, F.relu, torch.relu):
            return "relu"
        if _is(n.target, F.gelu) and n.kwargs.get("approximate", "none") == "none" and len(n.args) == 1:
            return "gelu"
        return None

    changed = {"dropout_add": 0, "act_dropout": 0, "activation": 0}
    for node in list(graph.nodes):
        if node.op != "call_function":
            continue
        if _is(node.target, operator.add) and len(node.args) == 2 and not node.kwargs:
            a, b = node.args
            drop, other = (b, a) if is_dropout(b) else ((a, b) if is_dropout(a) else (None, None))
            if drop is not None and len(drop.users) == 1 and isinstance(other, torch.fx.Node):
                x, p, training = dropout_args(drop)
                if isinstance(p, (int, float)) and training is True:
                    with graph.inserting_before(node):
                        new = graph.call_function(dropout_add, (x, other, float(p)))
                    node.replace_all_uses_with(new)
                    graph.erase_node(node)
                    graph.erase_node(drop)
                    changed["dropout_add"] += 1
        elif is_dropout(node):
            x, p, training = dropout_args(node)
            act = act_of(x)
            if act is not None and len(x.users) == 1 and isinstance(p, (int, float)) and training is True:
                with graph.inserting_before(node):
                    new = graph.call_function(act_dropout, (x.args[0], act, float(p)))
                node.replace_all_uses_with(new)
                graph.erase_node(node)
                graph.erase_node(x)
                changed["act_dropout"] += 1
    for node in list(graph.nodes):
        act = act_of(node)
        if act is not None:
            with graph.inserting_before(node):
                new = graph.call_function(act_dropout, (node.args[0], act, 0.0))
            node.replace_all_uses_with(new)
            graph.erase_node(node)
            changed["activation"] += 1
    graph.lint()
    return changed


def fuse_residual_norm(graph: torch.fx.Graph) -> int:
    """Pre-LN residual blocks, ``x_new = x + f(layer_norm(x))``: ``x`` feeds the normalisation and the residual
    addition, so autograd adds two gradients of ``x`` with a kernel of its own in every block.  Rewrites
    ``h = layer_norm(x, ...)`` into ``x_res, h = layer_norm_fork(x, ...)`` and hands ``x_res`` to the other
    users of ``x``; the two gradients then meet inside the normalisation's backward kernel.  Applies to this
    package's ``layer_norm`` nodes whose input has exactly one other user; returns the number rewritten."""
    import operator
    from .norm import layer_norm, layer_norm_fork
    changed = 0
    for node in list(graph.nodes):
        if node.op != "call_function" or not _is(node.target, layer_norm):
            continue
        x = node.args[0] if node.args else node.kwargs.get("input")
        if not isinstance(x, torch.fx.Node) or len(x.users) != 2:
            continue
        other = next(u for u in x.users if u is not node)
        with graph.inserting_before(node):
            fork = graph.call_function(layer_norm_fork, node.args, node.kwargs)
            x_res = graph.call_function(operator.getitem, (fork, 0))
            h = graph.call_function(operator.getitem, (fork, 1))
        other.replace_input_with(x, x_res)
        node.replace_all_uses_with(h)
        graph.erase_node(node)
        changed += 1
    graph.lint()
    return changed


def _peel(node, method: str):
    """If ``node`` is ``x.<method>(...)`` return ``x`` else ``node`` itself."""
    if isinstance(node, torch.fx.Node) and node.op == "call_method" and node.target == method:
        return node.args[0], node
    return node, None


def _fold_loss(graph: torch.fx.Graph, nll: torch.fx.Node, fused) -> bool:
    if nll.kwargs.get("reduction") != "sum" or len(nll.args) < 2 or len(nll.args) > 2:
        return False
    if any(k not in ("reduction",) for k in nll.kwargs):
        return False
    logp, tgt = nll.args[0], nll.args[1]
    logp_src, reshape_node = _peel(logp, "reshape")
    if not (isinstance(logp_src, torch.fx.Node) and logp_src.op == "call_function"
            and _is(logp_src.target, F.log_softmax, torch.log_softmax)):
        return False
    dim = logp_src.args[1] if len(logp_src.args) > 1 else logp_src.kwargs.get("dim")
    if dim != -1:
        return False
    logits, float_node = _peel(logp_src.args[0], "float")
    tgt_src, tgt_reshape = _peel(tgt, "reshape")
    if tgt_reshape is not None and tuple(tgt_reshape.args[1:]) != (-1,):
        return False
    # the intermediates must feed nothing else
    for n in (logp_src, reshape_node, float_node):
        if n is not None and len(n.users) != 1:
            return False
    with graph.inserting_before(nll):
        new = graph.call_function(fused, (logits, tgt_src))
    nll.replace_all_uses_with(new)
    for n in (nll, reshape_node, logp_src, float_node, tgt_reshape):
        if n is not None and not n.users:
            graph.erase_node(n)
    return True
