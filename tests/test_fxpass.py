"""Rewriting a program that names torch's functions (as the planner emits it) onto the package's ops."""
import copy

import pytest
import torch
import torch.nn.functional as F

from tests import spmd_common as C


def _names(graph):
    return [getattr(n.target, "__name__", str(n.target)) for n in graph.nodes if n.op == "call_function"]


def test_targets_are_swapped_and_the_loss_pair_is_folded():
    import hap_b200
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    model = C.lm_model()
    graph = P.emit_lm(copy.deepcopy(model), "dp_zero", C.RATIOS, 0, C.LM_BATCH, C.lm_cpu_namespace(), dropout_p=0.1)   # torch's functions
    before = _names(graph)
    assert "log_softmax" in before and "nll_loss" in before
    changed = fxpass.retarget_tensor_ops(graph)
    nl = C.LM_SMALL["nlayers"]
    assert changed == {"linear": 2 * nl + 1, "multi_head_attention_forward": nl, "einsum": 0, "layer_norm": 2 * nl + 1, "dropout": 3 * nl, "embedding": 1, "loss": 1}
    after = [n for n in graph.nodes if n.op == "call_function"]
    assert not any(n.target in (F.linear, F.layer_norm, F.multi_head_attention_forward, F.nll_loss, F.log_softmax, F.dropout) for n in after)
    assert all(n.kwargs["dropout_p"] == 0.1 for n in after if n.target is hap_b200.attention.multi_head_attention_forward)
    assert sum(n.target is hap_b200.nll_log_softmax_sum for n in after) == 1
    assert not any(n.op == "call_method" and n.target == "float" for n in graph.nodes)
    # collectives are left alone (they belong to the other pass)
    assert _names(graph).count("all_gather") == before.count("all_gather")

    moe = C.moe_model()
    g2 = P.emit_moe(copy.deepcopy(moe), C.RATIOS, 0, C.LM_BATCH, C.moe_cpu_namespace())
    changed = fxpass.retarget_tensor_ops(g2)
    assert changed["einsum"] == 4 * C.MOE_SMALL["nlayers"] and changed["loss"] == 1


def test_loss_is_not_folded_when_the_log_probabilities_are_used_elsewhere():
    from hap_b200 import fxpass
    g = torch.fx.Graph()
    x, y = g.placeholder("x"), g.placeholder("y")
    logp = g.call_function(F.log_softmax, (x, -1))
    loss = g.call_function(F.nll_loss, (logp, y), {"reduction": "sum"})
    g.output((loss, logp))
    assert fxpass.retarget_tensor_ops(g)["loss"] == 0
    g2 = torch.fx.Graph()
    x, y = g2.placeholder("x"), g2.placeholder("y")
    loss = g2.call_function(F.nll_loss, (g2.call_function(F.log_softmax, (x, -1)), y), {"reduction": "mean"})
    g2.output(loss)
    assert fxpass.retarget_tensor_ops(g2)["loss"] == 0


@pytest.mark.gpu
def test_rewritten_program_matches_the_natively_emitted_one():
    import hap_b200
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    from hap_b200.spmd import LockstepWorld
    dev = torch.device("cuda:0")
    model = C.lm_model(torch.bfloat16)
    tok, tgt = (t.to(dev) for t in C.lm_batch())
    comm = hap_b200.local_comm(2, dev, stage_bytes=16 << 20, heap_bytes=32 << 20)
    try:
        native = LockstepWorld(C.lm_rank_modules(model, "dp_zero", P.default_namespace(), device=dev), hap_b200.LocalCollectives(comm))
        # the same program with torch's functions as targets, then rewritten
        ns = P.default_namespace()
        torch_ns = type(ns)(collectives=ns.collectives, linear=F.linear, mha=F.multi_head_attention_forward)
        mods = C.lm_rank_modules(model, "dp_zero", torch_ns, device=dev)
        for m in mods:
            assert fxpass.retarget_tensor_ops(m.graph)["loss"] == 1
            m.recompile()
        rewritten = LockstepWorld(mods, hap_b200.LocalCollectives(comm))
        a = native.forward([(tok, tgt), (tok, tgt)])
        b = rewritten.forward([(tok, tgt), (tok, tgt)])
        for x, y in zip(a, b):
            assert float(x) == float(y)
        comm.check()
    finally:
        comm.destroy()


def test_elementwise_fusion_folds_the_dropout_sites():
    import operator
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    from hap_b200.dropout import act_dropout, dropout_add
    nl = C.LM_SMALL["nlayers"]
    model = C.lm_model()
    graph = P.emit_lm(copy.deepcopy(model), "dp_zero", C.RATIOS, 0, C.LM_BATCH, C.lm_cpu_namespace(), dropout_p=0.1)
    assert fxpass.fuse_elementwise(graph) == {"dropout_add": 2 * nl, "act_dropout": nl, "activation": 0}
    targets = [n.target for n in graph.nodes if n.op == "call_function"]
    assert F.dropout not in targets and F.relu not in targets
    assert targets.count(dropout_add) == 2 * nl and targets.count(act_dropout) == nl
    for n in graph.nodes:
        if n.op == "call_function" and n.target is act_dropout:
            assert n.args[1] == "relu" and n.args[2] == 0.1
    # without dropout only the activations are left to replace
    graph = P.emit_lm(copy.deepcopy(model), "dp", C.RATIOS, 0, C.LM_BATCH, C.lm_cpu_namespace())
    assert fxpass.fuse_elementwise(graph) == {"dropout_add": 0, "act_dropout": 0, "activation": nl}
    vit = C.vit_model()
    graph = P.emit_vit(copy.deepcopy(vit), "dp", C.RATIOS, 0, C.LM_BATCH, C.lm_cpu_namespace(), dropout_p=0.2)
    changed = fxpass.fuse_elementwise(graph)
    assert changed == {"dropout_add": 2 * C.VIT_SMALL["nlayers"], "act_dropout": C.VIT_SMALL["nlayers"], "activation": 0}
    assert all(n.args[1] == "gelu" for n in graph.nodes if n.op == "call_function" and n.target is act_dropout)
    # a dropout whose result is used twice is left alone
    g = torch.fx.Graph()
    x, y = g.placeholder("x"), g.placeholder("y")
    d = g.call_function(F.dropout, (x, 0.1))
    s1 = g.call_function(operator.add, (y, d))
    g.output(g.call_function(operator.add, (s1, d)))
    assert fxpass.fuse_elementwise(g)["dropout_add"] == 0


def test_residual_norms_are_forked():
    """x + f(layer_norm(x)): the normalisation hands x through, so the residual user reads the fork's first result."""
    import operator
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    from hap_b200.norm import layer_norm, layer_norm_fork
    nl = C.LM_SMALL["nlayers"]
    for p_drop in (0.0, 0.1):
        graph = P.emit_lm(copy.deepcopy(C.lm_model()), "dp_zero", C.RATIOS, 0, C.LM_BATCH, P.default_namespace(), dropout_p=p_drop)
        fxpass.fuse_elementwise(graph)
        assert fxpass.fuse_residual_norm(graph) == 2 * nl
        targets = [n.target for n in graph.nodes if n.op == "call_function"]
        assert targets.count(layer_norm_fork) == 2 * nl and targets.count(layer_norm) == 1      # the final norm has no residual
        for n in graph.nodes:
            if n.op == "call_function" and n.target is layer_norm_fork:
                parts = {u.args[1]: u for u in n.users}
                assert set(parts) == {0, 1} and all(u.target is operator.getitem for u in n.users)
                assert len(parts[0].users) == 1 and len(n.args[0].users) == 1               # x now feeds the fork only
    vit = P.emit_vit(copy.deepcopy(C.vit_model()), "dp", C.RATIOS, 0, C.LM_BATCH, P.default_namespace(), dropout_p=0.1)
    assert fxpass.fuse_residual_norm(vit) == 2 * C.VIT_SMALL["nlayers"]
    # the post-LN MoE blocks normalise the sum itself: nothing to fork
    moe = P.emit_moe(copy.deepcopy(C.moe_model()), C.RATIOS, 0, C.LM_BATCH, P.default_namespace())
    assert fxpass.fuse_residual_norm(moe) == 0


def test_parameter_gathers_are_hoisted():
    from hap_b200 import collectives, fxpass
    from hap_b200 import plan as P
    nl = C.LM_SMALL["nlayers"]
    model = C.lm_model()
    ns = C.lm_cpu_namespace()
    ns.collectives = collectives            # the pass looks for this package's (or the reference's) collectives module
    graph = P.emit_lm(copy.deepcopy(model), "dp_zero", C.RATIOS, 0, C.LM_BATCH, ns)
    gathers = sum(1 for n in graph.nodes if n.op == "call_function" and n.target is collectives.all_gather)
    assert gathers == 6 * nl + 2
    assert fxpass.prefetch_parameter_gathers(graph) == gathers
    nodes = list(graph.nodes)
    starts = [i for i, n in enumerate(nodes) if n.op == "call_function" and n.target is collectives.all_gather_start]
    waits = [i for i, n in enumerate(nodes) if n.op == "call_function" and n.target is collectives.all_gather_wait]
    first_compute = min(i for i, n in enumerate(nodes) if n.op in ("call_function", "call_method")
                        and n.target not in (collectives.all_gather_start,))
    assert len(starts) == len(waits) == gathers and max(starts) < first_compute
    assert not any(n.op == "call_function" and n.target is collectives.all_gather for n in nodes)
    # program order of the gathers is kept (all ranks must issue the same sequence of collectives)
    order = [nodes[i].args[0].target for i in starts]
    assert order == [nodes[w].args[0].args[0].target for w in waits]


def test_moe_einsums_fed_by_a_gating_function_become_gathers():
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    from hap_b200.einsum import sparse_combine, sparse_dispatch
    moe = C.moe_model()
    g = P.emit_moe(copy.deepcopy(moe), C.RATIOS, 0, C.LM_BATCH, C.moe_cpu_namespace())
    nl = C.MOE_SMALL["nlayers"]
    assert fxpass.sparsify_moe(g) == 2 * nl
    targets = [n.target for n in g.nodes if n.op == "call_function"]
    assert targets.count(sparse_dispatch) == nl and targets.count(sparse_combine) == nl
    assert targets.count(torch.einsum) == 2 * nl          # the two expert contractions stay dense
    # two ranks: a real all_to_all follows the dispatch, so its rows stay batch-major; the combine's result is only read
    # through transpose(0, 1), so it is written in that order
    for n in g.nodes:
        if n.op == "call_function" and n.target is sparse_dispatch:
            assert n.args[2] is False
        if n.op == "call_function" and n.target is sparse_combine:
            assert n.args[2] is True
    # one rank: the rows go straight to the expert contractions, in their memory layout
    g1 = P.emit_moe(copy.deepcopy(moe), [1.0], 0, C.LM_BATCH, C.moe_cpu_namespace())
    assert fxpass.sparsify_moe(g1) == 2 * nl
    assert all(n.args[2] is True for n in g1.nodes if n.op == "call_function" and n.target is sparse_dispatch)
    # an einsum whose second operand is not a gating output is left alone
    g2 = torch.fx.Graph()
    x, d = g2.placeholder("x"), g2.placeholder("d")
    g2.output(g2.call_function(torch.einsum, ("bsd,bsec->becd", x, d)))
    assert fxpass.sparsify_moe(g2) == 0
