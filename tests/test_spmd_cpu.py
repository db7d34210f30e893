"""Host logic of the SPMD path on the CPU: the plan emitter and the lockstep executor replay the
synthesized MLP programs (data parallel and column parallel, ratios [.6,.4]) with the CPU oracle
backend and must reproduce the unsharded model; the same programs run as 2 gloo processes with
the port of the reference's collectives (the N>1 host path)."""
import os
import sys
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from oracle.cpu_executors import CpuLockstepWorld as LockstepWorld, CpuProcessWorker as ProcessWorker
from oracle.lockstep_backend import OracleCollectives
from tests import spmd_common as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("plan", ["dp", "tp"])
def test_lockstep_program_reproduces_the_unsharded_model(plan):
    model, dims = C.reference_model(small=True)
    x, y = C.batch(dims)
    want_loss, want_grads = C.full_gradients(model, x, y)
    world = LockstepWorld(C.rank_modules(model, plan, C.cpu_namespace()), OracleCollectives())
    losses = world.forward([(x, y), (x, y)])
    assert abs(float(sum(losses)) - want_loss) <= 1e-5 * abs(want_loss)
    torch.stack(losses).sum().backward()
    for r, m in enumerate(world.modules):
        for name, p in m.named_parameters():
            want = C.expected_shard(want_grads[name], name, plan, r, dims)
            assert p.grad.shape == want.shape, (plan, r, name)
            torch.testing.assert_close(p.grad.double(), want, rtol=1e-4, atol=1e-4 * float(want.abs().max()))


def test_emitted_programs_have_the_planner_node_sequence():
    model, dims = C.reference_model(small=True)
    ns = C.cpu_namespace()
    import copy
    dp = C.P.emit_mlp(copy.deepcopy(model), "dp", C.RATIOS, 1, C.BATCH, ns)
    names = [n.target.__name__ if callable(n.target) else n.target for n in dp.nodes if n.op in ("call_function", "call_method")]
    assert names == ["split", "getitem", "split", "getitem", "replicate", "replicate", "replicate", "replicate",
                     "linear", "gelu", "linear", "mse_loss"]
    m = copy.deepcopy(model)
    tp = C.P.emit_mlp(m, "tp", C.RATIOS, 1, C.BATCH, ns)
    names = [n.target.__name__ if callable(n.target) else n.target for n in tp.nodes if n.op in ("call_function", "call_method")]
    assert names == ["linear", "all_gather", "gelu", "linear", "split", "getitem", "mse_loss"]
    # parameters were cut in place: rank 1 holds the second shard (hap.rs:929-944)
    assert tuple(m.fc1.weight.shape) == (136 - 82, 64) and tuple(m.fc2.bias.shape) == (72 - 43,)
    gather = next(n for n in tp.nodes if n.op == "call_function" and n.target.__name__ == "all_gather")
    assert gather.args[1:] == (1, [82, 54], 1)


def _gloo_worker(rank, world, store, plan, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from tests import spmd_common as C2
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}")
    model, dims = C2.reference_model(small=True)
    x, y = C2.batch(dims)
    import copy
    m = copy.deepcopy(model)
    graph = C2.P.emit_mlp(m, plan, C2.RATIOS, rank, C2.BATCH, C2.cpu_namespace())
    worker = ProcessWorker(torch.fx.GraphModule(m, graph), reduce_loss=lambda t: (dist.all_reduce(t), t)[1])
    totals = [float(worker.step(x, y)) for _ in range(2)]
    torch.save({"totals": totals, "params": {n: p.detach().clone() for n, p in worker.module.named_parameters()}},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("plan", ["dp", "tp"])
def test_two_gloo_processes_match_the_lockstep_replay(plan):
    model, dims = C.reference_model(small=True)
    x, y = C.batch(dims)
    world = LockstepWorld(C.rank_modules(model, plan, C.cpu_namespace()), OracleCollectives())
    want_totals = [float(world.step([(x, y), (x, y)])) for _ in range(2)]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_gloo_worker, args=(2, os.path.join(d, "store"), plan, d), nprocs=2, join=True)
        for r in range(2):
            got = torch.load(os.path.join(d, f"rank{r}.pt"), weights_only=False)
            for a, b in zip(got["totals"], want_totals):
                assert abs(a - b) <= 1e-5 * abs(b)
            for name, p in world.modules[r].named_parameters():
                torch.testing.assert_close(got["params"][name], p.detach(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("plan", ["dp", "dp_zero", "tp"])
def test_language_model_programs_reproduce_the_unsharded_model(plan):
    """Transformer LM (pre-LN, causal MHA, summed NLL): data parallel, and data parallel with
    ZeRO-style dim-0 sharded weights gathered at use (hap.rs:2527-2555)."""
    import copy
    from hap_b200 import sharding_round
    model = C.lm_model()
    tok, tgt = C.lm_batch()
    ref = copy.deepcopy(model)
    want = ref(tok, tgt)
    want.backward()
    world = LockstepWorld(C.lm_rank_modules(model, plan, C.lm_cpu_namespace()), OracleCollectives())
    losses = world.forward([(tok, tgt), (tok, tgt)])
    assert abs(float(sum(losses)) - float(want)) <= 1e-5 * abs(float(want))
    torch.stack(losses).sum().backward()
    full = dict(ref.named_parameters())
    n_sharded = 0
    for r, m in enumerate(world.modules):
        for name, p in m.named_parameters():
            g = full[name].grad
            if p.shape != g.shape:
                g = torch.split(g, sharding_round(g.shape[0], C.RATIOS), dim=0)[r]
                n_sharded += 1
            torch.testing.assert_close(p.grad, g, rtol=1e-3, atol=1e-4)
    assert (n_sharded > 0) == (plan in ("dp_zero", "tp"))
    if plan == "tp":      # the FFN is column-parallel: gathers on the last dimension and on the batch dimension, a slice back
        names = [getattr(n.target, "__name__", "") for n in world.modules[0].graph.nodes if n.op == "call_function"]
        nl = C.LM_SMALL["nlayers"]
        assert names.count("dynamic_slice") == nl and names.count("all_gather") == 3 * nl + 3 * nl + 2


@pytest.mark.parametrize("plan", ["dp", "dp_zero", "tp"])
def test_vit_programs_reproduce_the_unsharded_model(plan):
    """ViT (patch embedding as a linear map of flattened patches, class token, unmasked MHA, GELU MLP,
    summed NLL over the class token), ratios [.6,.4]; also checked against a convolutional patch
    embedding, which is what the reference's model uses (models.py:147-177)."""
    import copy
    from hap_b200 import sharding_round
    model = C.vit_model()
    img, lab = C.vit_batch()
    ref = copy.deepcopy(model)
    want = ref(img, lab)
    want.backward()
    # the reshape/permute + linear equals Conv2d(kernel = stride = patch)
    k = C.VIT_SMALL
    conv = torch.nn.functional.conv2d(img, model.patch_w.detach().view(k["d_model"], k["channels"], k["patch"], k["patch"]),
                                      model.patch_b.detach(), stride=k["patch"])
    mine = torch.nn.functional.linear(
        img.reshape(-1, k["channels"], 4, k["patch"], 4, k["patch"]).permute(0, 2, 4, 1, 3, 5).reshape(-1, 16, 48),
        model.patch_w.detach(), model.patch_b.detach())
    torch.testing.assert_close(mine, conv.flatten(2).transpose(1, 2), rtol=1e-5, atol=1e-5)
    world = LockstepWorld(C.vit_rank_modules(model, plan, C.lm_cpu_namespace()), OracleCollectives())
    losses = world.forward([(img, lab), (img, lab)])
    assert abs(float(sum(losses)) - float(want)) <= 1e-5 * abs(float(want))
    torch.stack(losses).sum().backward()
    full = dict(ref.named_parameters())
    n_sharded = 0
    for r, m in enumerate(world.modules):
        for name, p in m.named_parameters():
            g = full[name].grad
            if p.shape != g.shape:
                g = torch.split(g, sharding_round(g.shape[0], C.RATIOS), dim=0)[r]
                n_sharded += 1
            torch.testing.assert_close(p.grad, g, rtol=1e-3, atol=1e-4)
    assert (n_sharded > 0) == (plan in ("dp_zero", "tp"))
    if plan == "tp":      # the MLP is column-parallel, as in the language model's tp plan
        names = [getattr(n.target, "__name__", "") for n in world.modules[0].graph.nodes if n.op == "call_function"]
        nl = C.VIT_SMALL["nlayers"]
        assert names.count("dynamic_slice") == nl and names.count("all_gather") == 3 * nl + 3 * nl + 3


def test_expert_parallel_moe_program_reproduces_the_unsharded_model():
    """MoE Transformer: experts sharded by sharding_round(n_expert, ratios), tokens batch-sharded, two
    uneven all_to_all per layer (hap.rs:2713-2744) around the expert einsums (models.py:356-364)."""
    import copy
    from hap_b200 import sharding_round
    model = C.moe_model()
    tok, tgt = C.lm_batch()
    ref = copy.deepcopy(model)
    want = ref(tok, tgt)
    want.backward()
    world = LockstepWorld(C.moe_rank_modules(model, C.moe_cpu_namespace()), OracleCollectives())
    names = [n.target.__name__ for n in world.modules[0].graph.nodes if n.op == "call_function" and hasattr(n.target, "__name__")]
    assert names.count("all_to_all") == 2 * C.MOE_SMALL["nlayers"] and names.count("einsum") == 4 * C.MOE_SMALL["nlayers"]
    losses = world.forward([(tok, tgt), (tok, tgt)])
    assert abs(float(sum(losses)) - float(want)) <= 1e-5 * abs(float(want))
    torch.stack(losses).sum().backward()
    full = dict(ref.named_parameters())
    for r, m in enumerate(world.modules):
        for name, p in m.named_parameters():
            g = full[name].grad
            if p.shape != g.shape:
                g = torch.split(g, sharding_round(g.shape[0], C.RATIOS), dim=0)[r]
            torch.testing.assert_close(p.grad, g, rtol=1e-3, atol=1e-4)


def _gloo_program_worker(rank, world, store, kind, out_dir):
    sys.path.insert(0, ROOT)
    import copy
    import torch.distributed as dist
    from tests import spmd_common as C2
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}")
    if kind == "lm":
        m = copy.deepcopy(C2.lm_model())
        graph, inputs = C2.P.emit_lm(m, "dp_zero", C2.RATIOS, rank, C2.LM_BATCH, C2.lm_cpu_namespace()), C2.lm_batch()
    elif kind == "vit":
        m = copy.deepcopy(C2.vit_model())
        graph, inputs = C2.P.emit_vit(m, "dp_zero", C2.RATIOS, rank, C2.LM_BATCH, C2.lm_cpu_namespace()), C2.vit_batch()
    else:
        m = copy.deepcopy(C2.moe_model())
        graph, inputs = C2.P.emit_moe(m, C2.RATIOS, rank, C2.LM_BATCH, C2.moe_cpu_namespace()), C2.lm_batch()
    worker = ProcessWorker(torch.fx.GraphModule(m, graph), reduce_loss=lambda t: (dist.all_reduce(t), t)[1])
    totals = [float(worker.step(*inputs)) for _ in range(2)]
    torch.save({"totals": totals, "params": {n: p.detach().clone() for n, p in worker.module.named_parameters()}},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["lm", "vit", "moe"])
def test_two_gloo_processes_run_the_transformer_programs(kind):
    """The N > 1 host path for the Transformer programs: one process per rank over gloo with the port of the
    reference's collectives (all_to_all included) must walk the same two steps as the lockstep replay."""
    if kind == "lm":
        mods, inputs = C.lm_rank_modules(C.lm_model(), "dp_zero", C.lm_cpu_namespace()), C.lm_batch()
    elif kind == "vit":
        mods, inputs = C.vit_rank_modules(C.vit_model(), "dp_zero", C.lm_cpu_namespace()), C.vit_batch()
    else:
        mods, inputs = C.moe_rank_modules(C.moe_model(), C.moe_cpu_namespace()), C.lm_batch()
    world = LockstepWorld(mods, OracleCollectives())
    want_totals = [float(world.step([inputs, inputs])) for _ in range(2)]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_gloo_program_worker, args=(2, os.path.join(d, "store"), kind, d), nprocs=2, join=True)
        for r in range(2):
            got = torch.load(os.path.join(d, f"rank{r}.pt"), weights_only=False)
            for a, b in zip(got["totals"], want_totals):
                assert abs(a - b) <= 1e-4 * abs(b), (kind, got["totals"], want_totals)
            for name, p in world.modules[r].named_parameters():
                # Adam moves every entry by about lr per step whatever the gradient's size: entries whose
                # gradient is rounding noise may differ by the distance of two steps (lr = 5e-4)
                assert float((got["params"][name] - p.detach()).abs().max()) <= 2.5 * 5e-4, (kind, name)
