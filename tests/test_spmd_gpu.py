"""The synthesized SPMD training step on the GPU against its CPU replay.

Configuration: the 2-layer MLP (in 1024, hidden 4096, out 1024, GELU, sum-MSE), batch 64, world 2,
ratios [.6,.4], both candidate plans.  GPU side: CUDA collectives (2 virtual ranks on one device)
and the package's linear kernels.  CPU side: the same fx programs with the oracle collectives and
torch's CPU linear.  Tolerance from the north star: 1e-5 relative in fp32, 1e-2 in bf16."""
import pytest
import torch

import hap_b200
from hap_b200.spmd import LockstepWorld
from oracle.cpu_executors import CpuLockstepWorld
from oracle.lockstep_backend import OracleCollectives
from tests import spmd_common as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_close(got, want, tol, what):
    """Relative error of the whole tensor (Frobenius norm) within tol; every element within
    tol * (|want| + rms) in fp32, and within 4x that in bf16, where a single rounding flip early in
    the chain (one bf16 ulp = 0.8 %) shows up in a handful of the millions of entries."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float(want.pow(2).mean().sqrt()) + 1e-30
    assert float((got - want).norm()) <= tol * float(want.norm()) + 1e-30, f"{what}: relative error {float((got - want).norm() / want.norm()):.3g}"
    slack = 1.0 if tol < 1e-3 else 4.0
    excess = (got - want).abs() - slack * tol * (want.abs() + rms)
    assert float(excess.max()) <= 0, f"{what}: {int((excess > 0).sum())} of {want.numel()} entries off by up to {float(excess.max()):.3g} (rms {rms:.3g})"


@pytest.mark.parametrize("plan", ["dp", "tp"])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_training_step_matches_cpu_replay(plan, dtype, tol):
    model, dims = C.reference_model(dtype)
    x, y = C.batch(dims, dtype)
    # the CPU replay runs in the same dtype, so both sides round at the same places and differ only
    # in accumulation order
    cpu = CpuLockstepWorld(C.rank_modules(model, plan, C.cpu_namespace()), OracleCollectives())
    comm = hap_b200.local_comm(2, DEV, stage_bytes=64 << 20, heap_bytes=96 << 20)
    try:
        gpu = LockstepWorld(C.rank_modules(model.to(dtype), plan, hap_b200.plan.default_namespace(), device=DEV),
                            hap_b200.LocalCollectives(comm))
        xf, yf = x, y
        xg, yg = x.to(DEV), y.to(DEV)
        # forward + backward of the first step: partial losses and every parameter-gradient shard
        want_losses = cpu.forward([(xf, yf), (xf, yf)])
        got_losses = gpu.forward([(xg, yg), (xg, yg)])
        for r in range(2):
            assert abs(float(got_losses[r]) - float(want_losses[r])) <= tol * abs(float(want_losses[r])), (plan, r)
        torch.stack(want_losses).sum().backward()
        torch.stack(got_losses).sum().backward()
        for r in range(2):
            for (name, pw), (_, pg) in zip(cpu.modules[r].named_parameters(), gpu.modules[r].named_parameters()):
                assert pg.grad.shape == pw.grad.shape
                rel_close(pg.grad, pw.grad, tol, f"{plan} rank {r} grad {name}")
        # two full iterations (clip + Adam included): global loss and updated parameters
        for it in range(2):
            want = float(cpu.step([(xf, yf), (xf, yf)]))
            got = float(gpu.step([(xg, yg), (xg, yg)]))
            assert abs(got - want) <= tol * abs(want), (plan, it, got, want)
        for r in range(2):
            for (name, pw), (_, pg) in zip(cpu.modules[r].named_parameters(), gpu.modules[r].named_parameters()):
                # Adam normalises each element's update to about +-lr whatever the gradient's size, so
                # entries whose gradient is near zero may move differently: allow 5 % of the distance
                # two steps can travel (lr = 5e-4) in fp32, one bf16 ulp of the parameter scale in bf16
                diff = (pg.detach().float().cpu() - pw.detach().float())
                if dtype == torch.float32:
                    assert float(diff.abs().max()) <= 0.05 * 2 * 5e-4, (plan, r, name)
                else:
                    # in bf16 a near-zero gradient can even change sign, so single entries may differ by the
                    # full distance of two steps (2 * lr each way); the tensor as a whole must still agree
                    assert float(diff.abs().max()) <= 2 * 2 * 5e-4 + 2.0 ** -7 * float(pw.abs().max()), (plan, r, name)
                    assert float(diff.norm()) <= 2e-2 * float(pw.float().norm()), (plan, r, name)
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


@pytest.mark.parametrize("plan", ["dp", "dp_zero", "tp"])
def test_language_model_step_matches_cpu_replay(plan):
    """Transformer LM step in bf16: package linear + attention + collectives on the GPU (2 virtual
    ranks) against the same fx programs replayed on the CPU in bf16 with torch's own ops."""
    dtype = torch.bfloat16
    model = C.lm_model(dtype)
    tok, tgt = C.lm_batch()
    cpu = CpuLockstepWorld(C.lm_rank_modules(model, plan, C.lm_cpu_namespace()), OracleCollectives())
    comm = hap_b200.local_comm(2, DEV, stage_bytes=16 << 20, heap_bytes=32 << 20)
    try:
        gpu = LockstepWorld(C.lm_rank_modules(model, plan, hap_b200.plan.default_namespace(), device=DEV),
                            hap_b200.LocalCollectives(comm))
        want = cpu.forward([(tok, tgt), (tok, tgt)])
        got = gpu.forward([(tok.to(DEV), tgt.to(DEV)), (tok.to(DEV), tgt.to(DEV))])
        for r in range(2):
            assert abs(float(got[r]) - float(want[r])) <= 1e-2 * abs(float(want[r])), (plan, r, float(got[r]), float(want[r]))
        torch.stack(want).sum().backward()
        torch.stack(got).sum().backward()
        for r in range(2):
            for (name, pw), (_, pg) in zip(cpu.modules[r].named_parameters(), gpu.modules[r].named_parameters()):
                assert pg.grad.shape == pw.grad.shape, name
                d = (pg.grad.detach().float().cpu() - pw.grad.detach().float())
                assert float(d.norm()) <= 5e-2 * float(pw.grad.float().norm()) + 1e-3, (plan, r, name, float(d.norm()), float(pw.grad.float().norm()))
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


@pytest.mark.parametrize("plan", ["dp", "dp_zero", "tp"])
def test_vit_step_matches_cpu_replay(plan):
    """ViT step in bf16 with the heterogeneous ratios [.3,.25,.2,.25] on 4 virtual ranks: patch
    embedding, unmasked attention with an odd sequence length (17), GELU MLP and the class-token
    head on the package's GPU path against the CPU replay of the same fx programs."""
    dtype = torch.bfloat16
    r4 = [.3, .25, .2, .25]
    model = C.vit_model(dtype)
    img, lab = C.vit_batch(dtype)
    cpu = CpuLockstepWorld(C.vit_rank_modules(model, plan, C.lm_cpu_namespace(), world=4, ratios=r4), OracleCollectives())
    comm = hap_b200.local_comm(4, DEV, stage_bytes=16 << 20, heap_bytes=32 << 20)
    try:
        gpu = LockstepWorld(C.vit_rank_modules(model, plan, hap_b200.plan.default_namespace(), world=4, device=DEV, ratios=r4),
                            hap_b200.LocalCollectives(comm))
        want = cpu.forward([(img, lab)] * 4)
        got = gpu.forward([(img.to(DEV), lab.to(DEV))] * 4)
        for r in range(4):
            assert abs(float(got[r]) - float(want[r])) <= 2e-2 * abs(float(want[r])), (plan, r, float(got[r]), float(want[r]))
        torch.stack(want).sum().backward()
        torch.stack(got).sum().backward()
        for r in range(4):
            for (name, pw), (_, pg) in zip(cpu.modules[r].named_parameters(), gpu.modules[r].named_parameters()):
                assert pg.grad.shape == pw.grad.shape, name
                d = (pg.grad.detach().float().cpu() - pw.grad.detach().float())
                assert float(d.norm()) <= 5e-2 * float(pw.grad.float().norm()) + 1e-3, (plan, r, name, float(d.norm()), float(pw.grad.float().norm()))
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


def test_bucketed_gradient_reduction_gives_the_same_step():
    """ProcessWorker on a world of one: one flat all_reduce over the replicated parameters' gradients
    (views of a heap buffer) must leave exactly the parameters the per-parameter all_reduces leave."""
    import copy
    from hap_b200 import plan as P
    from hap_b200.spmd import ProcessWorker
    model = C.lm_model(torch.bfloat16).to(DEV)
    tok, tgt = (t.to(DEV) for t in C.lm_batch())
    comm = hap_b200.single_comm(DEV, stage_bytes=16 << 20, heap_bytes=48 << 20)
    hap_b200.collectives.set_default_comm(comm)
    try:
        workers = []
        for use_bucket in (False, True):
            m = copy.deepcopy(model)
            graph = P.emit_lm(m, "dp", [1.0], 0, C.LM_BATCH)
            workers.append(ProcessWorker(torch.fx.GraphModule(m, graph), comm=comm if use_bucket else None))
        for _ in range(2):
            a, b = (float(w.step(tok, tgt)) for w in workers)
            assert a == b
        for (name, pa), (_, pb) in zip(workers[0].module.named_parameters(), workers[1].module.named_parameters()):
            assert torch.equal(pa, pb), name
        comm.check()
    finally:
        hap_b200.collectives.set_default_comm(None)
        comm.destroy()


def test_cuda_graph_replay_follows_the_eager_step():
    """The whole iteration captured into a CUDA graph (ProcessWorker.capture) must walk the same loss
    trajectory as the eager step."""
    import copy
    from hap_b200 import plan as P
    from hap_b200.spmd import ProcessWorker
    model = C.lm_model(torch.bfloat16).to(DEV)
    tok, tgt = (t.to(DEV) for t in C.lm_batch())
    comm = hap_b200.single_comm(DEV, stage_bytes=16 << 20, heap_bytes=48 << 20)
    hap_b200.collectives.set_default_comm(comm)
    try:
        m1, m2 = copy.deepcopy(model), copy.deepcopy(model)
        eager = ProcessWorker(torch.fx.GraphModule(m1, P.emit_lm(m1, "dp_zero", [1.0], 0, C.LM_BATCH)), comm=comm)
        graphed = ProcessWorker(torch.fx.GraphModule(m2, P.emit_lm(m2, "dp_zero", [1.0], 0, C.LM_BATCH)), comm=comm)
        replay = graphed.capture(tok, tgt, warmup=3)
        want = [float(eager.step(tok, tgt)) for _ in range(6)]
        got = [float(replay(tok, tgt)) for _ in range(3)]
        comm.set_stream_ordering(True)
        for a, b in zip(got, want[3:]):
            assert abs(a - b) <= 1e-2 * abs(b), (got, want)
        assert got[-1] < want[0]          # it is training
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        hap_b200.collectives.set_default_comm(None)
        comm.destroy()


def test_language_model_on_eight_virtual_ranks_with_empty_shards():
    """World 8, ratios r8, batch 8: sharding_round gives [2,2,1,1,1,1,0,0]-like splits, so some ranks
    hold no samples at all and still take part in every collective."""
    import copy
    from hap_b200 import plan as P
    r8 = [.22, .18, .15, .13, .11, .09, .07, .05]
    lb = hap_b200.sharding_round(C.LM_BATCH, r8)
    assert 0 in lb and sum(lb) == C.LM_BATCH
    model = C.lm_model(torch.bfloat16)
    tok, tgt = C.lm_batch()

    def modules(ns, device):
        mods = []
        for r in range(8):
            m = copy.deepcopy(model).to(device)
            mods.append(torch.fx.GraphModule(m, P.emit_lm(m, "dp_zero", r8, r, C.LM_BATCH, ns)))
        return mods

    cpu = CpuLockstepWorld(modules(C.lm_cpu_namespace(), "cpu"), OracleCollectives())
    comm = hap_b200.local_comm(8, DEV, stage_bytes=8 << 20, heap_bytes=16 << 20)
    try:
        gpu = LockstepWorld(modules(hap_b200.plan.default_namespace(), DEV), hap_b200.LocalCollectives(comm))
        want = float(cpu.step([(tok, tgt)] * 8))
        got = float(gpu.step([(tok.to(DEV), tgt.to(DEV))] * 8))
        assert abs(got - want) <= 1e-2 * abs(want), (got, want)
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


def test_expert_parallel_moe_step_matches_cpu_replay():
    """MoE Transformer step in bf16 on 2 virtual ranks: package attention, linear, einsums and the uneven
    all_to_all against the CPU replay of the same fx programs."""
    dtype = torch.bfloat16
    model = C.moe_model(dtype)
    tok, tgt = C.lm_batch()
    cpu = CpuLockstepWorld(C.moe_rank_modules(model, C.moe_cpu_namespace()), OracleCollectives())
    comm = hap_b200.local_comm(2, DEV, stage_bytes=16 << 20, heap_bytes=32 << 20)
    try:
        gpu = LockstepWorld(C.moe_rank_modules(model, hap_b200.plan.default_namespace(), device=DEV), hap_b200.LocalCollectives(comm))
        want = cpu.forward([(tok, tgt), (tok, tgt)])
        got = gpu.forward([(tok.to(DEV), tgt.to(DEV))] * 2)
        for r in range(2):
            assert abs(float(got[r]) - float(want[r])) <= 2e-2 * abs(float(want[r])), (r, float(got[r]), float(want[r]))
        torch.stack(want).sum().backward()
        torch.stack(got).sum().backward()
        for r in range(2):
            for (name, pw), (_, pg) in zip(cpu.modules[r].named_parameters(), gpu.modules[r].named_parameters()):
                assert pg.grad.shape == pw.grad.shape, name
                d = (pg.grad.detach().float().cpu() - pw.grad.detach().float())
                # top-2 routing is discrete: a bf16-level difference in a gate logit sends a token to another
                # expert, which moves the gradients of the gate, of both experts and of everything upstream.
                # The contractions themselves are held to 1e-2 in test_einsum_gpu.py; here a flip must be survivable
                tol = 0.5
                assert float(d.norm()) <= tol * float(pw.grad.float().norm()) + 1e-2, (r, name, float(d.norm()), float(pw.grad.float().norm()))
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


# ---- one step of each program at the configurations' full layer widths ----------------------------------
# One layer instead of 12 / 12 / 8 and batch 8, but every tensor has the width the benchmark configuration
# gives it (d_model, FFN, vocabulary, sequence length, image and patch size, expert count and capacity), so
# the vocabulary projection with its split-K input gradient, the 197-token attention and the 32-expert
# einsums run inside a real step.  The CPU side replays the same fx programs in float32 on the
# bf16-rounded parameters (torch's CPU kernels; seconds).
def _full_width_case(kind):
    import copy
    from hap_b200 import plan as P
    torch.manual_seed(39)
    g = torch.Generator().manual_seed(2024)
    B = 8
    if kind in ("lm", "lm_tp"):
        model = P.TransformerLM(nlayers=1)
        inputs = (torch.randint(0, 33278, (B, 256), generator=g), torch.randint(0, 33278, (B, 256), generator=g))
        emit = lambda m, r, ns: P.emit_lm(m, "tp" if kind == "lm_tp" else "dp_zero", C.RATIOS, r, B, ns)
        cpu_ns = C.lm_cpu_namespace()
    elif kind in ("vit", "vit_tp"):
        model = P.ViT(nlayers=1)
        inputs = (torch.randn(B, 3, 224, 224, generator=g), torch.randint(0, 1000, (B,), generator=g))
        emit = lambda m, r, ns: P.emit_vit(m, "tp" if kind == "vit_tp" else "dp_zero", C.RATIOS, r, B, ns)
        cpu_ns = C.lm_cpu_namespace()
    else:
        model = P.MoETransformerLM(nlayers=1)
        inputs = (torch.randint(0, 33278, (B, 512), generator=g), torch.randint(0, 33278, (B, 512), generator=g))
        emit = lambda m, r, ns: P.emit_moe(m, C.RATIOS, r, B, ns)
        cpu_ns = C.moe_cpu_namespace()
    model = model.to(torch.bfloat16)

    def modules(ns, device, dtype):
        mods = []
        for r in range(2):
            m = copy.deepcopy(model).to(device=device, dtype=dtype)
            mods.append(torch.fx.GraphModule(m, emit(m, r, ns)))
        return mods

    return modules, cpu_ns, inputs


@pytest.mark.parametrize("kind", ["lm", "lm_tp", "vit", "vit_tp", "moe"])
def test_full_width_single_layer_step_matches_cpu_replay(kind):
    modules, cpu_ns, inputs = _full_width_case(kind)
    cpu = CpuLockstepWorld(modules(cpu_ns, "cpu", torch.float32), OracleCollectives())
    cpu_in = tuple(t.float() if t.is_floating_point() else t for t in inputs)
    gpu_in = tuple((t.to(torch.bfloat16) if t.is_floating_point() else t).to(DEV) for t in inputs)
    comm = hap_b200.local_comm(2, DEV, stage_bytes=128 << 20, heap_bytes=192 << 20)
    try:
        gpu = LockstepWorld(modules(hap_b200.plan.default_namespace(), DEV, torch.bfloat16), hap_b200.LocalCollectives(comm))
        want = cpu.forward([cpu_in] * 2)
        got = gpu.forward([gpu_in] * 2)
        for r in range(2):
            assert abs(float(got[r]) - float(want[r])) <= 1e-2 * abs(float(want[r])), (kind, r, float(got[r]), float(want[r]))
        torch.stack(want).sum().backward()
        torch.stack(got).sum().backward()
        # bf16 activations against a float32 replay: whole-tensor agreement of every parameter gradient;
        # with top-2 routing a flipped token moves the gradients of two experts, hence the looser bound
        tol = 0.5 if kind == "moe" else 6e-2
        for r in range(2):
            for (name, pw), (_, pg) in zip(cpu.modules[r].named_parameters(), gpu.modules[r].named_parameters()):
                assert pg.grad is not None and pg.grad.shape == pw.grad.shape, name
                d = (pg.grad.detach().float().cpu() - pw.grad.detach().float())
                assert float(d.norm()) <= tol * float(pw.grad.float().norm()) + 1e-2, (kind, r, name, float(d.norm()), float(pw.grad.float().norm()))
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


def test_moe_step_with_sparse_dispatch_follows_the_dense_program():
    """The expert-parallel program after fxpass.sparsify_moe (dispatch / combine as row gathers) and
    fxpass.fuse_elementwise must walk the same loss trajectory as the program as emitted."""
    import copy
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    model = C.moe_model(torch.bfloat16)
    tok, tgt = C.lm_batch()

    def modules(rewrite):
        mods = []
        for r in range(2):
            m = copy.deepcopy(model).to(DEV)
            g = P.emit_moe(m, C.RATIOS, r, C.LM_BATCH)
            if rewrite:
                assert fxpass.sparsify_moe(g) == 2 * C.MOE_SMALL["nlayers"]
                fxpass.fuse_elementwise(g)
            mods.append(torch.fx.GraphModule(m, g))
        return mods

    comm = hap_b200.local_comm(2, DEV, stage_bytes=16 << 20, heap_bytes=32 << 20)
    try:
        dense = LockstepWorld(modules(False), hap_b200.LocalCollectives(comm))
        sparse = LockstepWorld(modules(True), hap_b200.LocalCollectives(comm))
        feed = [(tok.to(DEV), tgt.to(DEV))] * 2
        for it in range(3):
            a, b = float(dense.step(feed)), float(sparse.step(feed))
            assert abs(a - b) <= 1e-2 * abs(a), (it, a, b)
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()


@pytest.mark.parametrize("kind", ["lm", "vit"])
def test_step_with_forked_residual_norms_follows_the_program_as_emitted(kind):
    """fxpass.fuse_residual_norm only moves an addition into the normalisation's backward kernel: the pre-LN
    programs give the same gradients (one bf16 rounding apart) and walk the same loss trajectory."""
    import copy
    from hap_b200 import fxpass
    from hap_b200 import plan as P
    if kind == "lm":
        model, feed1 = C.lm_model(torch.bfloat16), C.lm_batch()
        emit, nl = (lambda m, r: P.emit_lm(m, "dp_zero", C.RATIOS, r, C.LM_BATCH)), C.LM_SMALL["nlayers"]
    else:
        model, feed1 = C.vit_model(torch.bfloat16), C.vit_batch(torch.bfloat16)
        emit, nl = (lambda m, r: P.emit_vit(m, "dp_zero", C.RATIOS, r, C.LM_BATCH)), C.VIT_SMALL["nlayers"]

    def modules(rewrite):
        mods = []
        for r in range(2):
            m = copy.deepcopy(model).to(DEV)
            g = emit(m, r)
            if rewrite:
                assert fxpass.fuse_residual_norm(g) == 2 * nl
            mods.append(torch.fx.GraphModule(m, g))
        return mods

    comm = hap_b200.local_comm(2, DEV, stage_bytes=16 << 20, heap_bytes=32 << 20)
    try:
        plain = LockstepWorld(modules(False), hap_b200.LocalCollectives(comm))
        forked = LockstepWorld(modules(True), hap_b200.LocalCollectives(comm))
        feed = [tuple(t.to(DEV) for t in feed1)] * 2
        # first the gradients of one backward pass (before Adam's sign-like first steps amplify rounding differences) ...
        la, lb = plain.forward(feed), forked.forward(feed)
        torch.stack(la).sum().backward()
        torch.stack(lb).sum().backward()
        for r in range(2):
            assert abs(float(la[r]) - float(lb[r])) <= 1e-3 * abs(float(la[r]))
            for (name, pa), (_, pb) in zip(plain.modules[r].named_parameters(), forked.modules[r].named_parameters()):
                d = (pa.grad.float() - pb.grad.float()).norm()
                assert float(d) <= 3e-2 * float(pa.grad.float().norm()) + 1e-3, (name, float(d), float(pa.grad.float().norm()))
        # ... then the loss trajectory of whole steps
        for it in range(3):
            a, b = float(plain.step(feed)), float(forked.step(feed))
            assert abs(a - b) <= 1e-2 * abs(a), (it, a, b)
        comm.check()
        hap_b200.linear_ops.gemm_status()
    finally:
        comm.destroy()
