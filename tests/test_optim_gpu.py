"""Fused clip + Adam kernels against the CPU oracle (and against torch's own pair on the GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(dtype, dev, seed=0, big=False):
    g = torch.Generator().manual_seed(seed)
    shapes = [(37, 19), (128,), (5, 3, 7), (1,), (1000, 33), (8193,), (3, 8191)]
    if big:
        shapes += [(3072, 768), (33280, 96)] + [(768,)] * 70      # more than one kernel-parameter list
    params = [torch.randn(s, generator=g).to(dtype) for s in shapes]
    grads = [[(torch.randn(s, generator=g) * sc).to(dtype) for s in shapes] for sc in (3.0, 0.01, 0.5)]
    return params, grads


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("max_norm", [0.5, None])
@pytest.mark.parametrize("big", [False, True])
def test_clip_adam_matches_oracle(dtype, max_norm, big):
    from hap_b200.optim import ClipAdam
    from oracle import optim_math
    dev = torch.device("cuda:0")
    params, grads_per_step = _make(dtype, dev, seed=11, big=big)
    ps = [torch.nn.Parameter(p.clone().to(dev)) for p in params]
    opt = ClipAdam(ps, lr=5e-4, max_norm=max_norm)
    want = [p.clone() for p in params]
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    for step, grads in enumerate(grads_per_step):
        opt.zero_grad()
        for p, g in zip(ps, grads):
            p.grad = g.clone().to(dev)
        opt.step()
        norm = optim_math.clip_adam_step(want, grads, m, v, step, lr=5e-4, max_norm=max_norm)
        if max_norm is not None:
            assert abs(float(opt.grad_norm) - norm) <= 1e-5 * norm
        for p, g in zip(ps, grads):     # gradients are left as they were
            assert torch.equal(p.grad.cpu(), g)
    assert float(opt.steps) == len(grads_per_step)
    if dtype == torch.float32:
        for a, b, mm, em, vv, ev in zip(ps, want, opt.exp_avg, m, opt.exp_avg_sq, v):
            torch.testing.assert_close(a.detach().cpu(), b, rtol=2e-6, atol=1e-7)
            torch.testing.assert_close(mm.cpu(), em, rtol=1e-5, atol=1e-6)     # a moment crossing zero: cancellation
            torch.testing.assert_close(vv.cpu(), ev, rtol=1e-5, atol=1e-10)
    else:
        # the same fp32 arithmetic rounded once per step: fused multiply-adds against separate ones
        # flip a bf16 rounding now and then, and a flipped moment carries into the next step, so
        # after three steps values are at most a few bf16 steps (2^-7 relative each) apart; a
        # parameter near zero is compared against the size of its update (lr = 5e-4) instead
        for a, b, mm, em, vv, ev in zip(ps, want, opt.exp_avg, m, opt.exp_avg_sq, v):
            # (a first moment that crosses zero loses relative accuracy to cancellation: its floor is a
            # bf16 step of the tensor's typical magnitude)
            for got, exp, floor in ((a.detach(), b, 3 * 5e-4 * 2 ** -7), (mm, em, 2 ** -7 * float(em.float().abs().mean())),
                                    (vv, ev, 1e-30)):
                got, exp = got.cpu().float(), exp.float()
                assert bool(((got - exp).abs() <= exp.abs() * 3 * 2 ** -7 + floor).all())
            assert (mm.cpu() != em).float().mean() < 0.1


def test_clip_adam_misaligned_views_and_missing_grads():
    """Gradients that are odd-offset views of one flat bucket, and a parameter without a gradient."""
    from hap_b200.optim import ClipAdam
    from oracle import optim_math
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(2)
    shapes = [(33,), (7, 5), (129,), (64,)]
    params = [torch.randn(s, generator=g) for s in shapes]
    ps = [torch.nn.Parameter(p.clone().to(dev)) for p in params]
    opt = ClipAdam(ps, lr=1e-3, max_norm=0.5)
    flat = torch.randn(1 + sum(p.numel() for p in params[:3]), generator=g)
    bucket = flat.to(dev)
    off = 1
    grads = []
    for p, q in zip(ps[:3], params[:3]):
        p.grad = bucket[off:off + q.numel()].view(q.shape)
        grads.append(flat[off:off + q.numel()].view(q.shape).clone())
        off += q.numel()
    opt.step()
    want = [p.clone() for p in params[:3]]
    m = [torch.zeros_like(p) for p in want]
    v = [torch.zeros_like(p) for p in want]
    optim_math.clip_adam_step(want, grads, m, v, 0, lr=1e-3, max_norm=0.5)
    for a, b in zip(ps[:3], want):
        torch.testing.assert_close(a.detach().cpu(), b, rtol=2e-6, atol=1e-7)
    assert torch.equal(ps[3].detach().cpu(), params[3])        # untouched, like torch's Adam


def test_clip_adam_matches_torch_pair_on_gpu():
    """Same step as clip_grad_norm_ + torch.optim.Adam (what worker.py runs), fp32."""
    from hap_b200.optim import ClipAdam
    dev = torch.device("cuda:0")
    params, grads_per_step = _make(torch.float32, dev, seed=21)
    a = [torch.nn.Parameter(p.clone().to(dev)) for p in params]
    b = [torch.nn.Parameter(p.clone().to(dev)) for p in params]
    mine, ref = ClipAdam(a, lr=5e-4, max_norm=0.5), torch.optim.Adam(b, lr=5e-4)
    for grads in grads_per_step:
        for p, q, g in zip(a, b, grads):
            p.grad, q.grad = g.clone().to(dev), g.clone().to(dev)
        mine.step()
        torch.nn.utils.clip_grad_norm_(b, 0.5)
        ref.step()
    for p, q in zip(a, b):
        torch.testing.assert_close(p.detach(), q.detach(), rtol=2e-6, atol=1e-7)


def test_clip_adam_in_cuda_graph():
    from hap_b200.optim import ClipAdam
    dev = torch.device("cuda:0")
    params, grads_per_step = _make(torch.float32, dev, seed=31)
    a = [torch.nn.Parameter(p.clone().to(dev)) for p in params]
    b = [torch.nn.Parameter(p.clone().to(dev)) for p in params]
    eager, graphed = ClipAdam(a, lr=5e-4, max_norm=0.5), ClipAdam(b, lr=5e-4, max_norm=0.5)
    for p, q in zip(a, b):
        p.grad, q.grad = torch.zeros_like(p), torch.zeros_like(q)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            graphed.step()
    graphed.state.zero_()                                  # capture does not run the kernels; start from step 0
    for grads in grads_per_step:
        for p, q, g in zip(a, b, grads):
            p.grad.copy_(g.to(dev)); q.grad.copy_(g.to(dev))
        eager.step()
        graph.replay()
    torch.cuda.synchronize()
    for p, q in zip(a, b):
        assert torch.equal(p.detach(), q.detach())
