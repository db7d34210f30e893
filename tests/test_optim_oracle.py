"""The step-tail oracle against the torch functions the reference calls (worker.py:47, 74, 76)."""
import torch

from oracle import optim_math


def _make(dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = [(37, 19), (128,), (5, 3, 7), (1,), (1000, 33)]
    params = [torch.randn(s, generator=g).to(dtype) for s in shapes]
    grads = [[(torch.randn(s, generator=g) * sc).to(dtype) for s in shapes] for sc in (3.0, 0.01, 0.5)]
    return params, grads


def _torch_reference(params, grads_per_step, lr, max_norm):
    ps = [torch.nn.Parameter(p.clone()) for p in params]
    opt = torch.optim.Adam(ps, lr=lr)
    norms = []
    for grads in grads_per_step:
        opt.zero_grad()
        for p, g in zip(ps, grads):
            p.grad = g.clone()
        if max_norm is not None:
            norms.append(float(torch.nn.utils.clip_grad_norm_(ps, max_norm)))
        opt.step()
    return ps, opt, norms


def test_oracle_matches_torch_fp32():
    params, grads_per_step = _make(torch.float32)
    ps, opt, norms = _torch_reference(params, grads_per_step, 5e-4, 0.5)
    mine = [p.clone() for p in params]
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    for step, grads in enumerate(grads_per_step):
        norm = optim_math.clip_adam_step(mine, grads, m, v, step, lr=5e-4, max_norm=0.5)
        assert abs(norm - norms[step]) <= 1e-5 * norms[step]
    for a, b, mm, vv in zip(mine, ps, m, v):
        torch.testing.assert_close(a, b.detach(), rtol=1e-6, atol=1e-7)
        torch.testing.assert_close(mm, opt.state[b]["exp_avg"], rtol=1e-5, atol=1e-8)
        torch.testing.assert_close(vv, opt.state[b]["exp_avg_sq"], rtol=1e-5, atol=1e-10)


def test_oracle_matches_torch_without_clipping():
    params, grads_per_step = _make(torch.float32, seed=3)
    ps, opt, _ = _torch_reference(params, grads_per_step, 1e-3, None)
    mine = [p.clone() for p in params]
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    for step, grads in enumerate(grads_per_step):
        optim_math.clip_adam_step(mine, grads, m, v, step, lr=1e-3)
    for a, b in zip(mine, ps):
        torch.testing.assert_close(a, b.detach(), rtol=1e-6, atol=1e-7)


def test_oracle_close_to_torch_bf16():
    # torch rounds to bf16 after every elementwise op, the oracle once: parameters agree to bf16 resolution
    params, grads_per_step = _make(torch.bfloat16, seed=5)
    ps, opt, _ = _torch_reference(params, grads_per_step, 5e-4, 0.5)
    mine = [p.clone() for p in params]
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    for step, grads in enumerate(grads_per_step):
        optim_math.clip_adam_step(mine, grads, m, v, step, lr=5e-4, max_norm=0.5)
    for a, b in zip(mine, ps):
        torch.testing.assert_close(a.float(), b.detach().float(), rtol=1e-2, atol=1e-2)
