"""layer_norm kernels against torch's CPU implementation in float64/float32 (the op the reference's
programs call, hap.rs:1637-1660)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,E", [(8192, 768), (197 * 3, 768), (1000, 1024), (33, 64), (7, 8), (130, 2048), (64, 1288)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_layer_norm_forward_backward(dtype, rows, E, with_bias):
    from hap_b200.norm import layer_norm
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(rows + E)
    x = (torch.randn(rows, E, generator=g) * 2 + 0.5).to(dtype)
    w = (torch.rand(E, generator=g) + 0.5).to(dtype)
    b = torch.randn(E, generator=g).to(dtype) if with_bias else None
    dy = torch.randn(rows, E, generator=g).to(dtype)
    # reference in float64 from the same (rounded) inputs
    xr, wr = x.double().requires_grad_(True), w.double().requires_grad_(True)
    br = b.double().requires_grad_(True) if with_bias else None
    yr = F.layer_norm(xr, (E,), wr, br, 1e-5)
    yr.backward(dy.double())
    xg, wg = x.to(dev).requires_grad_(True), w.to(dev).requires_grad_(True)
    bg = b.to(dev).requires_grad_(True) if with_bias else None
    y = layer_norm(xg, (E,), wg, bg, 1e-5)
    assert y.dtype == dtype and y.shape == x.shape
    y.backward(dy.to(dev))
    if dtype == torch.float32:
        rtol, atol = 1e-5, 1e-5
    else:
        rtol, atol = 2 ** -7, 2 ** -7       # one bf16 rounding of values of order 1
    torch.testing.assert_close(y.detach().cpu().double(), yr.detach(), rtol=rtol, atol=atol)
    torch.testing.assert_close(xg.grad.cpu().double(), xr.grad, rtol=rtol, atol=atol * 2)
    # parameter gradients are sums over the rows: compare against their size
    scale = float(wr.grad.abs().max())
    assert float((wg.grad.cpu().double() - wr.grad).abs().max()) <= (1e-5 if dtype == torch.float32 else 2 ** -7) * max(scale, 1.0)
    if with_bias:
        scale = float(br.grad.abs().max())
        assert float((bg.grad.cpu().double() - br.grad).abs().max()) <= (1e-5 if dtype == torch.float32 else 2 ** -7) * max(scale, 1.0)


def test_layer_norm_is_deterministic_and_handles_leading_dimensions():
    from hap_b200.norm import layer_norm
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    x = torch.randn(17, 5, 768, generator=g).to(torch.bfloat16).to(dev)
    w = torch.ones(768, dtype=torch.bfloat16, device=dev).requires_grad_(True)
    b = torch.zeros(768, dtype=torch.bfloat16, device=dev).requires_grad_(True)
    grads = []
    for _ in range(2):
        w.grad = b.grad = None
        xx = x.clone().requires_grad_(True)
        layer_norm(xx, (768,), w, b).square().sum().backward()
        grads.append((xx.grad.clone(), w.grad.clone(), b.grad.clone()))
    for a, c in zip(*grads):
        assert torch.equal(a, c)
    # a transposed view is copied, not misread
    xt = x.transpose(0, 1)
    torch.testing.assert_close(layer_norm(xt, (768,), w, b), layer_norm(xt.contiguous(), (768,), w, b), rtol=0, atol=0)
    # shapes the kernels do not cover go to torch's implementation
    odd = torch.randn(4, 10, device=dev)
    torch.testing.assert_close(layer_norm(odd, (10,), torch.ones(10, device=dev), None), F.layer_norm(odd, (10,), torch.ones(10, device=dev)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(256, 8, 768), (197, 3, 768), (40, 1024), (9, 2, 64)])
def test_layer_norm_fork_adds_the_residual_gradient_in_the_same_kernel(dtype, shape):
    """(x, layer_norm(x)) for the pre-LN residual pattern: same values as layer_norm, and the gradient of x is the
    normalisation's gradient plus the residual path's, in float64 from the same rounded inputs."""
    from hap_b200.norm import layer_norm, layer_norm_fork
    dev = torch.device("cuda:0")
    E = shape[-1]
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 2 + 0.5).to(dtype)
    w = (torch.rand(E, generator=g) + 0.5).to(dtype)
    b = torch.randn(E, generator=g).to(dtype)
    dres, dy = torch.randn(*shape, generator=g).to(dtype), torch.randn(*shape, generator=g).to(dtype)
    xr, wr, br = x.double().requires_grad_(True), w.double().requires_grad_(True), b.double().requires_grad_(True)
    (F.layer_norm(xr, (E,), wr, br, 1e-5) * dy.double()).sum().backward()
    want_dx = xr.grad + dres.double()
    xg, wg, bg = x.to(dev).requires_grad_(True), w.to(dev).requires_grad_(True), b.to(dev).requires_grad_(True)
    x_res, h = layer_norm_fork(xg, (E,), wg, bg, 1e-5)
    assert x_res.data_ptr() == xg.data_ptr() and torch.equal(h, layer_norm(xg.detach(), (E,), wg.detach(), bg.detach(), 1e-5))
    ((x_res * dres.to(dev)).sum() + (h * dy.to(dev)).sum()).backward()
    rtol, atol = (1e-5, 2e-5) if dtype == torch.float32 else (2 ** -7, 2 ** -6)
    torch.testing.assert_close(xg.grad.cpu().double(), want_dx, rtol=rtol, atol=atol)
    for got, ref in ((wg.grad, wr.grad), (bg.grad, br.grad)):
        assert float((got.cpu().double() - ref).abs().max()) <= (1e-5 if dtype == torch.float32 else 2 ** -7) * max(float(ref.abs().max()), 1.0)
    # only one of the two results used
    for use in (0, 1):
        xg2 = x.to(dev).requires_grad_(True)
        out = layer_norm_fork(xg2, (E,), wg, bg, 1e-5)[use]
        (out * dy.to(dev)).sum().backward()
        want = dy.double() if use == 0 else xr.grad
        torch.testing.assert_close(xg2.grad.cpu().double(), want, rtol=rtol, atol=atol)
