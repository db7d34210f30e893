"""The dropout kernel (``F.dropout`` of the synthesized programs, ``hap.rs:1446-1464``) on the GPU.

The random mask cannot match torch's generator, so parity is checked GIVEN the mask: the library
exports the keep mask a call draws, and the output must equal ``x * mask / (1 - p)`` (rounded once to
the tensor's dtype) bit for bit; the backward pass must use the same mask; the keep rate must be
1 - p within sampling error; a new iteration must draw a new mask."""
import pytest
import torch

import hap_b200
from hap_b200 import dropout as D

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [1, 7, 8, 4099, 1 << 20])
def test_output_equals_masked_input(dtype, n):
    D.manual_seed(1234, DEV)
    D.advance(DEV)
    p = 0.1
    x = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(dtype).to(DEV).requires_grad_(True)
    y = D.dropout(x, p)
    call_id = D._next_call_id                       # the id this call took
    mask = D.keep_mask(n, p, call_id, DEV).bool()
    want = torch.where(mask, (x.detach().float() * (1.0 / (1.0 - p))), torch.zeros((), device=DEV)).to(dtype)
    assert torch.equal(y.detach(), want)
    g = torch.randn(n, generator=torch.Generator().manual_seed(n + 1)).to(dtype).to(DEV)
    y.backward(g)
    want_g = torch.where(mask, (g.float() * (1.0 / (1.0 - p))), torch.zeros((), device=DEV)).to(dtype)
    assert torch.equal(x.grad, want_g)


def test_keep_rate_and_fresh_masks_per_iteration_and_site():
    D.manual_seed(7, DEV)
    n, p = 1 << 22, 0.1
    D.advance(DEV)
    a = D.keep_mask(n, p, 1, DEV)
    b = D.keep_mask(n, p, 2, DEV)            # another site in the same iteration
    assert torch.equal(a, D.keep_mask(n, p, 1, DEV))   # the same site again: the same mask
    D.advance(DEV)
    c = D.keep_mask(n, p, 1, DEV)            # the same site in the next iteration
    for m in (a, b, c):
        rate = float(m.float().mean())
        assert abs(rate - (1 - p)) < 5 * (p * (1 - p) / n) ** 0.5 + 1e-5, rate     # 5 sigma + threshold rounding
    for u, v in ((a, b), (a, c), (b, c)):
        agree = float((u == v).float().mean())
        assert abs(agree - ((1 - p) ** 2 + p ** 2)) < 2e-3, agree                    # independent masks
    D.manual_seed(7, DEV)
    D.advance(DEV)
    assert torch.equal(a, D.keep_mask(n, p, 1, DEV))   # reseeding reproduces the sequence


def test_graph_replay_draws_new_masks():
    D.manual_seed(99, DEV)
    x = torch.ones(4096, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(x)

    def step():
        D.advance(DEV)
        out.copy_(D.dropout(x, 0.5))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    seen = []
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        seen.append(out.clone())
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[1], seen[2])


def test_eval_mode_and_p_zero_are_the_identity_and_bad_inputs_raise():
    x = torch.randn(64, device=DEV)
    assert D.dropout(x, 0.3, training=False) is x
    assert D.dropout(x, 0.0) is x
    with pytest.raises(ValueError):
        D.dropout(x, 1.0)
    with pytest.raises(RuntimeError):
        D.dropout(x.cpu(), 0.1)
    with pytest.raises(TypeError):
        D.dropout(x.half(), 0.1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,p", [(4099, 0.1), (1 << 18, 0.3), (64, 0.0)])
def test_dropout_add_equals_the_separate_ops_given_the_mask(dtype, n, p):
    D.manual_seed(5, DEV)
    D.advance(DEV)
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g).to(dtype).to(DEV).requires_grad_(True)
    r = torch.randn(n, generator=g).to(dtype).to(DEV).requires_grad_(True)
    y = D.dropout_add(x, r, p)
    mask = D.keep_mask(n, p, D._next_call_id, DEV).bool() if p > 0 else torch.ones(n, dtype=torch.bool, device=DEV)
    scale = 1.0 / (1.0 - p)
    # the kernel computes residual + x * scale as ONE fused multiply-add in float32: evaluate it exactly in float64
    # (the float32 scale factor included) and round once to float32, then to the tensor's dtype
    scale32 = float(torch.tensor(scale, dtype=torch.float32))
    want = (r.detach().double() + torch.where(mask, x.detach().double() * scale32, torch.zeros((), device=DEV, dtype=torch.float64)))
    want = want.float().to(dtype)
    assert torch.equal(y.detach(), want)
    gy = torch.randn(n, generator=g).to(dtype).to(DEV)
    y.backward(gy)
    assert torch.equal(r.grad, gy)
    assert torch.equal(x.grad, torch.where(mask, gy.float() * scale, torch.zeros((), device=DEV)).to(dtype))


@pytest.mark.parametrize("act", ["relu", "gelu"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,p", [(4099, 0.1), (1 << 18, 0.25), (96, 0.0)])
def test_act_dropout_equals_the_separate_ops_given_the_mask(act, dtype, n, p):
    D.manual_seed(6, DEV)
    D.advance(DEV)
    g = torch.Generator().manual_seed(n + 1)
    x = torch.randn(n, generator=g).to(dtype).to(DEV).requires_grad_(True)
    y = D.act_dropout(x, act, p)
    mask = D.keep_mask(n, p, D._next_call_id, DEV).bool() if p > 0 else torch.ones(n, dtype=torch.bool, device=DEV)
    scale = 1.0 / (1.0 - p)
    ref_in = x.detach().double().requires_grad_(True)
    fn = torch.relu if act == "relu" else torch.nn.functional.gelu
    ref = fn(ref_in) * mask.double() * scale
    gy = torch.randn(n, generator=g).to(dtype).to(DEV)
    y.backward(gy)
    ref.backward(gy.double())
    tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(y.detach().double(), ref.detach(), **tol)
    torch.testing.assert_close(x.grad.double(), ref_in.grad, **tol)
    if act == "relu":       # exact: one rounding of max(x, 0) * scale, and the gradient passes exactly where the output is non-zero
        assert torch.equal(y.detach(), (torch.relu(x.detach().float()) * mask * scale).to(dtype))
        assert torch.equal(x.grad, torch.where(y.detach() != 0, gy.float() * scale, torch.zeros((), device=DEV)).to(dtype))


@pytest.mark.parametrize("act", ["relu", "gelu"])
def test_permuted_views_keep_their_layout_and_their_mask(act):
    """A dense permuted view (the expert-major activations of the MoE layers) goes through without a copy,
    comes out with the same strides, and the backward pass applies the forward's mask whatever layout the
    incoming gradient has."""
    D.manual_seed(8, DEV)
    D.advance(DEV)
    base = torch.randn(6, 4, 5, 16, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    x = base.permute(1, 0, 2, 3).requires_grad_(True)            # (b, e, c, h) view of (e, b, c, h) memory
    y = D.act_dropout(x, act, 0.25)
    call_id = D._next_call_id
    assert y.stride() == x.stride()
    y2 = D.act_dropout(x.detach().contiguous().requires_grad_(True), act, 0.0)      # the bare activation, other layout
    kept = (y.detach() != 0) | (y2.detach() == 0)
    torch.testing.assert_close(torch.where(y.detach() != 0, y.detach().float() * 0.75, y2.detach().float()), y2.detach().float(), rtol=1e-2, atol=1e-2)
    g = torch.randn(4, 6, 5, 16, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(DEV)     # contiguous gradient
    y.backward(g)
    dropped = (y.detach() == 0) & (y2.detach() != 0)
    assert float(x.grad[dropped].abs().max()) == 0.0 if bool(dropped.any()) else True
    z = D.dropout(x.detach().requires_grad_(True), 0.5)
    zid = D._next_call_id
    assert z.stride() == x.stride()
    xin = x.detach().requires_grad_(True)
    z = D.dropout(xin, 0.5)
    z.backward(torch.ones(4, 6, 5, 16, dtype=torch.bfloat16, device=DEV))
    assert torch.equal(xin.grad != 0, z.detach() != 0) or bool((xin.detach() == 0).any())
