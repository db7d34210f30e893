"""The embedding backward kernel against torch's own gradient (the op the models look their tokens up with,
models.py:66-71): unique tokens, heavy repetition (one token at a third of the positions, chains longer than one
window of the kernel), indices in several layouts, float32 and bfloat16."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,V,E,repeat", [((256, 32), 33280, 768, 0.0), ((512, 16), 33280, 1024, 0.0), ((64, 50), 100, 64, 0.0),
                                              ((3000,), 5000, 128, 0.35), ((7, 3, 5), 11, 8, 0.0), ((1,), 9, 2048, 0.0)])
def test_embedding_backward_equals_torch(dtype, shape, V, E, repeat):
    from hap_b200.embedding import embedding
    g = torch.Generator().manual_seed(V + E)
    idx = torch.randint(0, V, shape, generator=g)
    if repeat:
        idx[torch.rand(shape, generator=g) < repeat] = 3          # one token at a third of the positions
    w = torch.randn(V, E, generator=g).to(dtype)
    gy = torch.randn(*shape, E, generator=g).to(dtype)
    wr = w.double().requires_grad_(True)
    F.embedding(idx, wr).backward(gy.double())
    wg = w.to(DEV).requires_grad_(True)
    out = embedding(idx.to(DEV), wg)
    assert torch.equal(out.detach().cpu(), F.embedding(idx, w))
    out.backward(gy.to(DEV))
    tol = dict(rtol=1e-5, atol=1e-4) if dtype == torch.float32 else dict(rtol=2 ** -7, atol=2 ** -6)
    if repeat and dtype == torch.bfloat16:
        tol = dict(rtol=2 ** -7, atol=2 ** -3)        # a row that sums a thousand gradients: one rounding of a value of order 30
    torch.testing.assert_close(wg.grad.cpu().double(), wr.grad, **tol)
    untouched = torch.ones(V, dtype=torch.bool)
    untouched[idx.reshape(-1)] = False
    assert float(wg.grad.cpu()[untouched].abs().max()) == 0.0 if bool(untouched.any()) else True
    # bit-reproducible
    wg2 = w.to(DEV).requires_grad_(True)
    embedding(idx.to(DEV), wg2).backward(gy.to(DEV))
    assert torch.equal(wg.grad, wg2.grad)


def test_embedding_falls_back_to_torch_outside_the_kernels_range():
    from hap_b200.embedding import embedding
    w = torch.randn(10, 12, device=DEV, requires_grad=True)            # rows not a multiple of 8 wide
    idx = torch.tensor([1, 2, 2, 9], device=DEV)
    embedding(idx, w).sum().backward()
    want = torch.zeros(10, 12, device=DEV)
    want[1] += 1; want[2] += 2; want[9] += 1
    assert torch.equal(w.grad, want)
    w2 = torch.randn(10, 16, device=DEV, requires_grad=True)
    out = embedding(idx, w2, padding_idx=2)                             # a padding index: torch's path
    out.sum().backward()
    assert float(w2.grad[2].abs().max()) == 0.0
