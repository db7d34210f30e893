"""MoE einsums (dispatch, two expert FFN contractions, combine) on the batched tensor-core GEMM
against float64 torch.einsum, forward and backward; shapes follow the MoE configuration
(capacity 20, d_model 1024, expert FFN 4096) at reduced batch / expert counts, including the
uneven per-GPU expert counts [7, 3, 2]."""
import pytest
import torch

import hap_b200
from hap_b200.einsum import einsum
from oracle.einsum_math import einsum as oracle_einsum

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, want, what, tol=1e-2):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    rms = float(want.pow(2).mean().sqrt()) + 1e-30
    assert float((got - want).norm()) <= tol * float(want.norm()) + 1e-30, f"{what}: relative error {float((got - want).norm() / want.norm()):.3g}"
    excess = (got - want).abs() - 4 * tol * (want.abs() + rms)
    assert float(excess.max()) <= 0, f"{what}: {int((excess > 0).sum())} entries off (rms {rms:.3g})"


def run(code, a, b, grad_a=True, grad_b=True):
    ra, rb = a.double().requires_grad_(grad_a), b.double().requires_grad_(grad_b)
    want = oracle_einsum(code, ra, rb)
    g = torch.randn(want.shape, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    (want * g.double()).sum().backward()
    da, db = a.to(DEV).requires_grad_(grad_a), b.to(DEV).requires_grad_(grad_b)
    got = einsum(code, da, db)
    (got * g.to(DEV)).sum().backward()
    hap_b200.linear_ops.gemm_status()
    close(got, want, code)
    if grad_a:
        close(da.grad, ra.grad, code + " grad a", 2e-2)
    if grad_b:
        close(db.grad, rb.grad, code + " grad b", 2e-2)


def gen(shape, seed, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("b,s,e,c,d", [(4, 64, 4, 8, 64), (3, 512, 32, 20, 128), (2, 128, 8, 20, 1024)])
def test_dispatch_and_combine(b, s, e, c, d):
    x = gen((b, s, d), 1)
    disp = (torch.rand(b, s, e, c, generator=torch.Generator().manual_seed(2)) < 0.05).to(torch.bfloat16)
    run("bsd,bsec->becd", x, disp, grad_b=False)
    eo = gen((b, e, c, d), 3)
    comb = (torch.rand(b, s, e, c, generator=torch.Generator().manual_seed(4)) * disp.float()).to(torch.bfloat16)
    run("becd,bsec->bsd", eo, comb)


@pytest.mark.parametrize("b,e,c,d,h", [(4, 4, 8, 64, 128), (16, 7, 20, 256, 512), (16, 3, 20, 1024, 4096), (8, 2, 20, 1024, 4096)])
def test_expert_ffn(b, e, c, d, h):
    w1 = gen((e, d, h), 5, d ** -0.5)
    inp = gen((b, e, c, d), 6)
    run("edh,becd->bech", w1, inp)
    w2 = gen((e, h, d), 7, h ** -0.5)
    hid = gen((b, e, c, h), 8)
    run("ehd,bech->becd", w2, hid)


def test_moe_block_chain_matches_oracle():
    """dispatch -> FFN1 -> relu -> FFN2 -> combine, as in models.py:356-364, through views."""
    b, s, e, c, d, h = 4, 128, 4, 20, 128, 256
    x, w1, w2 = gen((b, s, d), 1), gen((e, d, h), 2, d ** -0.5), gen((e, h, d), 3, h ** -0.5)
    disp = (torch.rand(b, s, e, c, generator=torch.Generator().manual_seed(4)) < 0.05).to(torch.bfloat16)
    comb = (disp.float() * 0.5).to(torch.bfloat16)

    def block(f, x, w1, w2, disp, comb):
        ei = f("bsd,bsec->becd", x, disp)
        hh = torch.relu(f("edh,becd->bech", w1, ei))
        eo = f("ehd,bech->becd", w2, hh)
        return f("becd,bsec->bsd", eo, comb)

    want = block(oracle_einsum, x, w1, w2, disp, comb)
    got = block(einsum, x.to(DEV), w1.to(DEV), w2.to(DEV), disp.to(DEV), comb.to(DEV))
    close(got, want, "moe block", 3e-2)


def test_unsupported_code_raises():
    with pytest.raises(NotImplementedError):
        einsum("ab,bc->ac", torch.ones(8, 8, device=DEV, dtype=torch.bfloat16), torch.ones(8, 8, device=DEV, dtype=torch.bfloat16))


@pytest.mark.parametrize("b,s,e,c,d", [(2, 64, 4, 20, 64), (3, 96, 32, 20, 1024), (1, 17, 5, 6, 8)])
def test_sparse_dispatch_and_combine_equal_the_dense_einsums(b, s, e, c, d):
    """Gating-shaped dispatch / combine tensors (at most one token per slot, two slots per token) through the
    gather kernels against float64 einsums; dispatch is exact (a pure row move)."""
    from hap_b200.einsum import sparse_combine, sparse_dispatch
    from hap_b200.plan import top2_gating
    g = torch.Generator().manual_seed(b * 1000 + s)
    x = torch.randn(b, s, d, generator=g).to(torch.bfloat16)
    gate_w = (torch.randn(d, e, generator=g) * d ** -0.5).to(torch.bfloat16)
    disp, comb = top2_gating(x, gate_w, e, c)
    assert int((disp.sum(dim=1) > 1).sum()) == 0 and int((disp.flatten(2).sum(dim=2) > 2).sum()) == 0
    xd = x.to(DEV).requires_grad_(True)
    got = sparse_dispatch(xd, disp.to(DEV))
    want = torch.einsum("bsd,bsec->becd", x.double(), disp.double())
    assert torch.equal(got.detach().cpu().double(), want)
    w1 = torch.randn(b, e, c, d, generator=g).to(torch.bfloat16)
    got.backward(w1.to(DEV))
    want_dx = torch.einsum("becd,bsec->bsd", w1.double(), disp.double())
    torch.testing.assert_close(xd.grad.cpu().double(), want_dx, rtol=1e-2, atol=1e-2)
    eo = torch.randn(b, e, c, d, generator=g).to(torch.bfloat16)
    eod, combd = eo.to(DEV).requires_grad_(True), comb.to(DEV).requires_grad_(True)
    y = sparse_combine(eod, combd)
    ref_eo, ref_comb = eo.double().requires_grad_(True), comb.double().requires_grad_(True)
    ref = torch.einsum("becd,bsec->bsd", ref_eo, ref_comb)
    torch.testing.assert_close(y.detach().cpu().double(), ref.detach(), rtol=1e-2, atol=1e-2)
    gy = torch.randn(b, s, d, generator=g).to(torch.bfloat16)
    y.backward(gy.to(DEV))
    ref.backward(gy.double())
    torch.testing.assert_close(eod.grad.cpu().double(), ref_eo.grad, rtol=1e-2, atol=1e-2)
    # the gradient of the combine weights where the gating function reads it: at the non-zero positions
    nz = comb != 0
    torch.testing.assert_close(combd.grad.cpu().double()[nz], ref_comb.grad[nz], rtol=2e-2, atol=2e-2 * float(ref_comb.grad[nz].abs().max()))
    assert float(combd.grad.cpu()[~nz].abs().max()) == 0.0


@pytest.mark.parametrize("b,s,e,c,d", [(3, 96, 8, 20, 256), (2, 40, 5, 6, 64)])
def test_sparse_gathers_work_in_the_neighbours_layouts(b, s, e, c, d):
    """No copy between the gathers and their neighbours: tokens as a (b, s, d) view of sequence-major memory, rows in
    the expert-major memory the expert contractions use; values and gradients equal the batch-major call's, and the
    gradients come out in the layout of the tensors they belong to."""
    from hap_b200.einsum import sparse_combine, sparse_dispatch
    from hap_b200.plan import top2_gating
    g = torch.Generator().manual_seed(b * 77 + s)
    x_sb = torch.randn(s, b, d, generator=g).to(torch.bfloat16).to(DEV)             # sequence-major memory
    gate_w = (torch.randn(d, e, generator=g) * d ** -0.5).to(torch.bfloat16).to(DEV)
    x_view = x_sb.transpose(0, 1).requires_grad_(True)                               # (b, s, d) view
    x_flat = x_sb.transpose(0, 1).contiguous().requires_grad_(True)
    disp, comb = top2_gating(x_flat.detach(), gate_w, e, c)
    plain = sparse_dispatch(x_flat, disp)
    major = sparse_dispatch(x_view, disp, expert_major=True)
    assert plain.is_contiguous() and major.permute(1, 0, 2, 3).is_contiguous() and torch.equal(plain, major)
    w = torch.randn(e, b, c, d, generator=g).to(torch.bfloat16).to(DEV).permute(1, 0, 2, 3)   # a gradient in expert-major memory
    plain.backward(w.contiguous())
    major.backward(w)
    assert torch.equal(x_flat.grad, x_view.grad) and x_view.grad.stride() == x_view.stride()
    eo_major = torch.randn(e, b, c, d, generator=g).to(torch.bfloat16).to(DEV).permute(1, 0, 2, 3).requires_grad_(True)
    eo_plain = eo_major.detach().contiguous().requires_grad_(True)
    comb_a, comb_b = comb.detach().requires_grad_(True), comb.detach().requires_grad_(True)
    y_a, y_b = sparse_combine(eo_plain, comb_a), sparse_combine(eo_major, comb_b)
    assert torch.equal(y_a, y_b)
    gy = torch.randn(s, b, d, generator=g).to(torch.bfloat16).to(DEV).transpose(0, 1)          # sequence-major gradient
    y_a.backward(gy.contiguous())
    y_b.backward(gy)
    assert torch.equal(eo_plain.grad, eo_major.grad) and eo_major.grad.permute(1, 0, 2, 3).is_contiguous()
    assert torch.equal(comb_a.grad, comb_b.grad)
    # the combine written in sequence-major order, for a program that transposes it right away
    y_c = sparse_combine(eo_major.detach(), comb.detach(), sequence_major=True)
    assert y_c.transpose(0, 1).is_contiguous() and torch.equal(y_c, y_a.detach())
