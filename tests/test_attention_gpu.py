"""Self-attention on the GPU path against the float64 oracle: the shapes of the Transformer-LM
(L 256, 12 heads of 64, causal), ViT (L 197, no mask) and MoE (L 512, 16 heads) configurations at
reduced batch, forward and backward.  bf16 tolerance: 1e-2 of (|value| + rms), and 1e-2 relative
error of the whole tensor."""
import pytest
import torch

import hap_b200
from hap_b200 import attention as A
from oracle import attention_math as am

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, want, what, tol=1e-2):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float(want.pow(2).mean().sqrt()) + 1e-30
    assert float((got - want).norm()) <= tol * float(want.norm()), f"{what}: relative error {float((got - want).norm() / want.norm()):.3g}"
    excess = (got - want).abs() - 4 * tol * (want.abs() + rms)
    assert float(excess.max()) <= 0, f"{what}: {int((excess > 0).sum())} entries off by up to {float(excess.max()):.3g} (rms {rms:.3g})"


@pytest.mark.parametrize("L,n,H,D,causal", [(256, 4, 12, 64, True), (197, 3, 12, 64, False), (512, 2, 16, 64, True),
                                             (64, 2, 2, 32, True), (40, 1, 3, 16, False)])
def test_attention_core_forward_backward(L, n, H, D, causal):
    E = H * D
    g = torch.Generator().manual_seed(11)
    qkv = (torch.randn(L, n, 3 * E, generator=g)).to(torch.bfloat16)
    w = torch.randn(L, n, E, generator=g).to(torch.bfloat16)
    mask = am.causal_mask(L) if causal else None
    ref_in = qkv.double().requires_grad_(True)
    want = am.attention_core(ref_in, H, mask)
    (want * w.double()).sum().backward()
    x = qkv.to(DEV).requires_grad_(True)
    got = A.attention(x, H, mask.to(DEV) if causal else None)
    (got * w.to(DEV)).sum().backward()
    hap_b200.linear_ops.gemm_status()
    close(got, want, "attention output")
    close(x.grad, ref_in.grad, "attention dqkv", tol=2e-2)
    if causal:      # the built-in causal masking gives the same bits as the -inf mask tensor
        assert torch.equal(A.attention(x.detach(), H, "causal"), got.detach())


def test_general_additive_mask():
    L, n, H, D = 48, 2, 2, 32
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(L, n, 3 * H * D, generator=g).to(torch.bfloat16)
    mask = torch.randn(L, L, generator=g)
    mask[:, 5] = float("-inf")
    want = am.attention_core(qkv, H, mask)
    got = A.attention(qkv.to(DEV), H, mask.to(DEV))
    close(got, want, "masked attention")


def test_multi_head_attention_forward_drop_in():
    L, n, E, H = 128, 3, 256, 4
    g = torch.Generator().manual_seed(7)
    x = torch.randn(L, n, E, generator=g).to(torch.bfloat16)
    in_w, in_b = (torch.randn(3 * E, E, generator=g) * E ** -0.5).to(torch.bfloat16), torch.randn(3 * E, generator=g).to(torch.bfloat16)
    out_w, out_b = (torch.randn(E, E, generator=g) * E ** -0.5).to(torch.bfloat16), torch.randn(E, generator=g).to(torch.bfloat16)
    mask = am.causal_mask(L)
    want = am.multi_head_attention(x, in_w, in_b, out_w, out_b, H, mask)
    xd = x.to(DEV)
    got, weights = A.multi_head_attention_forward(query=xd, key=xd, value=xd, embed_dim_to_check=E, num_heads=H,
                                                  in_proj_weight=in_w.to(DEV), in_proj_bias=in_b.to(DEV), bias_k=None, bias_v=None,
                                                  add_zero_attn=False, dropout_p=0.0, out_proj_weight=out_w.to(DEV),
                                                  out_proj_bias=out_b.to(DEV), attn_mask=mask.to(DEV))
    assert weights is None
    close(got, want, "mha", tol=2e-2)
    # head dimension 64 has the fused kernels with dropout; other head dimensions refuse it
    dropped, _ = A.multi_head_attention_forward(xd, xd, xd, E, H, in_w.to(DEV), in_b.to(DEV), dropout_p=0.1, out_proj_weight=out_w.to(DEV),
                                                out_proj_bias=out_b.to(DEV))
    assert dropped.shape == got.shape and not torch.equal(dropped, got)
    same, _ = A.multi_head_attention_forward(xd, xd, xd, E, H, in_w.to(DEV), in_b.to(DEV), dropout_p=0.1, out_proj_weight=out_w.to(DEV),
                                             out_proj_bias=out_b.to(DEV), training=False, attn_mask=mask.to(DEV))
    assert torch.equal(same, got)
    with pytest.raises(NotImplementedError):
        A.multi_head_attention_forward(xd, xd, xd, E, 8, in_w.to(DEV), in_b.to(DEV), dropout_p=0.1, out_proj_weight=out_w.to(DEV),
                                       out_proj_bias=out_b.to(DEV))


def test_empty_batch_shard():
    """sharding_round can hand a rank zero samples; every op must then produce empty tensors."""
    qkv = torch.zeros(16, 0, 3 * 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = A.attention(qkv, 2, "causal")
    assert out.shape == (16, 0, 64)
    out.sum().backward()
    assert qkv.grad.shape == qkv.shape
    x = torch.zeros(0, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(32, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = hap_b200.linear(x, w, None)
    assert y.shape == (0, 32)
    y.sum().backward()
    assert float(w.grad.abs().sum()) == 0.0 and x.grad.shape == (0, 64)
