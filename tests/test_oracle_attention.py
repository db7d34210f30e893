"""Pin the attention oracle against the function the reference calls
(torch.nn.functional.multi_head_attention_forward, CPU, fp32), forward and backward."""
import pytest
import torch
import torch.nn.functional as F

from oracle import attention_math as am


@pytest.mark.parametrize("L,n,E,H,causal", [(16, 3, 32, 4, True), (10, 2, 24, 3, False), (33, 1, 64, 1, True)])
def test_oracle_matches_torch_mha(L, n, E, H, causal):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(L, n, E, generator=g, requires_grad=True)
    in_w, in_b = torch.randn(3 * E, E, generator=g) * E ** -0.5, torch.randn(3 * E, generator=g)
    out_w, out_b = torch.randn(E, E, generator=g) * E ** -0.5, torch.randn(E, generator=g)
    mask = am.causal_mask(L) if causal else None
    want, _ = F.multi_head_attention_forward(x, x, x, E, H, in_w, in_b, None, None, False, 0.0, out_w, out_b, attn_mask=mask)
    x2 = x.detach().clone().requires_grad_(True)
    got = am.multi_head_attention(x2, in_w, in_b, out_w, out_b, H, mask)
    torch.testing.assert_close(got.float(), want, rtol=1e-4, atol=1e-5)
    w = torch.randn(L, n, E, generator=g)
    (want * w).sum().backward()
    (got * w.double()).sum().backward()
    torch.testing.assert_close(x2.grad, x.grad, rtol=1e-4, atol=1e-5)
