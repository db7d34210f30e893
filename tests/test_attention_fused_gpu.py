"""The fused attention kernels (head dimension 64) against the float64 oracle.

Without dropout: output and input gradient at the head shapes of the Transformer-LM (L 256, causal), ViT
(L 197, no mask, ragged tiles) and MoE (L 512, causal) configurations and at odd lengths, with the mask
given as the built-in causal rule, as the -inf tensor of the reference's language model, and as an
arbitrary additive tensor.  With dropout the random mask cannot match torch's generator, so parity is
checked GIVEN the mask: the library exports the keep mask a call draws and the oracle applies it to the
probabilities; forward and backward must both agree with that, which also shows that the two backward
kernels regenerate the mask the forward kernel used.  bf16 tolerance: 1e-2 (2e-2 for gradients) relative
error of the whole tensor and 4x that per entry relative to (|value| + rms)."""
import pytest
import torch

import hap_b200
from hap_b200 import attention as A
from hap_b200 import dropout as D
from oracle import attention_math as am

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, want, what, tol=1e-2):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float(want.pow(2).mean().sqrt()) + 1e-30
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    assert float((got - want).norm()) <= tol * float(want.norm()), f"{what}: relative error {float((got - want).norm() / want.norm()):.3g}"
    excess = (got - want).abs() - 4 * tol * (want.abs() + rms)
    assert float(excess.max()) <= 0, f"{what}: {int((excess > 0).sum())} entries off by up to {float(excess.max()):.3g} (rms {rms:.3g})"


def run_case(L, n, H, mask_kind, p=0.0, seed=11):
    E = H * 64
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(L, n, 3 * E, generator=g).to(torch.bfloat16)
    w = torch.randn(L, n, E, generator=g).to(torch.bfloat16)
    if mask_kind == "none":
        mask_cpu, mask_arg = None, None
    elif mask_kind == "causal":
        mask_cpu, mask_arg = am.causal_mask(L), "causal"
    elif mask_kind == "causal_tensor":
        mask_cpu = am.causal_mask(L)
        mask_arg = mask_cpu.to(DEV)
    else:
        mask_cpu = torch.randn(L, L, generator=g)
        mask_cpu[:, 3] = float("-inf")
        mask_cpu[:, L // 2:L // 2 + 5] = float("-inf")
        mask_arg = mask_cpu.to(DEV)
    x = qkv.to(DEV).requires_grad_(True)
    keep = None
    if p > 0.0:
        D.manual_seed(4321 + seed, DEV)
        D.advance(DEV)
    got = A.attention(x, H, mask_arg, dropout_p=p)
    if p > 0.0:
        call_id = D._next_call_id
        keep = A.attention_keep_mask(L, n, H, p, call_id, DEV).cpu().reshape(n, H, L, L)
    (got * w.to(DEV)).sum().backward()
    hap_b200.linear_ops.gemm_status()
    ref_in = qkv.double().requires_grad_(True)
    want = am.attention_core(ref_in, H, mask_cpu, keep, p)
    (want * w.double()).sum().backward()
    close(got, want, f"output L={L} {mask_kind} p={p}")
    close(x.grad, ref_in.grad, f"dqkv L={L} {mask_kind} p={p}", tol=2e-2)
    return got.detach(), x.grad.detach(), keep


@pytest.mark.parametrize("L,n,H,mask_kind", [
    (256, 4, 12, "causal"), (197, 3, 12, "none"), (512, 2, 16, "causal"),      # LM, ViT, MoE head shapes
    (16, 2, 2, "none"), (130, 2, 3, "causal"), (129, 1, 1, "none"), (300, 1, 2, "causal"), (128, 3, 1, "causal"),
    (256, 2, 2, "causal_tensor"), (200, 2, 2, "general"), (384, 1, 2, "general"),
])
def test_forward_backward_without_dropout(L, n, H, mask_kind):
    run_case(L, n, H, mask_kind)


def test_causal_rule_and_causal_tensor_give_the_same_bits():
    a, ga, _ = run_case(256, 2, 3, "causal")
    b, gb, _ = run_case(256, 2, 3, "causal_tensor")
    assert torch.equal(a, b) and torch.equal(ga, gb)


@pytest.mark.parametrize("L,n,H,mask_kind,p", [(256, 2, 12, "causal", 0.1), (197, 2, 4, "none", 0.1), (512, 1, 3, "causal", 0.25),
                                               (72, 2, 2, "general", 0.5)])
def test_forward_backward_given_the_dropout_mask(L, n, H, mask_kind, p):
    _, _, keep = run_case(L, n, H, mask_kind, p)
    rate = float(keep.float().mean())
    count = keep.numel()
    assert abs(rate - (1 - p)) < 5 * (p * (1 - p) / count) ** 0.5 + 1e-4, rate


def test_results_are_reproducible_bit_for_bit():
    a, ga, _ = run_case(256, 3, 4, "causal", 0.1, seed=5)
    b, gb, _ = run_case(256, 3, 4, "causal", 0.1, seed=5)
    assert torch.equal(a, b) and torch.equal(ga, gb)


def test_a_new_iteration_draws_a_new_mask():
    L, n, H = 128, 1, 2
    qkv = torch.randn(L, n, 3 * H * 64, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    D.manual_seed(77, DEV)
    D.advance(DEV)
    a = A.attention(qkv, H, None, dropout_p=0.3)
    D.advance(DEV)
    b = A.attention(qkv, H, None, dropout_p=0.3)
    assert not torch.equal(a, b)
