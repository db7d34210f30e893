"""Fused log_softmax + summed nll_loss kernels against the reference's two ops on the CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-5)])
@pytest.mark.parametrize("rows,V", [(37, 33278), (64, 1000), (5, 7), (300, 64), (1, 33280)])
def test_matches_the_two_reference_ops(dtype, tol, rows, V):
    # the inputs are identical bf16 (or fp32) values on both sides, and both sides compute in fp32:
    # the 1e-5 of the fp32 configurations applies to either dtype
    from hap_b200.loss import nll_log_softmax_sum
    from oracle import loss_math
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(rows * 131 + V)
    logits = (torch.randn(rows, V, generator=g) * 3).to(dtype)
    targets = torch.randint(0, V, (rows,), generator=g)
    if rows > 3:
        targets[1] = -100                       # torch's ignore_index: no loss, zero gradient row
    want_in = logits.clone().requires_grad_(True)
    want = loss_math.nll_log_softmax_sum(want_in, targets)
    (want * 0.37).backward()
    got_in = logits.to(dev).requires_grad_(True)
    got = nll_log_softmax_sum(got_in, targets.to(dev))
    (got * 0.37).backward()
    assert got.dtype == torch.float32
    assert abs(float(got) - float(want)) <= tol * abs(float(want))
    assert got_in.grad.dtype == dtype
    if dtype == torch.float32:
        torch.testing.assert_close(got_in.grad.cpu(), want_in.grad, rtol=1e-4, atol=1e-7)
    else:
        # both round an fp32 gradient to bf16 once
        torch.testing.assert_close(got_in.grad.cpu().float(), want_in.grad.float(), rtol=2 ** -7, atol=1e-9)
    if rows > 3:
        assert not bool(got_in.grad[1].any())


def test_leading_dimensions_views_and_empty_input():
    from hap_b200.loss import nll_log_softmax_sum
    from oracle import loss_math
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    # (S, B, V) logits with (B, S) targets transposed, as the language-model program passes them
    logits = torch.randn(6, 4, 50, generator=g).to(torch.bfloat16)
    targets = torch.randint(0, 50, (4, 6), generator=g)
    want = loss_math.nll_log_softmax_sum(logits, targets.transpose(0, 1))
    got = nll_log_softmax_sum(logits.to(dev), targets.to(dev).transpose(0, 1))
    assert abs(float(got) - float(want)) <= 1e-5 * abs(float(want))
    # rows that are slices of a wider matrix (row pitch larger than the class count), odd base offset
    wide = torch.randn(9, 40, generator=g)
    view = wide[:, 3:36]
    t = torch.randint(0, 33, (9,), generator=g)
    a = view.to(dev)                                  # contiguous copy
    b = wide.to(dev)[:, 3:36]                         # strided view
    la, lb = nll_log_softmax_sum(a, t.to(dev)), nll_log_softmax_sum(b, t.to(dev))
    assert float(la) == float(lb)
    assert abs(float(la) - float(loss_math.nll_log_softmax_sum(view, t))) <= 1e-5 * abs(float(la))
    empty = nll_log_softmax_sum(torch.empty(0, 10, device=dev), torch.empty(0, dtype=torch.int64, device=dev))
    assert float(empty) == 0.0
