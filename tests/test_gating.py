"""``plan.top2_gating`` against the reference's own ``_top_2_gating`` (``models.py:477-502``).

The fixture ``tests/golden/gating.pt`` was produced by ``tests/golden/make_gating_golden.py``, which
imports the reference's ``models.py`` unmodified.  Dispatch must agree entry for entry, combine to
1e-6 (both sides compute the softmax in float32)."""
import os

import pytest
import torch

from hap_b200.plan import top2_gating

GOLDEN = torch.load(os.path.join(os.path.dirname(__file__), "golden", "gating.pt"))


def _dense(shape, idx, values=None):
    t = torch.zeros(shape)
    t[tuple(idx.long().t())] = 1.0 if values is None else values
    return t


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_top2_gating_matches_reference(name):
    case = GOLDEN[name]
    dispatch, combine = top2_gating(case["x"], case["gate_weight"], case["n_expert"], case["capacity"])
    want_dispatch = _dense(case["shape"], case["dispatch_nonzero"])
    want_combine = _dense(case["shape"], case["combine_nonzero"], case["combine_values"])
    assert tuple(dispatch.shape) == tuple(case["shape"])
    assert torch.equal(dispatch, want_dispatch)
    torch.testing.assert_close(combine, want_combine, rtol=1e-6, atol=1e-6)


def test_fixture_covers_the_second_choice_offset():
    """At least one case must drop a second choice that a count-based offset would have kept."""
    case = GOLDEN["second_choice_offset"]
    x, w, e, c = case["x"], case["gate_weight"], case["n_expert"], case["capacity"]
    gates = torch.softmax(x @ w, dim=2)
    top_i = torch.topk(gates, 2, dim=2)[1]
    chosen = torch.nn.functional.one_hot(top_i, e)
    first, second = chosen[:, :, 0, :], chosen[:, :, 1, :]
    by_count = (torch.cumsum(second, 1) + first.sum(1, keepdim=True)) * second
    kept_by_count = int(((by_count > 0) & (by_count < c)).sum()) + int((((torch.cumsum(first, 1) * first) > 0) & ((torch.cumsum(first, 1) * first) < c)).sum())
    assert kept_by_count > case["dispatch_nonzero"].shape[0]


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_top2_gating_on_a_view_of_sequence_first_memory(name):
    """The MoE program is sequence-first: the gating function sees a (b, s, d) view of (s, b, d) memory.  Same
    outputs and the same gradient of the gate weights and of x as with a contiguous tensor."""
    case = GOLDEN[name]
    x = case["x"]
    x_a = x.clone().requires_grad_(True)
    w_a = case["gate_weight"].clone().requires_grad_(True)
    base = x.transpose(0, 1).contiguous().requires_grad_(True)            # (s, b, d) memory
    w_b = case["gate_weight"].clone().requires_grad_(True)
    d_a, c_a = top2_gating(x_a, w_a, case["n_expert"], case["capacity"])
    d_b, c_b = top2_gating(base.transpose(0, 1), w_b, case["n_expert"], case["capacity"])
    assert torch.equal(d_a, d_b) and torch.equal(c_a, c_b)
    probe = torch.randn(c_a.shape, generator=torch.Generator().manual_seed(5))
    (c_a * probe).sum().backward()
    (c_b * probe).sum().backward()
    # the products sum over (b, s) in a different order: float32 rounding apart
    torch.testing.assert_close(w_a.grad, w_b.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x_a.grad, base.grad.transpose(0, 1), rtol=1e-4, atol=1e-6)
