"""Pin the CPU oracle: against outputs of the reference's own collectives.py (golden files made
by tests/golden/make_golden.py) and against the known answers written as comments in the
reference's manual test (collectives.py:198-323)."""
import pytest
import torch

from oracle import collectives_math as cm
from tests.helpers import exact_op, load_golden, oracle_backward, oracle_forward


@pytest.mark.parametrize("world", [2, 4])
def test_oracle_matches_reference_outputs(world):
    data = load_golden(world)
    assert data["world"] == world
    n_ref = 0
    for name, per_rank in data["cases"].items():
        op, args = per_rank[0]["op"], per_rank[0]["args"]
        xs = [p["x"] for p in per_rank]
        ws = [p["w"] for p in per_rank]
        outs = oracle_forward(op, xs, args)
        grads = oracle_backward(op, xs, ws, args)
        for r in range(world):
            want_out, want_grad = per_rank[r]["out"], per_rank[r]["grad"]
            assert outs[r].shape == want_out.shape, name
            if exact_op(op):
                assert torch.equal(outs[r], want_out), name
            else:
                torch.testing.assert_close(outs[r], want_out, rtol=1e-5, atol=1e-6)
            torch.testing.assert_close(grads[r], want_grad, rtol=1e-5, atol=1e-6)
        n_ref += per_rank[0]["source"] == "reference"
    assert n_ref >= 30  # everything but all_to_all comes from the reference itself


L = [1, 2, 3, 4]


def test_known_answers_all_gather():
    # collectives.py:198, 213: ones(5, rank+1) gathered on dim 1, .sum()/4 -> 12.5 on every rank, grads all 1
    outs = cm.all_gather([torch.ones(5, r + 1) for r in range(4)], 1, L)
    assert [float(o.sum() / 4) for o in outs] == [12.5] * 4
    grads = cm.all_gather_backward([torch.full((5, 10), 0.25) for _ in range(4)], 1, L)
    for r in range(4):
        assert torch.equal(grads[r], torch.ones(5, r + 1))


def test_known_answers_all_reduce():
    # collectives.py:228: ones(5,4)*rank summed -> every element 6, .sum()/4 = 30; grads all 1
    outs = cm.all_reduce([torch.ones(5, 4) * r for r in range(4)])
    assert [float(o.sum() / 4) for o in outs] == [30.0] * 4
    grads = cm.all_reduce([torch.full((5, 4), 0.25) for _ in range(4)])
    assert all(torch.equal(g, torch.ones(5, 4)) for g in grads)


def test_known_answers_reduce_scatter():
    # collectives.py:243, 258: ones(5,10) reduce-scattered on dim 1 -> loss 20*(rank+1); grads all 1
    outs = cm.reduce_scatter([torch.ones(5, 10) for _ in range(4)], 1, L)
    assert [float(o.sum()) for o in outs] == [20.0 * (r + 1) for r in range(4)]
    grads = cm.reduce_scatter_backward([torch.ones(5, r + 1) for r in range(4)], 1, L)
    assert all(torch.equal(g, torch.ones(5, 10)) for g in grads)


def test_known_answers_dynamic_slice():
    # collectives.py:273: loss 5*(rank+1); grad 1 inside the own slice, 0 elsewhere
    for r in range(4):
        out = cm.dynamic_slice(torch.ones(5, 10), 1, L, r)
        assert float(out.sum()) == 5.0 * (r + 1)
        g = cm.dynamic_slice_backward(torch.ones(5, r + 1), (5, 10), 1, L, r)
        assert float(g.sum()) == 5.0 * (r + 1)
        assert torch.equal(g[:, sum(L[:r]):sum(L[:r + 1])], torch.ones(5, r + 1))


def test_known_answers_all_to_all():
    # collectives.py:288: ones(10, rank+1), split 0 by [4,3,2,1], cat 1 by [1,2,3,4] -> (4-rank, 10), loss 10*(4-rank)
    outs = cm.all_to_all([torch.ones(10, r + 1) for r in range(4)], 0, 1, [4, 3, 2, 1], L)
    assert [tuple(o.shape) for o in outs] == [(4 - r, 10) for r in range(4)]
    assert [float(o.sum()) for o in outs] == [10.0 * (4 - r) for r in range(4)]
    grads = cm.all_to_all_backward([torch.ones(4 - r, 10) for r in range(4)], 0, 1, [4, 3, 2, 1], L)
    assert all(torch.equal(g, torch.ones(10, r + 1)) for r, g in enumerate(grads))


def test_known_answers_all_to_all_zero_lengths():
    # collectives.py:300-308: shapes only
    cat = [0, 2, 0, 8]
    outs = cm.all_to_all([torch.ones(10, cat[r]) for r in range(4)], 0, 1, [5, 0, 5, 0], cat)
    assert [tuple(o.shape) for o in outs] == [(5, 10), (0, 10), (5, 10), (0, 10)]


def test_known_answers_replicate():
    # collectives.py:317: identity forward (sum/4 = 6.25), gradient all-reduce backward -> all 1
    assert float(torch.ones(5, 5).sum() / 4) == 6.25
    grads = cm.all_reduce([torch.full((5, 5), 0.25) for _ in range(4)])
    assert all(torch.equal(g, torch.ones(5, 5)) for g in grads)
