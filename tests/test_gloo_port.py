"""World-size-2 and -4 gloo runs on CPU: the multi-process port of the reference's collectives
(the timed CPU baseline) against the single-process oracle, forward and backward, plus the
known answers of collectives.py:198-323 through a real transport."""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, store, dtype_name):
    sys.path.insert(0, ROOT)
    from oracle import collectives_math as cm
    from oracle import gloo_port as gp
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}")
    dtype = getattr(torch, dtype_name)
    L = [1, 2, 3, 4][:world] if world == 4 else [3, 2]
    tot = sum(L)

    def gen(shape, seed):
        return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).to(dtype)

    def everyone(t):
        got = [None] * world
        dist.all_gather_object(got, t)
        return got

    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for dim in (0, 1):
        shape = [4, 6]
        shape[dim] = L[rank]
        x = gen(shape, 1000 + rank)
        xs = everyone(x)
        for fn in (gp.all_gather, gp.all_gather_by_group_call):
            assert torch.equal(fn(x, dim, L, rank), cm.all_gather(xs, dim, L)[rank])
        shape[dim] = tot
        y = gen(shape, 3000 + rank)
        ys = everyone(y)
        for fn in (gp.reduce_scatter, gp.reduce_scatter_by_group_call):
            torch.testing.assert_close(fn(y, dim, L, rank), cm.reduce_scatter(ys, dim, L)[rank], **tol)
        assert torch.equal(gp.dynamic_slice(y, dim, L, rank), cm.dynamic_slice(y, dim, L, rank))
    z = gen([5, 7], 4000 + rank)
    torch.testing.assert_close(gp.all_reduce(z), cm.all_reduce(everyone(z))[rank], **tol)
    if world == 4 and dtype == torch.float32:
        # known answers, collectives.py:198-323
        p = torch.ones(5, rank + 1, requires_grad=True)
        loss = gp.all_gather(p, 1, [1, 2, 3, 4], rank).sum() / 4
        loss.backward()
        assert float(loss) == 12.5 and torch.equal(p.grad, torch.ones(5, rank + 1))
        p = (torch.ones(5, 4) * rank).requires_grad_(True)
        loss = gp.all_reduce(p).sum() / 4
        loss.backward()
        assert float(loss) == 30.0 and torch.equal(p.grad, torch.ones(5, 4))
        p = torch.ones(5, 10, requires_grad=True)
        loss = gp.reduce_scatter_by_group_call(p, 1, [1, 2, 3, 4], rank).sum()
        loss.backward()
        assert float(loss) == 20.0 * (rank + 1) and torch.equal(p.grad, torch.ones(5, 10))
        p = torch.ones(10, rank + 1, requires_grad=True)
        out = gp.all_to_all(p, 0, 1, [4, 3, 2, 1], [1, 2, 3, 4], rank)
        out.sum().backward()
        assert tuple(out.shape) == (4 - rank, 10) and torch.equal(p.grad, torch.ones(10, rank + 1))
        p = torch.ones(10, [0, 2, 0, 8][rank])
        assert tuple(gp.all_to_all(p, 0, 1, [5, 0, 5, 0], [0, 2, 0, 8], rank).shape) == ([5, 0, 5, 0][rank], 10)
        p = torch.ones(5, 5, requires_grad=True)
        loss = gp.replicate(p).sum() / 4
        loss.backward()
        assert float(loss) == 6.25 and torch.equal(p.grad, torch.ones(5, 5))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,dtype_name", [(2, "float32"), (2, "bfloat16"), (4, "float32")])
def test_gloo_port_against_oracle(world, dtype_name):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "store"), dtype_name), nprocs=world, join=True)
