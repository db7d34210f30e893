"""Generate the golden fixtures in this directory from the reference itself.

Run once, on a machine that has the reference checkout (it is NOT needed to run
the tests):

    python tests/golden/make_golden.py --reference /path/to/hap --out tests/golden

What it does, per world size W in {2, 4}: spawns W CPU ranks on the gloo
backend, imports the reference's ``collectives.py`` UNMODIFIED from the given
checkout and runs forward + backward of every collective that backend can run,
on seeded float32 inputs.  The same cases are run through ``oracle/gloo_port.py``
and ``oracle/collectives_math.py``; the script refuses to write fixtures unless
gathers agree bit-exactly and reductions within 1e-6.  One shim is applied from
the outside: ``torch.distributed.distributed_c10d._coalescing_manager`` is
replaced by a ``(group, reqs)`` context manager that only yields, because the
reference targets torch 1.13's signature (``collectives.py:42,58,113,132``).

The reference's ``all_to_all`` cannot run on gloo ("Backend gloo does not
support alltoall"); its cases are produced by the port only and are pinned by
the shapes and sums stated in ``collectives.py:288-308`` (see
``tests/test_oracle_golden.py``).

Inputs: rank r draws ``x`` from ``torch.Generator().manual_seed(1000 + r)`` and
the loss weights from ``manual_seed(2000 + r)``; loss = ``(out * w).sum()``.
"""
from __future__ import annotations

import argparse
import contextlib
import importlib.util
import os
import sys
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# (name, op, shape builder, args builder).  L = sharding lengths.
LENGTHS = {2: [[3, 2], [1, 4]], 4: [[1, 2, 3, 4], [3, 0, 2, 5]]}


def randn(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def cases(world):
    out = []
    for li, L in enumerate(LENGTHS[world]):
        tot = sum(L)
        for dim in (0, 1, 2):
            def shard_shape(rank, dim=dim, L=L):
                s = [4, 5, 3]
                s[dim] = L[rank]
                return s

            def full_shape(rank, dim=dim, tot=tot):
                s = [4, 5, 3]
                s[dim] = tot
                return s
            tag = f"L{li}_d{dim}"
            out.append((f"all_gather_{tag}", "all_gather", shard_shape, (dim, L)))
            out.append((f"all_gather_by_group_call_{tag}", "all_gather_by_group_call", shard_shape, (dim, L)))
            out.append((f"reduce_scatter_{tag}", "reduce_scatter", full_shape, (dim, L)))
            out.append((f"reduce_scatter_by_group_call_{tag}", "reduce_scatter_by_group_call", full_shape, (dim, L)))
            out.append((f"dynamic_slice_{tag}", "dynamic_slice", full_shape, (dim, L)))
    out.append(("all_reduce", "all_reduce", lambda rank: [6, 7], ()))
    out.append(("replicate", "replicate", lambda rank: [6, 7], ()))
    # all_to_all: rank holds cat_L[rank] on cat_dim and sum(split_L) on split_dim
    for li, (sl, cl) in enumerate({2: [([3, 2], [1, 4])], 4: [([4, 3, 2, 1], [1, 2, 3, 4]), ([5, 0, 5, 0], [0, 2, 0, 8])]}[world]):
        for (sd, cd) in ((0, 1), (1, 0), (2, 0), (1, 2)):
            def shape(rank, sd=sd, cd=cd, sl=sl, cl=cl):
                s = [3, 3, 3]
                s[sd] = sum(sl)
                s[cd] = cl[rank]
                return s
            out.append((f"all_to_all_L{li}_s{sd}_c{cd}", "all_to_all", shape, (sd, cd, sl, cl)))
    return out


def load_reference(path):
    spec = importlib.util.spec_from_file_location("ref_collectives", os.path.join(path, "collectives.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@contextlib.contextmanager
def _legacy_coalescing_manager(group, reqs):
    yield


def run_one(mod, opname, x, args, rank, w=None):
    x = x.clone().requires_grad_(True)
    fn = getattr(mod, opname)
    if opname in ("all_reduce", "replicate"):
        out = fn(x)
    elif opname == "all_to_all":
        out = fn(x, *args, rank)
    else:
        out = fn(x, args[0], list(args[1]), rank)
    if w is None:
        w = randn(out.shape, 2000 + rank) if out.numel() else torch.zeros(out.shape)
    (out * w).sum().backward()
    return out.detach().clone(), x.grad.detach().clone(), w


def worker(rank, world, ref_path, store_path, out_dir):
    sys.path.insert(0, ROOT)
    from oracle import gloo_port
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store_path}")
    dist.distributed_c10d._coalescing_manager = _legacy_coalescing_manager
    ref = load_reference(ref_path)
    record = {}
    for name, opname, shape_fn, args in cases(world):
        x = randn(shape_fn(rank), 1000 + rank)
        port_out, port_grad, w = run_one(gloo_port, opname, x, args, rank)
        entry = {"op": opname, "args": args, "x": x, "w": w, "source": "port"}
        if opname != "all_to_all":
            ref_out, ref_grad, _ = run_one(ref, opname, x, args, rank, w)
            exact = opname.startswith("all_gather") or opname == "dynamic_slice"
            for a, b, what in ((ref_out, port_out, "out"), (ref_grad, port_grad, "grad")):
                assert a.shape == b.shape, (name, what, a.shape, b.shape)
                if exact and what == "out":
                    assert torch.equal(a, b), (name, what)
                else:
                    torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-6)
            entry.update(out=ref_out, grad=ref_grad, source="reference")
        else:
            entry.update(out=port_out, grad=port_grad)
        record[name] = entry
    gathered = [None] * world
    dist.all_gather_object(gathered, record)
    if rank == 0:
        from oracle import collectives_math as cm
        for name in record:
            per_rank = [g[name] for g in gathered]
            op, args = per_rank[0]["op"], per_rank[0]["args"]
            xs = [p["x"] for p in per_rank]
            if op.startswith("all_gather"):
                want = cm.all_gather(xs, *args)
            elif op.startswith("reduce_scatter"):
                want = cm.reduce_scatter(xs, *args)
            elif op == "all_reduce":
                want = cm.all_reduce(xs)
            elif op == "replicate":
                want = xs
            elif op == "dynamic_slice":
                want = [cm.dynamic_slice(xs[r], args[0], args[1], r) for r in range(world)]
            else:
                want = cm.all_to_all(xs, *args)
            for r in range(world):
                torch.testing.assert_close(per_rank[r]["out"], want[r], rtol=1e-6, atol=1e-6)
        torch.save({"world": world, "cases": {n: [g[n] for g in gathered] for n in record}},
                   os.path.join(out_dir, f"collectives_w{world}.pt"))
        print(f"wrote collectives_w{world}.pt with {len(record)} cases")
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    for world in (2, 4):
        with tempfile.TemporaryDirectory() as d:
            mp.spawn(worker, args=(world, a.reference, os.path.join(d, "store"), a.out), nprocs=world, join=True)


if __name__ == "__main__":
    main()
