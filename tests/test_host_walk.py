"""Index arithmetic of the pull kernels, checked on the CPU.

hapx_debug_host_walk runs the same segment builder and tile decoder the kernels use over
host buffers, bounds-checking every byte range.  Here its result must equal the oracle and
cover every output byte exactly once, for gathers, slices and all-to-all on awkward shapes."""
import ctypes as C
import random

import numpy as np
import pytest
import torch

from hap_b200 import _native as N
from oracle import collectives_math as cm

OP_GATHER, OP_EXCHANGE, OP_SLICE, OP_UNSLICE = 0, 1, 2, 3
NP = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}


def prod(xs):
    out = 1
    for x in xs:
        out *= int(x)
    return out


def walk(op, world, rank, es, a, b, c, split_first, l1, l2, srcs, dst_shape):
    dst = np.zeros(dst_shape, dtype=NP[es])
    cover = np.zeros(dst.nbytes, dtype=np.uint8)
    keep = [np.ascontiguousarray(s) for s in srcs]
    ptrs = N.ptr_array([k.ctypes.data if k.size else 0 for k in keep])
    sizes = (C.c_size_t * world)(*[k.nbytes for k in keep])
    rc = N.lib.hapx_debug_host_walk(op, world, rank, es, a, b, c, split_first, N.i64_array(l1),
                                    N.i64_array(l2) if l2 is not None else None, ptrs, sizes,
                                    dst.ctypes.data if dst.size else None, dst.nbytes,
                                    cover.ctypes.data if dst.size else None)
    assert rc == 0, N.lib.hapx_last_error()
    return dst, cover


def rand(shape, es, rng):
    return rng.integers(1, np.iinfo(NP[es]).max, size=shape, dtype=NP[es])


def to_t(x):
    return torch.from_numpy(x.astype(np.int64))


@pytest.mark.parametrize("es", [1, 2, 4, 8])
@pytest.mark.parametrize("world,lengths", [(2, [3, 2]), (4, [1, 2, 3, 4]), (4, [3, 0, 2, 5]), (8, [56, 46, 39, 33, 28, 23, 18, 13]),
                                           (3, [700, 1, 333])])
def test_gather_and_slice_geometry(es, world, lengths):
    rng = np.random.default_rng(es * 100 + world)
    for shape, dim in (((5, 0, 3), 1), ((0, 7), 0), ((1, 0, 129), 1), ((3, 4, 0), 2), ((2, 0, 1, 5), 1)):
        base = list(shape)
        shards = []
        for r in range(world):
            s = list(base)
            s[dim] = lengths[r]
            shards.append(rand(s, es, rng))
        full_shape = list(base)
        full_shape[dim] = sum(lengths)
        want = np.concatenate(shards, axis=dim)
        outer, inner = prod(base[:dim]), prod(base[dim + 1:])
        for r in range(world):
            got, cover = walk(OP_GATHER, world, r, es, outer, 0, inner, 0, lengths, None, shards, full_shape)
            assert np.array_equal(got, want)
            assert np.all(cover == 1)
            # slice the gathered tensor back: must give the shard, each byte once
            srcs = [want if p == r else np.zeros(0, NP[es]) for p in range(world)]
            back, cover = walk(OP_SLICE, world, r, es, outer, 0, inner, 0, lengths, None, srcs, shards[r].shape)
            assert np.array_equal(back, shards[r])
            assert np.all(cover == 1)
            # and the backward of slice scatters it into a zero tensor
            srcs = [shards[r] if p == r else np.zeros(0, NP[es]) for p in range(world)]
            scat, cover = walk(OP_UNSLICE, world, r, es, outer, 0, inner, 0, lengths, None, srcs, full_shape)
            ref = np.zeros(full_shape, NP[es])
            sl = [slice(None)] * len(full_shape)
            sl[dim] = slice(sum(lengths[:r]), sum(lengths[:r + 1]))
            ref[tuple(sl)] = shards[r]
            assert np.array_equal(scat, ref)
            assert int(cover.sum()) == shards[r].nbytes


@pytest.mark.parametrize("es", [2, 4])
def test_all_to_all_geometry(es):
    rng = np.random.default_rng(11)
    cases = [
        (4, [4, 3, 2, 1], [1, 2, 3, 4]), (4, [5, 0, 5, 0], [0, 2, 0, 8]), (2, [3, 2], [1, 4]),
        (8, [7, 6, 5, 4, 3, 3, 2, 2], [56, 46, 39, 33, 28, 23, 18, 13]),
    ]
    for world, sl, cl in cases:
        for nd, sd, cd in ((2, 0, 1), (2, 1, 0), (3, 0, 2), (3, 2, 0), (3, 1, 2), (4, 3, 1), (4, 1, 2)):
            base = [3, 2, 5, 2][:nd]
            xs = []
            for r in range(world):
                s = list(base)
                s[sd] = sum(sl)
                s[cd] = cl[r]
                xs.append(rand(s, es, rng))
            want = cm.all_to_all([to_t(x) for x in xs], sd, cd, sl, cl)
            d1, d2 = min(sd, cd), max(sd, cd)
            a, b, c = prod(base[:d1]), prod(base[d1 + 1:d2]), prod(base[d2 + 1:])
            for r in range(world):
                shape = list(base)
                shape[sd] = sl[r]
                shape[cd] = sum(cl)
                got, cover = walk(OP_EXCHANGE, world, r, es, a, b, c, int(sd < cd), sl, cl, xs, shape)
                assert np.array_equal(got.astype(np.int64), want[r].numpy()), (world, sd, cd, r)
                assert np.all(cover == 1)


def test_random_gather_shapes_large_rows():
    rng = np.random.default_rng(5)
    pyrng = random.Random(5)
    for _ in range(40):
        world = pyrng.choice([2, 3, 4, 8])
        es = pyrng.choice([2, 4])
        lengths = [pyrng.choice([0, 1, 5, 17, 64, 300]) for _ in range(world)]
        outer = pyrng.choice([1, 2, 7])
        inner = pyrng.choice([1, 3, 8, 127, 1025])
        shards = [rand((outer, l, inner), es, rng) for l in lengths]
        want = np.concatenate(shards, axis=1)
        r = pyrng.randrange(world)
        got, cover = walk(OP_GATHER, world, r, es, outer, 0, inner, 0, lengths, None, shards, want.shape)
        assert np.array_equal(got, want)
        assert np.all(cover == 1)
