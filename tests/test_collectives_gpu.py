"""Parity of the CUDA collectives with the oracle, on ONE GPU.

A local communicator hosts `world` virtual ranks on the device; every collective is one
cooperative launch of the same kernels (and flag protocol) the multi-GPU path runs.  All
calls go through the C ABI (ctypes).  Gathers / re-sharding must be bit-exact; reductions
within 1e-5 relative for fp32 and 1e-2 for bf16/fp16, as the north star states."""
import pytest
import torch

import hap_b200
from hap_b200 import _native as N
from oracle import collectives_math as cm
from tests.helpers import exact_op, load_golden

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: dict(rtol=1e-5, atol=1e-5), torch.bfloat16: dict(rtol=1e-2, atol=1e-2),
       torch.float16: dict(rtol=1e-2, atol=1e-2)}
_comms = {}


def comm_for(world):
    if world not in _comms:
        _comms[world] = hap_b200.local_comm(world, DEV, stage_bytes=160 << 20, heap_bytes=(160 << 20) + (128 << 20))
    return _comms[world]


@pytest.fixture(scope="module", autouse=True)
def _teardown():
    yield
    for c in _comms.values():
        c.destroy()
    _comms.clear()


def gen(shape, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)


def gpu(ts):
    return [t.to(DEV) for t in ts]


def cpu(ts):
    return [t.cpu() for t in ts]


# ---- golden fixtures: outputs of the reference's own collectives.py ------------------------------
@pytest.mark.parametrize("world", [2, 4])
def test_golden_forward_and_backward(world):
    data = load_golden(world)
    comm = comm_for(world)
    lc = hap_b200.LocalCollectives(comm)
    for name, per_rank in data["cases"].items():
        op, args = per_rank[0]["op"], per_rank[0]["args"]
        xs = [p["x"].to(DEV).requires_grad_(True) for p in per_rank]
        if op in ("all_reduce", "replicate"):
            outs = getattr(lc, op)(xs)
        elif op == "all_to_all":
            outs = lc.all_to_all(xs, *args)
        else:
            outs = getattr(lc, op)(xs, args[0], list(args[1]))
        loss = sum((o * p["w"].to(DEV)).sum() for o, p in zip(outs, per_rank))
        loss.backward()
        comm.check()
        for r in range(world):
            want_out, want_grad = per_rank[r]["out"], per_rank[r]["grad"]
            got = outs[r].detach().cpu()
            assert got.shape == want_out.shape, name
            if exact_op(op):
                assert torch.equal(got, want_out), name
            else:
                torch.testing.assert_close(got, want_out, rtol=1e-5, atol=1e-5, msg=name)
            torch.testing.assert_close(xs[r].grad.cpu(), want_grad, rtol=1e-5, atol=1e-5, msg=name)


# ---- known answers written in the reference's manual test (collectives.py:198-323) ---------------
def test_reference_known_answers():
    comm = comm_for(4)
    lc = hap_b200.LocalCollectives(comm)
    L = [1, 2, 3, 4]
    ones = lambda *s: torch.ones(*s, device=DEV)
    for fn in (lc.all_gather, lc.all_gather_by_group_call):      # Mod1, Mod1v2
        ps = [ones(5, r + 1).requires_grad_(True) for r in range(4)]
        losses = [o.sum() / 4 for o in fn(ps, 1, L)]
        sum(losses).backward()
        assert [float(l) for l in losses] == [12.5] * 4
        assert all(torch.equal(p.grad, ones(5, r + 1)) for r, p in enumerate(ps))
    ps = [(ones(5, 4) * r).requires_grad_(True) for r in range(4)]  # Mod2
    losses = [o.sum() / 4 for o in lc.all_reduce(ps)]
    sum(losses).backward()
    assert [float(l) for l in losses] == [30.0] * 4
    assert all(torch.equal(p.grad, ones(5, 4)) for p in ps)
    for fn in (lc.reduce_scatter, lc.reduce_scatter_by_group_call):  # Mod3, Mod3v2
        ps = [ones(5, 10).requires_grad_(True) for _ in range(4)]
        losses = [o.sum() for o in fn(ps, 1, L)]
        sum(losses).backward()
        assert [float(l) for l in losses] == [20.0 * (r + 1) for r in range(4)]
        assert all(torch.equal(p.grad, ones(5, 10)) for p in ps)
    ps = [ones(5, 10).requires_grad_(True) for _ in range(4)]      # Mod4
    losses = [o.sum() for o in lc.dynamic_slice(ps, 1, L)]
    sum(losses).backward()
    assert [float(l) for l in losses] == [5.0 * (r + 1) for r in range(4)]
    for r, p in enumerate(ps):
        want = torch.zeros(5, 10, device=DEV)
        want[:, sum(L[:r]):sum(L[:r + 1])] = 1
        assert torch.equal(p.grad, want)
    ps = [ones(10, r + 1).requires_grad_(True) for r in range(4)]   # Mod5
    outs = lc.all_to_all(ps, 0, 1, [4, 3, 2, 1], L)
    sum(o.sum() for o in outs).backward()
    assert [tuple(o.shape) for o in outs] == [(4 - r, 10) for r in range(4)]
    assert [float(o.sum()) for o in outs] == [10.0 * (4 - r) for r in range(4)]
    assert all(torch.equal(p.grad, ones(10, r + 1)) for r, p in enumerate(ps))
    cat = [0, 2, 0, 8]                                                # Mod5_v2: zero-length shards
    outs = lc.all_to_all([ones(10, cat[r]) for r in range(4)], 0, 1, [5, 0, 5, 0], cat)
    assert [tuple(o.shape) for o in outs] == [(5, 10), (0, 10), (5, 10), (0, 10)]
    ps = [ones(5, 5).requires_grad_(True) for _ in range(4)]        # Mod6
    losses = [o.sum() / 4 for o in lc.replicate(ps)]
    sum(losses).backward()
    assert [float(l) for l in losses] == [6.25] * 4
    assert all(torch.equal(p.grad, ones(5, 5)) for p in ps)
    comm.check()


# ---- seeded sweeps against the oracle -------------------------------------------------------------
R8 = [.22, .18, .15, .13, .11, .09, .07, .05]
SHAPES = [  # (world, lengths, base shape with a placeholder on `dim`, dim)
    (2, [141, 115], (0, 64), 0),
    (2, [2458, 1638], (64, 0), 1),                # column-TP hidden activation of the MLP config
    (4, [83, 68, 56, 49], (0, 33), 0),
    (4, [3, 0, 2, 5], (3, 0, 7), 1),
    (8, [56, 46, 39, 33, 28, 23, 18, 13], (0, 1024), 0),
    (8, [56, 46, 39, 33, 28, 23, 18, 13], (256, 0), 1),
    (8, [7, 6, 5, 4, 3, 3, 2, 2], (5, 0, 3, 11), 1),
    (8, [676, 553, 461, 399, 338, 276, 215, 154], (0, 96), 0),
    (8, [1, 1, 1, 1, 1, 1, 1, 1], (9, 0), 1),       # rows of a single element
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.uint8])
@pytest.mark.parametrize("world,lengths,base,dim", SHAPES)
def test_all_gather_bit_exact(world, lengths, base, dim, dtype):
    comm = comm_for(world)
    shards = []
    for r in range(world):
        s = list(base)
        s[dim] = lengths[r]
        t = gen(s, 1000 + r)
        shards.append((t * 50).to(dtype) if not dtype.is_floating_point else t.to(dtype))
    want = cm.all_gather(shards, dim, lengths)
    for mode in (N.MODE_PADDING, N.MODE_GROUP_CALL):
        got = comm.all_gather(gpu(shards), dim, lengths, mode)
        comm.check()
        for r in range(world):
            assert torch.equal(got[r].cpu(), want[r])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world,lengths,base,dim", SHAPES)
def test_reduce_scatter_and_all_reduce(world, lengths, base, dim, dtype):
    comm = comm_for(world)
    s = list(base)
    s[dim] = sum(lengths)
    xs = [gen(s, 3000 + r, dtype) for r in range(world)]
    want = cm.reduce_scatter(xs, dim, lengths)
    for mode in (N.MODE_PADDING, N.MODE_GROUP_CALL):
        got = comm.reduce_scatter(gpu(xs), dim, lengths, mode)
        comm.check()
        for r in range(world):
            assert got[r].shape == want[r].shape
            torch.testing.assert_close(got[r].cpu(), want[r], **TOL[dtype])
    want = cm.all_reduce(xs)
    got = comm.all_reduce(gpu(xs))
    comm.check()
    for r in range(world):
        torch.testing.assert_close(got[r].cpu(), want[r], **TOL[dtype])
        assert torch.equal(got[r], got[0])          # every rank holds the same bits


def test_reduce_scatter_fused_scale_and_cast():
    world, lengths = 8, [56, 46, 39, 33, 28, 23, 18, 13]
    comm = comm_for(world)
    for in_dt, out_dt in ((torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16), (torch.float16, torch.float32),
                          (torch.float32, torch.float16), (torch.bfloat16, torch.float16)):
        xs = [gen((256, 37), 10 + r, in_dt) for r in range(world)]
        want = cm.reduce_scatter(xs, 0, lengths, scale=1.0 / world, out_dtype=out_dt)
        got = comm.reduce_scatter(gpu(xs), 0, lengths, scale=1.0 / world, out_dtype=out_dt)
        comm.check()
        for r in range(world):
            assert got[r].dtype == out_dt
            torch.testing.assert_close(got[r].cpu(), want[r], **TOL[out_dt if out_dt != torch.float32 else in_dt])
        want = cm.rank_sum(xs, 0.5, out_dt)
        got = comm.all_reduce(gpu(xs), scale=0.5, out_dtype=out_dt)
        for r in range(world):
            torch.testing.assert_close(got[r].cpu(), want, **TOL[out_dt if out_dt != torch.float32 else in_dt])


@pytest.mark.parametrize("n", [1, 3, 1000, 65536, 65537, 300001, (1 << 20) + 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_all_reduce_sizes_and_in_place(n, dtype):
    world = 4
    comm = comm_for(world)
    xs = [gen((n,), 77 + r, dtype) for r in range(world)]
    want = cm.all_reduce(xs)[0]
    got = comm.all_reduce(gpu(xs))
    bufs = gpu(xs)
    same = comm.all_reduce(bufs, inplace=True)
    comm.check()
    for r in range(world):
        torch.testing.assert_close(got[r].cpu(), want, **TOL[dtype])
        assert same[r].data_ptr() == bufs[r].data_ptr()
        assert torch.equal(same[r], got[r])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_all_reduce_one_launch_form(world, dtype):
    """The one-launch all_reduce (reduce own slice, announce, gather) is the default between processes; the
    emulated communicator runs it when forced, as a cooperative launch over all virtual ranks."""
    comm = comm_for(world)
    comm.set_fused_all_reduce(True)
    try:
        for n in (65537, 300001, (1 << 20) + 5, (1 << 22)):
            xs = [gen((n,), 911 + r, dtype) for r in range(world)]
            want = cm.all_reduce(xs)[0]
            got = comm.all_reduce(gpu(xs))
            bufs = gpu(xs)
            same = comm.all_reduce(bufs, inplace=True)
            comm.check()
            for r in range(world):
                torch.testing.assert_close(got[r].cpu(), want, **TOL[dtype])
                assert torch.equal(same[r], got[r])
    finally:
        comm.set_fused_all_reduce(None)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_all_reduce_written_into_the_peers_outputs(world, dtype):
    """Form 2: when every output lies in its rank's heap the slice owners write the sums straight into all outputs
    (in place on heap tensors, and into separate heap tensors); if one output is an ordinary tensor the same
    launch falls back to reduce + gather.  All three against the oracle, bit-identical across ranks."""
    n = (1 << 20) + 64
    comm = hap_b200.local_comm(world, DEV, stage_bytes=8 << 20, heap_bytes=(8 << 20) + 3 * n * 4 + (1 << 20))
    try:
        comm.set_fused_all_reduce("push")
        xs = [gen((n,), 1311 + r, dtype) for r in range(world)]
        want = cm.rank_sum(xs, 0.25, dtype)
        src = [comm.symm_empty((n,), dtype, i) for i in range(world)]
        dst = [comm.symm_empty((n,), dtype, i) for i in range(world)]
        for s_, x in zip(src, xs):
            s_.copy_(x.to(DEV))
        got = comm.all_reduce(src, scale=0.25, out=dst)                       # heap -> heap
        comm.check()
        for r in range(world):
            assert got[r].data_ptr() == dst[r].data_ptr()
            torch.testing.assert_close(got[r].cpu(), want, **TOL[dtype])
            assert torch.equal(got[r], got[0])
            torch.testing.assert_close(src[r].cpu(), xs[r])                    # inputs untouched
        mixed = list(dst)
        mixed[world - 1] = torch.empty(n, dtype=dtype, device=DEV)             # one ordinary output: reduce + gather
        for d in dst:
            d.zero_()
        got = comm.all_reduce(src, scale=0.25, out=mixed)
        comm.check()
        for r in range(world):
            torch.testing.assert_close(got[r].cpu(), want, **TOL[dtype])
        same = comm.all_reduce(src, scale=0.25, inplace=True)                 # in place on heap tensors
        comm.check()
        for r in range(world):
            assert same[r].data_ptr() == src[r].data_ptr()
            torch.testing.assert_close(same[r].cpu(), want, **TOL[dtype])
            assert torch.equal(same[r], same[0])
        ordinary = comm.all_reduce(gpu(xs), scale=0.25)                       # staged inputs, ordinary outputs
        comm.check()
        for r in range(world):
            torch.testing.assert_close(ordinary[r].cpu(), want, **TOL[dtype])
        # a byte count that is not a multiple of 16: heap tensors all the same, but the launch reduces and gathers
        m = n - 3
        odd_src = [s_[:m] for s_ in src]
        for s_, x in zip(odd_src, xs):
            s_.copy_(x[:m].to(DEV))
        odd = comm.all_reduce(odd_src, scale=0.25, out=[d[:m] for d in dst])
        comm.check()
        for r in range(world):
            torch.testing.assert_close(odd[r].cpu(), cm.rank_sum([x[:m] for x in xs], 0.25, dtype), **TOL[dtype])
    finally:
        comm.destroy()


def test_all_to_all_against_oracle():
    for world, sl, cl in ((4, [4, 3, 2, 1], [1, 2, 3, 4]), (4, [5, 0, 5, 0], [0, 2, 0, 8]), (2, [3, 2], [1, 4]),
                          (8, [7, 6, 5, 4, 3, 3, 2, 2], [56, 46, 39, 33, 28, 23, 18, 13])):
        comm = comm_for(world)
        for dtype in (torch.float32, torch.bfloat16):
            for nd, sd, cd in ((2, 0, 1), (2, 1, 0), (3, 0, 2), (3, 2, 0), (3, 1, 2), (4, 3, 1), (4, 1, 2)):
                base = [3, 2, 5, 2][:nd]
                xs = []
                for r in range(world):
                    s = list(base)
                    s[sd] = sum(sl)
                    s[cd] = cl[r]
                    xs.append(gen(s, 500 + r, dtype))
                want = cm.all_to_all(xs, sd, cd, sl, cl)
                got = comm.all_to_all(gpu(xs), sd, cd, sl, cl)
                comm.check()
                for r in range(world):
                    assert got[r].shape == want[r].shape
                    assert torch.equal(got[r].cpu(), want[r]), (world, sd, cd, r)


def test_moe_sized_all_to_all_round_trip():
    # expert-parallel re-sharding of (b, e, c, d): Gather(0) -> Gather(1) and back is the identity
    world = 8
    comm = comm_for(world)
    e_l = hap_b200.sharding_round(32, R8)
    b_l = hap_b200.sharding_round(32, R8)
    xs = [gen((b_l[r], 32, 20, 64), 900 + r, torch.bfloat16).to(DEV) for r in range(world)]
    mid = comm.all_to_all(xs, 1, 0, e_l, b_l)
    assert [tuple(m.shape) for m in mid] == [(32, e_l[r], 20, 64) for r in range(world)]
    back = comm.all_to_all(mid, 0, 1, b_l, e_l)
    comm.check()
    for r in range(world):
        assert torch.equal(back[r], xs[r])


def test_dynamic_slice_and_backward():
    for shape, dim, lengths in (((64, 1024), 0, [38, 26]), ((64, 4096), 1, [2458, 1638]), ((7, 10, 3), 1, [1, 2, 3, 4]),
                                ((5, 9), 1, [3, 0, 6])):
        for dtype in (torch.float32, torch.bfloat16, torch.int64):
            x = (gen(shape, 5) * 10).to(dtype)
            for r in range(len(lengths)):
                got = hap_b200.comm.dynamic_slice(x.to(DEV), dim, lengths, r)
                want = cm.dynamic_slice(x, dim, lengths, r)
                assert torch.equal(got.cpu(), want)
                back = hap_b200.comm.dynamic_slice_backward(got, dim, lengths, r)
                assert torch.equal(back.cpu(), cm.dynamic_slice_backward(want, shape, dim, lengths, r))


# ---- inputs that already live in the peer-visible heap are read in place ---------------------------
def test_heap_resident_inputs_match_staged_inputs():
    world, lengths = 8, [56, 46, 39, 33, 28, 23, 18, 13]
    comm = comm_for(world)
    comm.symm_reset()
    shards = [gen((lengths[r], 515), 40 + r, torch.bfloat16) for r in range(world)]
    resident = []
    for r in range(world):
        t = comm.symm_empty(shards[r].shape, torch.bfloat16, r)
        t.copy_(shards[r])
        resident.append(t)
    a = comm.all_gather(resident, 0, lengths)
    b = comm.all_gather(gpu(shards), 0, lengths)
    fulls = []
    for r in range(world):
        t = comm.symm_empty((256, 515), torch.bfloat16, r)
        t.copy_(gen((256, 515), 60 + r, torch.bfloat16))
        fulls.append(t)
    c = comm.reduce_scatter(fulls, 0, lengths)
    d = comm.reduce_scatter([f.clone() for f in fulls], 0, lengths)
    e = comm.all_reduce(fulls)
    want = cm.all_reduce(cpu(fulls))[0]
    f = comm.all_reduce(fulls, inplace=True)
    comm.check()
    for r in range(world):
        assert torch.equal(a[r], b[r]) and torch.equal(c[r], d[r])
        torch.testing.assert_close(e[r].cpu(), want, **TOL[torch.bfloat16])
        assert torch.equal(f[r], e[r])
    comm.symm_reset()


# ---- benchmark-sized tensors: size-independent properties -----------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_large_round_trips(dtype):
    world = 8
    comm = comm_for(world)
    lengths = hap_b200.sharding_round(256, R8)
    cols = (64 << 20) // (256 * torch.empty((), dtype=dtype).element_size())    # 64 MiB tensor
    shards = [torch.randn(lengths[r], cols, device=DEV, generator=torch.Generator(DEV).manual_seed(1000 + r)).to(dtype)
              for r in range(world)]
    full = comm.all_gather(shards, 0, lengths)
    # gather -> slice gives the shard back; every rank holds identical bytes
    for r in range(world):
        assert torch.equal(hap_b200.comm.dynamic_slice(full[r], 0, lengths, r), shards[r])
        assert torch.equal(full[r], full[0])
    # reduce_scatter of W copies of the same tensor: the kernel adds in rank order in fp32, so the
    # result must equal the same chain of fp32 additions done with plain tensor ops, bit for bit
    def chain(x, scale=None):
        acc = x.float().clone()
        for _ in range(world - 1):
            acc += x.float()
        return (acc if scale is None else acc * scale).to(dtype)
    rs = comm.reduce_scatter([full[0]] * world, 0, lengths)
    for r in range(world):
        assert torch.equal(rs[r], chain(shards[r]))
    ar = comm.all_reduce([full[0]] * world, scale=1.0 / world)
    want = chain(full[0], 1.0 / world)
    assert all(torch.equal(a, want) for a in ar)
    comm.check()
    # checksum of checksums: sum over ranks of reduce_scatter outputs == sum of all inputs
    if dtype == torch.float32:
        xs = [torch.randn(256, 4096, device=DEV, generator=torch.Generator(DEV).manual_seed(r)) for r in range(world)]
        rs = comm.reduce_scatter(xs, 0, lengths)
        total = sum(float(o.double().sum()) for o in rs)
        want = sum(float(x.double().sum()) for x in xs)
        assert abs(total - want) <= 1e-6 * max(1.0, abs(want)) + 1e-2


# ---- error behaviour ---------------------------------------------------------------------------------
def test_shape_errors_raise():
    comm = comm_for(2)
    x = torch.ones(4, 4, device=DEV)
    with pytest.raises(ValueError):
        comm.all_gather([x, x], 0, [4, 3])
    with pytest.raises(ValueError):
        comm.reduce_scatter([x, x], 0, [1, 2])
    with pytest.raises(ValueError):
        comm.all_gather([x], 0, [4, 4])
    with pytest.raises(TypeError):
        comm.all_reduce([x.long(), x.long()])
    with pytest.raises(N.HapxError):
        big = torch.ones((200 << 20) // 4, device=DEV)     # larger than the 160 MiB staging area
        comm.all_gather([big, big], 0, [big.numel(), big.numel()])


def test_peer_that_never_arrives_times_out_cleanly():
    """A rank whose peer never launches: the bounded wait runs out, the kernel records the error
    and returns, the host reads it, and the device stays usable.  (The 'peer' is a zeroed buffer
    attached by hand, so no flag is ever written.)"""
    import ctypes as C
    h = C.c_void_p()
    N.check(N.lib.hapx_comm_create(C.byref(h), 2, 0, 0, 8 << 20, 1 << 20))
    fake_peer = torch.zeros(8 << 20, dtype=torch.uint8, device=DEV)
    N.check(N.lib.hapx_comm_attach_peer(h, 1, fake_peer.data_ptr()))
    comm = hap_b200.Comm(h.value, torch.device(DEV))
    comm.set_timeout_ms(200)
    x = torch.ones(3, 8, device=DEV)
    comm.all_gather([x], 0, [3, 5])
    with pytest.raises(N.HapxError) as err:
        comm.check()
    assert err.value.code == N.ERR_PEER_TIMEOUT
    comm.check()                                            # status was cleared
    assert float((x + 1).sum()) == 48.0                   # the context is alive
    comm.destroy()
