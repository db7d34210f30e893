"""The all_reduce entry point that allocates nothing (hapx_local_all_reduce_noalloc).

Some hosts cannot call cudaMalloc when a collective is due: all device memory already belongs to
another allocator, or the thread must not take the device-wide synchronisation an allocation
implies.  For them the library carries its scratch (control blocks, staged inputs, reduced
slices) in a built-in 16 MiB device array.  This file checks, through the C ABI, that the entry
point gives the same bits as the communicator-based hapx_all_reduce on two calls in a row (the
second with other data and another size, so leftovers of the first call in the shared scratch
would show), and that oversized calls are refused.  It is collected last on purpose.
"""

import pytest
import torch

import hap_b200
from hap_b200 import _native as N
from hap_b200.comm import local_all_reduce_noalloc

DEV = "cuda:0"


def test_oversized_and_malformed_calls_are_refused_without_a_device():
    arr = N.ptr_array([1, 1])          # never dereferenced: the size checks come first
    too_many = 600_000                  # float32 elements at world 2: 2.4 MB staged input > 2 MiB of scratch per rank
    rc = N.lib.hapx_local_all_reduce_noalloc(2, arr, arr, N.F32, N.F32, 1.0, too_many, None)
    assert rc == N.ERR_STAGING
    assert b"scratch" in N.lib.hapx_last_error()
    assert N.lib.hapx_local_all_reduce_noalloc(9, arr, arr, N.F32, N.F32, 1.0, 16, None) == N.ERR_ARGUMENT
    assert N.lib.hapx_local_all_reduce_noalloc(2, arr, arr, N.B64, N.B64, 1.0, 16, None) == N.ERR_DTYPE
    assert N.lib.hapx_local_all_reduce_noalloc(2, arr, arr, N.F32, N.F32, 1.0, -1, None) == N.ERR_EXTENT


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 4, 8])
def test_matches_the_communicator_all_reduce_on_two_calls_in_a_row(world):
    comm = hap_b200.local_comm(world, DEV, stage_bytes=16 << 20, heap_bytes=24 << 20)
    try:
        for dtype, out_dtype in ((torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)):
            for call, n in enumerate((200_001, 4099)):       # two calls in a row, second smaller and different data
                xs = [torch.randn(n, device=DEV, generator=torch.Generator(DEV).manual_seed(10 * call + r)).to(dtype)
                      for r in range(world)]
                want = comm.all_reduce(xs, scale=0.5, out_dtype=out_dtype)
                outs = [torch.full((n,), float("nan"), device=DEV, dtype=out_dtype) for _ in range(world)]
                local_all_reduce_noalloc(xs, outs, scale=0.5)
                torch.cuda.synchronize()
                for r in range(world):
                    assert torch.equal(outs[r], want[r]), (world, dtype, n, r)
        # in place: outputs are the inputs
        xs = [torch.randn(70_000, device=DEV, generator=torch.Generator(DEV).manual_seed(99 + r)) for r in range(world)]
        want = comm.all_reduce(xs)
        local_all_reduce_noalloc(xs, xs)
        for r in range(world):
            assert torch.equal(xs[r], want[r])
        comm.check()
    finally:
        comm.destroy()


@pytest.mark.gpu
def test_too_large_for_the_built_in_scratch_raises():
    xs = [torch.zeros(1 << 20, device=DEV) for _ in range(8)]
    with pytest.raises(N.HapxError) as err:
        local_all_reduce_noalloc(xs, xs)
    assert err.value.code == N.ERR_STAGING
