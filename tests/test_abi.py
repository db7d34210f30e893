"""The C-ABI library loads, exports every symbol include/hapx.h declares, and rejects bad
arguments before touching a device (no compute calls here: this file runs without a GPU)."""
import ctypes as C
import os
import re

import pytest

from hap_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hapx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hapx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 20
    lib = C.CDLL(N.LIB_PATH)
    for name in names:
        assert hasattr(lib, name), f"{name} declared in hapx.h but not exported"
        assert name in N.SIGNATURES, f"{name} has no ctypes signature"
    assert set(N.SIGNATURES) == set(names)


def test_version_and_launch_counter():
    assert N.lib.hapx_version() == 1
    assert N.lib.hapx_launch_count() == 0


@pytest.mark.parametrize("world", [0, -1, N.MAX_WORLD + 1])
def test_comm_create_rejects_bad_world(world):
    h = C.c_void_p()
    assert N.lib.hapx_comm_create(C.byref(h), world, 0, 0, 1 << 20, 0) == N.ERR_ARGUMENT
    assert N.lib.hapx_comm_create_local(C.byref(h), world, 0, 1 << 20, 0) == N.ERR_ARGUMENT
    assert b"world" in N.lib.hapx_last_error()


def test_comm_create_rejects_bad_sizes():
    h = C.c_void_p()
    assert N.lib.hapx_comm_create(C.byref(h), 2, 0, 0, 1 << 20, 100) == N.ERR_ARGUMENT       # stage not /256
    assert N.lib.hapx_comm_create(C.byref(h), 2, 0, 0, 1024, 256) == N.ERR_ARGUMENT          # heap too small
    assert N.lib.hapx_comm_create(C.byref(h), 2, 5, 0, 1 << 20, 0) == N.ERR_ARGUMENT         # rank >= world
    assert N.lib.hapx_comm_create(None, 2, 0, 0, 1 << 20, 0) == N.ERR_ARGUMENT


def test_null_communicator_is_rejected():
    null = C.c_void_p()
    arr = N.ptr_array([0])
    lens = N.i64_array([1, 1])
    assert N.lib.hapx_all_gather(null, arr, arr, N.F32, 1, 1, lens, 0, None) == N.ERR_ARGUMENT
    assert N.lib.hapx_reduce_scatter(null, arr, arr, N.F32, N.F32, 1.0, 1, 1, lens, 0, None) == N.ERR_ARGUMENT
    assert N.lib.hapx_all_reduce(null, arr, arr, N.F32, N.F32, 1.0, 4, None) == N.ERR_ARGUMENT
    assert N.lib.hapx_all_to_all(null, arr, arr, N.F32, 1, 1, 1, 1, lens, lens, None) == N.ERR_ARGUMENT
    assert N.lib.hapx_comm_check(null) == N.ERR_ARGUMENT


def test_dynamic_slice_rejects_bad_arguments_before_any_launch():
    lens = N.i64_array([1, 2])
    assert N.lib.hapx_dynamic_slice(None, None, 99, 1, 1, lens, 2, 0, None) == N.ERR_DTYPE
    assert N.lib.hapx_dynamic_slice(None, None, N.F32, 1, 1, lens, 2, 7, None) == N.ERR_ARGUMENT
    assert N.lib.hapx_dynamic_slice(None, None, N.F32, -1, 1, lens, 2, 0, None) == N.ERR_EXTENT
    assert N.lib.hapx_dynamic_slice(None, None, N.F32, 1, 1, N.i64_array([1, -2]), 2, 0, None) == N.ERR_EXTENT


def test_python_layer_refuses_cpu_tensors():
    import torch
    from hap_b200 import comm
    with pytest.raises(RuntimeError, match="no CPU path"):
        comm.dynamic_slice(torch.ones(4, 4), 0, [2, 2], 0)
