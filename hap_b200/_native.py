"""ctypes binding of ``libhapx.so`` (the C ABI declared in ``include/hapx.h``).

There is no CPU or eager fallback: if the library has not been built, importing
this module raises and so does every operation of the package.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libhapx.so")

MAX_WORLD = 16
IPC_HANDLE_BYTES = 64

OK, ERR_ARGUMENT, ERR_EXTENT, ERR_DTYPE, ERR_CUDA, ERR_PEER_TIMEOUT, ERR_STAGING, ERR_STATE = 0, -1, -2, -3, -4, -5, -6, -7
F32, BF16, F16, F64, B8, B16, B32, B64 = range(8)
MODE_PADDING, MODE_GROUP_CALL = 0, 1
OPTIM_STATE_FLOATS = 2056

_i64, _int, _dbl, _vp, _sz, _u64 = C.c_int64, C.c_int, C.c_double, C.c_void_p, C.c_size_t, C.c_uint64
_pp = C.POINTER(C.c_void_p)
_pi64 = C.POINTER(C.c_int64)

# name -> (restype, argtypes); every symbol include/hapx.h declares
SIGNATURES = {
    "hapx_last_error": (C.c_char_p, []),
    "hapx_version": (_int, []),
    "hapx_launch_count": (_i64, []),
    "hapx_sharding_round": (_int, [_i64, C.POINTER(_dbl), _int, _pi64]),
    "hapx_comm_create": (_int, [_pp, _int, _int, _int, _sz, _sz]),
    "hapx_comm_create_local": (_int, [_pp, _int, _int, _sz, _sz]),
    "hapx_comm_ipc_handle": (_int, [_vp, _vp]),
    "hapx_comm_open_peers": (_int, [_vp, _vp]),
    "hapx_comm_attach_peer": (_int, [_vp, _int, _vp]),
    "hapx_comm_close_peers": (_int, [_vp]),
    "hapx_comm_destroy": (_int, [_vp]),
    "hapx_comm_poll": (_int, [_vp]),
    "hapx_comm_calls_issued": (_int, [_vp, C.POINTER(_i64)]),
    "hapx_comm_world": (_int, [_vp, C.POINTER(_int), C.POINTER(_int), C.POINTER(_int)]),
    "hapx_comm_heap": (_int, [_vp, _int, _pp, C.POINTER(_sz)]),
    "hapx_comm_set_timeout_ms": (_int, [_vp, _int]),
    "hapx_comm_set_max_ctas": (_int, [_vp, _int]),
    "hapx_comm_set_stream_ordering": (_int, [_vp, _int]),
    "hapx_comm_set_fused_all_reduce": (_int, [_vp, _int]),
    "hapx_comm_check": (_int, [_vp]),
    "hapx_comm_get": (_int, [_vp, _int, _sz, _vp, _sz, _vp]),
    "hapx_all_gather": (_int, [_vp, _pp, _pp, _int, _i64, _i64, _pi64, _int, _vp]),
    "hapx_reduce_scatter": (_int, [_vp, _pp, _pp, _int, _int, _dbl, _i64, _i64, _pi64, _int, _vp]),
    "hapx_all_reduce": (_int, [_vp, _pp, _pp, _int, _int, _dbl, _i64, _vp]),
    "hapx_all_to_all": (_int, [_vp, _pp, _pp, _int, _i64, _i64, _i64, _int, _pi64, _pi64, _vp]),
    "hapx_dynamic_slice": (_int, [_vp, _vp, _int, _i64, _i64, _pi64, _int, _int, _vp]),
    "hapx_dynamic_slice_backward": (_int, [_vp, _vp, _int, _i64, _i64, _pi64, _int, _int, _vp]),
    "hapx_linear_forward": (_int, [_vp, _vp, _vp, _vp, _int, _int, _i64, _i64, _i64, _int, _vp]),
    "hapx_linear_dgrad": (_int, [_vp, _vp, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hapx_linear_wgrad": (_int, [_vp, _vp, _vp, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hapx_gemm_batched": (_int, [_vp, _vp, _vp, _int, _int, _int] + [_i64] * 14 + [_vp]),
    "hapx_gemm_status": (_int, []),
    "hapx_moe_index": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "hapx_moe_rows_from_tokens": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "hapx_moe_tokens_from_rows": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "hapx_moe_weight_grad": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "hapx_moe_rows_from_tokens_strided": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "hapx_moe_tokens_from_rows_strided": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "hapx_moe_weight_grad_strided": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "hapx_attention_forward": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp]),
    "hapx_attention_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "hapx_attention_classify_mask": (_int, [_vp, _i64, _vp, _vp]),
    "hapx_attention_fused_forward": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _dbl, _u64, _vp]),
    "hapx_attention_fused_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _dbl, _u64, _vp]),
    "hapx_attention_dropout_mask": (_int, [_vp, _i64, _i64, _i64, _dbl, _u64, _vp]),
    "hapx_grad_sqnorm": (_int, [_int, _pp, _pi64, _int, _vp, _int, _vp]),
    "hapx_clip_adam_apply": (_int, [_int, _pp, _pp, _pp, _pp, _pi64, _int, _dbl, _dbl, _dbl, _dbl, _dbl, _dbl, _vp, _int, _vp]),
    "hapx_nll_logsoftmax_forward": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    "hapx_nll_logsoftmax_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _i64, _vp]),
    "hapx_layer_norm_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _dbl, _vp]),
    "hapx_embedding_backward": (_int, [_vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    "hapx_layer_norm_backward_blocks": (_int, [_i64, _i64]),
    "hapx_layer_norm_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _vp]),
    "hapx_layer_norm_backward_add": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _vp]),
    "hapx_rng_seed": (_int, [_u64, _vp]),
    "hapx_rng_advance": (_int, [_vp]),
    "hapx_dropout": (_int, [_vp, _vp, _int, _i64, _dbl, _u64, _vp]),
    "hapx_dropout_mask": (_int, [_vp, _i64, _dbl, _u64, _vp]),
    "hapx_dropout_add": (_int, [_vp, _vp, _vp, _int, _i64, _dbl, _u64, _vp]),
    "hapx_act_dropout": (_int, [_vp, _vp, _int, _i64, _int, _dbl, _u64, _vp]),
    "hapx_act_dropout_backward": (_int, [_vp, _vp, _vp, _int, _i64, _int, _dbl, _u64, _vp]),
    "hapx_local_all_reduce_noalloc": (_int, [_int, _pp, _pp, _int, _int, _dbl, _i64, _vp]),
    "hapx_local_all_reduce_noalloc_status": (_int, []),
    "hapx_debug_host_walk": (_int, [_int, _int, _int, _int, _i64, _i64, _i64, _int, _pi64, _pi64, _pp,
                                     C.POINTER(_sz), _vp, _sz, _vp]),
}


class HapxError(RuntimeError):
    """A hapx entry point returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"hapx error {code}: {message}")
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python hap_b200/csrc/build.py` (needs nvcc, targets sm_100a). "
            "hap_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(code: int) -> None:
    if code != 0:
        raise HapxError(code, (lib.hapx_last_error() or b"").decode("utf-8", "replace"))


def ptr_array(ptrs):
    return (C.c_void_p * len(ptrs))(*[C.c_void_p(p) for p in ptrs])


_I64_CACHE = {}


def i64_array(vals):
    """ctypes int64 array of `vals`; sharding-length vectors repeat on every call, so small arrays are cached."""
    key = tuple(vals)
    arr = _I64_CACHE.get(key)
    if arr is None:
        arr = (C.c_int64 * len(key))(*[int(v) for v in key])
        if len(_I64_CACHE) < 4096:
            _I64_CACHE[key] = arr
    return arr
