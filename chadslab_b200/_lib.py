"""ctypes binding of libb200q.so (the C ABI declared in include/b200q.h).

There is no fallback: if the shared library is missing or a call fails, a BqError is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200q.so")

FMT_Q8, FMT_Q4 = 0, 1
DT_F32, DT_BF16 = 0, 1
PATH_AUTO, PATH_SIMT, PATH_TENSOR, PATH_MMA = 0, 1, 2, 3

OK, ERR_ARG, ERR_HANDLE, ERR_CUDA, ERR_STATE, ERR_TIMEOUT, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5, -6
_ERR_NAMES = {ERR_ARG: "BQ_ERR_ARG", ERR_HANDLE: "BQ_ERR_HANDLE", ERR_CUDA: "BQ_ERR_CUDA",
              ERR_STATE: "BQ_ERR_STATE", ERR_TIMEOUT: "BQ_ERR_TIMEOUT", ERR_UNSUPPORTED: "BQ_ERR_UNSUPPORTED"}


class BqError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{_ERR_NAMES.get(code, code)}: {msg}")
        self.code = code


_i64, _i32, _vp = C.c_int64, C.c_int, C.c_void_p
_h = C.c_uint64

# name -> (restype, argtypes); must list every symbol that include/b200q.h declares
PROTOTYPES = {
    "bq_init": (_i32, [_i32]),
    "bq_last_error": (C.c_char_p, []),
    "bq_version": (_i32, []),
    "bq_status_poll": (_i32, []),
    "bq_reserve": (_i32, [_i64, _i64, _i64]),
    "bq_weight_create": (_i32, [_vp, _vp, _i64, _i64, _i32, C.POINTER(_h)]),
    "bq_weight_create_device": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp, C.POINTER(_h)]),
    "bq_weight_destroy": (_i32, [_h]),
    "bq_weight_slice_rows": (_i32, [_h, _i64, _i64, C.POINTER(_h)]),
    "bq_weight_info": (_i32, [_h, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i32)]),
    "bq_weight_export": (_i32, [_h, _vp, _vp]),
    "bq_quantize": (_i32, [_vp, _i32, _i64, _i64, _i32, _vp, _vp, _vp]),
    "bq_dequant": (_i32, [_h, _vp, _i32, _vp]),
    "bq_unpack_codes": (_i32, [_h, _vp, _vp]),
    "bq_qlinear": (_i32, [_h, _vp, _i32, _i64, _vp, _i32, _vp]),
    "bq_qlinear_ex": (_i32, [_h, _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    "bq_qlinear_host": (_i32, [_h, _vp, _i32, _i64, _vp, _i32]),
    "bq_qlinear_gated": (_i32, [_h, _vp, _i32, _i64, _vp, _i32, _vp]),
    "bq_lm_head": (_i32, [_h, _vp, _i32, _i64, _vp, _i32, _vp, _vp]),
    "bq_last_path": (_i32, []),
    "bq_launch_count": (_i64, []),
    "bq_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, C.c_float, _i32, _vp]),
    "bq_rope_kv_append": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i64, C.c_float, _i32, _vp]),
    "bq_decode_attention": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _i32, _vp]),
    "bq_decode_attention_rope": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i64, C.c_float, _i32, _vp]),
    "bq_gated_act": (_i32, [_vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "bq_moe_route": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bq_moe_route_linear": (_i32, [_h, _vp, _i64, _i32, _i32, _vp, _vp, _vp]),
    "bq_moe_permute_scratch_bytes": (_i64, [_i64, _i32, _i32]),
    "bq_moe_permute": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "bq_moe_permute_noalloc_max_bytes": (_i64, []),
    "bq_moe_permute_noalloc": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bq_moe_gather": (_i32, [_vp, _i32, _i64, _vp, _i64, _i32, _vp, _vp]),
    "bq_moe_create": (_i32, [C.POINTER(_h), C.POINTER(_h), C.POINTER(_h), _i32, C.POINTER(_h)]),
    "bq_moe_destroy": (_i32, [_h]),
    "bq_moe_experts": (_i32, [_h, _vp, _vp, _i64, _vp, _vp, _i32, _vp]),
    "bq_moe_experts_ex": (_i32, [_h, _vp, _vp, _i64, _i64, _vp, _vp, _i32, _vp]),
    "bq_moe_experts_tokens": (_i32, [_h, _vp, _vp, _i32, _vp, _i64, _i64, _vp, _vp, _vp, _i32, _vp]),
    "bq_moe_combine": (_i32, [_vp, _vp, _vp, _i64, _i32, _i64, _vp, _i32, _vp]),
    "bq_comm_create": (_i32, [_i32, _i32, _i64, C.POINTER(_h)]),
    "bq_comm_handle": (_i32, [_h, _vp]),
    "bq_comm_connect": (_i32, [_h, _vp]),
    "bq_comm_connect_loopback": (_i32, [_h]),
    "bq_comm_set_timeout_ms": (_i32, [_h, _i32]),
    "bq_comm_destroy": (_i32, [_h]),
    "bq_comm_reset": (_i32, [_h]),
    "bq_lm_head_sharded": (_i32, [_h, _vp, _i32, _i64, _i64, _h, _vp, _vp, _vp]),
    "bq_ep_create": (_i32, [_i32, _i32, _i32, _i64, _i64, _i64, C.POINTER(_h)]),
    "bq_ep_handle": (_i32, [_h, _vp]),
    "bq_ep_connect": (_i32, [_h, _vp]),
    "bq_ep_set_timeout_ms": (_i32, [_h, _i32]),
    "bq_ep_destroy": (_i32, [_h]),
    "bq_ep_dispatch": (_i32, [_h, _vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "bq_ep_layout_selftest": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "bq_ep_recv_view": (_i32, [_h, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i64)]),
    "bq_ep_combine": (_i32, [_h, _vp, _vp, _vp, _i64, _i32, _vp, _i32, _vp]),
    "bq_qlinear_push": (_i32, [_h, _vp, _i32, _i64, _h, _vp]),
    "bq_allreduce": (_i32, [_h, _vp, _vp, _i64, _vp]),
    "bq_allreduce_add_rmsnorm": (_i32, [_h, _vp, _vp, _vp, _vp, _i64, _i64, C.c_float, _i32, _vp]),
}

_lock = threading.Lock()
_lib = None
_inited_device = None


def load() -> C.CDLL:
    """Load the shared library (no CUDA call is made here)."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise BqError(ERR_STATE, f"{LIB_PATH} not found: build it with "
                                         f"`python -m chadslab_b200.build` (there is no CPU fallback)")
            lib = C.CDLL(LIB_PATH)
            for name, (res, args) in PROTOTYPES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().bq_last_error()
        raise BqError(rc, msg.decode() if msg else "")


def init(device: int = 0) -> C.CDLL:
    """Load the library and bind it to a CUDA device (one process per GPU)."""
    global _inited_device
    lib = load()
    if _inited_device != device:
        check(lib.bq_init(int(device)))
        _inited_device = device
    return lib


def lib() -> C.CDLL:
    if _inited_device is None:
        raise BqError(ERR_STATE, "chadslab_b200._lib.init(device) has not been called")
    return _lib
