"""ctypes binding of ``liblmoe.so`` (the C ABI declared in ``include/lmoe.h``).

There is no fallback: if the library is missing it is built with nvcc, and if
that fails the import of any op raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_LIB = None

c_i32, c_i64, c_f32, c_sz, c_vp = C.c_int32, C.c_int64, C.c_float, C.c_size_t, C.c_void_p

# name -> (restype, argtypes); one line per declaration of include/lmoe.h
PROTOTYPES = {
    "lmoe_version": (C.c_char_p, []),
    "lmoe_last_error": (C.c_char_p, []),
    "lmoe_mm_id_min_seq": (c_i64, []),
    "lmoe_expert_stack_create": (c_i32, [c_i32, c_i64, c_i64, c_i64, c_vp, c_sz, c_sz, C.POINTER(c_vp)]),
    "lmoe_expert_stack_wrap": (c_i32, [c_i32, c_i64, c_i64, c_i64, c_vp, c_sz, c_sz, C.POINTER(c_vp)]),
    "lmoe_expert_stack_destroy": (None, [c_vp]),
    "lmoe_expert_stack_device_ptr": (c_vp, [c_vp]),
    "lmoe_expert_stack_info": (c_i32, [c_vp, C.POINTER(c_i32), C.POINTER(c_i64), C.POINTER(c_i64),
                                       C.POINTER(c_i64), C.POINTER(c_sz)]),
    "lmoe_quantize": (c_i32, [c_i32, c_vp, c_i64, c_vp, c_vp]),
    "lmoe_dequantize": (c_i32, [c_i32, c_vp, c_i64, c_vp, c_vp]),
    "lmoe_route_workspace_bytes": (c_sz, [c_i64, c_i64]),
    "lmoe_route": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_f32, c_i32, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_route_noalloc": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_f32, c_i32, c_vp, c_vp, c_vp]),
    "lmoe_route_from_logits": (c_i32, [c_vp, c_vp, c_i64, c_i64, c_i64, c_f32, c_i32, c_vp, c_vp, c_vp]),
    "lmoe_mul_mv_id": (c_i32, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "lmoe_mul_mv": (c_i32, [c_vp, c_i32, c_i64, c_i64, c_vp, c_i64, c_vp, c_vp]),
    "lmoe_map0_scratch_bytes": (c_sz, [c_i64, c_i64]),
    "lmoe_prepare_map0": (c_i32, [c_vp, c_i64, c_i64, c_i64, c_vp, c_sz, c_vp]),
    "lmoe_mm_id_supported": (c_i32, [c_i32, c_i64]),
    "lmoe_mm_id_workspace_bytes": (c_sz, [c_vp, c_i64, c_i64, c_i64]),
    "lmoe_mul_mm_id_shared": (c_i32, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_i64, c_i64, c_vp, c_i64, c_i64,
                                      c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_mul_mm_id": (c_i32, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_silu_mul": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp]),
    "lmoe_combine": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "lmoe_layer_create": (c_i32, [c_i64, c_i64, c_i64, c_i64, c_f32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                  c_vp, c_vp, C.POINTER(c_vp)]),
    "lmoe_layer_destroy": (None, [c_vp]),
    "lmoe_layer_workspace_bytes": (c_sz, [c_vp, c_i64]),
    "lmoe_moe_forward_decode": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_experts_workspace_bytes": (c_sz, [c_vp, c_i64]),
    "lmoe_experts_forward": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_experts_forward_ep": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_moe_forward_prefill": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_peer_alloc": (c_i32, [c_sz, C.POINTER(c_vp), c_vp]),
    "lmoe_peer_open": (c_i32, [c_vp, C.POINTER(c_vp)]),
    "lmoe_peer_close": (c_i32, [c_vp]),
    "lmoe_peer_free": (c_i32, [c_vp]),
    "lmoe_peer_ctrl_bytes": (c_sz, []),
    "lmoe_peer_put": (c_i32, [c_vp, c_i64, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "lmoe_peer_wait": (c_i32, [c_vp, c_i32, c_i32, c_vp]),
    "lmoe_moe_forward_host": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_moe_forward_host_async": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_experts_forward_rows": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_ep_pack_workspace_bytes": (c_sz, [c_i64, c_i64]),
    "lmoe_ep_pack": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_ep_localize_ids": (c_i32, [c_vp, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "lmoe_ep_combine": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "lmoe_experts_forward_rows_f16": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_rows_workspace_bytes": (c_sz, [c_vp, c_i64]),
    "lmoe_rms_norm": (c_i32, [c_vp, c_vp, C.c_float, c_i64, c_i64, c_vp, c_vp]),
    "lmoe_moe_layer_workspace_bytes": (c_sz, [c_vp, c_i64]),
    "lmoe_moe_layer_forward": (c_i32, [c_vp, c_vp, c_vp, C.c_float, c_i64, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_tokens_workspace_bytes": (c_sz, [c_vp, c_i64, c_i64]),
    "lmoe_experts_forward_tokens_f16": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_shared_forward": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "lmoe_check_device_flag": (c_i32, [c_vp, c_vp]),
}


class LmoeError(RuntimeError):
    """An entry point returned a non-zero status (the reference's ``Err``)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"lmoe status {status}: {message}")
        self.status = status
        self.message = message


def lib_path() -> str:
    return _build.LIB


def lib():
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path):
            path = _build.build()
        handle = C.CDLL(path)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(status: int):
    if status != 0:
        raise LmoeError(status, lib().lmoe_last_error().decode())
