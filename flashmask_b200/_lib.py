"""ctypes binding of libflashmask_b200.so (the C ABI in include/flashmask_b200.h).

The library is loaded lazily and never replaced by a fallback: if the shared
object is missing or a call fails, a RuntimeError is raised with the native
error message.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashmask_b200.so")

FM_OK = 0
FM_DTYPE_BF16, FM_DTYPE_FP16 = 0, 1
FM_ORDER_FWD, FM_ORDER_BWD_DQ, FM_ORDER_BWD_DKDV = 0, 1, 2
FM_BWD_DQ_CARRY, FM_BWD_DQ_LEAVE = 1, 2
TILE_SKIP, TILE_PARTIAL, TILE_FULL = 0, 1, 2

I64x3 = C.c_int64 * 3


class AttnArgs(C.Structure):
    """Mirror of ``fm_attn_args``."""
    _fields_ = [
        ("B", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32), ("Hq", C.c_int32),
        ("Hkv", C.c_int32), ("Hm", C.c_int32), ("d", C.c_int32), ("dv", C.c_int32),
        ("ncols", C.c_int32), ("causal", C.c_int32), ("dtype", C.c_int32),
        ("mask_B", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32),
        ("deterministic", C.c_int32), ("bwd_flags", C.c_int32),
        ("softmax_scale", C.c_float), ("reserved1", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("o", C.c_void_p), ("lse", C.c_void_p),
        ("mask", C.c_void_p), ("minmax", C.c_void_p), ("sink", C.c_void_p),
        ("d_o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p),
        ("dv_out", C.c_void_p), ("dsink", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3), ("o_stride", I64x3),
        ("do_stride", I64x3), ("dq_stride", I64x3), ("dk_stride", I64x3), ("dv_stride", I64x3),
        ("fwd_order", C.c_void_p), ("dq_order", C.c_void_p), ("dkdv_order", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/flashmask_b200.h declares
SIGNATURES = {
    "fm_version": (C.c_char_p, []),
    "fm_last_error": (C.c_char_p, []),
    "fm_mask_nblk_pad": (C.c_int, [C.c_int, C.c_int]),
    "fm_mask_prepare": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fm_mask_count_visible": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_int, C.c_void_p, C.c_void_p]),
    "fm_fwd_tile_shape": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "fm_bwd_tile_shape": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "fm_reload_options": (C.c_int, []),
    "fm_launch_count": (C.c_ulonglong, []),
    "fm_fwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fm_fwd_block_score": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "fm_launch_order_ints": (C.c_int64, [C.POINTER(AttnArgs), C.c_int]),
    "fm_launch_order": (C.c_int, [C.POINTER(AttnArgs), C.c_int, C.c_void_p, C.c_void_p]),
    "fm_launch_orders": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fm_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "fm_bwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fm_bwd_accumulates": (C.c_int, [C.POINTER(AttnArgs)]),
    "fm_kernel_status": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "fm_selftest_bounded_wait": (C.c_int, [C.c_int, C.c_void_p]),
    "fm_bwd_static_scratch": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fm_cp_chunk_workload": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "fm_cp_partition_heap": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "fm_cp_partition_ipo": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "fm_cp_rerank": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, C.c_void_p]),
    "fm_cp_localize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "fm_cp_shard_visible": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_void_p, C.c_void_p]),
    "fm_cp_merge_partial": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fm_cp_merge_two": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fm_cp_accumulate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "fm_cp_cast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "fm_cp_reduce_partials": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_int64, C.c_int,
                                        C.c_void_p]),
}

_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m flashmask_b200.build` "
                    "(nvcc, sm_100a). There is no fallback path.")
            lib = C.CDLL(LIB_PATH, mode=C.RTLD_LOCAL)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != FM_OK:
        msg = load().fm_last_error().decode()
        cls = {1: ValueError, 2: NotImplementedError}.get(rc, RuntimeError)
        raise cls(f"{what} failed (status {rc}): {msg}")


def reload_options() -> None:
    """Have the library read its FLASHMASK_B200_* switches from the environment again (it reads
    them once at load; nothing on the call path does)."""
    check(load().fm_reload_options(), "fm_reload_options")
