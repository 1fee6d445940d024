"""ctypes binding of libtorpor_swap.so (include/torpor_swap.h).

The library is the product: there is no Python or CPU implementation behind
these calls.  Importing this module fails loudly when the library has not been
built (``python -c "import __graft_entry__ as g; g.build()"`` or
``make -C torpor_b200/csrc``).
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libtorpor_swap.so")

OK = 0
ERR_INVALID, ERR_NO_DEVICE, ERR_CUDA, ERR_POOL_EXHAUSTED, ERR_UNKNOWN_MODEL = -1, -2, -3, -4, -5
ERR_TIMEOUT, ERR_NOT_FOUND, ERR_BUFFER, ERR_STATE, ERR_KERNEL = -6, -7, -8, -9, -10
READY_HOST, READY_PINNED, READY_CUDA = 0, 1, 2
MODEL_FULL, MODEL_INCOMPLETE, MODEL_PARTIAL, MODEL_NODATA = 0, 1, 2, 3
POOL_BUDDY, POOL_FIXED = 0, 1
STORE_DEFAULT, STORE_WRITE_COMBINED, STORE_HUGE_PAGES = 0, 1, 2

_ERR_NAMES = {
    -1: "TSW_ERR_INVALID", -2: "TSW_ERR_NO_DEVICE", -3: "TSW_ERR_CUDA", -4: "TSW_ERR_POOL_EXHAUSTED",
    -5: "TSW_ERR_UNKNOWN_MODEL", -6: "TSW_ERR_TIMEOUT", -7: "TSW_ERR_NOT_FOUND", -8: "TSW_ERR_BUFFER",
    -9: "TSW_ERR_STATE", -10: "TSW_ERR_KERNEL",
}


class SwapError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{_ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class Config(C.Structure):
    _fields_ = [
        ("device", C.c_int),
        ("server_id", C.c_int),
        ("gpu_count", C.c_int),
        ("budget_bytes", C.c_uint64),
        ("pool_policy", C.c_int),
        ("host_arena_bytes", C.c_uint64),
        ("host_arena_shm", C.c_char_p),
        ("grid_ctas", C.c_int),
        ("tile_bytes_host", C.c_int),
        ("tile_bytes_device", C.c_int),
        ("mover", C.c_int),
        ("shard_static", C.c_int),
        ("host_store_mode", C.c_int),
        ("ticket_chunk", C.c_int),
        ("grid_ctas_host", C.c_int),
    ]


class Segment(C.Structure):
    _fields_ = [("src", C.c_uint64), ("dst", C.c_uint64), ("bytes", C.c_uint64), ("row_dst", C.c_uint64),
                ("row", C.c_uint32), ("row_tiles", C.c_uint32)]


class Publish(C.Structure):
    _fields_ = [("done_count", C.c_uint64), ("table_phys", C.c_uint64), ("table_flag", C.c_uint64),
                ("host_phys", C.c_uint64), ("host_flag", C.c_uint64), ("flag_value", C.c_uint32),
                ("ticket_chunk", C.c_uint32), ("ticket", C.c_uint64)]


class IpcRegion(C.Structure):
    _fields_ = [("base", C.c_uint64), ("size", C.c_uint64), ("handle", C.c_ubyte * 64)]


# Every symbol include/torpor_swap.h declares: name -> (restype, argtypes)
_u64, _i32, _i64, _vp, _cp = C.c_uint64, C.c_int, C.c_int64, C.c_void_p, C.c_char_p
SIGNAL_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int, C.c_char_p)    # tsw_signal_fn
ACK_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int)                    # tsw_ack_fn
_pu64 = C.POINTER(C.c_uint64)
SIGNATURES = {
    "tsw_config_default": (None, [C.POINTER(Config)]),
    "tsw_last_error": (_cp, []),
    "tsw_version": (_cp, []),
    "tsw_repo_reset": (_i32, []),
    "tsw_repo_add_model_info": (_i32, [_cp, _i32]),
    "tsw_repo_remove_model_info": (_i32, [_cp, _i32]),
    "tsw_repo_model_status": (_i32, [_cp, _i32]),
    "tsw_repo_total_size": (_u64, [_cp]),
    "tsw_repo_active_devices": (_i32, [_cp, C.POINTER(C.c_int), _i32]),
    "tsw_engine_create": (_i32, [C.POINTER(Config), C.POINTER(_vp)]),
    "tsw_engine_destroy": (_i32, [_vp]),
    "tsw_track_begin": (_i32, [_vp, _cp]),
    "tsw_track_end": (_i32, [_vp, _cp]),
    "tsw_malloc": (_i32, [_vp, _cp, _u64, _i32, _pu64]),
    "tsw_free": (_i32, [_vp, _cp, _u64]),
    "tsw_memcpy_h2d_model": (_i32, [_vp, _cp, _u64, _vp, _u64, _vp]),
    "tsw_sync_done": (_i32, [_vp, _cp]),
    "tsw_mark_access": (_i32, [_vp, _u64]),
    "tsw_memcpy_h2d": (_i32, [_vp, _cp, _u64, _vp, _u64, _vp]),
    "tsw_memcpy_d2h": (_i32, [_vp, _cp, _vp, _u64, _u64, _vp]),
    "tsw_memcpy_d2d": (_i32, [_vp, _cp, _u64, _u64, _u64, _vp]),
    "tsw_memset": (_i32, [_vp, _cp, _u64, _i32, _u64, _vp]),
    "tsw_swap_in": (_i32, [_vp, _cp, _i32]),
    "tsw_swap_in_sharded": (_i32, [_vp, _cp, C.POINTER(_vp), _i32]),
    "tsw_wait_ready": (_i32, [_vp, _cp, _i64]),
    "tsw_poll_ready": (_i32, [_vp, _cp]),
    "tsw_check_alloc": (_i32, [_vp, _cp]),
    "tsw_evict": (_i32, [_vp, _cp, _i32]),
    "tsw_translate": (_i32, [_vp, _cp, _u64, _i32, _i64, _pu64]),
    "tsw_translate_async": (_i32, [_vp, _cp, _u64, _vp, _pu64, C.POINTER(C.c_int)]),
    "tsw_release_waiters": (_i32, [_vp, _cp]),
    "tsw_is_model_address": (_i32, [_vp, _cp, _u64]),
    "tsw_valid_memory_address": (_i32, [_vp, _cp, _u64]),
    "tsw_dump_blocks": (_i32, [_vp, _cp, _i32, _vp, _i32]),
    "tsw_dump_params": (_i32, [_vp, _cp, _i32, _vp, _i32]),
    "tsw_pool_info": (_i32, [_vp, _pu64, _pu64, _pu64]),
    "tsw_canonical_address": (_i32, [_vp, _cp, _u64, _pu64]),
    "tsw_read_phys": (_i32, [_vp, _u64, _vp, _u64]),
    "tsw_read_host_store": (_i32, [_vp, _cp, _u64, _vp, _u64]),
    "tsw_checksum_resident": (_i32, [_vp, _cp, _vp, _i32]),
    "tsw_place_segments": (_i32, [_vp, _vp, _i32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _vp, _i32]),
    "tsw_swap_plan": (_i32, [_vp, _cp, _vp, _i32, C.POINTER(C.c_uint32), _vp]),
    "tsw_swap_commit": (_i32, [_vp, _cp]),
    "tsw_ipc_regions": (_i32, [_vp, _vp, _i32]),
    "tsw_ipc_open": (_i32, [_vp, _vp, _pu64]),
    "tsw_pointer_info": (_i32, [_vp, _u64, C.POINTER(C.c_int), C.POINTER(C.c_int), _pu64, _pu64]),
    "tsw_arena_info": (_i32, [_vp, _pu64, _pu64, _pu64, _pu64]),
    "tsw_arena_attach": (_i32, [_vp, _cp, _u64, _pu64]),
    "tsw_place_segments_pipelined": (_i32, [_vp, _vp, _i32, C.c_uint32, C.c_uint32, C.c_uint32, _vp, C.c_uint32, _i32]),
    "tsw_place_segments_static": (_i32, [_i32, _vp, _i32, C.c_uint32, C.c_uint32, C.c_uint32, _vp, _vp]),
    "tsw_place_segments_static_status": (_i32, [_i32, _vp, C.POINTER(C.c_uint32), _i32]),
    "tsw_stats": (_i32, [_vp, _pu64, _pu64, _pu64]),
    "tsw_evictor_create": (_i32, [_cp, _i32, _u64, C.POINTER(_vp)]),
    "tsw_evictor_destroy": (_i32, [_vp]),
    "tsw_evictor_check_and_add": (_i32, [_vp, _i32, _cp, _u64, _i32, _vp, _i32]),
    "tsw_evictor_force_evict": (_i32, [_vp, _i32, _cp]),
    "tsw_evictor_lock": (_i32, [_vp, _i32, _cp]),
    "tsw_evictor_unlock": (_i32, [_vp, _i32, _cp]),
    "tsw_topology_discover": (_i32, [_i32, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tsw_sched_create": (_i32, [_i32, _cp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(_vp)]),
    "tsw_sched_destroy": (_i32, [_vp]),
    "tsw_sched_set_status": (_i32, [_vp, _i32, _i32]),
    "tsw_sched_set_level": (_i32, [_vp, _cp, _i32]),
    "tsw_sched_decide": (_i32, [_vp, _cp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tsw_sched_helpers": (_i32, [_vp, _i32, _i32, C.POINTER(C.c_int), _i32]),
    "tsw_ctrl_helpers": (_i32, [_vp, _i32, _i32, C.POINTER(C.c_int), _i32]),
    "tsw_ctrl_create": (_i32, [_i32, _u64, _cp, _cp, C.POINTER(C.c_int), C.POINTER(C.c_int), SIGNAL_FN, ACK_FN, _vp,
                               C.POINTER(_vp)]),
    "tsw_ctrl_destroy": (_i32, [_vp]),
    "tsw_ctrl_request": (_i32, [_vp, _i32, _cp, _cp]),
    "tsw_ctrl_complete": (_i32, [_vp, _i32]),
    "tsw_ctrl_executor_status": (_i32, [_vp, _i32, C.POINTER(C.c_int), C.c_char_p, _i32]),
    "tsw_ctrl_queue_depth": (_i32, [_vp]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library, with argument types set."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: the swap engine has no fallback path. Build it with "
                "`make -C torpor_b200/csrc` (needs nvcc).")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> int:
    if rc < 0:
        raise SwapError(rc, lib().tsw_last_error().decode(errors="replace"))
    return rc
