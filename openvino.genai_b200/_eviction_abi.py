"""ctypes mirror of include/eviction_b200.h."""
from __future__ import annotations

import ctypes as C

EVICTION_OK = 0
AGG_SUM = 0
AGG_NORM_SUM = 1


class eviction_config_b200(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("start_size", C.c_int32), ("recent_size", C.c_int32), ("max_cache_size", C.c_int32),
                ("block_size", C.c_int32), ("aggregation", C.c_int32), ("snapkv_window_size", C.c_int32), ("max_pool_window", C.c_int32),
                ("num_layers", C.c_int32), ("num_slots", C.c_int32), ("max_tracked_tokens", C.c_int32), ("max_evicted_blocks", C.c_int32)]


class eviction_step_args(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("layer", C.c_int32), ("num_sequences", C.c_int32), ("scores", C.c_void_p),
                ("span_begin", C.c_void_p), ("span_len", C.c_void_p), ("slot", C.c_void_p), ("num_snapkv_scores", C.c_void_p),
                ("do_evict", C.c_int32), ("evicted_count", C.c_void_p), ("evicted_blocks", C.c_void_p), ("stream", C.c_void_p)]


EVICTION_SYMBOLS = {
    "eviction_b200_last_error": (C.c_char_p, []),
    "eviction_b200_create": (C.c_int, [C.POINTER(eviction_config_b200), C.c_int, C.POINTER(C.c_void_p)]),
    "eviction_b200_destroy": (C.c_int, [C.c_void_p]),
    "eviction_b200_reset_slot": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "eviction_b200_step": (C.c_int, [C.c_void_p, C.POINTER(eviction_step_args)]),
    "eviction_b200_last_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "eviction_b200_read_slot": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
}
