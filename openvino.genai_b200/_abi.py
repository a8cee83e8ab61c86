"""ctypes mirror of include/pa_b200.h and include/sampler_b200.h (struct layouts and prototypes)."""
from __future__ import annotations

import ctypes as C

PA_OK = 0
PA_ERR_INVALID_ARG = 1
PA_ERR_UNSUPPORTED = 2
PA_ERR_CUDA = 3
PA_ERR_BAD_INDEX = 4
PA_ERR_NO_DEVICE = 5
PA_ERR_TOO_LARGE = 6

PA_DTYPE_F32 = 0
PA_DTYPE_F16 = 1
PA_DTYPE_BF16 = 2
PA_DTYPE_U8 = 3

PA_DEV_BAD_BLOCK_INDEX = 0x1
PA_DEV_BAD_BEGINS = 0x2
PA_DEV_BAD_PAST_LEN = 0x4
PA_DEV_BAD_ROTATION = 0x8
PA_DEV_WAIT_TIMEOUT_SCORES = 0x20000000
PA_DEV_WAIT_TIMEOUT_PREFILL = 0x40000000
PA_DEV_WAIT_TIMEOUT_DECODE = 0x80000000


class pa_model_desc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_size", C.c_int32),
        ("block_size", C.c_int32),
        ("act_dtype", C.c_int32),
        ("cache_dtype", C.c_int32),
    ]


class pa_cache_layout(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("elem_dtype", C.c_int32),
        ("key_shape", C.c_int64 * 4),
        ("value_shape", C.c_int64 * 4),
        ("key_block_bytes", C.c_int64),
        ("value_block_bytes", C.c_int64),
        ("base_alignment", C.c_int32),
    ]


class pa_forward_args(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("query", C.c_void_p),
        ("key", C.c_void_p),
        ("value", C.c_void_p),
        ("output", C.c_void_p),
        ("num_tokens", C.c_int32),
        ("key_cache", C.c_void_p),
        ("value_cache", C.c_void_p),
        ("num_blocks", C.c_int32),
        ("past_lens", C.c_void_p),
        ("subsequence_begins", C.c_void_p),
        ("block_indices", C.c_void_p),
        ("block_indices_begins", C.c_void_p),
        ("num_sequences", C.c_int32),
        ("num_block_indices", C.c_int32),
        ("max_context_len", C.c_int32),
        ("scale", C.c_float),
        ("sliding_window", C.c_int32),
        ("alibi_slopes", C.c_void_p),
        ("score_aggregation_window", C.c_void_p),
        ("scores", C.c_void_p),
        ("scores_len", C.c_int64),
        ("rotated_block_indices", C.c_void_p),
        ("rotation_deltas", C.c_void_p),
        ("num_rotated_blocks", C.c_int32),
        ("rotation_trig_lut", C.c_void_p),
        ("rotation_lut_rows", C.c_int32),
        ("stream", C.c_void_p),
    ]


class pa_marshal_args(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("block_table", C.c_void_p),
        ("block_table_len", C.c_void_p),
        ("table_stride", C.c_int32),
        ("num_slots", C.c_int32),
        ("slot", C.c_void_p),
        ("num_processed_tokens", C.c_void_p),
        ("num_evicted_tokens", C.c_void_p),
        ("num_scheduled_tokens", C.c_void_p),
        ("skip_mask", C.c_void_p),
        ("skip_words", C.c_int32),
        ("num_sequences", C.c_int32),
        ("past_lens", C.c_void_p),
        ("subsequence_begins", C.c_void_p),
        ("block_indices", C.c_void_p),
        ("block_indices_begins", C.c_void_p),
        ("totals", C.c_void_p),
        ("block_indices_capacity", C.c_int32),
        ("stream", C.c_void_p),
    ]


PA_SYMBOLS = {
    "pa_b200_abi_version": (C.c_int, []),
    "pa_b200_last_error": (C.c_char_p, []),
    "pa_b200_query_cache_layout": (C.c_int, [C.POINTER(pa_model_desc), C.POINTER(pa_cache_layout)]),
    "pa_b200_create": (C.c_int, [C.POINTER(pa_model_desc), C.c_int, C.POINTER(C.c_void_p)]),
    "pa_b200_destroy": (C.c_int, [C.c_void_p]),
    "pa_b200_workspace_bytes": (C.c_int64, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64]),
    "pa_b200_reserve": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32]),
    "pa_b200_forward": (C.c_int, [C.c_void_p, C.POINTER(pa_forward_args)]),
    "pa_b200_forward_host": (C.c_int, [C.c_void_p, C.POINTER(pa_forward_args)]),
    "pa_b200_last_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "pa_b200_launch_count": (C.c_int64, [C.c_void_p]),
    "pa_b200_last_prefill_kernel": (C.c_int, [C.c_void_p]),
    "pa_b200_set_kernel_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "pa_b200_get_kernel_timing": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
    "pa_b200_write_kv": (C.c_int, [C.c_void_p, C.POINTER(pa_forward_args)]),
    "pa_b200_rotate_blocks": (C.c_int, [C.c_void_p, C.POINTER(pa_forward_args)]),
    "pa_b200_decode_step_static": (C.c_int, [C.POINTER(pa_model_desc), C.POINTER(pa_forward_args), C.c_int]),
    "pa_b200_cache_pool_last_error": (C.c_char_p, []),
    "pa_b200_cache_pool_create": (C.c_int, [C.POINTER(pa_model_desc), C.c_int, C.c_int64, C.c_int64, C.POINTER(C.c_void_p)]),
    "pa_b200_cache_pool_grow": (C.c_int, [C.c_void_p, C.c_int64]),
    "pa_b200_cache_pool_get": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64)]),
    "pa_b200_cache_pool_destroy": (C.c_int, [C.c_void_p]),
    "pa_b200_marshal_inputs": (C.c_int, [C.c_void_p, C.POINTER(pa_marshal_args)]),
    "pa_b200_copy_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
}


def bind(lib: C.CDLL, table: dict) -> None:
    """Sets restype/argtypes for every symbol of `table`; raises AttributeError if one is missing."""
    for name, (res, args) in table.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
