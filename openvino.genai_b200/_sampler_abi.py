"""ctypes mirror of include/sampler_b200.h."""
from __future__ import annotations

import ctypes as C

SAMPLER_OK = 0
SAMPLER_ERR_INVALID_ARG = 1
SAMPLER_ERR_UNSUPPORTED = 2
SAMPLER_ERR_CUDA = 3
SAMPLER_ERR_BAD_TOKEN_ID = 4
SAMPLER_ERR_TOO_LARGE = 5

HIST_IN_PROMPT = 0x1
HIST_GENERATED = 0x2
HIST_STOP_MASK = 0x4

TOP_K_OFF = 2 ** 63 - 1

ROW_MULTINOMIAL = 0x1
ROW_RAW_LOG_PROB = 0x2


class sampler_row_params(C.Structure):
    _fields_ = [
        ("logits_row", C.c_int64),
        ("top_k", C.c_int64),
        ("do_sample", C.c_int32),
        ("temperature", C.c_float),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repetition_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("rand_u", C.c_float),
    ]


class sampler_step_args(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("logits", C.c_void_p),
        ("num_logit_rows", C.c_int64),
        ("vocab", C.c_int64),
        ("num_rows", C.c_int32),
        ("rows", C.c_void_p),
        ("hist_offsets", C.c_void_p),
        ("hist_ids", C.c_void_p),
        ("hist_meta", C.c_void_p),
        ("out_token", C.c_void_p),
        ("out_log_prob", C.c_void_p),
        ("stream", C.c_void_p),
        ("hist_raw", C.c_void_p),
        ("extra_offsets", C.c_void_p),
        ("extra_rand_u", C.c_void_p),
        ("extra_out_token", C.c_void_p),
        ("extra_out_log_prob", C.c_void_p),
        ("token_bitmasks", C.c_void_p),
        ("bitmask_index", C.c_void_p),
        ("bitmask_words", C.c_int64),
    ]


ROW_DTYPE = [("logits_row", "<i8"), ("top_k", "<i8"), ("do_sample", "<i4"), ("temperature", "<f4"), ("top_p", "<f4"),
             ("min_p", "<f4"), ("repetition_penalty", "<f4"), ("presence_penalty", "<f4"), ("frequency_penalty", "<f4"),
             ("rand_u", "<f4")]

SAMPLER_SYMBOLS = {
    "sampler_b200_last_error": (C.c_char_p, []),
    "sampler_b200_create": (C.c_int, [C.c_int, C.c_int32, C.c_int64, C.POINTER(C.c_void_p)]),
    "sampler_b200_destroy": (C.c_int, [C.c_void_p]),
    "sampler_b200_step": (C.c_int, [C.c_void_p, C.POINTER(sampler_step_args)]),
    "sampler_b200_step_host": (C.c_int, [C.c_void_p, C.POINTER(sampler_step_args), C.c_int]),
    "sampler_b200_last_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "sampler_b200_launch_count": (C.c_int64, [C.c_void_p]),
    "sampler_b200_selftest_expf": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]),
}
