"""ctypes mirror of include/exchange_b200.h."""
from __future__ import annotations

import ctypes as C

EXCHANGE_OK = 0
EXCHANGE_ERR_INVALID_ARG = 1
EXCHANGE_ERR_NO_NCCL = 2
EXCHANGE_ERR_NCCL = 3
EXCHANGE_ERR_CUDA = 4
ID_BYTES = 128

EXCHANGE_SYMBOLS = {
    "exchange_b200_last_error": (C.c_char_p, []),
    "exchange_b200_unique_id": (C.c_int, [C.c_void_p]),
    "exchange_b200_create": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "exchange_b200_destroy": (C.c_int, [C.c_void_p]),
    "exchange_b200_local_row": (C.c_void_p, [C.c_void_p]),
    "exchange_b200_all_rows": (C.c_void_p, [C.c_void_p]),
    "exchange_b200_all_gather_ids": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
}
