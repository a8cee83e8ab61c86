"""numpy-facing wrapper of oracle/pa_oracle.cpp (TEST INFRASTRUCTURE, CPU only).

The oracle takes the product's own `pa_forward_args` struct with HOST pointers, so a test builds
one set of inputs and hands it to both sides.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build_oracle

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = build_oracle.BUILD / "libpa_oracle.so"
        if not path.exists():
            build_oracle.build_restatements()
        _lib = C.CDLL(str(path))
        for name in ("pa_oracle_forward", "pa_oracle_attend"):
            getattr(_lib, name).restype = C.c_int
            getattr(_lib, name).argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        for name in ("pa_oracle_rotate_blocks", "pa_oracle_write_kv"):
            getattr(_lib, name).restype = C.c_int
            getattr(_lib, name).argtypes = [C.c_void_p, C.c_void_p]
        _lib.pa_oracle_gather_dense.restype = None
        _lib.pa_oracle_gather_dense.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        _lib.pa_oracle_hardware_threads.restype = C.c_int
    return _lib


def hardware_threads() -> int:
    return int(lib().pa_oracle_hardware_threads())


def forward(desc, args, threads: int = 0) -> int:
    """rotate listed blocks -> write the chunk -> attend; `desc`/`args` are ctypes structs."""
    return int(lib().pa_oracle_forward(C.byref(desc), C.byref(args), threads or hardware_threads()))


def attend(desc, args, threads: int = 0) -> int:
    return int(lib().pa_oracle_attend(C.byref(desc), C.byref(args), threads or hardware_threads()))


def write_kv(desc, args) -> int:
    return int(lib().pa_oracle_write_kv(C.byref(desc), C.byref(args)))


def rotate_blocks(desc, args) -> int:
    return int(lib().pa_oracle_rotate_blocks(C.byref(desc), C.byref(args)))


def gather_dense(desc, key_cache: np.ndarray, value_cache: np.ndarray, table: np.ndarray, ctx: int, kv_head: int, head_size: int):
    k = np.empty((ctx, head_size), np.float32)
    v = np.empty((ctx, head_size), np.float32)
    table = np.ascontiguousarray(table, np.int32)
    lib().pa_oracle_gather_dense(C.byref(desc), key_cache.ctypes.data, value_cache.ctypes.data, table.ctypes.data, ctx, kv_head,
                                 k.ctypes.data, v.ctypes.data)
    return k, v
