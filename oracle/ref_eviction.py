"""ctypes wrapper of oracle/_ref/libref_eviction.so: the reference's own cache_eviction.cpp and
kvcrush.cpp compiled unmodified (oracle/ref_eviction_bridge.cpp).  TEST INFRASTRUCTURE, CPU only."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_oracle

_lib = None


def lib():
    """The library, or None when it was never built (the reference tree is absent and no prebuilt file travelled)."""
    global _lib
    if _lib is None:
        path = build_oracle.REF_OUT / "libref_eviction.so"
        if not path.exists():
            build_oracle.build_reference()
        if not path.exists():
            return None
        _lib = C.CDLL(str(path))
        _lib.ref_eviction_select.restype = C.c_int
        _lib.ref_eviction_select.argtypes = [C.c_int] * 7 + [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_char_p, C.c_int]
        _lib.ref_snapkv_window.restype = C.c_int
        _lib.ref_snapkv_window.argtypes = [C.c_int] * 4
        _lib.ref_rotation_lut.restype = C.c_int
        _lib.ref_rotation_lut.argtypes = [C.c_int, C.c_int, C.c_int, C.c_double, C.c_void_p, C.c_void_p]
        if hasattr(_lib, "ref_eviction_new"):
            _lib.ref_eviction_new.restype = C.c_void_p
            _lib.ref_eviction_new.argtypes = [C.c_int] * 7
            _lib.ref_eviction_free.restype = None
            _lib.ref_eviction_free.argtypes = [C.c_void_p]
            _lib.ref_eviction_register.restype = C.c_int
            _lib.ref_eviction_register.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_char_p, C.c_int]
            _lib.ref_eviction_evict.restype = C.c_int
            _lib.ref_eviction_evict.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_char_p, C.c_int]
    return _lib


class Algorithm:
    """The reference's CacheEvictionAlgorithm for one sequence and one layer, kept alive over several steps."""

    def __init__(self, *, start_size, recent_size, max_cache_size, block_size, aggregation="NORM_SUM", snapkv_window=0, max_pool_window=7):
        self._h = lib().ref_eviction_new(start_size, recent_size, max_cache_size, 0 if aggregation == "SUM" else 1, snapkv_window, block_size, max_pool_window)
        if not self._h:
            raise RuntimeError("the reference rejected the eviction configuration")

    def register(self, scores, num_snapkv_scores=0):
        s = np.ascontiguousarray(scores, np.float32)
        err = C.create_string_buffer(512)
        if lib().ref_eviction_register(self._h, s.ctypes.data, len(s), int(num_snapkv_scores), err, 512) != 0:
            raise RuntimeError(err.value.decode())

    def evict(self):
        out = np.zeros(8192, np.int32)
        err = C.create_string_buffer(512)
        n = lib().ref_eviction_evict(self._h, out.ctypes.data, len(out), err, 512)
        if n < 0:
            raise RuntimeError(err.value.decode())
        return sorted(int(b) for b in out[:n])

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ref_eviction_free(self._h)
            self._h = None


def select_blocks(score_steps, snapkv_counts, *, start_size, recent_size, max_cache_size, block_size, aggregation="NORM_SUM",
                  snapkv_window=8, max_pool_window=1):
    """Registers the given per-step score vectors of ONE sequence and returns the sorted logical
    blocks CacheEvictionAlgorithm::evict_logical_blocks() selects."""
    flat = np.ascontiguousarray(np.concatenate([np.asarray(s, np.float32) for s in score_steps]))
    lens = np.array([len(s) for s in score_steps], np.int64)
    snap = np.array(snapkv_counts, np.int32)
    out = np.zeros(4096, np.int32)
    err = C.create_string_buffer(512)
    n = lib().ref_eviction_select(start_size, recent_size, max_cache_size, 0 if aggregation == "SUM" else 1, snapkv_window, block_size,
                                  max_pool_window, flat.ctypes.data, lens.ctypes.data, snap.ctypes.data, len(lens), out.ctypes.data, len(out),
                                  err, 512)
    if n < 0:
        raise RuntimeError(err.value.decode())
    return sorted(int(b) for b in out[:n])


def snapkv_window(snapkv_window_size, prompt_len, num_processed, num_scheduled) -> int:
    return int(lib().ref_snapkv_window(snapkv_window_size, prompt_len, num_processed, num_scheduled))


def rotation_lut(block_size, rows, head_size, theta):
    """The model_rotation_trig_lut layout: row i = cos row | sin row (the minus sign is in the reference's sin table)."""
    c = np.zeros((rows, head_size // 2), np.float32)
    s = np.zeros((rows, head_size // 2), np.float32)
    lib().ref_rotation_lut(block_size, rows, head_size, float(theta), c.ctypes.data, s.ctypes.data)
    return np.concatenate([c, s], axis=1)
