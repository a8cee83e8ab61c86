"""numpy-facing wrapper of oracle/sampler_oracle.cpp and of the compiled reference transforms
(oracle/_ref/libref_sampler.so).  TEST INFRASTRUCTURE, CPU only."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_oracle

_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = build_oracle.BUILD / "libsampler_oracle.so"
        if not path.exists():
            build_oracle.build_restatements()
        _lib = C.CDLL(str(path))
        _lib.sampler_oracle_step.restype = C.c_int
        _lib.sampler_oracle_step.argtypes = [C.c_void_p, C.c_int]
        _lib.sampler_oracle_transform.restype = C.c_int
        _lib.sampler_oracle_transform.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p]
        _lib.sampler_oracle_uniform_stream.restype = None
        _lib.sampler_oracle_uniform_stream.argtypes = [C.c_uint32, C.c_int, C.c_void_p]
        _lib.sampler_oracle_hardware_threads.restype = C.c_int
    return _lib


def ref_lib():
    """The reference's own transforms, or None when oracle/_ref was never built."""
    global _ref
    if _ref is None:
        path = build_oracle.REF_OUT / "libref_sampler.so"
        if not path.exists():
            build_oracle.build_reference()
        if not path.exists():
            return None
        _ref = C.CDLL(str(path))
        _ref.ref_transform.restype = C.c_int
        _ref.ref_transform.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p]
        _ref.ref_penalty.restype = C.c_int
        _ref.ref_penalty.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        _ref.ref_eos_mask.restype = C.c_int
        _ref.ref_eos_mask.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        _ref.ref_filter_chain.restype = C.c_int
        _ref.ref_filter_chain.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
    return _ref


def hardware_threads() -> int:
    return int(lib().sampler_oracle_hardware_threads())


def step(args, threads: int = 0) -> int:
    """`args` is the product's sampler_step_args ctypes struct over HOST buffers."""
    return int(lib().sampler_oracle_step(C.byref(args), threads or hardware_threads()))


def transform(which: int, data, param: float, use_reference: bool = False):
    x = np.array(data, np.float32)
    p = np.zeros(len(x), np.float32)
    idx = np.zeros(len(x), np.int64)
    fn = ref_lib().ref_transform if use_reference else lib().sampler_oracle_transform
    n = fn(which, x.ctypes.data, len(x), float(param), p.ctypes.data, idx.ctypes.data)
    return p[:n].copy(), idx[:n].copy(), x


def uniform_stream(seed: int, n: int) -> np.ndarray:
    out = np.zeros(n, np.float32)
    lib().sampler_oracle_uniform_stream(seed, n, out.ctypes.data)
    return out
