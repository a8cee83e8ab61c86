"""B200-native per-step compute of a continuous-batching pipeline: the PagedAttention operator
and the Sampler, as hand-written sm_100a CUDA behind a C ABI (include/*.h).

This Python layer is a thin host-side mirror of the operator / sampler interface used by tests
and the benchmark.  It never computes anything itself: if the CUDA library is missing the
import of `load_library()` fails loudly.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

from . import _abi
from .build import LIB_PATH, build_all

__all__ = ["load_library", "library_path", "build_all", "PagedAttentionExtension", "GenaiB200Error"]

_lib = None


class GenaiB200Error(RuntimeError):
    """Raised where the reference would raise ov::Exception."""


def library_path() -> Path:
    return LIB_PATH


def load_library(build_if_missing: bool = False) -> ctypes.CDLL:
    """Loads lib/libgenai_b200.so and binds every symbol the headers declare."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if not build_if_missing:
            raise GenaiB200Error(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; there is no CPU fallback")
        build_all()
    lib = ctypes.CDLL(str(LIB_PATH))
    _abi.bind(lib, _abi.PA_SYMBOLS)
    from . import _sampler_abi
    _abi.bind(lib, _sampler_abi.SAMPLER_SYMBOLS)
    from . import _exchange_abi
    _abi.bind(lib, _exchange_abi.EXCHANGE_SYMBOLS)
    from . import _eviction_abi
    _abi.bind(lib, _eviction_abi.EVICTION_SYMBOLS)
    _lib = lib
    return lib


from .paged_attention import PagedAttentionExtension  # noqa: E402
