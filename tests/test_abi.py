"""The C-ABI library loads without a GPU and exports every symbol the headers declare."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared(header: Path):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b((?:pa|sampler|exchange|eviction)_b200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib(pkg):
    pkg.build_all()
    return pkg.load_library()


@pytest.mark.parametrize("header", sorted((ROOT / "include").glob("*.h")), ids=lambda p: p.name)
def test_every_declared_symbol_is_exported(lib, header):
    names = _declared(header)
    assert names, f"no entry points found in {header}"
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"{header.name} declares symbols the library does not export: {missing}"


def test_abi_version(lib):
    assert lib.pa_b200_abi_version() == 1


def test_cache_layout_query(pkg, lib):
    from openvino_genai_b200 import _abi
    desc = _abi.pa_model_desc(C.sizeof(_abi.pa_model_desc), 32, 8, 128, 32, _abi.PA_DTYPE_BF16, _abi.PA_DTYPE_U8)
    out = _abi.pa_cache_layout()
    out.struct_size = C.sizeof(_abi.pa_cache_layout)
    assert lib.pa_b200_query_cache_layout(C.byref(desc), C.byref(out)) == _abi.PA_OK
    assert list(out.key_shape) == [0, 8, 32, 136]
    assert out.key_block_bytes == 8 * 32 * 136 and out.value_block_bytes == out.key_block_bytes
    desc.cache_dtype = _abi.PA_DTYPE_F16
    assert lib.pa_b200_query_cache_layout(C.byref(desc), C.byref(out)) == _abi.PA_OK
    assert list(out.key_shape) == [0, 8, 32, 128] and out.key_block_bytes == 8 * 32 * 128 * 2


def test_invalid_descriptors_are_rejected(pkg, lib):
    from openvino_genai_b200 import _abi
    out = _abi.pa_cache_layout()
    out.struct_size = C.sizeof(_abi.pa_cache_layout)
    bad_heads = _abi.pa_model_desc(C.sizeof(_abi.pa_model_desc), 30, 8, 128, 32, _abi.PA_DTYPE_BF16, _abi.PA_DTYPE_U8)
    assert lib.pa_b200_query_cache_layout(C.byref(bad_heads), C.byref(out)) == _abi.PA_ERR_INVALID_ARG
    bad_size = _abi.pa_model_desc(C.sizeof(_abi.pa_model_desc), 32, 8, 96, 32, _abi.PA_DTYPE_BF16, _abi.PA_DTYPE_U8)
    assert lib.pa_b200_query_cache_layout(C.byref(bad_size), C.byref(out)) == _abi.PA_ERR_UNSUPPORTED
    wrong_struct = _abi.pa_model_desc(4, 32, 8, 128, 32, _abi.PA_DTYPE_BF16, _abi.PA_DTYPE_U8)
    assert lib.pa_b200_query_cache_layout(C.byref(wrong_struct), C.byref(out)) == _abi.PA_ERR_INVALID_ARG
    assert b"struct_size" in lib.pa_b200_last_error()
