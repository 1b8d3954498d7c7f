"""CPU tests of the boundary: the library builds, loads, and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    import importlib
    build = importlib.import_module("ojasx-vector-24x96_b200.build")
    return build.build()


def _declared():
    names = []
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"OJASX_API\s+[^;(]*?\b(ojasx_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_reference_handle_api():
    want = """ojasx_get_version ojasx_get_backend_name ojasx_create_linear ojasx_set_linear_outliers
    ojasx_linear_forward ojasx_get_compressed_size ojasx_get_dense_size ojasx_get_lut_sram_size
    ojasx_get_compression_ratio ojasx_destroy_linear ojasx_create_kv_cache ojasx_kv_cache_append
    ojasx_kv_cache_attention ojasx_kv_cache_get_memory_size ojasx_kv_cache_get_compression_ratio
    ojasx_destroy_kv_cache ojasx_create_moe ojasx_moe_forward ojasx_moe_get_compressed_size
    ojasx_moe_get_compression_ratio ojasx_destroy_moe""".split()
    declared = _declared()
    assert all(n in declared for n in want)


def test_library_exports_every_declared_symbol(built_lib):
    L = ctypes.CDLL(built_lib)
    missing = [n for n in _declared() if not hasattr(L, n)]
    assert not missing, missing
    assert L.ojasx_get_backend_name is not None
    L.ojasx_get_version.restype = ctypes.c_char_p
    L.ojasx_get_backend_name.restype = ctypes.c_char_p
    assert b"B200" in L.ojasx_get_version()
    assert b"sm_100a" in L.ojasx_get_backend_name()


def test_python_signatures_cover_the_header(built_lib):
    import ojasx_b200
    from ojasx_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    assert ojasx_b200.lib() is not None


def test_null_arguments_are_rejected_without_a_gpu(built_lib):
    """Argument checks of the handle API run before any CUDA call (ojasx_lut_c_api.cpp:100, 154, 267)."""
    import ojasx_b200
    L = ojasx_b200.lib()
    assert L.ojasx_linear_forward(None, None, None, 1, 0) == -1
    assert L.ojasx_moe_forward(None, None, None, None, None, 10) == -1
    assert L.ojasx_kv_cache_append(None, 0, None, None) == -1
    assert L.ojasx_kv_cache_attention(None, 0, None, None, 1.0) == -1
    assert L.ojasx_set_linear_outliers(None, 0, None, None, None) == -1
    assert L.ojasx_get_compressed_size(None) == 0
    assert L.ojasx_get_compression_ratio(None) == 0.0
    assert L.ojasx_b200_linear_forward(None, None, None, 1, 0, 0, 1, None) == -1
    assert L.ojasx_b200_moe_forward(None, None, None, None, None, 1, 1, 0, None) == -1
    assert L.ojasx_b200_kvq_decode(None, None, None, 1.0, 0, None) == -1
    assert L.ojasx_ggml_forward_linear(None, None, None, 0, 1, None) == -1       # ojasx_ggml_adapter.cpp:37
    assert L.ojasx_ggml_forward_moe(None, None, None, None, 1, None) == -1           # :68
    assert L.ojasx_ggml_forward_kv_attention(None, None, 0, 1.0, None) == -1         # :85
    L.ojasx_destroy_linear(None)
    L.ojasx_destroy_moe(None)
    L.ojasx_destroy_kv_cache(None)
