"""The GGML dispatch shim (ojasx_ggml_*) against the CPU oracle: same struct and calls a llama.cpp
node would make (reference: tests of the adapter's callees in native/tests/test_lut_linear.cpp and
test_moe_kv_cache.cpp; the adapter itself forwards, ojasx_ggml_adapter.cpp:29-92)."""
import ctypes as C

import numpy as np
import pytest

import ojasx_b200
from ojasx_b200 import lut_ctypes, synth
from ojasx_b200._lib import GgmlTensor

pytestmark = pytest.mark.gpu


def test_ggml_linear_node(cuda, oracle):
    L = ojasx_b200.lib()
    assert L.ojasx_ggml_init() == 0 and L.ojasx_ggml_init() == 0
    w = synth.make_vq_linear(21, 2560, 2560, block_dim=8)
    layer = lut_ctypes.NativeSplitManifoldLinear(2560, 2560, 8, 256)
    layer.initialize_weights(w.codebook, w.codes, np.ones(2560, np.float32))
    layer.set_outliers(*w.csr)
    for batch in (1, 3):
        x = np.random.default_rng(batch).standard_normal((batch, 2560)).astype(np.float32)
        y = np.zeros((batch, 2560), np.float32)
        src0, dst = GgmlTensor.of(x), GgmlTensor.of(y)
        weight = GgmlTensor.of(None, extra=layer._handle, type_=100)
        # a four-worker node: every worker calls, worker 0 computes
        for ith in range(4):
            assert L.ojasx_ggml_forward_linear(C.byref(dst), C.byref(src0), C.byref(weight), ith, 4, None) == 0
        want = oracle.linear_forward(w.codebook, w.codes, None, None, w.csr, x, block_dim=8)
        assert np.array_equal(y, want)
        # handle through userdata, single worker
        y[:] = 0
        bare = GgmlTensor.of(None, type_=100)
        assert L.ojasx_ggml_forward_linear(C.byref(dst), C.byref(src0), C.byref(bare), 0, 1, layer._handle) == 0
        assert np.array_equal(y, want)
    # error codes of ojasx_ggml_adapter.cpp:37-46
    assert L.ojasx_ggml_forward_linear(None, C.byref(src0), C.byref(weight), 0, 1, None) == -1
    assert L.ojasx_ggml_forward_linear(C.byref(dst), C.byref(src0), C.byref(bare), 0, 1, None) == -2
    empty = GgmlTensor.of(None)
    assert L.ojasx_ggml_forward_linear(C.byref(empty), C.byref(src0), C.byref(weight), 0, 1, None) == -3


def test_ggml_moe_and_kv_nodes(cuda, oracle):
    L = ojasx_b200.lib()
    w = synth.make_vq_moe(5, 16, 256, 64, block_dim=8, outlier_frac=0.0)
    moe = lut_ctypes.NativeSplitManifoldMoE(16, 256, 64, 4, 8)
    moe.initialize_weights(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                           w.down_scales)
    x = np.random.default_rng(3).standard_normal(256).astype(np.float32)
    idx = np.array([3, 9, 0, 15], np.int32)
    wt = np.array([0.4, 0.3, 0.2, 0.1], np.float32)
    y = np.zeros(256, np.float32)
    assert L.ojasx_ggml_forward_moe(C.byref(GgmlTensor.of(y)), C.byref(GgmlTensor.of(x)), idx.ctypes.data,
                                    wt.ctypes.data, 4, moe._handle) == 0
    want = oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                              w.down_scales, x, idx, wt, block_dim=8)
    assert np.all(np.abs(y - want) <= 1e-6 + 1e-5 * np.abs(want))
    assert L.ojasx_ggml_forward_moe(C.byref(GgmlTensor.of(y)), C.byref(GgmlTensor.of(x)), None, wt.ctypes.data, 4,
                                    moe._handle) == -1
    assert L.ojasx_ggml_forward_moe(C.byref(GgmlTensor.of(None)), C.byref(GgmlTensor.of(x)), idx.ctypes.data,
                                    wt.ctypes.data, 4, moe._handle) == -2

    cache = lut_ctypes.NativeKVCache(2, 64, 8, 32)
    rng = np.random.default_rng(4)
    ks = rng.standard_normal((5, 64)).astype(np.float32)
    vs = rng.standard_normal((5, 64)).astype(np.float32)
    for k, v in zip(ks, vs):
        cache.append(1, k, v)
    q = rng.standard_normal(64).astype(np.float32)
    out = np.zeros(64, np.float32)
    assert L.ojasx_ggml_forward_kv_attention(C.byref(GgmlTensor.of(out)), C.byref(GgmlTensor.of(q)), 1, 0.125,
                                             cache._handle) == 0
    assert np.array_equal(out, cache.attention(1, q, 0.125))
    assert L.ojasx_ggml_forward_kv_attention(C.byref(GgmlTensor.of(out)), C.byref(GgmlTensor.of(q)), 1, 0.125, None) == -1
