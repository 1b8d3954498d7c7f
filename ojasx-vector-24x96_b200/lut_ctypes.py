"""Host-array bindings with the class names and methods of the reference's
``split_manifold_lut_experiment/native/bindings/ojasx_lut_ctypes.py`` (``:98-241``), bound to
libojasx_lut_b200.so.  Inputs and outputs are numpy arrays in host memory; each forward copies
its activations to the GPU, runs the CUDA kernels and copies the result back.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib

_vp = C.c_void_p


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def get_engine_info():
    L = lib()
    return {"version": L.ojasx_get_version().decode(), "backend": L.ojasx_get_backend_name().decode()}


class NativeSplitManifoldLinear:
    """ojasx_lut_ctypes.py:98-157."""

    def __init__(self, in_features: int, out_features: int, block_dim: int = 16, codebook_size: int = 256):
        self.in_features = in_features
        self.out_features = out_features
        self.block_dim = block_dim
        self.codebook_size = codebook_size
        self._handle = None

    def initialize_weights(self, codebook, codes, scales, bias=None):
        cb = np.ascontiguousarray(codebook, dtype=np.float32)
        cd = np.ascontiguousarray(codes, dtype=np.uint8)
        sc = None if scales is None else np.ascontiguousarray(scales, dtype=np.float32)
        bi = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self._handle = lib().ojasx_create_linear(self.in_features, self.out_features, self.block_dim,
                                                 self.codebook_size, _p(cb), _p(cd), _p(sc), _p(bi))
        if not self._handle:
            check(-3, "ojasx_create_linear")

    def set_outliers(self, row_ptrs, col_indices, values):
        assert self._handle is not None
        rp = np.ascontiguousarray(row_ptrs, dtype=np.int32)
        ci = np.ascontiguousarray(col_indices, dtype=np.int32)
        va = np.ascontiguousarray(values, dtype=np.float32)
        check(lib().ojasx_set_linear_outliers(self._handle, len(va), _p(rp), _p(ci), _p(va)),
              "ojasx_set_linear_outliers")

    def forward(self, x, num_threads: int = 0):
        assert self._handle is not None
        batch = x.shape[0] if x.ndim > 1 else 1
        xf = np.ascontiguousarray(x.reshape(batch, self.in_features), dtype=np.float32)
        y = np.zeros((batch, self.out_features), dtype=np.float32)
        ret = lib().ojasx_linear_forward(self._handle, _p(xf), _p(y), batch, num_threads)
        assert ret == 0, f"Forward failed with code {ret}"
        return y.squeeze(0) if x.ndim == 1 else y

    @property
    def handle(self):
        return self._handle

    @property
    def compressed_bytes(self) -> int:
        return lib().ojasx_get_compressed_size(self._handle) if self._handle else 0

    @property
    def compression_ratio(self) -> float:
        return lib().ojasx_get_compression_ratio(self._handle) if self._handle else 0.0

    def __del__(self):
        if getattr(self, "_handle", None):
            lib().ojasx_destroy_linear(self._handle)
            self._handle = None


class NativeKVCache:
    """ojasx_lut_ctypes.py:160-190 (the reference's cache as shipped)."""

    def __init__(self, num_heads: int, head_dim: int = 128, max_seq_len: int = 4096, block_dim: int = 16):
        self.num_heads = num_heads
        self.head_dim = head_dim
        self._handle = lib().ojasx_create_kv_cache(num_heads, head_dim, max_seq_len, block_dim)
        if not self._handle:
            check(-3, "ojasx_create_kv_cache")

    def append(self, head_idx: int, k, v):
        kc = np.ascontiguousarray(k, dtype=np.float32)
        vc = np.ascontiguousarray(v, dtype=np.float32)
        ret = lib().ojasx_kv_cache_append(self._handle, head_idx, _p(kc), _p(vc))
        assert ret == 0, f"KV append failed with code {ret}"

    def attention(self, head_idx: int, q, scale_factor: float = -1.0):
        qc = np.ascontiguousarray(q, dtype=np.float32)
        out = np.zeros(self.head_dim, dtype=np.float32)
        ret = lib().ojasx_kv_cache_attention(self._handle, head_idx, _p(qc), _p(out), scale_factor)
        assert ret == 0, f"Attention failed with code {ret}"
        return out

    @property
    def total_bytes(self) -> int:
        return lib().ojasx_kv_cache_get_memory_size(self._handle)

    @property
    def compression_ratio(self) -> float:
        return lib().ojasx_kv_cache_get_compression_ratio(self._handle)

    def __del__(self):
        if getattr(self, "_handle", None):
            lib().ojasx_destroy_kv_cache(self._handle)
            self._handle = None


class NativeSplitManifoldMoE:
    """ojasx_lut_ctypes.py:193-241."""

    def __init__(self, num_experts: int = 512, hidden_dim: int = 2560, intermediate_dim: int = 640, top_k: int = 10,
                 block_dim: int = 16):
        self.num_experts = num_experts
        self.hidden_dim = hidden_dim
        self.intermediate_dim = intermediate_dim
        self.top_k = top_k
        self.block_dim = block_dim
        self._handle = None

    def initialize_weights(self, codebook_in, codebook_down, gate_up_codes, gate_up_scales, down_codes, down_scales):
        a = [np.ascontiguousarray(codebook_in, dtype=np.float32), np.ascontiguousarray(codebook_down, dtype=np.float32),
             np.ascontiguousarray(gate_up_codes, dtype=np.uint8), np.ascontiguousarray(gate_up_scales, dtype=np.float32),
             np.ascontiguousarray(down_codes, dtype=np.uint8), np.ascontiguousarray(down_scales, dtype=np.float32)]
        self._handle = lib().ojasx_create_moe(self.num_experts, self.hidden_dim, self.intermediate_dim, self.top_k,
                                              self.block_dim, *[_p(t) for t in a])
        assert self._handle is not None, "Failed to create Native MoE engine handle"

    def forward(self, x, top_k_indices, top_k_weights):
        assert self._handle is not None
        xc = np.ascontiguousarray(x, dtype=np.float32)
        ic = np.ascontiguousarray(top_k_indices, dtype=np.int32)
        wc = np.ascontiguousarray(top_k_weights, dtype=np.float32)
        y = np.zeros(self.hidden_dim, dtype=np.float32)
        ret = lib().ojasx_moe_forward(self._handle, _p(xc), _p(ic), _p(wc), _p(y), len(ic))
        assert ret == 0, f"MoE forward failed with code {ret}"
        return y

    @property
    def handle(self):
        return self._handle

    @property
    def compressed_bytes(self) -> int:
        return lib().ojasx_moe_get_compressed_size(self._handle) if self._handle else 0

    @property
    def compression_ratio(self) -> float:
        return lib().ojasx_moe_get_compression_ratio(self._handle) if self._handle else 0.0

    def __del__(self):
        if getattr(self, "_handle", None):
            lib().ojasx_destroy_moe(self._handle)
            self._handle = None
