"""RVQ half of the reference's backend ABI (``ojasx_24x96/backend_abi.py``): status codes, the
56-byte ``ojasx_rvq_layer_desc_t`` mirror and the ggml-style dispatch, with device pointers in the
descriptor instead of host pointers.  The Leech-lattice half is a different codec and out of scope.
"""
from __future__ import annotations

import ctypes
from enum import IntEnum
from typing import Dict, Optional, Tuple

import torch

from .math_engine import fused_rvq_gemm_native

OJASX_BACKEND_ABI_VERSION = 1
OJASX_MAX_STAGES = 8


class OjasxStatus(IntEnum):
    """ojasx_status_e (ojasx_24x96/native/ojasx_backend_abi.h:24-32) plus the CUDA-side codes of this library."""
    OK = 0
    INVALID_ARGUMENT = -1
    NULL_POINTER = -2
    MISSING_PRESENCE = -3
    GAIN_OUT_OF_RANGE = -5
    DECODE_POINT_FAILED = -6
    ABI_MISMATCH = -7


class CRVQLayerDesc(ctypes.Structure):
    """ojasx_rvq_layer_desc_t (ojasx_backend_abi.h:50-60): four pointers and five int32, 56 bytes."""
    _fields_ = [("packed_codes", ctypes.c_void_p), ("codebooks", ctypes.c_void_p), ("row_scales", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("stages", ctypes.c_int32), ("bits_per_stage", ctypes.c_int32),
                ("block_size", ctypes.c_int32), ("rows", ctypes.c_int32), ("columns", ctypes.c_int32)]


def build_c_layer_descriptor(layer) -> Tuple[CRVQLayerDesc, Dict[str, object]]:
    """Descriptor over the layer's DEVICE tensors; the metadata dict keeps them alive (borrowed pointers)."""
    enc = layer.encoded()
    desc = CRVQLayerDesc()
    desc.stages, desc.bits_per_stage, desc.block_size = enc.stages, enc.bits_per_stage, enc.block_size
    desc.rows, desc.columns = enc.original_shape
    pc, cb, rs = enc.packed_codes.contiguous(), enc.codebooks.contiguous(), enc.row_scales.contiguous()
    bias = None if layer.bias is None else layer.bias.contiguous()
    desc.packed_codes = pc.data_ptr() if pc.numel() else 0
    desc.codebooks = cb.data_ptr() if cb.numel() else 0
    desc.row_scales = rs.data_ptr() if rs.numel() else 0
    desc.bias = bias.data_ptr() if bias is not None and bias.numel() else 0
    tensors = {"packed_codes": pc, "codebooks": cb, "row_scales": rs}
    if bias is not None:
        tensors["bias"] = bias
    meta = {"codec": "OJASX_RVQ", "abi_version": OJASX_BACKEND_ABI_VERSION, "shape": (desc.rows, desc.columns),
            "rows": desc.rows, "columns": desc.columns, "stages": desc.stages, "bits_per_stage": desc.bits_per_stage,
            "block_size": desc.block_size, "workspace_bytes": 0, "has_bias": bias is not None,
            "device": str(pc.device), "tensors": tensors}
    return desc, meta


class LlamaCppGGMLAdapter:
    @staticmethod
    def dispatch_ggml_custom_matmul(layer, input_tensor: torch.Tensor, *, prefer_native: bool = True) -> torch.Tensor:
        """``backend_abi.py:457-516``: flatten, fused GEMM through the C ABI, no dense weight cache, reshape, input dtype."""
        if input_tensor.shape[-1] != layer.in_features:
            raise ValueError(f"Expected inputs with {layer.in_features} features, got {input_tensor.shape[-1]}")
        flat = input_tensor.reshape(-1, layer.in_features)
        out = fused_rvq_gemm_native(layer.encoded(), flat.to(torch.float32), 0, layer.out_features, bias=layer.bias)
        if layer.cached_weight_bytes != 0:
            raise RuntimeError(f"Unreported dense weight cache detected in ggml dispatch: {layer.cached_weight_bytes} bytes")
        return out.to(input_tensor.dtype).reshape(*input_tensor.shape[:-1], layer.out_features)
