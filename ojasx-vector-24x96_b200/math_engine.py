"""CUDA execution of the package's LUT GEMM entry points.

``subspace_lut_rvq_gemm`` keeps the signature, shape rules, error text and dtype behaviour of
``ojasx_24x96/math_engine.py:136-208`` (widen to fp32, compute, cast back to the input dtype) and
``fused_rvq_gemm_native`` those of ``ojasx_24x96/leech_native.py:384-447``; the arithmetic runs in
libojasx_lut_b200.so on the tensors' device memory.  CPU tensors are rejected: there is no
fallback in this package.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import OjasxB200Error, check, lib
from .codec import QuantizedWeight


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _is_table_layout(encoded: QuantizedWeight) -> bool:
    return encoded.bits_per_stage == 8 and encoded.stages == 1 and encoded.block_size in (4, 8, 16, 32)


def _run(encoded: QuantizedWeight, flat_x: torch.Tensor, bias: Optional[torch.Tensor], row_start: int,
         row_stop: int) -> torch.Tensor:
    rows, columns = encoded.original_shape
    dev = flat_x.device
    if encoded.packed_codes.device != dev:
        raise OjasxB200Error("encoded tensors and inputs must live on the same CUDA device")
    b32 = None if bias is None else bias.to(device=dev, dtype=torch.float32).contiguous()
    batch = flat_x.shape[0]
    n = row_stop - row_start
    if _is_table_layout(encoded) and flat_x.dtype in (torch.float32, torch.bfloat16):
        # split-manifold layout: activations stay in their dtype, the kernel widens and rounds
        x = flat_x.contiguous()
        out = torch.empty((batch, n), device=dev, dtype=x.dtype)
        nnz, rp, ci, va = 0, None, None, None
        if encoded.outliers is not None and encoded.outliers[2].numel() > 0:
            rp, ci, va = (t.data_ptr() for t in encoded.outliers)
            nnz = int(encoded.outliers[2].numel())
        rc = lib().ojasx_b200_linear_forward_raw(
            encoded.packed_codes.data_ptr(), encoded.codebooks.data_ptr(), encoded.row_scales.data_ptr(),
            0 if b32 is None else b32.data_ptr(), nnz, rp, ci, va, x.data_ptr(), out.data_ptr(), batch,
            0 if x.dtype == torch.float32 else 1, encoded.block_size, 256, rows, columns, row_start, row_stop,
            _stream(dev))
        check(rc, "ojasx_b200_linear_forward_raw")
        return out
    if encoded.outliers is not None and encoded.outliers[2].numel() > 0:
        raise OjasxB200Error("CSR outliers are carried for the 8-bit single-stage layout only")
    x = flat_x.to(torch.float32).contiguous()
    out = torch.empty((batch, n), device=dev, dtype=torch.float32)
    rc = lib().ojasx_b200_rvq_fused_gemm(
        encoded.packed_codes.data_ptr(), encoded.codebooks.data_ptr(), encoded.row_scales.data_ptr(),
        0 if b32 is None else b32.data_ptr(), x.data_ptr(), batch, encoded.stages, encoded.bits_per_stage,
        encoded.block_size, rows, columns, row_start, row_stop, out.data_ptr(), _stream(dev))
    check(rc, "ojasx_b200_rvq_fused_gemm")
    return out.to(flat_x.dtype)


def subspace_lut_rvq_gemm(inputs: torch.Tensor, encoded: QuantizedWeight, bias: Optional[torch.Tensor] = None, *,
                          row_block_size: int = 256) -> torch.Tensor:
    """``Y[..., m] = row_scales[m] * sum_{s,g} <X[..., g, :], C[s, code[s,m,g], :]> + bias[m]``; returns the input dtype.

    ``row_block_size`` is accepted for signature compatibility; the kernels tile on their own.
    """
    rows, columns = encoded.original_shape
    if inputs.shape[-1] != columns:
        raise ValueError(f"Input feature mismatch: expected {columns}, got {inputs.shape[-1]}")
    if not inputs.is_cuda:
        raise OjasxB200Error("subspace_lut_rvq_gemm needs CUDA tensors: this package has no CPU path")
    flat = inputs.reshape(-1, columns)
    if flat.shape[0] == 0:
        return inputs.new_zeros(*inputs.shape[:-1], rows)
    out = _run(encoded, flat, bias, 0, rows)
    return out.to(inputs.dtype).reshape(*inputs.shape[:-1], rows)


def fused_rvq_gemm_native(encoded: QuantizedWeight, inputs: torch.Tensor, row_start: int, row_stop: int,
                          bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``[row_start, row_stop)`` only; output ``[batch, row_stop - row_start]`` fp32 like the reference."""
    rows, columns = encoded.original_shape
    if not 0 <= row_start < row_stop <= rows:
        raise IndexError("Invalid row range")
    if inputs.ndim != 2 or inputs.shape[1] != columns:
        raise ValueError(f"Expected inputs with {columns} features")
    if not inputs.is_cuda:
        raise OjasxB200Error("fused_rvq_gemm_native needs CUDA tensors: this package has no CPU path")
    return _run(encoded, inputs.to(torch.float32), bias, row_start, row_stop)


def compression_aware_linear_forward(inputs: torch.Tensor, module, *, use_subspace_lut: bool = False) -> torch.Tensor:
    """Inference branch of ``ojasx_24x96/math_engine.py:384-424`` (no autograd path here)."""
    return subspace_lut_rvq_gemm(inputs, module.encoded(), bias=module.bias)
