"""Container and bit-packing of the package's residual-VQ layout.

Mirrors the parts of ``ojasx_24x96/codec.py`` that the execution path reads: ``QuantizedWeight``
(``:76-173``) and ``pack_codes`` / ``unpack_codes`` (``:176-214``).  The k-means encoder is offline
tooling and is not part of this package.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

SUPPORTED_WIDTHS = (1, 2, 4, 8)


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Little-endian packing: code i occupies bits [(i % per_byte)*bits, ...) of byte i // per_byte."""
    if bits not in SUPPORTED_WIDTHS:
        raise ValueError("Only 1-, 2-, 4-, and 8-bit codes are supported")
    if codes.dtype not in (torch.uint8, torch.int16, torch.int32, torch.int64):
        raise TypeError("Codes must have an integer dtype")
    flat = codes.reshape(-1)
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= (1 << bits)):
        raise ValueError("A code exceeds the requested bit width")
    if bits == 8:
        return flat.to(torch.uint8).clone()
    per_byte = 8 // bits
    n = flat.numel()
    padded = torch.zeros((n + per_byte - 1) // per_byte * per_byte, dtype=torch.int32, device=flat.device)
    padded[:n] = flat.to(torch.int32)
    lanes = padded.view(-1, per_byte)
    out = torch.zeros(lanes.shape[0], dtype=torch.int32, device=flat.device)
    for k in range(per_byte):
        out |= lanes[:, k] << (k * bits)
    return out.to(torch.uint8)


def unpack_codes(packed: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    if bits not in SUPPORTED_WIDTHS:
        raise ValueError("Only 1-, 2-, 4-, and 8-bit codes are supported")
    if packed.dtype != torch.uint8 or count < 0:
        raise ValueError("Packed codes must be uint8 and count nonnegative")
    expected = (count * bits + 7) // 8
    if packed.numel() != expected:
        raise ValueError(f"Expected {expected} packed bytes, received {packed.numel()}")
    if count == 0:
        return torch.empty(0, dtype=torch.uint8, device=packed.device)
    per_byte = 8 // bits
    wide = packed.reshape(-1, 1).to(torch.int32)
    shifts = torch.arange(per_byte, device=packed.device, dtype=torch.int32) * bits
    return ((wide >> shifts) & ((1 << bits) - 1)).reshape(-1)[:count].to(torch.uint8)


@dataclass
class QuantizedWeight:
    """Encoded rank-two weight: ``packed_codes u8[stages, ceil(M*G*bits/8)]``, ``codebooks f32[stages, 2^bits, D]``,
    ``row_scales f32[M]`` -- the tensor names and shapes of the reference container."""

    original_shape: Tuple[int, int]
    block_size: int
    bits_per_stage: int
    packed_codes: torch.Tensor
    codebooks: torch.Tensor
    row_scales: torch.Tensor
    metrics: Dict[str, object] = field(default_factory=dict)
    # CSR outliers added after the row scale, as SplitManifoldLinear does (ojasx_lut.h:66-71):
    # (row_ptrs i32[M+1], col_indices i32[nnz], values f32[nnz]) on the tensors' device.  The reference
    # container has no such field; it is carried for the 8-bit single-stage layout only.
    outliers: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None

    def __post_init__(self) -> None:
        if len(self.original_shape) != 2:
            raise ValueError("Only rank-two weights are supported")
        if self.bits_per_stage not in SUPPORTED_WIDTHS:
            raise ValueError("Unsupported code width")
        if self.packed_codes.dtype != torch.uint8:
            raise TypeError("packed_codes must be uint8")
        if self.codebooks.dtype != torch.float32 or self.row_scales.dtype != torch.float32:
            raise TypeError("Codebooks and scales use float32 storage")
        if not (self.packed_codes.device == self.codebooks.device == self.row_scales.device):
            raise ValueError("All encoded tensors must be on one device")
        rows, columns = self.original_shape
        if self.codebooks.ndim != 3 or self.codebooks.shape[0] < 1:
            raise ValueError("Codebooks must be a rank-three tensor with at least one stage")
        if tuple(self.codebooks.shape[1:]) != (1 << self.bits_per_stage, self.block_size):
            raise ValueError("Codebook shape is inconsistent with the codec")
        expected = (rows * self.blocks_per_row * self.bits_per_stage + 7) // 8
        if tuple(self.packed_codes.shape) != (self.stages, expected):
            raise ValueError("Packed-code shape is inconsistent with the weight shape")
        if tuple(self.row_scales.shape) != (rows,):
            raise ValueError("Row-scale shape is inconsistent with the weight shape")

    @property
    def stages(self) -> int:
        return int(self.codebooks.shape[0])

    @property
    def blocks_per_row(self) -> int:
        return (self.original_shape[1] + self.block_size - 1) // self.block_size

    @property
    def vector_count(self) -> int:
        return self.original_shape[0] * self.blocks_per_row

    @property
    def storage_bytes(self) -> int:
        return (self.packed_codes.numel() + self.codebooks.numel() * 4 + self.row_scales.numel() * 4)

    def codes(self, stage: int) -> torch.Tensor:
        if not 0 <= stage < self.stages:
            raise IndexError("Invalid residual stage")
        return unpack_codes(self.packed_codes[stage], self.bits_per_stage, self.vector_count)

    def to(self, device) -> "QuantizedWeight":
        outliers = None if self.outliers is None else tuple(t.to(device) for t in self.outliers)
        return QuantizedWeight(self.original_shape, self.block_size, self.bits_per_stage, self.packed_codes.to(device),
                               self.codebooks.to(device), self.row_scales.to(device), dict(self.metrics), outliers=outliers)


def dequantize_weight(encoded: QuantizedWeight) -> torch.Tensor:
    """Dense fp32 weight (test helper: the reference's tests compare fast paths against dequantise + F.linear)."""
    rows, columns = encoded.original_shape
    G, D = encoded.blocks_per_row, encoded.block_size
    w = torch.zeros(rows * G, D, dtype=torch.float32, device=encoded.codebooks.device)
    for s in range(encoded.stages):
        w += encoded.codebooks[s][encoded.codes(s).long()]
    w = w.view(rows, G * D)[:, :columns]
    return w * encoded.row_scales[:, None]
