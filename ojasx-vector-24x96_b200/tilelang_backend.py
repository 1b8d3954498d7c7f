"""``dispatch_universal_compressed_gemm`` with the contract of ``ojasx_24x96/tilelang_backend.py:272-338``.

The reference function picks between its CPU library and its torch LUT GEMM and returns the
result with the tile schedule it chose.  Here there is one backend (the sm_100a kernels), so the
schedule object only reports the tile those kernels use.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch

from .math_engine import fused_rvq_gemm_native, subspace_lut_rvq_gemm


@dataclass(frozen=True)
class HardwareTileSchedule:
    backend: str = "cuda_sm_100a"
    block_m: int = 1        # tokens per table
    block_n: int = 32       # rows per warp block
    block_k: int = 1024     # features per table slice (128 groups x block_dim 8)
    num_stages: int = 4     # cp.async ring depth
    threads: int = 512


def dispatch_universal_compressed_gemm(inputs: torch.Tensor, encoded: Any, bias: Optional[torch.Tensor] = None, *,
                                       prefer_subspace_lut: bool = True,
                                       row_block_size: int = 256) -> Tuple[torch.Tensor, HardwareTileSchedule]:
    rows, columns = encoded.original_shape
    schedule = HardwareTileSchedule(block_k=128 * encoded.block_size)
    if prefer_subspace_lut:
        return subspace_lut_rvq_gemm(inputs, encoded, bias=bias, row_block_size=row_block_size), schedule
    flat = inputs.reshape(-1, columns)
    out = fused_rvq_gemm_native(encoded, flat, 0, rows, bias=bias)
    return out.to(inputs.dtype).reshape(*inputs.shape[:-1], rows), schedule
