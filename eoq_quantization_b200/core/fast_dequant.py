"""Interface of the reference's ``core/fast_dequant.py``; the arithmetic is the
library's dequantisation kernel."""
from __future__ import annotations

import torch

from ..fused import dequant_packed, require_cuda


def _unpack(packed: torch.Tensor, out_features: int, in_features: int, bits: int) -> torch.Tensor:
    return dequant_packed(packed, None, out_features, in_features, bits, 128, dtype=torch.int8)      # the kernel writes the codes


def unpack_4bit_fast(packed: torch.Tensor, out_features: int, in_features: int) -> torch.Tensor:
    """uint8 (N, K/2) -> int8 (N, K) in [-7, 7]; low nibble first (core/fast_dequant.py:9-27)."""
    require_cuda(packed, "unpack_4bit_fast")
    return _unpack(packed, out_features, in_features, 4)


def unpack_2bit_fast(packed: torch.Tensor, out_features: int, in_features: int) -> torch.Tensor:
    """uint8 (N, K/4) -> int8 (N, K) in [-1, 1] (core/fast_dequant.py:30-44)."""
    require_cuda(packed, "unpack_2bit_fast")
    return _unpack(packed, out_features, in_features, 2)


def dequantize_weight_fast(packed: torch.Tensor, scales: torch.Tensor, out_features: int, in_features: int,
                           bits: int = 4, block_size: int = 128) -> torch.Tensor:
    """float32 (N, K): unpack, then multiply by the scale of the element's block in the
    FLATTENED matrix (core/fast_dequant.py:47-87)."""
    require_cuda(packed, "dequantize_weight_fast")
    return dequant_packed(packed, scales, out_features, in_features, bits, block_size)
