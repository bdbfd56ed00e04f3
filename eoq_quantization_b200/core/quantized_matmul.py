"""Interface of the reference's ``core/quantized_matmul.py``: matmul against a packed
quantised weight without the caller materialising it.  Dequantisation is the library's
kernel; the dense product is a library GEMM; ``QuantizedLinearFast`` additionally keeps
an entropy-coded resident copy and uses the fused decode+GEMV kernel for up to 8 rows."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..fused import GEMM_MAX_ROWS, EOQWeight, dequant_packed, fused_rows, gemv_packed, PACKED_TENSOR_ROWS, packed_gemv_rows, require_cuda

_SUPPORTED_BITS = (2, 4, 8)
_MEMORY_THRESHOLD = 16 * 1024 * 1024


def _mm_dtype(x: torch.Tensor) -> torch.dtype:
    return x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.float32


def fast_dequantize(packed_weight: torch.Tensor, scales: torch.Tensor, out_features: int, in_features: int,
                    bits: int = 4, block_size: int = 128) -> torch.Tensor:
    """float32 (N, K) (core/quantized_matmul.py:123-163)."""
    if bits not in _SUPPORTED_BITS:
        raise KeyError(bits)
    require_cuda(packed_weight, "fast_dequantize")
    return dequant_packed(packed_weight, scales, out_features, in_features, bits, block_size)


def dequantize_chunk(packed_weight: torch.Tensor, scales: torch.Tensor, start_row: int, end_row: int, in_features: int,
                     bits: int = 4, block_size: int = 128) -> torch.Tensor:
    """float32 rows [start_row, end_row) (core/quantized_matmul.py:170-225)."""
    if bits not in _SUPPORTED_BITS:
        raise KeyError(bits)
    require_cuda(packed_weight, "dequantize_chunk")
    return dequant_packed(packed_weight, scales, packed_weight.shape[0], in_features, bits, block_size, start_row, end_row)


def quantized_matmul_blocked(x, packed_weight, scales, out_features, in_features, bits=4, block_size=128, chunk_rows=64):
    """core/quantized_matmul.py:232-280: chunk_rows weight rows at a time, outputs concatenated."""
    require_cuda(x, "quantized_matmul_blocked")
    x2 = x.reshape(-1, in_features)
    dt = _mm_dtype(x)
    outs = []
    for lo in range(0, out_features, chunk_rows):
        hi = min(lo + chunk_rows, out_features)
        w = dequant_packed(packed_weight, scales, out_features, in_features, bits, block_size, lo, hi, dtype=dt)
        outs.append(x2 @ w.to(x.dtype).T)
    return torch.cat(outs, dim=-1).view(*x.shape[:-1], out_features)


def quantized_matmul_vectorized(x, packed_weight, scales, out_features, in_features, bits=4, block_size=128):
    """core/quantized_matmul.py:287-319."""
    require_cuda(x, "quantized_matmul_vectorized")
    w = dequant_packed(packed_weight, scales, out_features, in_features, bits, block_size, dtype=_mm_dtype(x))
    return F.linear(x, w.to(x.dtype))


def quantized_matmul(x: torch.Tensor, packed_weight: torch.Tensor, scales: torch.Tensor, out_features: int,
                     in_features: int, bits: int = 4, block_size: int = 128, *, strategy: str = "auto",
                     chunk_rows: int = 64, memory_threshold: int = _MEMORY_THRESHOLD) -> torch.Tensor:
    """core/quantized_matmul.py:331-380 (same dispatch rule and error)."""
    if strategy == "auto":
        strategy = "blocked" if out_features * in_features > memory_threshold else "vectorized"
    if strategy == "blocked":
        return quantized_matmul_blocked(x, packed_weight, scales, out_features, in_features, bits=bits,
                                        block_size=block_size, chunk_rows=chunk_rows)
    if strategy == "vectorized":
        return quantized_matmul_vectorized(x, packed_weight, scales, out_features, in_features, bits=bits,
                                           block_size=block_size)
    raise ValueError(f"Unknown strategy {strategy!r}; choose 'blocked', 'vectorized', or 'auto'")


class QuantizedLinearFast(nn.Module):
    """core/quantized_matmul.py:387-553."""

    def __init__(self, in_features: int, out_features: int, bits: int = 4, block_size: int = 128, bias: bool = False,
                 strategy: str = "auto", chunk_rows: int = 64):
        super().__init__()
        if bits not in _SUPPORTED_BITS:
            raise ValueError(f"Unsupported bits={bits}; choose from {list(_SUPPORTED_BITS)}")
        self.in_features, self.out_features = in_features, out_features
        self.bits, self.block_size, self.strategy, self.chunk_rows = bits, block_size, strategy, chunk_rows
        cols = (in_features + 1) // 2 if bits == 4 else (in_features + 3) // 4 if bits == 2 else in_features
        self.register_buffer("packed_weight", torch.zeros(out_features, cols, dtype=torch.uint8 if bits in (2, 4) else torch.int8))
        self.register_buffer("scales", torch.ones((out_features * in_features + block_size - 1) // block_size, dtype=torch.float16))
        if bias:
            self.register_buffer("bias_param", torch.zeros(out_features, dtype=torch.float16))
        else:
            self.bias_param = None
        self._eoq: Optional[EOQWeight] = None
        self._eoq_key = None

    @property
    def bias(self):
        return self.bias_param

    @bias.setter
    def bias(self, value):
        self.bias_param = value

    @classmethod
    def from_linear(cls, linear: nn.Linear, bits: int = 4, block_size: int = 128, strategy: str = "auto",
                    chunk_rows: int = 64) -> "QuantizedLinearFast":
        from .quantized_linear import QuantizedLinear
        return cls.from_quantized_linear(QuantizedLinear.from_float(linear, bits=bits, block_size=block_size),
                                         strategy=strategy, chunk_rows=chunk_rows)

    @classmethod
    def from_quantized_linear(cls, ql: nn.Module, strategy: str = "auto", chunk_rows: int = 64) -> "QuantizedLinearFast":
        """Shares (does not copy) the buffers of `ql`."""
        layer = cls(ql.in_features, ql.out_features, bits=ql.bits, block_size=ql.block_size,
                    bias=ql.bias_param is not None, strategy=strategy, chunk_rows=chunk_rows)
        layer.packed_weight = ql.packed_weight
        layer.scales = ql.scales
        if ql.bias_param is not None:
            layer.bias_param = ql.bias_param
        return layer

    def _fusable(self) -> bool:
        return (self.bits == 4 and self.in_features % 16 == 0 and self.block_size % 16 == 0
                and self.in_features % self.block_size == 0)

    def eoq_weight(self) -> EOQWeight:
        key = (self.packed_weight.data_ptr(), self.scales.data_ptr(), self.packed_weight._version, self.scales._version)
        if self._eoq is None or self._eoq_key != key:
            with torch.cuda.device(self.packed_weight.device):
                self._eoq = EOQWeight.from_int4_packed(self.packed_weight, self.scales, self.in_features, group=self.block_size)
            self._eoq_key = key
        return self._eoq

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        require_cuda(x, "QuantizedLinearFast.forward")
        rows = x.numel() // max(self.in_features, 1)
        if self.strategy == "auto" and x.dtype in (torch.float16, torch.bfloat16, torch.float32) and \
                1 <= rows <= PACKED_TENSOR_ROWS == packed_gemv_rows(self.in_features, self.bits, self.block_size, x.dtype):
            # one pass over the packed codes on the tensor cores (HBM-bound), see QuantizedLinear.forward
            return gemv_packed(self.packed_weight, self.scales, self.out_features, self.in_features, self.bits, self.block_size,
                               x, self.bias_param)
        if self.strategy == "auto" and self._fusable() and rows >= 1 and x.dtype in (torch.float16, torch.bfloat16, torch.float32):
            # up to fused_rows (4 rows of 16-bit activations, 8 of fp32): fused decode + GEMV, fp32 accumulate; beyond
            # that one dequantisation amortises over enough rows for a library GEMM to win (the fused tensor-core
            # kernel would take 9..GEMM_MAX_ROWS rows of 16-bit activations if that constant were raised)
            if rows <= fused_rows(x.dtype):
                return self.eoq_weight().gemv(x, self.bias_param)
            if 8 < rows <= GEMM_MAX_ROWS and x.dtype != torch.float32:
                return self.eoq_weight().gemm(x, self.bias_param)
        out = quantized_matmul(x, self.packed_weight, self.scales, self.out_features, self.in_features, bits=self.bits,
                               block_size=self.block_size, strategy=self.strategy, chunk_rows=self.chunk_rows)
        if self.bias_param is not None:
            out = out + self.bias_param.to(x.dtype)
        return out

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"block_size={self.block_size}, bias={self.bias_param is not None}, strategy={self.strategy!r}, "
                f"chunk_rows={self.chunk_rows}")

    def memory_bytes(self) -> int:
        total = self.packed_weight.numel() * self.packed_weight.element_size() + self.scales.numel() * self.scales.element_size()
        if self.bias_param is not None:
            total += self.bias_param.numel() * self.bias_param.element_size()
        return total

    def original_bytes(self) -> int:
        return self.out_features * self.in_features * 4 + (self.out_features * 4 if self.bias_param is not None else 0)

    def compression_ratio(self) -> float:
        return self.original_bytes() / self.memory_bytes()
