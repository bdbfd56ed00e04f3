"""``QuantizedLinear`` with the interface of the reference's
``core/quantized_linear.py``.  Buffers, packing and ``from_float`` are the
reference's; ``forward`` runs on the GPU: for up to 8 activation rows the
weights are kept entropy-coded in HBM and consumed by the fused
decode+dequantise+GEMV kernel, otherwise they are dequantised by the library
and multiplied with a library GEMM."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..fused import GEMM_MAX_ROWS, EOQWeight, dequant_packed, fused_rows, gemv_packed, PACKED_TENSOR_ROWS, packed_gemv_rows, require_cuda


class QuantizedLinear(nn.Module):
    """core/quantized_linear.py:19-285."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, bits: int = 4, block_size: int = 128):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.bits = bits
        self.block_size = block_size
        if bits == 4:
            self.register_buffer("packed_weight", torch.zeros(out_features, (in_features + 1) // 2, dtype=torch.uint8))
        elif bits == 2:
            self.register_buffer("packed_weight", torch.zeros(out_features, (in_features + 3) // 4, dtype=torch.uint8))
        else:
            self.register_buffer("packed_weight", torch.zeros(out_features, in_features, dtype=torch.int8))
        num_blocks = (out_features * in_features + block_size - 1) // block_size
        self.register_buffer("scales", torch.ones(num_blocks, dtype=torch.float16))
        if bias:
            self.register_buffer("bias_param", torch.zeros(out_features, dtype=torch.float32))
        else:
            self.bias_param = None
        self._eoq: Optional[EOQWeight] = None
        self._eoq_key = None

    # -- packing (host-side, exact) -------------------------------------------
    @staticmethod
    def pack_4bit(codes: torch.Tensor) -> torch.Tensor:
        """[-7, 7] -> code+7, two per byte, low nibble first (core/quantized_linear.py:76-91)."""
        u = (codes.flatten().to(torch.int32) + 7).to(torch.uint8)
        if len(u) % 2:
            u = torch.cat([u, torch.zeros(1, dtype=torch.uint8, device=u.device)])
        return u[0::2] | (u[1::2] << 4)

    @staticmethod
    def unpack_4bit(packed: torch.Tensor, num_elements: int) -> torch.Tensor:
        lo = (packed & 0x0F).to(torch.int32)
        hi = ((packed >> 4) & 0x0F).to(torch.int32)
        return (torch.stack([lo, hi], dim=-1).flatten()[:num_elements] - 7).to(torch.int8)

    @staticmethod
    def pack_2bit(codes: torch.Tensor) -> torch.Tensor:
        u = (codes.flatten().to(torch.int32) + 1).to(torch.uint8)
        pad = (4 - len(u) % 4) % 4
        if pad:
            u = torch.cat([u, torch.zeros(pad, dtype=torch.uint8, device=u.device)])
        return u[0::4] | (u[1::4] << 2) | (u[2::4] << 4) | (u[3::4] << 6)

    @staticmethod
    def unpack_2bit(packed: torch.Tensor, num_elements: int) -> torch.Tensor:
        parts = [((packed >> s) & 0x03).to(torch.int32) for s in (0, 2, 4, 6)]
        return (torch.stack(parts, dim=-1).flatten()[:num_elements] - 1).to(torch.int8)

    @classmethod
    def from_float(cls, linear: nn.Linear, bits: int = 4, block_size: int = 128) -> "QuantizedLinear":
        """Quantise an nn.Linear: per-block absmax over the flattened weight, fp16 scales,
        row-wise packing (core/quantized_linear.py:126-184)."""
        ql = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, bits=bits, block_size=block_size)
        with torch.no_grad():
            w = linear.weight.data.float().cpu()
            flat = w.flatten()
            n = flat.numel()
            pad = (block_size - n % block_size) % block_size
            if pad:
                flat = torch.cat([flat, torch.zeros(pad)])
            blocks = flat.view(-1, block_size)
            qmax = (1 << (bits - 1)) - 1
            scales = (blocks.abs().amax(dim=1) / qmax).clamp(min=1e-10)
            q = (blocks / scales.unsqueeze(1)).round().clamp(-qmax, qmax).to(torch.int8).flatten()[:n].view(w.shape)
            ql.scales.copy_(scales.to(torch.float16))
            if bits == 4:
                u = (q.to(torch.int32) + 7).to(torch.uint8)
                if u.shape[1] % 2:
                    u = torch.cat([u, torch.zeros(u.shape[0], 1, dtype=torch.uint8)], dim=1)
                ql.packed_weight.copy_(u[:, 0::2] | (u[:, 1::2] << 4))
            elif bits == 2:
                u = (q.to(torch.int32) + 1).to(torch.uint8)
                padc = (4 - u.shape[1] % 4) % 4
                if padc:
                    u = torch.cat([u, torch.zeros(u.shape[0], padc, dtype=torch.uint8)], dim=1)
                ql.packed_weight.copy_(u[:, 0::4] | (u[:, 1::4] << 2) | (u[:, 2::4] << 4) | (u[:, 3::4] << 6))
            else:
                ql.packed_weight.copy_(q)
            if linear.bias is not None:
                ql.bias_param.copy_(linear.bias.data.float())
        return ql.to(linear.weight.device)

    from_linear = from_float

    # -- GPU paths ---------------------------------------------------------------
    def _fusable(self) -> bool:
        return (self.bits in (2, 3, 4, 8) and self.in_features % 16 == 0 and self.block_size % 16 == 0
                and self.in_features % self.block_size == 0)

    def eoq_weight(self) -> EOQWeight:
        """The entropy-coded resident form of this layer's weight (built on first use, rebuilt if
        the buffers are replaced)."""
        key = (self.packed_weight.data_ptr(), self.scales.data_ptr(), self.packed_weight._version, self.scales._version)
        if self._eoq is None or self._eoq_key != key:
            with torch.cuda.device(self.packed_weight.device):
                self._eoq = EOQWeight.from_packed(self.packed_weight, self.scales, self.in_features, self.bits, group=self.block_size)
            self._eoq_key = key
        return self._eoq

    def _dequantize_weight(self) -> torch.Tensor:
        """float32 (out_features, in_features) (core/quantized_linear.py:189-217)."""
        require_cuda(self.packed_weight, "QuantizedLinear._dequantize_weight")
        return dequant_packed(self.packed_weight, self.scales, self.out_features, self.in_features, self.bits, self.block_size)

    _dequantize = _dequantize_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x of shape (..., in_features), any float dtype -> (..., out_features) in x.dtype."""
        require_cuda(x, "QuantizedLinear.forward")
        require_cuda(self.packed_weight, "QuantizedLinear.forward")
        rows = x.numel() // max(self.in_features, 1)
        if x.dtype in (torch.float16, torch.bfloat16, torch.float32) and \
                1 <= rows <= PACKED_TENSOR_ROWS == packed_gemv_rows(self.in_features, self.bits, self.block_size, x.dtype):
            # up to 32 rows: one pass over the packed codes this module keeps resident, codes to exact 16-bit floats in
            # registers and warp-level tensor-core products (fp32 activations as two fp16 halves each); the
            # entropy-coded form of the same weight (`eoq_weight()`) trades that speed for 7-15 % less memory and is
            # what `EOQLinear` holds.  Other group sizes take the routes below.
            return gemv_packed(self.packed_weight, self.scales, self.out_features, self.in_features, self.bits, self.block_size,
                               x, self.bias_param)
        if self._fusable() and rows >= 1 and x.dtype in (torch.float16, torch.bfloat16, torch.float32):
            # up to fused_rows (4 rows of 16-bit activations, 8 of fp32): fused decode + GEMV, fp32 accumulate; beyond
            # that one dequantisation amortises over enough rows for a library GEMM to win (the fused tensor-core
            # kernel would take 9..GEMM_MAX_ROWS rows of 16-bit activations if that constant were raised)
            if rows <= fused_rows(x.dtype):
                return self.eoq_weight().gemv(x, self.bias_param)
            if 8 < rows <= GEMM_MAX_ROWS and x.dtype != torch.float32 and self.bits == 4:          # the tensor-core kernel is built for the 4-bit layout
                return self.eoq_weight().gemm(x, self.bias_param)
        weight = dequant_packed(self.packed_weight, self.scales, self.out_features, self.in_features, self.bits,
                                self.block_size, dtype=x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.float32)
        bias = self.bias_param.to(x.dtype) if self.bias_param is not None else None
        return F.linear(x, weight.to(x.dtype), bias)

    # -- bookkeeping (core/quantized_linear.py:230-285) ---------------------------
    def memory_bytes(self) -> dict:
        packed = self.packed_weight.numel() * self.packed_weight.element_size()
        scales = self.scales.numel() * self.scales.element_size()
        bias = self.bias_param.numel() * self.bias_param.element_size() if self.bias_param is not None else 0
        orig = self.out_features * self.in_features * 4 + (self.out_features * 4 if self.bias_param is not None else 0)
        return {"packed_bytes": packed, "scales_bytes": scales, "bias_bytes": bias,
                "total_bytes": packed + scales + bias, "original_fp32_bytes": orig}

    def total_memory_bytes(self) -> int:
        return self.memory_bytes()["total_bytes"]

    def original_bytes(self) -> int:
        return self.memory_bytes()["original_fp32_bytes"]

    def compression_ratio(self) -> float:
        m = self.memory_bytes()
        return m["original_fp32_bytes"] / m["total_bytes"]

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"block_size={self.block_size}, bias={self.bias_param is not None}")

    @property
    def bias(self):
        return self.bias_param

    @bias.setter
    def bias(self, value):
        self.bias_param = value


def _pack_int4(codes: torch.Tensor) -> torch.Tensor:
    return QuantizedLinear.pack_4bit(codes.to(torch.int8))


def _unpack_int4(packed: torch.Tensor, numel: int) -> torch.Tensor:
    return QuantizedLinear.unpack_4bit(packed, numel).to(torch.int32)


def replace_linear_with_quantized(model: nn.Module, bits: int = 4, block_size: int = 128, min_size: int = 256) -> int:
    """Swap every nn.Linear with at least `min_size` weights for a QuantizedLinear, in place;
    returns the number replaced (core/quantized_linear.py:319-347)."""
    replaced = 0
    for name, module in list(model.named_children()):
        if isinstance(module, nn.Linear) and module.weight.numel() >= min_size:
            setattr(model, name, QuantizedLinear.from_float(module, bits=bits, block_size=block_size))
            replaced += 1
        elif not isinstance(module, QuantizedLinear):
            replaced += replace_linear_with_quantized(module, bits=bits, block_size=block_size, min_size=min_size)
    return replaced


def get_model_memory(model: nn.Module) -> dict:
    """Memory breakdown with the reference's keys (core/quantized_linear.py:350-400); storage shared
    between modules is counted once."""
    q_bytes = q_orig = other = n_q = n_reg = 0
    seen = set()
    for _, module in model.named_modules():
        if isinstance(module, QuantizedLinear):
            m = module.memory_bytes()
            q_bytes += m["total_bytes"]
            q_orig += m["original_fp32_bytes"]
            n_q += 1
            for _, t in list(module.named_buffers()) + list(module.named_parameters()):
                if t is not None:
                    seen.add(t.data_ptr())
        elif isinstance(module, nn.Linear):
            n_reg += 1
    for t in list(model.parameters()) + [b for _, b in model.named_buffers()]:
        if t is not None and t.data_ptr() not in seen:
            other += t.numel() * t.element_size()
            seen.add(t.data_ptr())
    total, total_orig = q_bytes + other, q_orig + other
    return {"quantized_layers": n_q, "regular_layers": n_reg, "quantized_bytes": q_bytes,
            "quantized_original_bytes": q_orig, "other_bytes": other, "total_bytes": total,
            "total_original_bytes": total_orig, "compression_ratio": total_orig / total if total > 0 else 1.0}
