"""``PolarLinear`` (kernels/polar_engine.py:144-360): a linear layer whose weight stays in PolarQuant form.

Buffers, constructors and the result type of ``forward`` are the reference's.  Where the reference rebuilds the
weight 64 rows at a time with torch operations (centroid look-up, inverse Hadamard, norm) and multiplies, this
module rotates the activations once per call (H is symmetric, so x . (c H) = (x H) . c) and never materialises the
weight: up to 32 rows of x (8 for blocks below 64 columns) are multiplied straight from the byte codes the module holds
(any bit width and block size the reference builds; one row on the CUDA cores, several on the tensor cores), or, with ``entropy_coded = True`` and
the configuration that path is built for (5-bit codes, blocks of 64), from an entropy-coded copy of the codes by
the fused decode + GEMV kernel.  Larger batches dequantise with torch operations on the same device.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib
from ..core.polar_quant import _ensure_centroids, hadamard_matrix, polar_quantize
from ..fused import EOQWeight, gemv_polar_codes, polar_codes_gemv_applies, require_cuda


class PolarLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bits: int = 4, block_size: int = 128,
                 bias_data: Optional[torch.Tensor] = None):
        super().__init__()
        self.in_features, self.out_features, self.bits, self.block_size = in_features, out_features, bits, block_size
        n = out_features * in_features
        self.register_buffer("codes", torch.zeros(n, dtype=torch.int8))
        self.register_buffer("norms", torch.zeros((n + block_size - 1) // block_size, dtype=torch.float16))
        self.register_buffer("centroids", torch.zeros(1 << bits, dtype=torch.float32))
        self.register_buffer("awq_scales", None)
        self.register_buffer("H", hadamard_matrix(block_size).clone())
        if bias_data is not None:
            self.register_buffer("bias", bias_data.half())
        else:
            self.bias = None
        self._eoq: Optional[EOQWeight] = None
        self._eoq_key = None
        # False: forward multiplies straight from the byte codes this module holds anyway (14336 x 4096 at 5 bits: 34 / 39 /
        # 40 us at 1 / 4 / 8 rows); True: from an entropy-coded copy (`eoq_weight()`, about 4.6 instead of 8 bits per
        # weight if the byte codes are then dropped; 48 / 64 / 116 us) where that path exists (5-bit codes, blocks of 64)
        self.entropy_coded = False

    _hadamard = staticmethod(lambda n: hadamard_matrix(n).clone())

    # -- construction (kernels/polar_engine.py:190-251) ---------------------------
    @classmethod
    def from_polar_quant(cls, codes: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor, shape: tuple, bits: int,
                         block_size: int = 128, awq_scales: Optional[torch.Tensor] = None,
                         bias: Optional[torch.Tensor] = None) -> "PolarLinear":
        out_f, in_f = shape
        layer = cls(in_f, out_f, bits, block_size, bias)
        layer.codes.copy_(codes[:out_f * in_f])
        layer.norms.copy_(norms)
        layer.centroids.copy_(centroids)
        if awq_scales is not None:
            layer.awq_scales = awq_scales.half()
        return layer

    @classmethod
    def from_linear(cls, linear: nn.Linear, bits: int = 4, block_size: int = 128,
                    centroids_t: Optional[torch.Tensor] = None, awq_imp: Optional[torch.Tensor] = None) -> "PolarLinear":
        if awq_imp is not None:
            raise NotImplementedError("importance-weighted PolarQuant belongs to the quantisation policy, which this package leaves out")
        cent = _ensure_centroids(bits) if centroids_t is None else centroids_t
        w = linear.weight.data
        res = polar_quantize(w, bits, block_size)          # the reference quantises with its default (use_qjl=True) and drops the signs
        layer = cls(linear.in_features, linear.out_features, bits, block_size, linear.bias.data if linear.bias is not None else None)
        layer.codes.copy_(res.codes[:linear.out_features * linear.in_features])
        layer.norms.copy_(res.norms)
        layer.centroids.copy_(cent.to(res.codes.device))
        return layer.to(w.device)

    # -- fused path ------------------------------------------------------------------
    def _fusable(self) -> bool:
        return self.bits == 5 and self.block_size == 64 and self.in_features % 64 == 0

    def eoq_weight(self) -> EOQWeight:
        """The entropy-coded resident form of the codes (built on first use, rebuilt if the buffers change)."""
        key = (self.codes.data_ptr(), self.norms.data_ptr(), self.codes._version, self.norms._version, self.centroids._version)
        if self._eoq is None or self._eoq_key != key:
            with torch.cuda.device(self.codes.device):
                sym = self.codes.view(self.out_features, self.in_features).to(torch.uint8)
                self._eoq = EOQWeight.from_symbols(sym, self.norms, kind=_lib.KIND_Q5_POLAR, group=64,
                                                   centroids=self.centroids.detach().cpu().tolist())
            self._eoq_key = key
        return self._eoq

    def _dequant_block(self, codes_block: torch.Tensor, norm: torch.Tensor) -> torch.Tensor:
        """One block, for inspection (kernels/polar_engine.py:257-264)."""
        return ((self.centroids[codes_block.long()] / math.sqrt(self.block_size)) @ self.H) * norm

    def _dense_rows(self, lo: int, hi: int) -> torch.Tensor:
        bs, in_f = self.block_size, self.in_features
        codes = self.codes[: self.out_features * in_f].view(self.out_features, in_f)[lo:hi]
        pad = (bs - in_f % bs) % bs
        if pad:
            codes = F.pad(codes, (0, pad))
        per_row = (in_f + bs - 1) // bs
        vals = (self.centroids[codes.long().view(hi - lo, -1, bs)] / math.sqrt(bs)).view(-1, bs) @ self.H
        vals = vals.view(hi - lo, -1, bs) * self.norms[lo * per_row:hi * per_row].float().view(hi - lo, -1, 1)
        return vals.reshape(hi - lo, -1)[:, :in_f]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x (..., in_features) -> float16 (..., out_features), fp32 accumulation (kernels/polar_engine.py:270-340)."""
        require_cuda(x, "PolarLinear.forward")
        require_cuda(self.codes, "PolarLinear.forward")
        x2 = x.reshape(-1, self.in_features)
        if self.awq_scales is not None:                       # W / s applied to x instead: (x / s) W^T
            x2 = x2.float() / self.awq_scales.float().unsqueeze(0)
        if self.entropy_coded and self._fusable() and x2.shape[0] <= 8:
            xin = x2 if x2.dtype in (torch.float16, torch.bfloat16, torch.float32) else x2.float()
            out = self.eoq_weight().gemv(xin, out_dtype=torch.float32)
        elif polar_codes_gemv_applies(self.in_features, self.bits, self.block_size, x2.shape[0]):
            # up to 8 rows (32 with blocks of 64 columns and more): one pass over the byte codes this module keeps resident
            # (any bit width and block size the reference builds), activations rotated once per call
            xin = x2 if x2.dtype in (torch.float16, torch.bfloat16, torch.float32) else x2.float()
            out = gemv_polar_codes(self.codes, self.norms, self.centroids, self.out_features, self.in_features, self.bits,
                                   self.block_size, xin)
        else:
            out = torch.empty(x2.shape[0], self.out_features, device=x.device, dtype=torch.float32)
            xf = x2.float()
            for lo in range(0, self.out_features, 1024):
                hi = min(self.out_features, lo + 1024)
                out[:, lo:hi] = xf @ self._dense_rows(lo, hi).t()
        res = out.half().view(*x.shape[:-1], self.out_features)
        return res + self.bias if self.bias is not None else res

    # -- bookkeeping (kernels/polar_engine.py:346-360) ---------------------------------
    def vram_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in (self.codes, self.norms, self.centroids, self.H))
        if self.awq_scales is not None:
            n += self.awq_scales.numel() * 2
        if self.bias is not None:
            n += self.bias.numel() * self.bias.element_size()
        return n

    def extra_repr(self) -> str:
        fp16_mb = self.out_features * self.in_features * 2 / 1e6
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"block_size={self.block_size}, vram={self.vram_bytes() / 1e6:.1f}MB (vs {fp16_mb:.1f}MB FP16)")
