"""Block-wise absmax quantiser of the reference's ``core/utils.py`` (lines 23-161):
the encode side of the hot path, plain torch ops on whatever device the tensor is on."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F


@dataclass
class QuantizedTensor:
    """core/utils.py:23-32."""
    data: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    bits: int
    shape: tuple
    block_size: Optional[int] = None


def quantize_absmax(tensor: torch.Tensor, bits: int, block_size: int = 128) -> QuantizedTensor:
    """core/utils.py:75-127: flatten, zero-pad to a multiple of the block, scale = max(absmax/qmax, 1e-10),
    codes = round(w/scale) clamped to [-qmax, qmax]."""
    t = tensor.detach().float().flatten()
    n = t.numel()
    pad = (block_size - n % block_size) % block_size
    if pad:
        t = F.pad(t, (0, pad), value=0.0)
    blocks = t.view(-1, block_size)
    qmax = (1 << (bits - 1)) - 1
    scale = (blocks.abs().amax(dim=1) / qmax).clamp(min=1e-10)
    q = (blocks / scale.unsqueeze(1)).round().clamp(-qmax, qmax).to(torch.int32)
    q = q.flatten()[:n].view(tensor.shape)
    return QuantizedTensor(data=q, scale=scale, zero_point=torch.zeros(blocks.shape[0]), bits=bits,
                           shape=tuple(tensor.shape), block_size=block_size)


def dequantize(quantized: QuantizedTensor) -> torch.Tensor:
    """core/utils.py:130-161."""
    q = quantized.data.float()
    if quantized.block_size is None:
        return q * quantized.scale + quantized.zero_point
    flat = q.flatten()
    n = flat.numel()
    bs = quantized.block_size
    pad = (bs - n % bs) % bs
    if pad:
        flat = F.pad(flat, (0, pad), value=0.0)
    return (flat.view(-1, bs) * quantized.scale.unsqueeze(1)).flatten()[:n].view(quantized.shape)
