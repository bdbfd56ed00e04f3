"""Bridge between the absmax quantiser and the rANS coder: interface of the reference's
``core/rans_bitpacked.py``.  Compression runs in the library's host encoder; decompression
decodes on the GPU."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import numpy as np
import torch

from .rans_blocked import (BlockedRANSDecoder, BlockedRANSEncoder, deserialize_blocked_rans, serialize_blocked_rans)
from .utils import QuantizedTensor, dequantize, quantize_absmax


@dataclass
class CompressedTensorData:
    """core/rans_bitpacked.py:43-55."""
    name: str
    shape: tuple
    bits: int
    block_size: int
    scales_bytes: bytes
    rans_bytes: bytes
    n_elements: int
    original_size: int
    compressed_size: int


def compress_tensor_rans(name: str, codes: torch.Tensor, scales: torch.Tensor, bits: int, block_size: int,
                         shape: tuple) -> CompressedTensorData:
    """Signed codes -> symbols code+qmax -> blocked rANS with 256-symbol blocks at 14-bit precision;
    scales stored as fp16 (core/rans_bitpacked.py:62-123)."""
    n = codes.numel()
    flat = codes.detach().cpu().flatten().numpy().astype(np.int64)
    qmax = (1 << (bits - 1)) - 1
    alphabet = 2 * qmax + 1
    unsigned = np.clip(flat + qmax, 0, alphabet - 1)
    blocked = BlockedRANSEncoder(block_size=256, precision_bits=14).encode(unsigned, alphabet)
    rans_bytes = serialize_blocked_rans(blocked)
    scales_bytes = scales.detach().cpu().float().numpy().astype(np.float16).tobytes()
    return CompressedTensorData(name=name, shape=shape, bits=bits, block_size=block_size, scales_bytes=scales_bytes,
                                rans_bytes=rans_bytes, n_elements=n, original_size=n * 2,
                                compressed_size=len(scales_bytes) + len(rans_bytes))


def decompress_tensor_rans(data: CompressedTensorData) -> Tuple[torch.Tensor, torch.Tensor]:
    """(int8 signed codes, float32 scales of fp16 precision) (core/rans_bitpacked.py:126-154)."""
    unsigned = BlockedRANSDecoder().decode_all(deserialize_blocked_rans(data.rans_bytes))
    qmax = (1 << (data.bits - 1)) - 1
    signed = unsigned.astype(np.int64) - qmax
    scales = np.frombuffer(data.scales_bytes, dtype=np.float16).copy()
    return torch.from_numpy(signed.astype(np.int8)).to(torch.int8), torch.from_numpy(scales.astype(np.float32))


def compress_model_rans(model, bits_fn: Callable, block_size: int = 128,
                        awq_scales: Optional[Dict[str, torch.Tensor]] = None) -> Tuple[Dict[str, CompressedTensorData], dict]:
    """Quantise and entropy-code every tensor with at least two dimensions
    (core/rans_bitpacked.py:161-251)."""
    compressed: Dict[str, CompressedTensorData] = {}
    metadata: dict = {"block_size": block_size, "has_awq": awq_scales is not None, "tensor_info": {}}
    named = list(model.items()) if isinstance(model, dict) else list(model.named_parameters())
    total_o = total_c = 0
    for name, param in named:
        t = param.detach().float() if hasattr(param, "detach") else param.float()
        if t.ndim < 2:
            continue
        bits = bits_fn(name, t)
        awq = None
        if awq_scales is not None and name in awq_scales:
            awq = awq_scales[name]
            if awq.shape[0] == t.shape[-1]:
                t = t * awq.unsqueeze(0)
            elif awq.shape[0] == t.shape[0]:
                t = t * awq.unsqueeze(1)
        qt = quantize_absmax(t, bits, block_size)
        ct = compress_tensor_rans(name=name, codes=qt.data, scales=qt.scale, bits=bits, block_size=block_size,
                                  shape=tuple(t.shape))
        compressed[name] = ct
        total_o += ct.original_size
        total_c += ct.compressed_size
        metadata["tensor_info"][name] = {"shape": tuple(t.shape), "bits": bits, "has_awq_scale": awq is not None}
    metadata["total_original_bytes"] = total_o
    metadata["total_compressed_bytes"] = total_c
    metadata["num_tensors"] = len(compressed)
    return compressed, metadata


def decompress_model_rans(compressed: Dict[str, CompressedTensorData], metadata: dict) -> Dict[str, torch.Tensor]:
    """name -> fp16 tensor (core/rans_bitpacked.py:254-294)."""
    out: Dict[str, torch.Tensor] = {}
    for name, ct in compressed.items():
        codes, scales = decompress_tensor_rans(ct)
        qt = QuantizedTensor(data=codes[:ct.n_elements].reshape(ct.shape).to(torch.int32), scale=scales,
                             zero_point=torch.zeros(len(scales)), bits=ct.bits, shape=ct.shape, block_size=ct.block_size)
        out[name] = dequantize(qt).to(torch.float16)
    return out


def estimate_savings(compressed: Dict[str, CompressedTensorData]) -> dict:
    """core/rans_bitpacked.py:301-357."""
    orig = packed = rans = 0
    for ct in compressed.values():
        orig += ct.original_size
        packed += math.ceil(ct.bits * ct.n_elements / 8) + len(ct.scales_bytes)
        rans += ct.compressed_size
    gb = 1 << 30
    return {"original_gb": orig / gb, "bitpacked_gb": packed / gb, "rans_gb": rans / gb,
            "rans_vs_bitpacked_savings": (packed - rans) / packed * 100.0 if packed > 0 else 0.0,
            "total_compression_ratio": orig / rans if rans > 0 else float("inf")}
