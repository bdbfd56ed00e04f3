"""Reader of the reference's ``.eoq`` container (core/eoq_format.py:7-33, load_eoq :187-254) that
takes the tensors straight to the GPU: two-dimensional INT4 tensors whose shape the fused kernel
can tile become resident entropy-coded weights (:class:`EOQWeight`); everything else is decoded
and dequantised on the GPU into a dense tensor.  This is the loading path the reference leaves
as a TODO in core/eoq_linear.py:49-51.

File layout (all little-endian):
    b'EOQ\\x01' | u32 version = 1 | u32 num_tensors | u32 json_size | json
    per tensor, in the order of json["tensors"]:  u32 scales_size | fp16 scales | u32 rans_size | RANS container
    u32 CRC32 of everything before it
"""
from __future__ import annotations

import json
import struct
import zlib
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Tuple, Union

import numpy as np

MAGIC = b"EOQ\x01"
VERSION = 1


@dataclass
class EOQTensorRecord:
    """One tensor of the container, still compressed (fields of EOQCompressedTensor, core/eoq.py:40-50)."""
    name: str
    shape: Tuple[int, ...]
    dtype: str
    bits: int
    quant_block_size: int
    scales: bytes
    rans_data: bytes
    num_elements: int


def read_eoq(path: Union[str, Path]) -> Tuple[dict, List[EOQTensorRecord]]:
    """Parse and verify a .eoq file.  ValueError on checksum, magic or version mismatch, as load_eoq."""
    data = Path(path).read_bytes()
    if len(data) < 20:
        raise ValueError("file too short to be an .eoq container")
    stored = struct.unpack("<I", data[-4:])[0]
    computed = zlib.crc32(data[:-4]) & 0xFFFFFFFF
    if stored != computed:
        raise ValueError(f"Checksum mismatch: expected {stored:08x}, got {computed:08x}")
    if data[:4] != MAGIC:
        raise ValueError(f"Invalid magic: {data[:4]!r}")
    version, num_tensors, json_size = struct.unpack_from("<3I", data, 4)
    if version != VERSION:
        raise ValueError(f"Unsupported version: {version}")
    at = 16
    header = json.loads(data[at:at + json_size].decode("utf-8"))
    at += json_size
    records = []
    for meta in header["tensors"]:
        (ssz,) = struct.unpack_from("<I", data, at); at += 4
        scales = data[at:at + ssz]; at += ssz
        (rsz,) = struct.unpack_from("<I", data, at); at += 4
        rans = data[at:at + rsz]; at += rsz
        records.append(EOQTensorRecord(meta["name"], tuple(meta["shape"]), meta["dtype"], meta["bits"],
                                       meta["quant_block_size"], scales, rans, meta["num_elements"]))
    if len(records) != num_tensors:
        raise ValueError(f"header lists {len(records)} tensors, file says {num_tensors}")
    return header, records


def fusable(rec: EOQTensorRecord) -> bool:
    """Can this tensor stay entropy-coded in HBM behind the fused kernel?"""
    return (rec.bits == 4 and len(rec.shape) == 2 and rec.shape[1] % 16 == 0 and rec.quant_block_size % 16 == 0
            and rec.shape[1] % rec.quant_block_size == 0)


def load_eoq_to_device(path: Union[str, Path], device="cuda", dense_dtype=None) -> Dict[str, object]:
    """name -> EOQWeight (fusable INT4 matrices) or dense torch tensor (anything else), all on `device`."""
    import torch
    from .core.rans_blocked import BlockedRANSDecoder, deserialize_blocked_rans
    from .fused import EOQWeight

    dense_dtype = dense_dtype or torch.float16
    _, records = read_eoq(path)
    out: Dict[str, object] = {}
    with torch.cuda.device(device):
        for rec in records:
            if fusable(rec):
                out[rec.name] = EOQWeight.from_rans(rec.rans_data, rec.scales, rec.shape, group=rec.quant_block_size)
                continue
            qmax = (1 << (rec.bits - 1)) - 1
            sym = BlockedRANSDecoder().decode_all(deserialize_blocked_rans(rec.rans_data))        # GPU decode
            codes = torch.from_numpy((sym - qmax).astype(np.float32)).to(device)
            scales = torch.from_numpy(np.frombuffer(rec.scales, np.float16).astype(np.float32)).to(device)
            n, bs = codes.numel(), rec.quant_block_size
            pad = (-n) % bs
            if pad:
                codes = torch.cat([codes, torch.zeros(pad, device=device)])
            dense = (codes.view(-1, bs) * scales[:, None]).flatten()[:n].view(rec.shape)          # core/utils.py:130-161
            out[rec.name] = dense.to(dense_dtype)
    return out
