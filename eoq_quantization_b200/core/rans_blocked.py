"""Blocked rANS with random access: interface of the reference's
``core/rans_blocked.py``.  Containers and tables are handled on the host;
``BlockedRANSDecoder`` decodes every block in one GPU launch."""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass

import numpy as np

from .rans import (RANSDecoder, RANSEncoder, _normalize_frequencies, compute_frequency_table, decode_blocks,
                   encode_blocks, estimate_compressed_size)  # noqa: F401


@dataclass
class BlockedRANSData:
    """core/rans_blocked.py:25-58 (same fields, same accessors)."""

    compressed_blocks: bytes
    block_offsets: list
    freq_table: np.ndarray
    num_symbols: int
    block_size: int
    num_blocks: int
    alphabet_size: int
    precision_bits: int

    def total_size_bytes(self) -> int:
        return len(self.compressed_blocks) + self.num_blocks * 4 + self.alphabet_size * 4 + 32

    def compression_ratio(self) -> float:
        bps = max(1, math.ceil(math.log2(max(self.alphabet_size, 2))))
        raw_size = (self.num_symbols * bps + 7) // 8
        total = self.total_size_bytes()
        return raw_size / total if total > 0 else 0.0

    def bits_per_symbol(self) -> float:
        if self.num_symbols == 0:
            return 0.0
        return (self.total_size_bytes() * 8) / self.num_symbols


class BlockedRANSEncoder:
    """core/rans_blocked.py:65-114: one global table, one independent stream per block."""

    def __init__(self, block_size: int = 256, precision_bits: int = 14):
        self.block_size = block_size
        self.precision_bits = precision_bits

    def encode(self, symbols: np.ndarray, alphabet_size: int) -> BlockedRANSData:
        symbols = np.asarray(symbols).ravel()
        n = len(symbols)
        freq = compute_frequency_table(symbols, alphabet_size)
        enc = RANSEncoder(freq, precision_bits=self.precision_bits)
        data, offsets = encode_blocks(enc.freq, self.precision_bits, symbols, self.block_size)
        return BlockedRANSData(compressed_blocks=data, block_offsets=offsets, freq_table=freq, num_symbols=n,
                               block_size=self.block_size, num_blocks=(n + self.block_size - 1) // self.block_size,
                               alphabet_size=alphabet_size, precision_bits=self.precision_bits)


class BlockedRANSDecoder:
    """core/rans_blocked.py:121-165."""

    def decode_all(self, data: BlockedRANSData) -> np.ndarray:
        if data.num_symbols == 0:
            return np.empty(0, dtype=np.int64)
        freq, _ = _normalize_frequencies(data.freq_table, data.precision_bits)
        return decode_blocks(freq, data.precision_bits, bytes(data.compressed_blocks), data.block_offsets,
                             data.block_size, data.num_symbols)

    def decode_block(self, data: BlockedRANSData, block_idx: int) -> np.ndarray:
        if block_idx < 0 or block_idx >= data.num_blocks:
            raise IndexError(f"block_idx {block_idx} out of range [0, {data.num_blocks})")
        start = block_idx * data.block_size
        count = min(start + data.block_size, data.num_symbols) - start
        lo = data.block_offsets[block_idx]
        hi = data.block_offsets[block_idx + 1] if block_idx + 1 < data.num_blocks else len(data.compressed_blocks)
        freq, _ = _normalize_frequencies(data.freq_table, data.precision_bits)
        return decode_blocks(freq, data.precision_bits, bytes(data.compressed_blocks[lo:hi]), [0], max(count, 1), count)


_MAGIC = b"RANS"
_VERSION = 1


def serialize_blocked_rans(data: BlockedRANSData) -> bytes:
    """`RANS` container of core/rans_blocked.py:176-214: magic, seven little-endian u32
    (version, num_symbols, block_size, num_blocks, alphabet_size, precision_bits, data_size),
    u32 freq_table[], u32 block_offsets[], data."""
    head = _MAGIC + struct.pack("<7I", _VERSION, data.num_symbols, data.block_size, data.num_blocks,
                                data.alphabet_size, data.precision_bits, len(data.compressed_blocks))
    return (head + np.asarray(data.freq_table).astype("<u4").tobytes()
            + np.asarray(data.block_offsets, dtype=np.int64).astype("<u4").tobytes() + bytes(data.compressed_blocks))


def deserialize_blocked_rans(raw: bytes) -> BlockedRANSData:
    """core/rans_blocked.py:217-259; ValueError on bad magic or version."""
    magic = raw[:4]
    if magic != _MAGIC:
        raise ValueError(f"Invalid magic: {magic!r}")
    version, n, bs, nb, a, p, dsz = struct.unpack_from("<7I", raw, 4)
    if version != _VERSION:
        raise ValueError(f"Unsupported version: {version}")
    at = 32
    freq = np.frombuffer(raw, "<u4", a, at).astype(np.int64)
    at += 4 * a
    offsets = np.frombuffer(raw, "<u4", nb, at).astype(np.int64).tolist()
    at += 4 * nb
    return BlockedRANSData(compressed_blocks=bytes(raw[at:at + dsz]), block_offsets=offsets, freq_table=freq,
                           num_symbols=n, block_size=bs, num_blocks=nb, alphabet_size=a, precision_bits=p)


def encode_quantized_tensor(quantized_codes: np.ndarray, bits: int, block_size: int = 256,
                            precision_bits: int = 14) -> BlockedRANSData:
    """Signed codes in [-qmax, qmax] -> symbols code+qmax -> blocked rANS (core/rans_blocked.py:266-295)."""
    codes = np.asarray(quantized_codes).ravel().astype(np.int64)
    qmax = (1 << (bits - 1)) - 1
    alphabet_size = 2 * qmax + 1
    unsigned = np.clip(codes + qmax, 0, alphabet_size - 1)
    return BlockedRANSEncoder(block_size=block_size, precision_bits=precision_bits).encode(unsigned, alphabet_size)


def decode_quantized_tensor(data: BlockedRANSData, bits: int) -> np.ndarray:
    """core/rans_blocked.py:298-309: int64 signed codes."""
    qmax = (1 << (bits - 1)) - 1
    return BlockedRANSDecoder().decode_all(data).astype(np.int64) - qmax
