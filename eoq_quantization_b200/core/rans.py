"""Single-stream rANS front end with the interface of the reference's
``core/rans.py``: table helpers on the host, encoding in the library's host
encoder, decoding on the GPU."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib


def compute_frequency_table(symbols: np.ndarray, alphabet_size: int) -> np.ndarray:
    """Histogram of symbol values (core/rans.py:32-55); ValueError if out of range."""
    symbols = np.asarray(symbols).ravel()
    if symbols.size == 0:
        return np.zeros(alphabet_size, dtype=np.int64)
    if symbols.min() < 0 or symbols.max() >= alphabet_size:
        raise ValueError(f"Symbols must be in [0, {alphabet_size}), got range [{symbols.min()}, {symbols.max()}]")
    return np.bincount(symbols, minlength=alphabet_size).astype(np.int64)[:alphabet_size]


def estimate_compressed_size(freq_table: np.ndarray, num_symbols: int) -> int:
    """ceil(H * n / 8) with H the Shannon entropy of the table (core/rans.py:58-78)."""
    f = np.asarray(freq_table, dtype=np.float64)
    tot = f.sum()
    if tot == 0 or num_symbols == 0:
        return 0
    pr = f[f > 0] / tot
    return int(np.ceil(-float(np.sum(pr * np.log2(pr))) * num_symbols / 8))


def _normalize_frequencies(raw_freq: np.ndarray, precision_bits: int):
    """(freq, cdf) summing to ``2**precision_bits``, every symbol >= 1.

    Same arithmetic as core/rans.py:85-153 -- float64 proportional scaling,
    truncation, then the residual dealt out round-robin over the symbols in
    descending order of scaled frequency.  The order comes from
    ``np.argsort(-scaled)`` exactly as in the reference, so a table built here
    agrees with one built by the reference on the same machine even where ties
    make that order implementation-defined (alphabets above 16 symbols).
    """
    M = 1 << precision_bits
    raw = np.asarray(raw_freq, dtype=np.int64).copy()
    a = len(raw)
    if a == 0:
        raise ValueError("Frequency table must not be empty")
    if a > M:
        raise ValueError(f"Alphabet size ({a}) exceeds probability space (2**{precision_bits} = {M}).  "
                         "Use a larger precision_bits.")
    raw = np.maximum(raw, 1)
    scaled = np.maximum((raw.astype(np.float64) / raw.sum() * M).astype(np.int64), 1)
    residual = int(M - scaled.sum())
    if residual:
        order = np.argsort(-scaled)
        at = 0
        while residual:
            step = 1 if residual > 0 else -1
            if scaled[order[at]] + step >= 1:
                scaled[order[at]] += step
                residual -= step
            at = (at + 1) % a
    cdf = np.zeros(a + 1, dtype=np.int64)
    np.cumsum(scaled, out=cdf[1:])
    return scaled, cdf


def _check_precision(p: int) -> None:
    if p < 8 or p > 20:
        raise ValueError(f"precision_bits must be in [8, 20], got {p}")


def encode_blocks(freq_norm: np.ndarray, precision_bits: int, symbols: np.ndarray, block_size: int):
    """Host encoder of the library -> (bytes, offsets), wire format of core/rans.py:210-276."""
    sym = np.ascontiguousarray(np.asarray(symbols).ravel().astype(np.uint32))
    if sym.size == 0:
        return b"", []
    f = np.ascontiguousarray(freq_norm, dtype=np.uint32)
    nb = (sym.size + block_size - 1) // block_size
    cap = C.c_size_t(3 * sym.size + 16 * nb + 64)
    out = np.empty(cap.value, np.uint8)
    offs = np.empty(nb, np.uint32)
    _lib.check(_lib.lib().eoq_b200_encode_blocked(f.ctypes.data, f.size, precision_bits, sym.ctypes.data, sym.size,
                                                  block_size, out.ctypes.data, C.byref(cap), offs.ctypes.data),
               "eoq_b200_encode_blocked")
    return out[:cap.value].tobytes(), offs.astype(np.int64).tolist()


def decode_blocks(freq_norm: np.ndarray, precision_bits: int, data: bytes, offsets, block_size: int, n: int) -> np.ndarray:
    """GPU decode of wire-format blocks -> int64 symbols (core/rans.py:368-419 per block)."""
    if n == 0 or len(data) == 0:
        return np.empty(0, dtype=np.int64)
    if precision_bits > 16:
        raise NotImplementedError("the GPU decoder keeps a 32-bit state: precision_bits must be <= 16")
    f = np.ascontiguousarray(freq_norm, dtype=np.uint32)
    if f.size > 65536:
        raise NotImplementedError("alphabets above 65536 symbols are not supported")
    buf = np.frombuffer(data, dtype=np.uint8)
    offs = np.ascontiguousarray(np.asarray(offsets, dtype=np.uint32))
    width = 1 if f.size <= 256 else 2
    out = np.empty(n, np.uint8 if width == 1 else np.uint16)
    _lib.check(_lib.lib().eoq_b200_decode_blocked(f.ctypes.data, f.size, precision_bits, buf.ctypes.data, buf.size,
                                                  offs.ctypes.data, offs.size, block_size, n, out.ctypes.data, width, 0, None),
               "eoq_b200_decode_blocked")
    return out.astype(np.int64)


class RANSEncoder:
    """core/rans.py:160-314."""

    def __init__(self, freq_table: np.ndarray, precision_bits: int = 16) -> None:
        _check_precision(precision_bits)
        self.precision_bits = precision_bits
        self.M = 1 << precision_bits
        freq_table = np.asarray(freq_table, dtype=np.int64)
        self.alphabet_size = len(freq_table)
        self.freq, self.cdf = _normalize_frequencies(freq_table, precision_bits)

    def encode(self, symbols: np.ndarray) -> bytes:
        symbols = np.asarray(symbols).ravel()
        if symbols.size == 0:
            return b""
        data, _ = encode_blocks(self.freq, self.precision_bits, symbols, max(int(symbols.size), 1))
        return data

    def encode_blocked(self, symbols: np.ndarray, block_size: int = 256):
        symbols = np.asarray(symbols).ravel()
        return encode_blocks(self.freq, self.precision_bits, symbols, block_size)


class RANSDecoder:
    """core/rans.py:321-439."""

    def __init__(self, freq_table: np.ndarray, precision_bits: int = 16) -> None:
        _check_precision(precision_bits)
        self.precision_bits = precision_bits
        self.M = 1 << precision_bits
        freq_table = np.asarray(freq_table, dtype=np.int64)
        self.alphabet_size = len(freq_table)
        self.freq, self.cdf = _normalize_frequencies(freq_table, precision_bits)

    def decode(self, data: bytes, num_symbols: int) -> np.ndarray:
        if num_symbols == 0 or len(data) == 0:
            return np.empty(0, dtype=np.int64)
        return decode_blocks(self.freq, self.precision_bits, bytes(data), [0], max(num_symbols, 1), num_symbols)

    def decode_block(self, data: bytes, offset: int, block_size: int) -> np.ndarray:
        return self.decode(data[offset:], block_size)
