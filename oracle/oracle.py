"""CPU checker for the EOQ hot path.  TEST INFRASTRUCTURE ONLY.

Thin numpy/ctypes front end over ``eoq_oracle.c`` (the C restatement of the
reference's rANS codec) plus numpy restatements of the reference's quantiser,
INT4 packing and dequantise-then-matmul composition.  The product package
never imports this module; only the tests, the smoke check and the benchmark's
CPU-baseline leg do.

Parity status: pinned -- see the header of ``eoq_oracle.c``.

When ``oracle/_ref/`` holds the reference's own C decoders (``make -C oracle
ref``), :class:`RefC` exposes them so that they can validate the restatement
and serve as the timed CPU baseline.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import struct
import subprocess
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def reference_dir(ref_root: Optional[str] = None) -> Optional[str]:
    """Where a checkout of the reference project is: the argument, else ``$EOQ_REFERENCE_DIR``, else a directory
    named ``reference`` beside this repository; None if there is none."""
    for cand in (ref_root, os.environ.get("EOQ_REFERENCE_DIR"),
                 os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "llamacpp_integration")):
            return os.path.abspath(cand)
    return None


def build(ref_root: Optional[str] = None) -> None:
    """Compile ``liboracle.so`` and, when a reference tree is present, ``_ref``."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    ref_root = reference_dir(ref_root)
    if ref_root:
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={ref_root}"], check=True, capture_output=True)
        import shutil
        if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
            nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
            # the reference's CUDA decoder, for timing beside this project's kernel; failure to build it is not an error
            subprocess.run(["make", "-C", _HERE, "ref_cuda", f"REF={ref_root}", f"NVCC={nvcc}"], check=False, capture_output=True)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "liboracle.so")
        src = os.path.join(_HERE, "eoq_oracle.c")
        if not os.path.exists(path) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(path)):
            build()
        L = C.CDLL(path)
        u8p, u16p, u32p, u64p, f32p = (C.POINTER(t) for t in (C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64, C.c_float))
        L.orc_normalize.argtypes = [u64p, C.c_uint32, C.c_uint32, u32p, u32p]
        L.orc_normalize.restype = C.c_int
        L.orc_build_lut.argtypes = [u32p, C.c_uint32, C.c_uint32, u16p]
        L.orc_decode_block.argtypes = [u32p, u32p, u16p, C.c_uint32, u8p, C.c_size_t, C.c_uint32, u32p]
        L.orc_decode_block.restype = C.c_int
        L.orc_encode_block.argtypes = [u32p, u32p, C.c_uint32, u32p, C.c_uint32, u8p, C.c_size_t]
        L.orc_encode_block.restype = C.c_long
        L.orc_decode_blocked.argtypes = [u64p, C.c_uint32, C.c_uint32, u8p, C.c_size_t, u32p, C.c_uint32,
                                         C.c_uint32, C.c_uint32, u32p]
        L.orc_decode_blocked.restype = C.c_int
        L.orc_decode_c_payload.argtypes = [u32p, u8p, C.c_size_t, u8p, C.c_size_t]
        L.orc_decode_c_payload.restype = C.c_int
        L.orc_int4_linear.argtypes = [u8p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, f32p, C.c_uint32, f32p, f32p]
        L.orc_int4_linear.restype = None
        _LIB = L
    return _LIB


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(C.POINTER(t))


def _bytes_arr(b) -> np.ndarray:
    a = np.frombuffer(bytes(b), dtype=np.uint8)
    return a if a.size else np.zeros(1, np.uint8)


# --------------------------------------------------------------------------
# rANS codec (C restatement)
# --------------------------------------------------------------------------

def normalize(raw_freq: Sequence[int], precision_bits: int) -> Tuple[np.ndarray, np.ndarray]:
    """(freq, cdf) summing to 2**p -- core/rans.py:85-153."""
    raw = np.ascontiguousarray(np.asarray(raw_freq, dtype=np.int64).clip(min=0).astype(np.uint64))
    a = raw.size
    freq = np.zeros(a, np.uint32)
    cdf = np.zeros(a + 1, np.uint32)
    rc = lib().orc_normalize(_p(raw, C.c_uint64), a, precision_bits, _p(freq, C.c_uint32), _p(cdf, C.c_uint32))
    if rc != 0:
        raise ValueError(f"orc_normalize failed: {rc}")
    return freq, cdf


class Table:
    """Normalised table + slot->symbol LUT for one (raw_freq, p)."""

    def __init__(self, raw_freq: Sequence[int], precision_bits: int):
        self.p = int(precision_bits)
        self.alphabet = len(raw_freq)
        self.freq, self.cdf = normalize(raw_freq, self.p)
        self.lut = np.zeros(1 << self.p, np.uint16)
        lib().orc_build_lut(_p(self.cdf, C.c_uint32), self.alphabet, self.p, _p(self.lut, C.c_uint16))

    def decode(self, data: bytes, n: int) -> np.ndarray:
        """core/rans.py:368-419."""
        out = np.zeros(max(n, 1), np.uint32)
        if n == 0 or len(data) == 0:
            return np.empty(0, np.int64)
        d = _bytes_arr(data)
        rc = lib().orc_decode_block(_p(self.freq, C.c_uint32), _p(self.cdf, C.c_uint32), _p(self.lut, C.c_uint16),
                                    self.p, _p(d, C.c_uint8), len(data), n, _p(out, C.c_uint32))
        if rc != 0:
            raise ValueError(f"orc_decode_block failed: {rc}")
        return out[:n].astype(np.int64)

    def encode(self, symbols: np.ndarray) -> bytes:
        """core/rans.py:210-276."""
        s = np.ascontiguousarray(np.asarray(symbols).ravel().astype(np.uint32))
        if s.size == 0:
            return b""
        cap = 16 + 3 * s.size
        out = np.zeros(cap, np.uint8)
        n = lib().orc_encode_block(_p(self.freq, C.c_uint32), _p(self.cdf, C.c_uint32), self.p,
                                   _p(s, C.c_uint32), s.size, _p(out, C.c_uint8), cap)
        if n < 0:
            raise ValueError(f"orc_encode_block failed: {n}")
        return out[:n].tobytes()


@dataclass
class Blocked:
    """Field-for-field twin of core/rans_blocked.py:25-36 (BlockedRANSData)."""
    compressed_blocks: bytes
    block_offsets: List[int]
    freq_table: np.ndarray          # RAW histogram, as the reference stores it
    num_symbols: int
    block_size: int
    num_blocks: int
    alphabet_size: int
    precision_bits: int


def encode_blocked(symbols: np.ndarray, alphabet: int, block_size: int = 256, precision_bits: int = 14) -> Blocked:
    """core/rans_blocked.py:72-114: global histogram, independent stream per block."""
    s = np.asarray(symbols).ravel().astype(np.int64)
    raw = np.bincount(s, minlength=alphabet).astype(np.int64)[:alphabet]
    t = Table(raw, precision_bits)
    nb = (s.size + block_size - 1) // block_size
    parts, offs, at = [], [], 0
    for b in range(nb):
        enc = t.encode(s[b * block_size:(b + 1) * block_size])
        offs.append(at)
        parts.append(enc)
        at += len(enc)
    return Blocked(b"".join(parts), offs, raw, int(s.size), block_size, nb, alphabet, precision_bits)


def decode_blocked(d: Blocked) -> np.ndarray:
    """core/rans_blocked.py:124-145."""
    if d.num_symbols == 0:
        return np.empty(0, np.int64)
    raw = np.ascontiguousarray(np.asarray(d.freq_table, dtype=np.int64).astype(np.uint64))
    data = _bytes_arr(d.compressed_blocks)
    offs = np.ascontiguousarray(np.asarray(d.block_offsets, dtype=np.uint32))
    out = np.zeros(d.num_symbols, np.uint32)
    rc = lib().orc_decode_blocked(_p(raw, C.c_uint64), d.alphabet_size, d.precision_bits,
                                  _p(data, C.c_uint8), len(d.compressed_blocks), _p(offs, C.c_uint32),
                                  d.num_blocks, d.block_size, d.num_symbols, _p(out, C.c_uint32))
    if rc != 0:
        raise ValueError(f"orc_decode_blocked failed: {rc}")
    return out.astype(np.int64)


def serialize_rans_v1(d: Blocked) -> bytes:
    """`RANS` container, core/rans_blocked.py:176-214 (8 x u32 header, all little-endian)."""
    head = b"RANS" + struct.pack("<7I", 1, d.num_symbols, d.block_size, d.num_blocks, d.alphabet_size,
                                 d.precision_bits, len(d.compressed_blocks))
    return (head + np.asarray(d.freq_table, dtype="<u4").tobytes()
            + np.asarray(d.block_offsets, dtype="<u4").tobytes() + d.compressed_blocks)


def deserialize_rans_v1(raw: bytes) -> Blocked:
    """core/rans_blocked.py:217-259."""
    if raw[:4] != b"RANS":
        raise ValueError(f"Invalid magic: {raw[:4]!r}")
    ver, n, bs, nb, a, p, dsz = struct.unpack_from("<7I", raw, 4)
    if ver != 1:
        raise ValueError(f"Unsupported version: {ver}")
    at = 32
    freq = np.frombuffer(raw, "<u4", a, at).astype(np.int64); at += 4 * a
    offs = np.frombuffer(raw, "<u4", nb, at).astype(np.int64).tolist(); at += 4 * nb
    return Blocked(bytes(raw[at:at + dsz]), offs, freq, n, bs, nb, a, p)


def make_c_payload(d: Blocked, original_type: int = 0) -> Tuple[np.ndarray, bytes]:
    """Assemble the C tensor payload `[u16 freq x A][u32 offsets x B][blocks]` and its
    7-word header (eoq_rans_v2.h:54-62) from blocked data.  The table written is the
    NORMALISED one (sum 2**p, all >= 1) so every normaliser is the identity on it; a
    frequency of 65536 does not fit a u16 and is refused."""
    t = Table(d.freq_table, d.precision_bits)
    if t.freq.max() > 0xFFFF:
        raise ValueError("frequency does not fit the u16 table of the C payload")
    body = t.freq.astype("<u2").tobytes() + np.asarray(d.block_offsets, "<u4").tobytes() + d.compressed_blocks
    hdr = np.array([original_type, d.num_blocks, d.alphabet_size, d.precision_bits, d.block_size,
                    len(body), d.num_symbols], np.uint32)
    return hdr, body


def decode_c_payload(header: np.ndarray, payload: bytes, out_cap: Optional[int] = None) -> Tuple[int, np.ndarray]:
    """eoq_rans_v2.c:577-782.  Returns (error code, uint8 symbols)."""
    h = np.ascontiguousarray(header, dtype=np.uint32)
    n = int(h[6])
    cap = n if out_cap is None else out_cap
    out = np.zeros(max(cap, 1), np.uint8)
    d = _bytes_arr(payload)
    rc = lib().orc_decode_c_payload(_p(h, C.c_uint32), _p(d, C.c_uint8), len(payload), _p(out, C.c_uint8), cap)
    return rc, out[:n]


# --------------------------------------------------------------------------
# Quantiser, INT4 packing, dequantise + linear (numpy restatements)
# --------------------------------------------------------------------------

def quantize_absmax(w: np.ndarray, bits: int, group: int = 128) -> Tuple[np.ndarray, np.ndarray]:
    """core/utils.py:75-127 in float32: (codes int32 of w.shape, scales float32 per group
    over the FLATTENED tensor)."""
    flat = np.asarray(w, np.float32).ravel()
    n = flat.size
    pad = (-n) % group
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, np.float32)])
    blocks = flat.reshape(-1, group)
    qmax = (1 << (bits - 1)) - 1
    scale = np.maximum(np.abs(blocks).max(axis=1) / np.float32(qmax), np.float32(1e-10)).astype(np.float32)
    q = np.clip(np.round(blocks / scale[:, None]), -qmax, qmax).astype(np.int32)
    return q.ravel()[:n].reshape(np.shape(w)), scale


def dequantize(codes: np.ndarray, scales: np.ndarray, group: int) -> np.ndarray:
    """core/utils.py:130-161."""
    flat = np.asarray(codes, np.float32).ravel()
    n = flat.size
    pad = (-n) % group
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, np.float32)])
    out = (flat.reshape(-1, group) * np.asarray(scales, np.float32)[:, None]).ravel()[:n]
    return out.reshape(np.shape(codes))


def pack_int4_rows(codes: np.ndarray) -> np.ndarray:
    """core/quantized_linear.py:76-91,165-170: per row, value code+7, low nibble = even column."""
    c = np.asarray(codes)
    u = (c.astype(np.int32) + 7).astype(np.uint8)
    if u.shape[1] % 2:
        u = np.concatenate([u, np.zeros((u.shape[0], 1), np.uint8)], axis=1)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def unpack_int4_rows(packed: np.ndarray, k: int) -> np.ndarray:
    """core/quantized_linear.py:93-102 / core/fast_dequant.py:9-27."""
    lo = (packed & 0x0F).astype(np.int32)
    hi = (packed >> 4).astype(np.int32)
    return (np.stack([lo, hi], axis=-1).reshape(packed.shape[0], -1)[:, :k] - 7).astype(np.int8)


def int4_dequant_matrix(packed: np.ndarray, scales: np.ndarray, n: int, k: int, group: int) -> np.ndarray:
    """core/quantized_linear.py:189-217 -> float32 (N, K)."""
    return dequantize(unpack_int4_rows(packed, k).astype(np.int32), np.asarray(scales, np.float32), group).reshape(n, k)


def int4_linear(packed: np.ndarray, scales: np.ndarray, n: int, k: int, group: int, x: np.ndarray,
                bias: Optional[np.ndarray] = None) -> np.ndarray:
    """dequantise-then-matmul (core/quantized_linear.py:222-228) with a double accumulator."""
    x2 = np.ascontiguousarray(np.asarray(x, np.float32).reshape(-1, k))
    pk = np.ascontiguousarray(packed, np.uint8)
    sc = np.ascontiguousarray(scales, np.float32)
    y = np.zeros((x2.shape[0], n), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().orc_int4_linear(_p(pk, C.c_uint8), _p(sc, C.c_float), n, k, group, _p(x2, C.c_float), x2.shape[0],
                          _p(b, C.c_float) if b is not None else None, _p(y, C.c_float))
    return y.reshape(*np.shape(x)[:-1], n)


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


# --------------------------------------------------------------------------
# The reference's own C decoders, when built into oracle/_ref
# --------------------------------------------------------------------------

class _Hdr(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("original_type", "num_blocks", "freq_table_size", "precision_bits",
                                          "rans_block_size", "compressed_size", "uncompressed_size")]


class _Task(C.Structure):
    _fields_ = [("header", C.POINTER(_Hdr)), ("compressed_data", C.c_void_p), ("compressed_size", C.c_size_t),
                ("output", C.c_void_p), ("output_capacity", C.c_size_t), ("result", C.c_int), ("task_index", C.c_int)]


class _POpts(C.Structure):
    _fields_ = [("num_threads", C.c_int), ("progress_cb", C.c_void_p), ("progress_ud", C.c_void_p)]


class RefC:
    """ctypes view of the reference C decoders compiled by `make -C oracle ref`."""

    def __init__(self):
        v2 = os.path.join(_HERE, "_ref", "libeoq_ref_v2.so")
        v1 = os.path.join(_HERE, "_ref", "libeoq_ref_v1.so")
        if not (os.path.exists(v1) and os.path.exists(v2)):
            raise FileNotFoundError("oracle/_ref is not built (make -C oracle ref)")
        self.v2 = C.CDLL(v2)
        self.v1 = C.CDLL(v1)
        self.v2.eoq_decode_tensor_v2.restype = C.c_int
        self.v2.eoq_decode_tensor_v2.argtypes = [C.POINTER(_Hdr), C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]
        self.v2.eoq_parallel_decode.restype = C.c_int
        self.v2.eoq_parallel_decode.argtypes = [C.POINTER(_Task), C.c_int, C.POINTER(_POpts)]
        self.v2.eoq_detect_num_threads.restype = C.c_int
        self.v1.eoq_encode_tensor.restype = C.c_int
        self.v1.eoq_encode_tensor.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(_Hdr)]

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(_HERE, "_ref", "libeoq_ref_v2.so"))

    def threads(self) -> int:
        return int(self.v2.eoq_detect_num_threads())

    def decode_v2(self, header: np.ndarray, payload: bytes, out_cap: Optional[int] = None) -> Tuple[int, np.ndarray]:
        h = _Hdr(*[int(v) for v in header])
        cap = int(header[6]) if out_cap is None else out_cap
        out = np.zeros(max(cap, 1), np.uint8)
        buf = _bytes_arr(payload)
        rc = self.v2.eoq_decode_tensor_v2(C.byref(h), buf.ctypes.data, len(payload), out.ctypes.data, cap, None)
        return rc, out[:int(header[6])]

    def encode_v1(self, data: np.ndarray) -> Tuple[np.ndarray, bytes]:
        """eoq_encode_tensor (llamacpp/eoq_rans.c:455-580): byte alphabet, p=16, 256-symbol blocks."""
        d = np.ascontiguousarray(data, np.uint8)
        cap = C.c_size_t(d.size * 2 + 4096)
        out = np.zeros(cap.value, np.uint8)
        h = _Hdr()
        rc = self.v1.eoq_encode_tensor(d.ctypes.data, d.size, 0, out.ctypes.data, C.byref(cap), C.byref(h))
        if rc != 0:
            raise RuntimeError("eoq_encode_tensor failed")
        hdr = np.array([getattr(h, n) for n, _ in _Hdr._fields_], np.uint32)
        return hdr, out[:cap.value].tobytes()

    def parallel_decode(self, items: Sequence[Tuple[np.ndarray, bytes]], num_threads: int = 0) -> Tuple[int, List[np.ndarray], float]:
        """Run eoq_parallel_decode over (header, payload) pairs.  Returns (rc, outputs, seconds)."""
        import time
        n = len(items)
        tasks = (_Task * n)()
        keep = []
        outs = []
        for i, (hdr, payload) in enumerate(items):
            h = _Hdr(*[int(v) for v in hdr])
            buf = _bytes_arr(payload)
            out = np.zeros(max(int(hdr[6]), 1), np.uint8)
            keep.append((h, buf))
            outs.append(out)
            tasks[i].header = C.pointer(h)
            tasks[i].compressed_data = buf.ctypes.data
            tasks[i].compressed_size = len(payload)
            tasks[i].output = out.ctypes.data
            tasks[i].output_capacity = int(hdr[6])
        opts = _POpts(num_threads, None, None)
        t0 = time.perf_counter()
        rc = self.v2.eoq_parallel_decode(tasks, n, C.byref(opts))
        dt = time.perf_counter() - t0
        return rc, [o[:int(h[6])] for o, (h, _) in zip(outs, items)], dt


class RefCuda:
    """ctypes view of the reference's CUDA decoder (llamacpp_integration/eoq_cuda_decompress.cu:529-567) compiled by
    `make -C oracle ref_cuda`: device pointers in, asynchronous launch of its one-thread-per-block kernel."""

    def __init__(self):
        path = os.path.join(_HERE, "_ref", "libeoq_ref_cuda.so")
        if not os.path.exists(path):
            raise FileNotFoundError("oracle/_ref/libeoq_ref_cuda.so is not built (make -C oracle ref_cuda)")
        self.lib = C.CDLL(path)
        vp = C.c_void_p
        self.lib.eoq_cuda_decode_tensor_device.restype = C.c_int
        self.lib.eoq_cuda_decode_tensor_device.argtypes = [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp]

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(_HERE, "_ref", "libeoq_ref_cuda.so"))

    def decode_device(self, d_stream, d_offsets, d_sizes, d_sym_info, d_out, nblocks, block_size, total, p, stream) -> int:
        return int(self.lib.eoq_cuda_decode_tensor_device(d_stream, d_offsets, d_sizes, d_sym_info, d_out, nblocks, block_size,
                                                          total, p, stream))


def decode_tiles(table: np.ndarray, p: int, g: int, bits: int, desc: np.ndarray, stream: np.ndarray,
                 rows: int, cols: int, head_bytes: int = 0) -> np.ndarray:
    """Scalar decode of the product's tiled device layout -> uint8 [rows, cols] (orc_decode_tiles)."""
    L = lib()
    L.orc_decode_tiles.restype = C.c_int
    L.orc_decode_tiles.argtypes = [C.POINTER(C.c_uint32), C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32),
                                   C.c_uint32, C.POINTER(C.c_uint8), C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32,
                                   C.POINTER(C.c_uint8)]
    table = np.ascontiguousarray(table, np.uint32)
    desc = np.ascontiguousarray(desc, np.uint32).reshape(-1, 6)
    stream = np.ascontiguousarray(stream, np.uint8)
    out = np.full((rows, cols), 255, np.uint8)
    rc = L.orc_decode_tiles(_p(table, C.c_uint32), p, g, bits, _p(desc, C.c_uint32), desc.shape[0],
                            _p(stream, C.c_uint8), stream.size, head_bytes, rows, cols, _p(out, C.c_uint8))
    if rc != 0:
        raise ValueError(f"orc_decode_tiles failed: {rc}")
    return out
