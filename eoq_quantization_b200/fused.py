"""Python face of the fused path: a weight matrix resident in HBM as
entropy-coded tiles (``eoq_b200_weight_t``) and the calls that consume it.

torch is used for device memory and streams only; every computation is a call
into ``libeoq_b200.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib

_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}
_I8 = 3        # EOQ_B200_I8: eoq_b200_dequant_packed writes the signed codes
_NP_DTYPES = {np.dtype(np.float16): _lib.F16, np.dtype(np.float32): _lib.F32}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: tensor is on {t.device}; this implementation computes on a CUDA device only "
                           "(there is no CPU path)")


# Rows up to which `linear` and the reference-API modules use the fused decode + GEMV: four rows of 16-bit activations
# (one launch), eight of fp32 activations.  Beyond, the weight is decoded once to a dense matrix (1.0 T symbols/s; a
# 16-bit matrix stays in the 126 MB L2) for a library GEMM.  Measured, graph replay, fp16: 11008 x 4096 at 4 / 5 / 8 rows
# 33.9 / 51.8 / 63.8 us fused (a second launch from the fifth row on) against 47.4 / 47.5 / 47.7 us decode + GEMM;
# 4096 x 4096: 28.7 / 42.8 / 52.8 against 26.8; at 16 rows and more the fused decode + tensor-core kernel
# (`EOQWeight.gemm`, still there to be called) loses as well, 39 against 34 us at 16 rows and 92 against 37 us at 256
# rows on 3584 x 8192: it decodes one tile per warp through a word ring, at half the rate of the two-tiles-per-warp decoders.
GEMV_MAX_ROWS = {torch.float16: 4, torch.bfloat16: 4, torch.float32: 8}
GEMM_MAX_ROWS = 8       # rows up to which the tensor-core kernel would be preferred to decode + library GEMM: none above the GEMV's
PACKED_TENSOR_ROWS = 32       # activation rows the tensor-core form of the packed GEMV takes per launch


def fused_rows(dtype: torch.dtype) -> int:
    """Activation rows up to which the fused decode + GEMV is the fastest route for this activation type."""
    return GEMV_MAX_ROWS.get(dtype, 0)


class EOQWeight:
    """Owner of one ``eoq_b200_weight_t`` (resident on the device that was current when it was built)."""

    def __init__(self, handle: int, kind: int):
        self._h = C.c_void_p(handle)
        self.kind = kind
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        info = _lib.WeightInfo()
        _lib.check(_lib.lib().eoq_b200_weight_info(self._h, C.byref(info)), "eoq_b200_weight_info")
        self.info = info
        self.rows, self.cols = info.rows, info.cols

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.lib().eoq_b200_weight_destroy(h)
            except Exception:
                pass

    # -- construction --------------------------------------------------------
    @staticmethod
    def _opts(kind: int, rows: int, cols: int, group: int, symbols_per_step: int, precision_bits: int,
              target_tiles: int, centroids: Optional[Sequence[float]]):
        cent = None
        if centroids is not None:
            cent = (C.c_float * 32)(*[float(v) for v in centroids])
        o = _lib.WeightOpts(kind, rows, cols, group, symbols_per_step, precision_bits, target_tiles,
                            C.cast(cent, C.POINTER(C.c_float)) if cent is not None else None)
        return o, cent

    @classmethod
    def from_symbols(cls, symbols, scales_fp16, *, kind: int = _lib.KIND_INT4_ABSMAX, group: int = 128,
                     symbols_per_step: int = 0, precision_bits: int = 0, target_tiles: int = 0,
                     centroids: Optional[Sequence[float]] = None) -> "EOQWeight":
        """symbols: uint8 [N, K] (INT4: code+7; polar: centroid index); scales_fp16: float16 [N*K/group]."""
        sym = np.ascontiguousarray(symbols.detach().cpu().numpy() if isinstance(symbols, torch.Tensor) else symbols,
                                   dtype=np.uint8)
        sc = scales_fp16.detach().cpu().numpy() if isinstance(scales_fp16, torch.Tensor) else np.asarray(scales_fp16)
        sc = np.ascontiguousarray(sc.astype(np.float16, copy=False))
        n, k = sym.shape
        if sc.size != n * k // group:
            raise ValueError(f"expected {n * k // group} scales, got {sc.size}")
        o, keep = cls._opts(kind, n, k, group, symbols_per_step, precision_bits, target_tiles, centroids)
        h = C.c_void_p()
        _lib.check(_lib.lib().eoq_b200_weight_from_symbols(sym.ctypes.data, sc.ctypes.data, C.byref(o), C.byref(h)),
                   "eoq_b200_weight_from_symbols")
        return cls(h.value, kind)

    @classmethod
    def replicas(cls, count: int, symbols, scales_fp16, *, kind: int = _lib.KIND_INT4_ABSMAX, group: int = 128,
                 symbols_per_step: int = 0, precision_bits: int = 0, target_tiles: int = 0,
                 centroids: Optional[Sequence[float]] = None) -> list:
        """Encode once on the host, upload `count` independent copies to the current device."""
        sym = np.ascontiguousarray(symbols.detach().cpu().numpy() if isinstance(symbols, torch.Tensor) else symbols,
                                   dtype=np.uint8)
        sc = scales_fp16.detach().cpu().numpy() if isinstance(scales_fp16, torch.Tensor) else np.asarray(scales_fp16)
        sc = np.ascontiguousarray(sc.astype(np.float16, copy=False))
        n, k = sym.shape
        o, keep = cls._opts(kind, n, k, group, symbols_per_step, precision_bits, target_tiles, centroids)
        L = _lib.lib()
        tiles = C.c_void_p()
        _lib.check(L.eoq_b200_tiles_build(sym.ctypes.data, C.byref(o), C.byref(tiles)), "eoq_b200_tiles_build")
        out = []
        try:
            for _ in range(count):
                h = C.c_void_p()
                _lib.check(L.eoq_b200_weight_from_tiles(tiles, sc.ctypes.data, keep, C.byref(h)), "eoq_b200_weight_from_tiles")
                out.append(cls(h.value, kind))
        finally:
            L.eoq_b200_tiles_free(tiles)
        return out

    @classmethod
    def from_device_symbols(cls, symbols: torch.Tensor, scales_fp16, *, kind: int = _lib.KIND_INT4_ABSMAX, group: int = 128,
                            symbols_per_step: int = 0, precision_bits: int = 0, target_tiles: int = 0,
                            centroids: Optional[Sequence[float]] = None) -> "EOQWeight":
        """symbols: uint8 [N, K] on a CUDA device; counted, encoded into tiles and laid out there (no copy to the host)."""
        require_cuda(symbols, "EOQWeight.from_device_symbols")
        sym = symbols.detach().to(torch.uint8).contiguous()
        sc = scales_fp16.detach().cpu().numpy() if isinstance(scales_fp16, torch.Tensor) else np.asarray(scales_fp16)
        sc = np.ascontiguousarray(sc.astype(np.float16, copy=False))
        n, k = sym.shape
        o, keep = cls._opts(kind, n, k, group, symbols_per_step, precision_bits, target_tiles, centroids)
        h = C.c_void_p()
        with torch.cuda.device(sym.device):
            torch.cuda.current_stream().synchronize()          # the library encodes on the default stream
            _lib.check(_lib.lib().eoq_b200_weight_from_device_symbols(sym.data_ptr(), sc.ctypes.data, C.byref(o), C.byref(h)),
                       "eoq_b200_weight_from_device_symbols")
            return cls(h.value, kind)

    @classmethod
    def from_int4_packed(cls, packed, scales_fp16, in_features: int, *, group: int = 128, **kw) -> "EOQWeight":
        """packed: QuantizedLinear.packed_weight, uint8 [N, K/2], low nibble = even column, value code+7."""
        return cls.from_packed(packed, scales_fp16, in_features, 4, group=group, **kw)

    @classmethod
    def from_packed(cls, packed, scales_fp16, in_features: int, bits: int, *, group: int = 128, **kw) -> "EOQWeight":
        """packed: QuantizedLinear.packed_weight of any width the fused kernels serve (core/quantized_linear.py:49-66):
        4 bits two per byte, 2 bits four per byte (low bits first), 3 and 8 bits one signed code per byte.  A tensor on
        a CUDA device is unpacked and encoded there."""
        if bits not in _lib.INT_KINDS:
            raise ValueError(f"no fused layout for {bits}-bit weights")
        qmax = (1 << (bits - 1)) - 1
        if isinstance(packed, torch.Tensor) and packed.is_cuda:
            pk = packed.detach()
            if bits == 4:
                sym = torch.stack([pk & 0x0F, pk >> 4], dim=-1).reshape(pk.shape[0], -1)
            elif bits == 2:
                sym = torch.stack([(pk >> s) & 0x03 for s in (0, 2, 4, 6)], dim=-1).reshape(pk.shape[0], -1)
            else:
                sym = (pk.view(torch.int8).to(torch.int16) + qmax).to(torch.uint8)
            return cls.from_device_symbols(sym[:, :in_features], scales_fp16, kind=_lib.INT_KINDS[bits], group=group, **kw)
        pk = packed.detach().cpu().numpy() if isinstance(packed, torch.Tensor) else np.asarray(packed)
        if bits == 4:
            sym = np.stack([pk & 0x0F, pk >> 4], axis=-1).reshape(pk.shape[0], -1)
        elif bits == 2:
            sym = np.stack([(pk >> s) & 0x03 for s in (0, 2, 4, 6)], axis=-1).reshape(pk.shape[0], -1)
        else:
            sym = (pk.view(np.int8).astype(np.int16) + qmax).astype(np.uint8)
        return cls.from_symbols(np.ascontiguousarray(sym[:, :in_features]), scales_fp16, kind=_lib.INT_KINDS[bits], group=group, **kw)

    @classmethod
    def from_rans(cls, rans_bytes: bytes, scales_fp16, shape, *, kind: int = _lib.KIND_INT4_ABSMAX, group: int = 128,
                  symbols_per_step: int = 0, precision_bits: int = 0, target_tiles: int = 0,
                  centroids: Optional[Sequence[float]] = None) -> "EOQWeight":
        """rans_bytes: the reference's serialised `RANS` container of the symbols of an [N, K] matrix."""
        buf = np.frombuffer(rans_bytes, dtype=np.uint8)
        sc = np.frombuffer(scales_fp16, dtype=np.float16) if isinstance(scales_fp16, (bytes, bytearray)) else \
            np.ascontiguousarray(np.asarray(scales_fp16).astype(np.float16, copy=False))
        n, k = shape
        o, keep = cls._opts(kind, n, k, group, symbols_per_step, precision_bits, target_tiles, centroids)
        h = C.c_void_p()
        _lib.check(_lib.lib().eoq_b200_weight_from_rans(buf.ctypes.data, buf.size, sc.ctypes.data, C.byref(o), C.byref(h)),
                   "eoq_b200_weight_from_rans")
        return cls(h.value, kind)

    def _on_device(self, x: torch.Tensor, what: str):
        """Context that makes the weight's device current; raises if x lives elsewhere (the kernels take raw pointers)."""
        require_cuda(x, what)
        if self.device is not None and x.device != self.device:
            raise RuntimeError(f"{what}: the activations are on {x.device} but the weight lives on {self.device}")
        return torch.cuda.device(x.device)

    # -- use -------------------------------------------------------------------
    def gemv(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """y = x @ W.T (+ bias) for x of shape (..., K) with at most 8 rows in total."""
        require_cuda(x, "EOQWeight.gemv")
        if x.shape[-1] != self.cols:
            raise ValueError(f"expected last dimension {self.cols}, got {x.shape[-1]}")
        if x.dtype not in _DTYPES:
            raise TypeError(f"unsupported activation dtype {x.dtype}")
        x2 = x.reshape(-1, self.cols).contiguous()
        rows = x2.shape[0]
        out_dtype = out_dtype or x.dtype
        y = torch.empty((rows, self.rows), dtype=out_dtype, device=x.device)
        b = None
        if bias is not None:
            b = bias.to(device=x.device, dtype=torch.float32).contiguous()
        with self._on_device(x, "EOQWeight.gemv"):
            for lo in range(0, rows, 8):
                hi = min(rows, lo + 8)
                _lib.check(_lib.lib().eoq_b200_gemv(self._h, x2[lo:hi].data_ptr(), _DTYPES[x.dtype], hi - lo,
                                                    y[lo:hi].data_ptr(), _DTYPES[out_dtype],
                                                    b.data_ptr() if b is not None else None, _stream_ptr()), "eoq_b200_gemv")
        return y.reshape(*x.shape[:-1], self.rows)

    def gemm(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """y = x @ W.T (+ bias) for any number of rows: decoded fp16 tiles feed tcgen05 MMAs (INT4 kind only).

        The fused counterpart of dequantize-then-matmul (core/quantized_linear.py:222-228) for prefill.
        """
        require_cuda(x, "EOQWeight.gemm")
        if x.shape[-1] != self.cols:
            raise ValueError(f"expected last dimension {self.cols}, got {x.shape[-1]}")
        if x.dtype not in _DTYPES:
            raise TypeError(f"unsupported activation dtype {x.dtype}")
        x2 = x.reshape(-1, self.cols).contiguous()
        out_dtype = out_dtype or x.dtype
        y = torch.empty((x2.shape[0], self.rows), dtype=out_dtype, device=x.device)
        b = None
        if bias is not None:
            b = bias.to(device=x.device, dtype=torch.float32).contiguous()
        with self._on_device(x, "EOQWeight.gemm"):
            _lib.check(_lib.lib().eoq_b200_gemm(self._h, x2.data_ptr(), _DTYPES[x.dtype], x2.shape[0], y.data_ptr(), _DTYPES[out_dtype],
                                                b.data_ptr() if b is not None else None, _stream_ptr()), "eoq_b200_gemm")
        return y.reshape(*x.shape[:-1], self.rows)

    def linear(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y = x @ W.T (+ bias) in x.dtype by the fastest route built for the number of rows: up to `fused_rows` the
        fused decode + GEMV; beyond, the weight is decoded to a dense matrix once (fused decode + dequantise kernel)
        for a library GEMM.  (Were GEMM_MAX_ROWS raised above 8, 16-bit activations on 4-bit weights would take the
        fused decode + tensor-core kernel, `gemm`, up to that many rows.)"""
        require_cuda(x, "EOQWeight.linear")
        rows = x.numel() // max(self.cols, 1)
        if rows >= 1 and x.dtype in _DTYPES:
            if rows <= fused_rows(x.dtype):
                return self.gemv(x, bias)
            if 8 < rows <= GEMM_MAX_ROWS and x.dtype != torch.float32 and self.kind == _lib.KIND_INT4_ABSMAX and self.cols % 16 == 0:
                return self.gemm(x, bias)
        dt = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.float32
        with self._on_device(x, "EOQWeight.linear"):
            w = self.dequantize(dt, device=x.device)
        return torch.nn.functional.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))

    def status(self) -> int:
        """0, or the status word a kernel left after a bounded wait gave up (synchronises the current stream)."""
        return int(_lib.lib().eoq_b200_weight_status(self._h, _stream_ptr()))

    def gemv_host(self, x: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
        """Same with numpy buffers on the host (copies in, runs, copies out, synchronises)."""
        x2 = np.ascontiguousarray(x).reshape(-1, self.cols)
        if x2.dtype not in _NP_DTYPES:
            raise TypeError(f"unsupported activation dtype {x2.dtype}")
        if x2.shape[0] > 8:
            raise ValueError("at most 8 rows per call")
        y = np.empty((x2.shape[0], self.rows), x2.dtype)
        b = None if bias is None else np.ascontiguousarray(bias, np.float32)
        code = _NP_DTYPES[x2.dtype]
        _lib.check(_lib.lib().eoq_b200_gemv_host(self._h, x2.ctypes.data, code, x2.shape[0], y.ctypes.data, code,
                                                 b.ctypes.data if b is not None else None, None), "eoq_b200_gemv_host")
        return y.reshape(*np.shape(x)[:-1], self.rows)

    def decode_symbols(self, packed: bool = False, device=None) -> torch.Tensor:
        """Decoded symbols: uint8 [N, K], or packed two per byte [N, K/2] as QuantizedLinear stores them."""
        dev = torch.device(device) if device is not None else (self.device or torch.device("cuda"))
        shape = (self.rows, self.cols // 2) if packed else (self.rows, self.cols)
        out = torch.empty(shape, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().eoq_b200_weight_decode(self._h, out.data_ptr(), int(packed), None, 0, _stream_ptr()),
                       "eoq_b200_weight_decode")
        return out

    def dequantize(self, dtype: torch.dtype = torch.float16, device=None) -> torch.Tensor:
        """Dense [N, K] matrix (INT4 kind): (sym - 7) * scale."""
        dev = torch.device(device) if device is not None else (self.device or torch.device("cuda"))
        out = torch.empty((self.rows, self.cols), dtype=dtype, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().eoq_b200_weight_decode(self._h, None, 0, out.data_ptr(), _DTYPES[dtype], _stream_ptr()),
                       "eoq_b200_weight_decode")
        return out


def dequant_packed(packed: torch.Tensor, scales: torch.Tensor, rows: int, cols: int, bits: int, group: int,
                   row_lo: int = 0, row_hi: Optional[int] = None, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Dense rows [row_lo, row_hi) of a packed QuantizedLinear weight, computed by the library's kernel; with
    dtype torch.int8 the signed codes themselves (scales may then be None)."""
    require_cuda(packed, "dequant_packed")
    row_hi = rows if row_hi is None else row_hi
    pk = packed.contiguous()
    sc = None if scales is None else scales.to(device=packed.device, dtype=torch.float16).contiguous()
    out = torch.empty((row_hi - row_lo, cols), dtype=dtype, device=packed.device)
    code = _I8 if dtype == torch.int8 else _DTYPES[dtype]
    with torch.cuda.device(packed.device):
        _lib.check(_lib.lib().eoq_b200_dequant_packed(pk.data_ptr(), sc.data_ptr() if sc is not None else None, rows, cols, bits, group,
                                                      row_lo, row_hi, out.data_ptr(), code, _stream_ptr()), "eoq_b200_dequant_packed")
    return out


def packed_gemv_rows(cols: int, bits: int, group: int, dtype: torch.dtype = torch.float16) -> int:
    """Activation rows `gemv_packed` takes for this shape: 32 on its tensor-core form (scale groups of whole 128-column
    spans; fp32 activations go in as two fp16 halves each), 8 on the general form, 0 if it does not apply."""
    if not (2 <= bits <= 8 and group > 0 and cols % group == 0):
        return 0
    if dtype in _DTYPES and cols % 128 == 0 and group % 128 == 0:
        return PACKED_TENSOR_ROWS
    per16 = 32 if bits == 4 else 64 if bits == 2 else 16                 # codes in the sixteen bytes a lane loads
    return 8 if cols % per16 == 0 and group % 8 == 0 else 0


def packed_gemv_applies(cols: int, bits: int, group: int, dtype: torch.dtype = torch.float16, rows: int = 1) -> bool:
    """Whether `gemv_packed` takes this shape and row count (else: `dequant_packed` and a GEMM)."""
    return 1 <= rows <= packed_gemv_rows(cols, bits, group, dtype)


def gemv_packed(packed: torch.Tensor, scales: torch.Tensor, rows: int, cols: int, bits: int, group: int, x: torch.Tensor,
                bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ W.T (+ bias) for at most `packed_gemv_rows` rows of x, straight from a packed QuantizedLinear weight
    (codes + fp16 scales resident on the device): one pass over the packed bytes, fp32 accumulation, no dense matrix
    in between."""
    require_cuda(packed, "gemv_packed")
    require_cuda(x, "gemv_packed")
    if x.device != packed.device:
        raise RuntimeError(f"gemv_packed: the activations are on {x.device} but the weight lives on {packed.device}")
    if x.shape[-1] != cols:
        raise ValueError(f"expected last dimension {cols}, got {x.shape[-1]}")
    if x.dtype not in _DTYPES:
        raise TypeError(f"unsupported activation dtype {x.dtype}")
    x2 = x.reshape(-1, cols).contiguous()
    n = x2.shape[0]
    if x2.data_ptr() % 16:
        x2 = x2.clone()
    if n > packed_gemv_rows(cols, bits, group, x.dtype):
        raise ValueError(f"at most {packed_gemv_rows(cols, bits, group, x.dtype)} rows per call for this shape and dtype")
    pk = packed.contiguous()
    sc = scales.to(device=packed.device, dtype=torch.float16).contiguous()
    out_dtype = out_dtype or x.dtype
    y = torch.empty((n, rows), dtype=out_dtype, device=x.device)
    b = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    # fp32 activations on the tensor-core form: room for their two fp16 halves
    scratch = torch.empty((n, cols), dtype=torch.float32, device=x.device) if x.dtype == torch.float32 and cols % 128 == 0 and group % 128 == 0 else None
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().eoq_b200_gemv_packed(pk.data_ptr(), sc.data_ptr(), rows, cols, bits, group, x2.data_ptr(), _DTYPES[x.dtype], n,
                                                   scratch.data_ptr() if scratch is not None else None,
                                                   y.data_ptr(), _DTYPES[out_dtype], b.data_ptr() if b is not None else None, _stream_ptr()),
                   "eoq_b200_gemv_packed")
    return y.reshape(*x.shape[:-1], rows)


def polar_codes_gemv_applies(cols: int, bits: int, block: int, rows: int = 1) -> bool:
    """Whether `gemv_polar_codes` takes this configuration and row count (8 rows on the CUDA cores, 32 on the tensor
    cores, which need blocks of 64 columns and more)."""
    return (1 <= rows <= (32 if block >= 64 else 8) and 1 <= bits <= 8 and 16 <= block <= 4096 and block & (block - 1) == 0 and
            cols % block == 0)


def gemv_polar_codes(codes: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor, rows: int, cols: int,
                     bits: int, block: int, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     out_dtype: torch.dtype = torch.float32, tensor_cores: Optional[bool] = None) -> torch.Tensor:
    """y = x @ W.T (+ bias) for at most 8 rows of x (32 on the tensor cores), straight from PolarLinear's buffers (one centroid index per byte, fp16
    norms, fp32 centroids; kernels/polar_engine.py:144-360): x is rotated once per call (every block times the symmetric
    normalised Hadamard matrix, divided by sqrt(block)), the weight is never materialised.  `tensor_cores`: True (blocks
    of 64 columns and more: centroids and activations as two fp16 halves each, fp32 accumulation, within about 1e-6 of
    the fp32 form), False (CUDA cores, fp32 throughout), None: the quicker of the two for this row count."""
    require_cuda(codes, "gemv_polar_codes")
    require_cuda(x, "gemv_polar_codes")
    if x.device != codes.device:
        raise RuntimeError(f"gemv_polar_codes: the activations are on {x.device} but the weight lives on {codes.device}")
    if x.shape[-1] != cols:
        raise ValueError(f"expected last dimension {cols}, got {x.shape[-1]}")
    if x.dtype not in _DTYPES:
        raise TypeError(f"unsupported activation dtype {x.dtype}")
    x2 = x.reshape(-1, cols).contiguous()
    n = x2.shape[0]
    if not polar_codes_gemv_applies(cols, bits, block, n) or (tensor_cores and block < 64) or (tensor_cores is False and n > 8):
        raise ValueError("at most 8 rows (tensor cores: 32); blocks that are powers of two from 16 (tensor cores: 64) to 4096 and divide the row")
    cd = codes.reshape(-1)[:rows * cols].contiguous().view(torch.uint8)
    nr = norms.to(device=codes.device, dtype=torch.float16).contiguous()
    ct = centroids.to(device=codes.device, dtype=torch.float32).contiguous()
    scratch = torch.empty((n, cols), dtype=torch.float32, device=x.device)          # the rotated activations
    y = torch.empty((n, rows), dtype=out_dtype, device=x.device)
    b = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().eoq_b200_gemv_polar_codes(cd.data_ptr(), nr.data_ptr(), ct.data_ptr(), rows, cols, bits, block, x2.data_ptr(),
                                                        _DTYPES[x.dtype], n, scratch.data_ptr(), y.data_ptr(), _DTYPES[out_dtype],
                                                        b.data_ptr() if b is not None else None,
                                                        -1 if tensor_cores is None else int(tensor_cores), _stream_ptr()),
                   "eoq_b200_gemv_polar_codes")
    return y.reshape(*x.shape[:-1], rows)
