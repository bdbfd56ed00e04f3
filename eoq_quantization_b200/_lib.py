"""ctypes binding of ``libeoq_b200.so`` (C ABI declared in ``include/eoq_b200.h``).

The library is the only compute path: if it cannot be loaded the import of any
compute function raises, and on a machine without a CUDA device every compute
entry point returns ``EOQ_ERR_CUDA`` -- there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libeoq_b200.so")

EOQ_OK = 0
EOQ_ERR_NULL_PTR = -1
EOQ_ERR_BUFFER_TOO_SMALL = -2
EOQ_ERR_CORRUPT_STREAM = -3
EOQ_ERR_INVALID_HEADER = -4
EOQ_ERR_ALLOC = -5
EOQ_ERR_THREAD = -6
EOQ_ERR_OVERFLOW = -7
EOQ_ERR_CUDA = -8
EOQ_ERR_UNSUPPORTED = -9

KIND_INT4_ABSMAX = 0
KIND_Q5_POLAR = 1
KIND_INT2_ABSMAX, KIND_INT3_ABSMAX, KIND_INT8_ABSMAX = 2, 3, 4
#: kind of the symmetric absmax code of a given width (symbol = code + qmax)
INT_KINDS = {2: KIND_INT2_ABSMAX, 3: KIND_INT3_ABSMAX, 4: KIND_INT4_ABSMAX, 8: KIND_INT8_ABSMAX}
F16, BF16, F32 = 0, 1, 2

#: every symbol include/eoq_b200.h declares
EXPORTS = [
    "eoq_error_string", "eoq_decode_tensor_v2", "eoq_decode_tensor", "eoq_validate_header",
    "eoq_decoder_init", "eoq_decoder_decode", "eoq_decoder_free",
    "eoq_parallel_decode", "eoq_detect_num_threads",
    "eoq_cuda_decode_tensor", "eoq_cuda_decode_tensor_device",
    "eoq_cuda_batch_init", "eoq_cuda_batch_create", "eoq_cuda_batch_prepare_tensor", "eoq_cuda_batch_launch",
    "eoq_cuda_batch_sync_and_free", "eoq_cuda_batch_destroy",
    "eoq_b200_decode_blocked", "eoq_b200_encode_blocked",
    "eoq_b200_tiles_build", "eoq_b200_tiles_view", "eoq_b200_tiles_free",
    "eoq_b200_weight_from_tiles", "eoq_b200_weight_from_symbols", "eoq_b200_weight_from_device_symbols", "eoq_b200_weight_from_rans", "eoq_b200_weight_destroy",
    "eoq_b200_weight_info", "eoq_b200_gemv", "eoq_b200_gemm",
    "eoq_b200_gather_create", "eoq_b200_gather_connect", "eoq_b200_gather_destroy", "eoq_b200_gather_buffer",
    "eoq_b200_gather_status", "eoq_b200_gather_set_timeout_ms", "eoq_b200_gather_wait", "eoq_b200_gemv_gather", "eoq_b200_gemv_static_scratch", "eoq_b200_gemv_host", "eoq_b200_gemv_host_async", "eoq_b200_weight_decode",
    "eoq_b200_dequant_packed", "eoq_b200_gemv_packed", "eoq_b200_gemv_polar_codes",
    "eoq_b200_weight_status",
]
#: exported for this project's benchmarks and tests only (declared in csrc/eoq_internal.h, not in the public header)
INTERNAL_EXPORTS = ["eoq_b200_tune", "eoq_b200_launch_count", "eoq_b200_weight_read"]


class EOQError(RuntimeError):
    def __init__(self, code: int, where: str = ""):
        self.code = int(code)
        msg = lib().eoq_error_string(self.code).decode()
        super().__init__(f"{where + ': ' if where else ''}{msg} (eoq_error_t {self.code})")


class TensorHeader(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("original_type", "num_blocks", "freq_table_size", "precision_bits",
                                          "rans_block_size", "compressed_size", "uncompressed_size")]


PROGRESS_FN = C.CFUNCTYPE(C.c_int, C.c_size_t, C.c_size_t, C.c_void_p)
PARALLEL_PROGRESS_FN = C.CFUNCTYPE(C.c_int, C.c_int, C.c_int, C.c_void_p)


class DecodeOpts(C.Structure):
    _fields_ = [("n_threads", C.c_uint32), ("progress_cb", PROGRESS_FN), ("progress_ud", C.c_void_p)]


class DecodeTask(C.Structure):
    _fields_ = [("header", C.POINTER(TensorHeader)), ("compressed_data", C.c_void_p), ("compressed_size", C.c_size_t),
                ("output", C.c_void_p), ("output_capacity", C.c_size_t), ("result", C.c_int), ("task_index", C.c_int)]


class ParallelOpts(C.Structure):
    _fields_ = [("num_threads", C.c_int), ("progress_cb", PARALLEL_PROGRESS_FN), ("progress_ud", C.c_void_p)]


class Decoder(C.Structure):
    _fields_ = [("state", C.c_uint32), ("stream", C.c_void_p), ("stream_pos", C.c_size_t), ("stream_end", C.c_size_t),
                ("precision_bits", C.c_uint32), ("precision_mask", C.c_uint32), ("sym_info", C.c_void_p)]


class WeightOpts(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("group", C.c_uint32),
                ("symbols_per_step", C.c_uint32), ("precision_bits", C.c_uint32), ("target_tiles", C.c_uint32),
                ("centroids", C.POINTER(C.c_float))]


class WeightInfo(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("padded_rows", C.c_uint32), ("group", C.c_uint32),
                ("kind", C.c_uint32), ("symbols_per_step", C.c_uint32), ("precision_bits", C.c_uint32),
                ("alphabet", C.c_uint32), ("num_tiles", C.c_uint32), ("num_col_segments", C.c_uint32),
                ("stream_bytes", C.c_uint64), ("table_bytes", C.c_uint64), ("scale_bytes", C.c_uint64),
                ("desc_bytes", C.c_uint64), ("scratch_bytes", C.c_uint64), ("bits_per_weight", C.c_double)]


class TilesView(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("padded_rows", C.c_uint32), ("group", C.c_uint32),
                ("kind", C.c_uint32), ("bits", C.c_uint32), ("symbols_per_step", C.c_uint32),
                ("precision_bits", C.c_uint32), ("num_tiles", C.c_uint32), ("num_col_segments", C.c_uint32),
                ("table", C.POINTER(C.c_uint32)), ("tiles", C.POINTER(C.c_uint32)), ("stream", C.POINTER(C.c_uint8)),
                ("stream_bytes", C.c_uint64), ("max_lane_drift", C.c_uint32), ("head_bytes", C.c_uint32)]


_LIB: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Load the library (building it first if it is missing and nvcc is present)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    L = C.CDLL(LIB_PATH)
    vp, u8p, u16p, u32p = C.c_void_p, C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.POINTER(C.c_uint32)
    hp = C.POINTER(TensorHeader)
    sig = {
        "eoq_error_string": (C.c_char_p, [C.c_int]),
        "eoq_decode_tensor_v2": (C.c_int, [hp, vp, C.c_size_t, vp, C.c_size_t, C.POINTER(DecodeOpts)]),
        "eoq_decode_tensor": (C.c_int, [hp, vp, vp]),
        "eoq_validate_header": (C.c_int, [hp]),
        "eoq_decoder_init": (C.c_int, [C.POINTER(Decoder), vp, C.c_uint32, C.c_uint32, vp, C.c_size_t]),
        "eoq_decoder_decode": (C.c_int, [C.POINTER(Decoder), vp, C.c_uint32]),
        "eoq_decoder_free": (None, [C.POINTER(Decoder)]),
        "eoq_parallel_decode": (C.c_int, [C.POINTER(DecodeTask), C.c_int, C.POINTER(ParallelOpts)]),
        "eoq_detect_num_threads": (C.c_int, []),
        "eoq_cuda_decode_tensor": (C.c_int, [hp, vp, vp, vp]),
        "eoq_cuda_decode_tensor_device": (C.c_int, [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp]),
        "eoq_cuda_batch_init": (None, [vp, vp]),
        "eoq_cuda_batch_create": (vp, [vp]),
        "eoq_cuda_batch_prepare_tensor": (C.c_int, [vp, hp, vp, vp]),
        "eoq_cuda_batch_launch": (C.c_int, [vp]),
        "eoq_cuda_batch_sync_and_free": (C.c_int, [vp]),
        "eoq_cuda_batch_destroy": (None, [vp]),
        "eoq_b200_decode_blocked": (C.c_int, [vp, C.c_uint32, C.c_uint32, vp, C.c_size_t, vp, C.c_uint32, C.c_uint32,
                                              C.c_uint32, vp, C.c_int, C.c_int, vp]),
        "eoq_b200_encode_blocked": (C.c_int, [vp, C.c_uint32, C.c_uint32, vp, C.c_uint32, C.c_uint32, vp,
                                              C.POINTER(C.c_size_t), vp]),
        "eoq_b200_tiles_build": (C.c_int, [vp, C.POINTER(WeightOpts), C.POINTER(vp)]),
        "eoq_b200_tiles_view": (C.c_int, [vp, C.POINTER(TilesView)]),
        "eoq_b200_tiles_free": (None, [vp]),
        "eoq_b200_weight_from_tiles": (C.c_int, [vp, vp, vp, C.POINTER(vp)]),
        "eoq_b200_weight_from_symbols": (C.c_int, [vp, vp, C.POINTER(WeightOpts), C.POINTER(vp)]),
        "eoq_b200_weight_from_device_symbols": (C.c_int, [vp, vp, C.POINTER(WeightOpts), C.POINTER(vp)]),
        "eoq_b200_weight_from_rans": (C.c_int, [vp, C.c_size_t, vp, C.POINTER(WeightOpts), C.POINTER(vp)]),
        "eoq_b200_weight_destroy": (None, [vp]),
        "eoq_b200_weight_info": (C.c_int, [vp, C.POINTER(WeightInfo)]),
        "eoq_b200_gemv": (C.c_int, [vp, vp, C.c_int, C.c_uint32, vp, C.c_int, vp, vp]),
        "eoq_b200_gather_create": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_size_t, C.POINTER(vp), vp]),
        "eoq_b200_gather_connect": (C.c_int, [vp, vp]),
        "eoq_b200_gather_destroy": (None, [vp]),
        "eoq_b200_gather_buffer": (vp, [vp, C.c_uint32]),
        "eoq_b200_gather_status": (C.c_int, [vp, vp]),
        "eoq_b200_gather_set_timeout_ms": (C.c_int, [vp, C.c_uint32]),
        "eoq_b200_gather_wait": (C.c_int, [vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_uint32, vp]),
        "eoq_b200_gemv_gather": (C.c_int, [vp, vp, C.c_int, C.c_uint32, C.c_int, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, vp]),
        "eoq_b200_gemm": (C.c_int, [vp, vp, C.c_int, C.c_uint32, vp, C.c_int, vp, vp]),
        "eoq_b200_gemv_static_scratch": (C.c_int, [vp, vp, C.c_int, C.c_uint32, vp, C.c_int, vp, vp]),
        "eoq_b200_gemv_host": (C.c_int, [vp, vp, C.c_int, C.c_uint32, vp, C.c_int, vp, vp]),
        "eoq_b200_gemv_host_async": (C.c_int, [vp, vp, C.c_int, C.c_uint32, vp, C.c_int, vp, vp]),
        "eoq_b200_weight_decode": (C.c_int, [vp, vp, C.c_int, vp, C.c_int, vp]),
        "eoq_b200_dequant_packed": (C.c_int, [vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                              C.c_uint32, vp, C.c_int, vp]),
        "eoq_b200_gemv_packed": (C.c_int, [vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp, C.c_int, C.c_uint32, vp, vp, C.c_int, vp, vp]),
        "eoq_b200_gemv_polar_codes": (C.c_int, [vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp, C.c_int, C.c_uint32, vp, vp, C.c_int, vp, C.c_int, vp]),
        "eoq_b200_weight_status": (C.c_int, [vp, vp]),
        "eoq_b200_tune": (C.c_int, [C.c_char_p, C.c_int]),
        "eoq_b200_launch_count": (C.c_uint64, []),
        "eoq_b200_weight_read": (C.c_uint64, [vp, C.c_int, vp, C.c_uint64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


def check(code: int, where: str = "") -> None:
    if code != EOQ_OK:
        raise EOQError(code, where)
