"""The allocation-free fused GEMV (eoq_b200_gemv_static_scratch) against the ordinary entry point.

Some callers -- a server that owns all of HBM through its own arena, a latency-critical thread,
a framework replaying recorded work -- cannot tolerate a library that allocates device memory,
so this entry point keeps its scratch in an array built into the library.  The array is shared by
every call and keeps the previous call's contents, so the check is made on two calls in a row,
with a different weight in between, and must hold both in a fresh process and after the rest of
the suite has used the GPU.  This file sorts last so that a run stopping at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.fused import EOQWeight
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _weight(n, k, seed, **kw):
    rng = np.random.default_rng(seed)
    codes, scales = O.quantize_absmax((rng.standard_normal((n, k)) * 0.02).astype(np.float32), 4, 128)
    return EOQWeight.from_symbols((codes + 7).astype(np.uint8), scales.astype(np.float16), **kw)


def _both(w, x, bias=None):
    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    rows = x.shape[0]
    y_ref = torch.empty(rows, w.rows, dtype=x.dtype, device="cuda")
    y_new = torch.full((rows, w.rows), float("nan"), dtype=x.dtype, device="cuda")
    code = {torch.float16: L.F16, torch.bfloat16: L.BF16, torch.float32: L.F32}[x.dtype]
    b = bias.data_ptr() if bias is not None else None
    L.check(lib.eoq_b200_gemv(w._h, x.data_ptr(), code, rows, y_ref.data_ptr(), code, b, stream))
    L.check(lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), code, rows, y_new.data_ptr(), code, b, stream))
    torch.cuda.synchronize()
    assert lib.eoq_b200_weight_status(w._h, stream) == 0
    return y_ref, y_new


def test_static_scratch_gemv_matches_allocating_entry_point_twice_in_a_row():
    w_a = _weight(300, 1408, 1)                 # several column segments, padded rows
    w_b = _weight(96, 4096, 2, symbols_per_step=2)
    g = torch.Generator(device="cuda").manual_seed(7)
    for call in range(2):                        # second pass starts from the first pass's leftovers
        for w, rows, dt in ((w_a, 1, torch.float16), (w_b, 5, torch.float32), (w_a, 8, torch.bfloat16)):
            x = torch.randn(rows, w.cols, device="cuda", generator=g).to(dt)
            bias = torch.randn(w.rows, device="cuda", generator=g)
            y_ref, y_new = _both(w, x, bias)
            assert torch.equal(y_ref, y_new), (call, rows, dt)     # same kernel, same order of additions
            assert O.rel_l2(y_new.float().cpu().numpy(), y_ref.float().cpu().numpy()) < 1e-3


def test_static_scratch_gemv_refuses_what_does_not_fit():
    lib = L.lib()
    # 2304 rows x 72 column segments x 8 rows of x x 4 B > 8 MiB
    w = _weight(2304, 4608, 3, target_tiles=72 * 24)
    assert w.info.num_col_segments >= 64
    x = torch.randn(8, w.cols, device="cuda")
    y = torch.empty(8, w.rows, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    need = w.info.num_col_segments * w.info.padded_rows * 8 * 4
    rc = lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), L.F32, 8, y.data_ptr(), L.F32, None, stream)
    if need > (8 << 20):
        assert rc == L.EOQ_ERR_BUFFER_TOO_SMALL
    else:
        assert rc == 0
    y1, y2 = _both(w, x[:1].contiguous())                          # one row of x fits, and still agrees
    assert torch.equal(y1, y2)
    assert lib.eoq_b200_gemv_static_scratch(None, x.data_ptr(), L.F32, 1, y.data_ptr(), L.F32, None, stream) == L.EOQ_ERR_NULL_PTR
    assert lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), L.F32, 9, y.data_ptr(), L.F32, None, stream) == L.EOQ_ERR_UNSUPPORTED
