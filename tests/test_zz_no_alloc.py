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


def _layer(n, k, seed):
    rng = np.random.default_rng(seed)
    codes, scales = O.quantize_absmax((rng.standard_normal((n, k)) * 0.02).astype(np.float32), 4, 128)
    return codes, scales.astype(np.float16)


def _weight(n, k, seed, **kw):
    codes, s16 = _layer(n, k, seed)
    return EOQWeight.from_symbols((codes + 7).astype(np.uint8), s16, **kw)


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
    codes_a, s16_a = _layer(300, 1408, 1)        # several column segments, padded rows
    w_a = EOQWeight.from_symbols((codes_a + 7).astype(np.uint8), s16_a)
    w_b = _weight(96, 4096, 2, symbols_per_step=2)
    packed_a = O.pack_int4_rows(codes_a)
    g = torch.Generator(device="cuda").manual_seed(7)
    for call in range(2):                        # second pass starts from the first pass's leftovers
        for w, rows, dt in ((w_a, 1, torch.float16), (w_b, 5, torch.float32), (w_a, 8, torch.bfloat16), (w_a, 3, torch.float32)):
            x = torch.randn(rows, w.cols, device="cuda", generator=g).to(dt)
            bias = torch.randn(w.rows, device="cuda", generator=g)
            y_ref, y_new = _both(w, x, bias)
            # the two entry points meet their partial rows differently, so the last bits may differ: same tolerance as
            # every GEMV parity test
            assert O.rel_l2(y_new.float().cpu().numpy(), y_ref.float().cpu().numpy()) < 1e-3, (call, rows, dt)
            if w is w_a:                          # and against the CPU oracle: dequantise, then multiply
                want = O.int4_linear(packed_a, s16_a.astype(np.float32).reshape(-1), 300, 1408, 128, x.float().cpu().numpy(),
                                     bias.cpu().numpy())
                tol = 1e-3 if dt != torch.bfloat16 else 5e-3       # bf16 output rounding alone is 1.1e-3
                assert O.rel_l2(y_new.float().cpu().numpy(), want) < tol, (call, rows, dt)


def test_static_scratch_gemv_allocates_nothing_in_steady_state():
    lib = L.lib()
    w = _weight(192, 2048, 5)
    x = torch.randn(1, w.cols, device="cuda", dtype=torch.float16)
    y = torch.empty(1, w.rows, device="cuda", dtype=torch.float16)
    stream = torch.cuda.current_stream().cuda_stream
    L.check(lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), L.F16, 1, y.data_ptr(), L.F16, None, stream))   # first call on this device: set-up
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(50):
        L.check(lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), L.F16, 1, y.data_ptr(), L.F16, None, stream))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0


@pytest.mark.parametrize("n,k,batch", [(28672, 8192, 1), (11008, 4096, 8)])
def test_static_scratch_takes_the_default_layout_at_full_size(n, k, batch):
    """The scratch request follows the kernel that runs: weights in the default layout need a few partial rows per
    pair of row blocks, so a Llama-70B gate projection and eight rows on a Llama-7B projection fit the built-in array."""
    g = torch.Generator(device="cuda").manual_seed(n)
    wt = torch.randn(n, k, device="cuda", generator=g) * 0.02
    scale = (wt.view(-1, 128).abs().amax(dim=1) / 7).clamp(min=1e-10)
    codes = (wt.view(-1, 128) / scale[:, None]).round().clamp(-7, 7).to(torch.int8).view(n, k)
    w = EOQWeight.from_symbols((codes + 7).to(torch.uint8), scale.half())
    x = torch.randn(batch, k, device="cuda", generator=g).half()
    y_ref, y_new = _both(w, x)
    assert O.rel_l2(y_new.float().cpu().numpy(), y_ref.float().cpu().numpy()) < 1e-3
    dense = (codes.float().view(-1, 128) * scale.half().float()[:, None]).view(n, k)
    assert O.rel_l2(y_new.float().cpu().numpy(), (x.float() @ dense.T).cpu().numpy()) < 1e-3


def test_static_scratch_gemv_refuses_what_does_not_fit():
    lib = L.lib()
    # two symbols per step: one tile per warp, one partial row per column segment (and eight rows of a 2304-column x
    # fit shared memory, so the call is not split): 36 column segments x 8192 rows x 8 rows of x x 4 B = 9.4 MB > 8 MiB
    w = _weight(8192, 2304, 3, symbols_per_step=2, target_tiles=36 * 128)
    assert w.info.num_col_segments == 36 and w.info.padded_rows == 8192
    x = torch.randn(8, w.cols, device="cuda")
    y = torch.full((8, w.rows), 5.0, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert w.info.num_col_segments * w.info.padded_rows * 8 * 4 > (8 << 20)
    rc = lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), L.F32, 8, y.data_ptr(), L.F32, None, stream)
    assert rc == L.EOQ_ERR_BUFFER_TOO_SMALL
    torch.cuda.synchronize()
    assert float(y.min()) == 5.0 and float(y.max()) == 5.0          # refused before anything ran
    y1, y2 = _both(w, x[:1].contiguous())                          # one row of x fits, and still agrees
    assert O.rel_l2(y2.cpu().numpy(), y1.cpu().numpy()) < 1e-3
    assert lib.eoq_b200_gemv_static_scratch(None, x.data_ptr(), L.F32, 1, y.data_ptr(), L.F32, None, stream) == L.EOQ_ERR_NULL_PTR
    assert lib.eoq_b200_gemv_static_scratch(w._h, x.data_ptr(), L.F32, 9, y.data_ptr(), L.F32, None, stream) == L.EOQ_ERR_UNSUPPORTED
