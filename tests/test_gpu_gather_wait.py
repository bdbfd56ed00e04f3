"""Host-visible behaviour of the fused all-gather's waiting half: a wait for words nobody sends runs out after the
limit set on the host, the kernel returns, the status call reports the failure once and the object stays usable.
Nothing here faults or hangs: the wait is bounded by design and the limit is set to a few milliseconds."""
import ctypes as C

import numpy as np
import pytest
import torch

from eoq_quantization_b200 import _lib as L

pytestmark = pytest.mark.gpu


def test_wait_for_a_peer_that_never_sends_expires_and_reports():
    lib = L.lib()
    torch.cuda.set_device(0)
    handle = (C.c_ubyte * 64)()
    g = C.c_void_p()
    L.check(lib.eoq_b200_gather_create(2, 0, 2, 2 * 96 * 2, C.byref(g), handle), "eoq_b200_gather_create")
    try:
        assert lib.eoq_b200_gather_set_timeout_ms(g, 0) == L.EOQ_ERR_UNSUPPORTED
        L.check(lib.eoq_b200_gather_set_timeout_ms(g, 5), "eoq_b200_gather_set_timeout_ms")
        assert lib.eoq_b200_gather_status(g, None) == 0
        # rank 1 does not exist: its 32 words of slot 0 never arrive
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        L.check(lib.eoq_b200_gather_wait(g, 0, 96, 1, L.F16, 3, torch.cuda.current_stream().cuda_stream), "eoq_b200_gather_wait")
        t1.record()
        torch.cuda.synchronize()
        assert 1.0 < t0.elapsed_time(t1) < 500.0            # gave up after about the limit, far below the default second
        assert lib.eoq_b200_gather_status(g, None) == L.EOQ_ERR_CUDA
        assert lib.eoq_b200_gather_status(g, None) == 0      # reported once; the context and the object are still usable
        assert lib.eoq_b200_gather_wait(g, 7, 96, 1, L.F16, 3, None) == L.EOQ_ERR_UNSUPPORTED
        assert lib.eoq_b200_gather_wait(g, 0, 1 << 20, 1, L.F16, 3, None) == L.EOQ_ERR_BUFFER_TOO_SMALL
        y = torch.ones(8, device="cuda") * 2                 # ordinary work still runs on the device
        assert float(y.sum()) == 16.0
    finally:
        lib.eoq_b200_gather_destroy(g)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_weight_used_with_another_device_current_is_refused_before_any_launch():
    from eoq_quantization_b200.fused import EOQWeight
    lib = L.lib()
    rng = np.random.default_rng(0)
    sym = rng.integers(0, 15, (96, 128), dtype=np.uint8)
    sc = np.ones(96, np.float16)
    with torch.cuda.device(0):
        w = EOQWeight.from_symbols(sym, sc)
        x0 = torch.zeros(1, 128, device="cuda:0", dtype=torch.float16)
    with torch.cuda.device(1):
        x1 = torch.zeros(1, 128, device="cuda:1", dtype=torch.float16)
        y1 = torch.full((1, 96), 3.0, device="cuda:1", dtype=torch.float16)
        n0 = lib.eoq_b200_launch_count()
        rc = lib.eoq_b200_gemv(w._h, x1.data_ptr(), L.F16, 1, y1.data_ptr(), L.F16, None, None)
        assert rc == L.EOQ_ERR_UNSUPPORTED and lib.eoq_b200_launch_count() == n0
        assert lib.eoq_b200_gemm(w._h, x1.data_ptr(), L.F16, 16, y1.data_ptr(), L.F16, None, None) == L.EOQ_ERR_UNSUPPORTED
        assert lib.eoq_b200_gemv_static_scratch(w._h, x1.data_ptr(), L.F16, 1, y1.data_ptr(), L.F16, None, None) == L.EOQ_ERR_UNSUPPORTED
        assert lib.eoq_b200_launch_count() == n0
        torch.cuda.synchronize()
        assert float(y1.float().min()) == 3.0
        with pytest.raises(RuntimeError):
            w.gemv(x1)                                        # the Python wrapper refuses activations on another device
        assert w.gemv(x0).shape == (1, 96)                    # and makes the weight's device current for its own
