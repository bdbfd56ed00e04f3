"""GPU parity of the tensor-core path: fused decode -> fp16 tiles -> tcgen05 MMA, through the C ABI.

Reference behaviour: dequantize, then matmul (core/quantized_linear.py:222-228, core/quantized_matmul.py:91-176).
Two checks per case: against the oracle's fp32 dequantize-then-matmul within rel-L2 1e-3 (operands are rounded
to fp16 on the way into the tensor cores), and against the same product of the fp16-rounded operands computed in
float64, which only fp32 accumulation order separates from the kernel (rel-L2 1e-5).
"""
import numpy as np
import pytest
import torch

from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.fused import EOQWeight
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _case(n, k, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    codes, scales = O.quantize_absmax(w, 4, 128)
    sym = (codes.reshape(n, k) + 7).astype(np.uint8)
    return sym, scales.reshape(n, k // 128).astype(np.float16)


def _refs(sym, s16, x, bias):
    n, k = sym.shape
    sc = np.repeat(s16.astype(np.float32), 128, axis=1)
    w32 = (sym.astype(np.float32) - 7.0) * sc
    ref32 = x.astype(np.float64) @ w32.astype(np.float64).T + bias
    w16 = w32.astype(np.float16).astype(np.float64)
    x16 = x.astype(np.float16).astype(np.float64)
    return ref32, x16 @ w16.T + bias


@pytest.mark.parametrize("n,k", [(96, 128), (100, 512), (200, 1408), (300, 4096), (1000, 2048)])
@pytest.mark.parametrize("m", [1, 16, 33, 128, 200])
def test_tensor_core_gemm_matches_dequant_then_matmul(n, k, m):
    sym, s16 = _case(n, k, 11 * n + k + m)
    w = EOQWeight.from_symbols(sym, s16)
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    ref32, ref16 = _refs(sym, s16, x, bias)
    y = w.gemm(torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda())
    assert y.shape == (m, n) and y.dtype == torch.float32
    assert w.status() == 0
    got = y.cpu().numpy().astype(np.float64)
    assert O.rel_l2(got, ref16) < 1e-5
    assert O.rel_l2(got, ref32) < 1e-3
    for dt in (torch.float16, torch.bfloat16):
        xh = torch.from_numpy(x).cuda().to(dt)
        yh = w.gemm(xh, torch.from_numpy(bias).cuda())
        assert yh.dtype == dt
        _, r16 = _refs(sym, s16, xh.float().cpu().numpy(), bias)
        want = torch.from_numpy(r16).to(dt).double().numpy()
        assert O.rel_l2(yh.double().cpu().numpy(), want) < (2e-3 if dt == torch.bfloat16 else 3e-4)
    # eight warps accumulate into one tensor-memory tile in arrival order, so two runs may differ in the last bits
    y2 = w.gemm(torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda())
    assert O.rel_l2(y2.cpu().numpy(), y.cpu().numpy()) < 1e-6
    # and the GEMV kernel agrees on the rows it can take
    y8 = w.gemv(torch.from_numpy(x[:8]).cuda(), torch.from_numpy(bias).cuda())
    assert O.rel_l2(y[:8].cpu().numpy(), y8.cpu().numpy()) < 1e-3


def test_tensor_core_gemm_rejects_other_layouts():
    sym, s16 = _case(64, 256, 5)
    w = EOQWeight.from_symbols(sym, s16, symbols_per_step=2)
    with pytest.raises(L.EOQError):
        w.gemm(torch.randn(16, 256, device="cuda"))
    with pytest.raises(RuntimeError):
        EOQWeight.from_symbols(sym, s16).gemm(torch.randn(16, 256))


def test_tensor_core_gemm_70b_shape_slice():
    """Llama-70B-shape K (8192) on a slice of rows, bf16 activations, 64 tokens."""
    n, k, m = 1024, 8192, 64
    rng = np.random.default_rng(70)
    wf = (rng.standard_normal((n, k)) * 0.015).astype(np.float32)
    codes, scales = O.quantize_absmax(wf, 4, 128)
    sym = (codes.reshape(n, k) + 7).astype(np.uint8)
    s16 = scales.reshape(n, k // 128).astype(np.float16)
    w = EOQWeight.from_symbols(sym, s16)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    y = w.gemm(x, out_dtype=torch.float32)
    ref32, ref16 = _refs(sym, s16, x.float().cpu().numpy(), np.zeros(n, np.float32))
    assert O.rel_l2(y.double().cpu().numpy(), ref16) < 1e-5
    assert O.rel_l2(y.double().cpu().numpy(), ref32) < 1e-3
    assert w.status() == 0


def test_reference_modules_take_the_tensor_core_path_for_prefill_rows():
    """QuantizedLinear / QuantizedLinearFast (core/quantized_linear.py:222-228, core/quantized_matmul.py:179-260) with
    9..128 rows of 16-bit activations agree with dequantize-then-matmul."""
    from eoq_quantization_b200.core.quantized_linear import QuantizedLinear
    from eoq_quantization_b200.core.quantized_matmul import QuantizedLinearFast
    torch.manual_seed(3)
    lin = torch.nn.Linear(512, 300, bias=True)
    ql = QuantizedLinear.from_float(lin).cuda()
    fast = QuantizedLinearFast.from_quantized_linear(ql)
    launches = L.lib().eoq_b200_launch_count()
    for rows, dt in ((33, torch.float16), (128, torch.bfloat16), (2 * 40, torch.float16)):
        x = torch.randn(rows, 512, device="cuda", dtype=dt)
        want = torch.nn.functional.linear(x.float(), ql._dequantize_weight().float(), ql.bias_param.float())
        for mod in (ql, fast):
            y = mod(x)
            assert y.dtype == dt and y.shape == (rows, 300)
            assert O.rel_l2(y.float().cpu().numpy(), want.to(dt).float().cpu().numpy()) < (4e-3 if dt == torch.bfloat16 else 1e-3)
    assert L.lib().eoq_b200_launch_count() > launches
    y3 = ql(torch.randn(2, 20, 512, device="cuda", dtype=torch.float16))       # 40 rows through a 3-D input
    assert y3.shape == (2, 20, 300)
