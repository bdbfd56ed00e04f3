"""``eoq_b200_gemv_packed``: the GEMV straight from QuantizedLinear's in-memory form (packed codes + fp16 scales), against
the oracle's dequantise-then-matmul (core/quantized_linear.py:189-228), for every bit width the reference packs."""
import numpy as np
import pytest
import torch

from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.core.quantized_linear import QuantizedLinear
from eoq_quantization_b200.fused import (dequant_packed, gemv_packed, gemv_polar_codes, packed_gemv_applies, packed_gemv_rows,
                                         polar_codes_gemv_applies)
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """Rows of codes as QuantizedLinear.packed_weight holds them (core/quantized_linear.py:49-66)."""
    qmax = (1 << (bits - 1)) - 1
    if bits == 4:
        u = (codes + qmax).astype(np.uint8)
        return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
    if bits == 2:
        u = (codes + qmax).astype(np.uint8)
        return (u[:, 0::4] | (u[:, 1::4] << 2) | (u[:, 2::4] << 4) | (u[:, 3::4] << 6)).astype(np.uint8)
    return codes.astype(np.int8).view(np.uint8)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("n,k,group", [(1, 128, 128), (101, 256, 64), (300, 1536, 128), (1000, 4096, 128), (77, 11008, 128)])
def test_packed_gemv_matches_dequantise_then_matmul(bits, n, k, group):
    rng = np.random.default_rng(bits * 1000 + n + k)
    wt = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    codes, scales = O.quantize_absmax(wt, bits, group)
    s16 = scales.astype(np.float16)
    dense = (codes.reshape(-1, group).astype(np.float64) * s16.astype(np.float64)[:, None]).reshape(n, k)
    packed = torch.from_numpy(_pack(codes, bits)).cuda()
    sc = torch.from_numpy(s16).cuda()
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    assert packed_gemv_applies(k, bits, group)
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        # 32 rows on the tensor-core form (16-bit activations, groups of whole 128-column spans), 8 on the general one
        most = packed_gemv_rows(k, bits, group, dt)
        assert most == (32 if group % 128 == 0 else 8)
        for rows in (1, 2, 3, 4, 7, 8, 9, 16, 17, 32):
            x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda().to(dt)
            if rows > most:
                with pytest.raises(ValueError):
                    gemv_packed(packed, sc, n, k, bits, group, x, bias)
                continue
            y = gemv_packed(packed, sc, n, k, bits, group, x, bias, out_dtype=torch.float32)
            want = x.float().cpu().numpy().astype(np.float64) @ dense.T + bias.cpu().numpy()
            # general form: codes ride in a float of magnitude 2**7 (2**15 for byte codes) whose constant is taken out per
            # eight columns, which leaves about 1e-5 of relative error on a single output; tensor-core form: exact
            # products, fp32 accumulation
            assert O.rel_l2(y.cpu().numpy(), want) < 3e-5, (rows, dt)
            assert torch.equal(y, gemv_packed(packed, sc, n, k, bits, group, x, bias, out_dtype=torch.float32))
            if dt != torch.float32:
                yh = gemv_packed(packed, sc, n, k, bits, group, x)
                assert yh.dtype == dt and yh.shape == (rows, n)
    # a view that starts two bytes into its allocation is realigned, not refused
    x = torch.from_numpy(rng.standard_normal(k + 1).astype(np.float32)).cuda().half()[1:].reshape(1, k)
    y = gemv_packed(packed, sc, n, k, bits, group, x, bias, out_dtype=torch.float32)
    assert O.rel_l2(y.cpu().numpy(), x.float().cpu().numpy().astype(np.float64) @ dense.T + bias.cpu().numpy()) < 3e-5


def test_quantized_linear_forward_takes_the_packed_route_for_few_rows():
    """The module's forward for up to 32 rows of 16-bit activations is the packed GEMV (no entropy-coded copy is built);
    more rows go through dequantise + GEMM; fp32 activations and shapes the kernel does not take go the other routes."""
    rng = np.random.default_rng(0)
    lin = torch.nn.Linear(512, 200, bias=True)
    ql = QuantizedLinear.from_float(lin, bits=4, block_size=128).cuda()
    dense = ql._dequantize_weight().double().cpu().numpy()
    for dt, tol in ((torch.float16, 1e-3), (torch.bfloat16, 6e-3)):
        for rows in (1, 5, 8, 9, 32, 40):
            n0 = L.lib().eoq_b200_launch_count()
            x = torch.from_numpy(rng.standard_normal((rows, 512)).astype(np.float32)).cuda().to(dt)
            y = ql(x)
            want = x.double().cpu().numpy() @ dense.T + ql.bias_param.double().cpu().numpy()
            assert y.dtype == dt and O.rel_l2(y.double().cpu().numpy(), want) < tol, (dt, rows)
            assert L.lib().eoq_b200_launch_count() == n0 + 1                   # one kernel of this library either way
    x = torch.from_numpy(rng.standard_normal((3, 512)).astype(np.float32)).cuda()       # fp32: two fp16 halves per activation
    want = x.double().cpu().numpy() @ dense.T + ql.bias_param.double().cpu().numpy()
    assert O.rel_l2(ql(x).double().cpu().numpy(), want) < 1e-5
    assert ql._eoq is None
    assert not packed_gemv_applies(100, 4, 100) and not packed_gemv_applies(260, 4, 130)
    assert packed_gemv_applies(4096, 4, 128, torch.float16, 32) and packed_gemv_applies(4096, 4, 128, torch.float32, 32)
    assert not packed_gemv_applies(4096, 4, 64, torch.float32, 9)
    odd = QuantizedLinear.from_float(torch.nn.Linear(100, 30, bias=False), bits=4, block_size=100).cuda()
    x = torch.from_numpy(rng.standard_normal((2, 100)).astype(np.float32)).cuda()
    want = x.double().cpu().numpy() @ odd._dequantize_weight().double().cpu().numpy().T
    assert O.rel_l2(odd(x).double().cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("n,k,group", [(37, 256, 128), (64, 200, 80), (5, 4096, 128), (33, 100, 50), (300, 1536, 64)])
def test_dequantised_rows_of_packed_codes_are_the_reference_product(bits, n, k, group):
    """`dequant_packed` (core/quantized_linear.py:189-217: codes.float() * scales.float(), scales indexed over the
    flattened matrix, so groups may straddle rows): bit-exact in fp32, rounded once for 16-bit outputs; the vector
    form (K and group multiples of 8) and the general form, whole matrices and row ranges."""
    rng = np.random.default_rng(bits + n + k)
    qmax = (1 << (bits - 1)) - 1
    codes = rng.integers(-qmax, qmax + 1, size=(n, k)).astype(np.int64)
    s16 = (rng.random(n * k // group).astype(np.float32) * 0.05 + 1e-3).astype(np.float16)
    want = (codes.reshape(-1, group).astype(np.float32) * s16.astype(np.float32)[:, None]).reshape(n, k)
    packed = torch.from_numpy(_pack(codes, bits)).cuda()
    sc = torch.from_numpy(s16).cuda()
    for lo, hi in ((0, n), (n // 3, n - 1)):
        got = dequant_packed(packed, sc, n, k, bits, group, lo, hi)
        assert got.dtype == torch.float32 and np.array_equal(got.cpu().numpy(), want[lo:hi])
        for dt in (torch.float16, torch.bfloat16):
            got = dequant_packed(packed, sc, n, k, bits, group, lo, hi, dtype=dt)
            assert torch.equal(got.cpu(), torch.from_numpy(want[lo:hi]).to(dt))
        got = dequant_packed(packed, None, n, k, bits, group, lo, hi, dtype=torch.int8)
        assert np.array_equal(got.cpu().numpy(), codes[lo:hi].astype(np.int8))


@pytest.mark.parametrize("bits", [3, 4, 5, 8])
@pytest.mark.parametrize("n,k,block", [(1, 64, 64), (37, 256, 16), (300, 1536, 128), (1000, 4096, 64), (77, 11008, 32)])
def test_polar_byte_codes_gemv_matches_the_dequantised_weight(bits, n, k, block):
    """`gemv_polar_codes` against the reference's dequantisation of the same buffers (kernels/polar_engine.py:257-264:
    centroids[codes] / sqrt(block) @ H * norm), fp64 on the host; random codes, norms and centroids."""
    from eoq_quantization_b200.core.polar_quant import hadamard_matrix
    rng = np.random.default_rng(bits * 100 + n + block)
    codes = rng.integers(0, 1 << bits, size=(n, k)).astype(np.int8 if bits < 8 else np.uint8)
    norms = (rng.random(n * k // block).astype(np.float32) * 2 + 0.1).astype(np.float16)
    cent = np.sort(rng.standard_normal(1 << bits)).astype(np.float32)
    H = hadamard_matrix(block).double().numpy()
    vals = cent.astype(np.float64)[codes.astype(np.uint8).astype(np.int64)].reshape(-1, block) / np.sqrt(block)
    dense = ((vals @ H) * norms.astype(np.float64)[:, None]).reshape(n, k)
    cd, nr, ct = torch.from_numpy(codes.view(np.int8)).cuda(), torch.from_numpy(norms).cuda(), torch.from_numpy(cent).cuda()
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    for rows in (1, 2, 3, 4, 5, 8) + ((9, 16, 17, 32) if block >= 64 else ()):
        assert polar_codes_gemv_applies(k, bits, block, rows)
        for dt in (torch.float16, torch.bfloat16, torch.float32):
            x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda().to(dt)
            want = x.float().cpu().numpy().astype(np.float64) @ dense.T + bias.cpu().numpy()
            for tensor_cores in (((True, False, None) if rows <= 8 else (True, None)) if block >= 64 else (False, None)):
                y = gemv_polar_codes(cd, nr, ct, n, k, bits, block, x, bias, tensor_cores=tensor_cores)
                assert y.dtype == torch.float32 and O.rel_l2(y.cpu().numpy(), want) < 1e-5, (rows, dt, tensor_cores)
            assert gemv_polar_codes(cd, nr, ct, n, k, bits, block, x, out_dtype=dt).dtype == dt
    most = 32 if block >= 64 else 8
    assert not polar_codes_gemv_applies(k, bits, block, most + 1) and not polar_codes_gemv_applies(100, bits, 50)
    with pytest.raises(ValueError):
        gemv_polar_codes(cd, nr, ct, n, k, bits, block, torch.zeros(most + 1, k, device="cuda"))
    with pytest.raises(ValueError):
        gemv_polar_codes(cd, nr, ct, n, k, bits, block, torch.zeros(9, k, device="cuda"), tensor_cores=False)
    if block < 64:
        with pytest.raises(ValueError):
            gemv_polar_codes(cd, nr, ct, n, k, bits, block, x, tensor_cores=True)
