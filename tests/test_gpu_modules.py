"""The module-level surface in front of the fused kernels: a model filled from a reference-written ``.eoq`` file
(core/eoq_linear.py:15-54), and ``PolarLinear`` (kernels/polar_engine.py:144-360), each against fixtures the imported
reference produced (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import GOLDEN
from eoq_quantization_b200.core.eoq_linear import EOQLinear, fill_model_from_eoq, load_eoq_to_quantized_model
from eoq_quantization_b200.core.polar_quant import PolarQuantResult, polar_dequantize, polar_quantize
from eoq_quantization_b200.kernels.polar_engine import PolarLinear
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _z(name):
    return np.load(f"{GOLDEN}/{name}.npz", allow_pickle=False)


class _Scale(nn.Module):
    def __init__(self, n):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(n))


class _Mlp(nn.Module):
    def __init__(self):
        super().__init__()
        self.up = nn.Linear(256, 48, bias=False)
        self.down = nn.Linear(384, 32, bias=True)


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.mlp = _Mlp()
        self.norm = _Scale(100)


class _Tiny(nn.Module):
    """The tensor names of tests/golden/sample.eoq: layers.0.mlp.{up,down}.weight, layers.0.norm.weight, embed.weight."""
    def __init__(self):
        super().__init__()
        self.layers = nn.ModuleList([_Block()])
        self.embed = nn.Embedding(10, 30)


def test_model_is_filled_from_a_reference_written_eoq_file():
    z = _z("ref_eoq_file")
    torch.manual_seed(0)
    model = _Tiny()
    down_bias = model.layers[0].mlp.down.bias.detach().clone()
    model, tok, stats = load_eoq_to_quantized_model(f"{GOLDEN}/sample.eoq", model, device="cuda")
    assert tok is None and stats == {"layers_replaced": 2, "tensors_copied": 2, "unmatched": 0}
    up, down = model.layers[0].mlp.up, model.layers[0].mlp.down
    assert isinstance(up, EOQLinear) and isinstance(down, EOQLinear)
    assert (up.out_features, up.in_features) == (48, 256) and up.bias is None
    # parameters the fused kernels do not serve hold the reference's dequantised values
    assert np.allclose(model.layers[0].norm.weight.detach().cpu().numpy(), z["layers.0.norm.weight"], atol=0, rtol=0)
    assert np.allclose(model.embed.weight.detach().cpu().numpy(), z["embed.weight"], atol=0, rtol=0)
    # the replaced layers compute x W^T (+ b) with the reference's decompressed W, at every batch size and dtype
    w_up, w_down = z["layers.0.mlp.up.weight"].astype(np.float64), z["layers.0.mlp.down.weight"].astype(np.float64)
    assert np.array_equal(up._dequantize_weight().cpu().numpy(), z["layers.0.mlp.up.weight"])
    rng = np.random.default_rng(1)
    for rows, dt in ((1, torch.float16), (3, torch.float32), (8, torch.bfloat16), (40, torch.float16), (20, torch.float32)):
        x = torch.from_numpy(rng.standard_normal((rows, 256)).astype(np.float32)).to(dt).cuda()
        y = up(x)
        assert y.dtype == dt and y.shape == (rows, 48)
        want = x.float().cpu().numpy().astype(np.float64) @ w_up.T
        assert O.rel_l2(y.float().cpu().numpy(), want) < (TOL if dt != torch.bfloat16 else 5e-3)
    x = torch.from_numpy(rng.standard_normal((2, 5, 384)).astype(np.float32)).cuda()
    y = down(x)
    want = x.cpu().numpy().astype(np.float64) @ w_down.T + down_bias.numpy().astype(np.float64)
    assert y.shape == (2, 5, 32) and O.rel_l2(y.cpu().numpy(), want) < 1e-5
    assert up.eoq.status() == 0 and down.eoq.status() == 0


def test_fill_model_reports_what_it_could_not_place():
    model = _Tiny()
    model.layers[0].mlp.up = nn.Linear(128, 48, bias=False)       # wrong shape: the record has no home
    stats = fill_model_from_eoq(model, f"{GOLDEN}/sample.eoq", "cuda")
    assert stats["layers_replaced"] == 1 and stats["unmatched"] == 1


def test_polar_linear_matches_the_reference_dequantised_weight():
    z = _z("ref_polar")
    n, k = 16, 256
    codes = torch.from_numpy(z["codes"]).to(torch.int8)
    norms = torch.from_numpy(z["norms"])
    layer = PolarLinear.from_polar_quant(codes, norms, torch.from_numpy(z["centroids5"]), (n, k), bits=5, block_size=64,
                                         bias=torch.linspace(-1, 1, n)).cuda()
    assert layer._fusable()
    dense = z["dequant"].astype(np.float64)                            # the reference's polar_dequantize
    rng = np.random.default_rng(3)
    assert not layer.entropy_coded                                     # the default: straight from the byte codes
    for entropy_coded in (False, True):                                # from the byte codes; from the entropy-coded copy
        layer.entropy_coded = entropy_coded
        for rows in (1, 4, 8, 20, 40):                                 # 40: beyond every kernel, torch operations
            x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda()
            y = layer(x)
            assert y.dtype == torch.float16 and y.shape == (rows, n)
            want = x.cpu().numpy().astype(np.float64) @ dense.T + np.linspace(-1, 1, n)
            assert O.rel_l2(y.float().cpu().numpy(), want) < 2e-3          # fp16 output
        assert (layer._eoq is not None) == entropy_coded
    # a configuration the entropy-coded path is not built for (4 bits, blocks of 128): the byte-code kernel takes it
    lin = nn.Linear(256, 24, bias=False)
    other = PolarLinear.from_linear(lin, bits=4, block_size=128).cuda()
    assert not other._fusable()
    res = polar_quantize(lin.weight.data, 4, 128)
    dense4 = polar_dequantize(PolarQuantResult(res.codes, res.norms, 4, 128, (24, 256), 24 * 256, False)).float().numpy()
    x = torch.from_numpy(rng.standard_normal((2, 256)).astype(np.float32)).cuda()
    assert O.rel_l2(other(x).float().cpu().numpy(), x.cpu().numpy() @ dense4.T) < 2e-3
    assert "vram=" in repr(other) and other.vram_bytes() > 0


@pytest.mark.parametrize("bits", [2, 3, 8])
def test_other_integer_widths_stay_on_the_fused_path(bits):
    """Mixed-bit models (bits_fn of core/rans_bitpacked.py:161-251) quantise some tensors to 2, 3 or 8 bits: their
    symbols are tiled and entropy-coded like the 4-bit ones and run through the same fused decode + GEMV.  Checked
    against the reference's own codes, scales and dequantised matrix (tests/golden/ref_tensor.npz)."""
    from eoq_quantization_b200 import _lib as L
    from eoq_quantization_b200.fused import EOQWeight
    z = _z("ref_tensor")
    key = f"bits{bits}"
    codes = z[key + "/codes"].reshape(24, 256)
    qmax = (1 << (bits - 1)) - 1
    sym = (codes + qmax).astype(np.uint8)
    s16 = np.frombuffer(z[key + "/scales_bytes"].tobytes(), np.float16)
    w = EOQWeight.from_symbols(sym, s16, kind=L.INT_KINDS[bits])
    assert w.info.kind == L.INT_KINDS[bits] and w.info.symbols_per_step == (1 if bits == 8 else 3)
    assert np.array_equal(w.decode_symbols().cpu().numpy(), sym)
    dense = z[key + "/dequant"].reshape(24, 256)
    assert np.array_equal(w.dequantize(torch.float32).cpu().numpy(), dense)          # bit-exact with the reference's dequantize
    rng = np.random.default_rng(bits)
    for rows, dt in ((1, torch.float16), (2, torch.float32), (4, torch.bfloat16), (8, torch.float32)):
        x = torch.from_numpy(rng.standard_normal((rows, 256)).astype(np.float32)).to(dt).cuda()
        y = w.gemv(x, out_dtype=torch.float32)
        want = x.float().cpu().numpy().astype(np.float64) @ dense.astype(np.float64).T
        # narrow codes sit high in the float mantissa (the unpack is one logic instruction), which costs fp32 activations a
        # few bits of headroom: 2e-5 at two bits, far inside the 1e-3 bar
        assert O.rel_l2(y.cpu().numpy(), want) < 1e-4, (rows, dt)
    # a larger matrix with several column segments and row blocks, against the oracle's quantiser
    n, k = 500, 1536
    wt = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    c2, s2 = O.quantize_absmax(wt, bits, 128)
    w2 = EOQWeight.from_symbols((c2 + qmax).astype(np.uint8), s2.astype(np.float16), kind=L.INT_KINDS[bits])
    dense2 = (c2.reshape(-1, 128) * s2.astype(np.float16).astype(np.float32)[:, None]).reshape(n, k)
    x = torch.from_numpy(rng.standard_normal((3, k)).astype(np.float32)).cuda().half()
    y = w2.gemv(x, out_dtype=torch.float32)
    assert O.rel_l2(y.cpu().numpy(), x.float().cpu().numpy().astype(np.float64) @ dense2.astype(np.float64).T) < 1e-4
    assert w2.status() == 0
    # stream bytes only; a 32-row tile of 8-bit codes is short, so its 128 bytes of initial states and the padding to the
    # longest lane weigh more than on the 96-row tiles of the narrow widths
    assert w2.info.bits_per_weight < bits + (0.8 if bits == 8 else 0.3)


def test_quantized_linear_of_other_widths_runs_fused():
    from eoq_quantization_b200.core.quantized_linear import QuantizedLinear
    torch.manual_seed(3)
    lin = nn.Linear(512, 96, bias=True)
    x = torch.randn(2, 512)
    for bits in (2, 3, 8):
        ql = QuantizedLinear.from_float(lin, bits=bits, block_size=128).cuda()
        assert ql._fusable()
        y = ql(x.cuda())
        want = torch.nn.functional.linear(x.cuda(), ql._dequantize_weight(), ql.bias_param)
        assert O.rel_l2(y.cpu().numpy(), want.cpu().numpy()) < 1e-4, bits
        assert ql.eoq_weight().info.symbols_per_step == (1 if bits == 8 else 3)


def test_linear_picks_a_route_by_the_number_of_rows_and_all_routes_agree():
    """EOQWeight.linear: fused GEMV (up to fused_rows of the activation type), decode + library GEMM beyond;
    each against the dense matrix the oracle's dequantiser gives (tolerance: fp16 operands on the tensor-core routes)."""
    from eoq_quantization_b200.fused import GEMM_MAX_ROWS, EOQWeight
    rng = np.random.default_rng(5)
    n, k = 300, 1024
    wt = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    codes, scales = O.quantize_absmax(wt, 4, 128)
    w = EOQWeight.from_symbols((codes + 7).astype(np.uint8), scales.astype(np.float16))
    dense = (codes.reshape(-1, 128) * scales.astype(np.float16).astype(np.float32)[:, None]).reshape(n, k).astype(np.float64)
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    for rows in (1, 4, 5, 8, 9, GEMM_MAX_ROWS, GEMM_MAX_ROWS + 1, 300):
        for dt in (torch.float16, torch.bfloat16, torch.float32):
            x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda().to(dt)
            y = w.linear(x, bias)
            assert y.dtype == dt and y.shape == (rows, n)
            want = x.float().cpu().numpy().astype(np.float64) @ dense.T + bias.cpu().numpy()
            tol = 1e-5 if dt == torch.float32 else 6e-3 if dt == torch.bfloat16 else 2e-3
            assert O.rel_l2(y.float().cpu().numpy(), want) < tol, (rows, dt)
    assert w.status() == 0
