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
    for rows in (1, 4, 8, 20):
        x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda()
        y = layer(x)
        assert y.dtype == torch.float16 and y.shape == (rows, n)
        want = x.cpu().numpy().astype(np.float64) @ dense.T + np.linspace(-1, 1, n)
        assert O.rel_l2(y.float().cpu().numpy(), want) < 2e-3          # fp16 output
    # a configuration outside the fused path (4 bits, blocks of 128) still answers, through torch on the device
    lin = nn.Linear(256, 24, bias=False)
    other = PolarLinear.from_linear(lin, bits=4, block_size=128).cuda()
    assert not other._fusable()
    res = polar_quantize(lin.weight.data, 4, 128)
    dense4 = polar_dequantize(PolarQuantResult(res.codes, res.norms, 4, 128, (24, 256), 24 * 256, False)).float().numpy()
    x = torch.from_numpy(rng.standard_normal((2, 256)).astype(np.float32)).cuda()
    assert O.rel_l2(other(x).float().cpu().numpy(), x.cpu().numpy() @ dense4.T) < 2e-3
    assert "vram=" in repr(other) and other.vram_bytes() > 0
