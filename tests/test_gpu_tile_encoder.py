"""The device-side tile encoder (behind ``eoq_b200_weight_from_symbols`` / ``eoq_b200_weight_from_rans``) against the host
encoder (``eoq_b200_tiles_build``), which the oracle's tile decoder checks in tests/test_host_codec.py: stream, tile
descriptors and decode table byte for byte, then the symbols back out of the resident weight."""
import ctypes as C

import numpy as np
import pytest
import torch

from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.core import rans_blocked as RB
from eoq_quantization_b200.fused import EOQWeight
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _read(w, what):
    lib = L.lib()
    n = lib.eoq_b200_weight_read(w._h, what, None, 0)
    buf = np.zeros(n, np.uint8)
    assert lib.eoq_b200_weight_read(w._h, what, buf.ctypes.data, n) == n
    return buf


def _host_tiles(sym, kind, group, target_tiles=0, centroids=None):
    lib = L.lib()
    n, k = sym.shape
    o, keep = EOQWeight._opts(kind, n, k, group, 0, 0, target_tiles, centroids)
    tiles = C.c_void_p()
    L.check(lib.eoq_b200_tiles_build(np.ascontiguousarray(sym).ctypes.data, C.byref(o), C.byref(tiles)), "tiles_build")
    v = L.TilesView()
    L.check(lib.eoq_b200_tiles_view(tiles, C.byref(v)), "tiles_view")
    out = {"stream": np.ctypeslib.as_array(v.stream, (v.stream_bytes,)).copy(),
           "tiles": np.ctypeslib.as_array(v.tiles, (v.num_tiles * 6,)).copy().view(np.uint8),
           "table": np.ctypeslib.as_array(v.table, (1 << v.precision_bits,)).copy().view(np.uint8),
           "head_bytes": v.head_bytes, "num_tiles": v.num_tiles}
    lib.eoq_b200_tiles_free(tiles)
    return out


CASES = [
    # rows, cols, kind, alphabet, group, target_tiles
    (96, 256, L.KIND_INT4_ABSMAX, 15, 128, 0),            # one row block
    (500, 1536, L.KIND_INT4_ABSMAX, 15, 128, 0),          # rows padded to 576: the last lanes repeat real rows
    (1000, 4096, L.KIND_INT4_ABSMAX, 15, 128, 0),
    (4096, 4096, L.KIND_INT4_ABSMAX, 15, 128, 0),
    (2048, 11008, L.KIND_INT4_ABSMAX, 15, 128, 0),        # 96- and 112-column tiles, heads of 2 KB
    (1376, 4096, L.KIND_INT4_ABSMAX, 15, 128, 15 * 128),  # 32-column tiles: heads of 1 KB
    (70, 64, L.KIND_INT4_ABSMAX, 15, 64, 0),              # tiles shorter than a kilobyte: no head region
    (300, 512, L.INT_KINDS[2], 3, 128, 0),
    (300, 512, L.INT_KINDS[3], 7, 128, 0),
    (300, 512, L.INT_KINDS[8], 255, 128, 0),
    (512, 1024, L.KIND_Q5_POLAR, 32, 64, 0),
]


@pytest.mark.parametrize("rows,cols,kind,alphabet,group,target", CASES)
def test_device_built_tiles_equal_host_built_tiles(rows, cols, kind, alphabet, group, target):
    rng = np.random.default_rng(rows * 7 + cols)
    mid = (alphabet - 1) / 2
    sym = np.clip(np.round(rng.normal(mid, max(alphabet / 6, 0.7), (rows, cols))), 0, alphabet - 1).astype(np.uint8)
    scales = (rng.random(rows * cols // group) * 0.01 + 0.001).astype(np.float16)
    cent = np.linspace(-2.5, 2.5, 32).astype(np.float32) if kind == L.KIND_Q5_POLAR else None
    host = _host_tiles(sym, kind, group, target, cent)
    w = EOQWeight.from_symbols(sym, scales, kind=kind, group=group, target_tiles=target, centroids=cent)
    assert w.info.num_tiles == host["num_tiles"]
    assert np.array_equal(_read(w, 2), host["table"])
    assert np.array_equal(_read(w, 1), host["tiles"])
    assert np.array_equal(_read(w, 0), host["stream"])
    assert np.array_equal(w.decode_symbols().cpu().numpy(), sym)
    assert w.status() == 0


def test_from_rans_decodes_and_encodes_on_the_device():
    """Wire format in, resident tiles out, with the symbols never on the host: same tiles as from the symbols directly,
    and the GEMV of the result against the oracle's dequantise-then-matmul."""
    rng = np.random.default_rng(3)
    n, k = 1000, 2048
    wt = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    codes, scales = O.quantize_absmax(wt, 4, 128)
    sym = (codes + 7).astype(np.uint8)
    raw = RB.serialize_blocked_rans(RB.BlockedRANSEncoder(256, 14).encode(sym.reshape(-1), 15))
    w = EOQWeight.from_rans(raw, scales.astype(np.float16), (n, k))
    host = _host_tiles(sym, L.KIND_INT4_ABSMAX, 128)
    assert np.array_equal(_read(w, 0), host["stream"]) and np.array_equal(_read(w, 1), host["tiles"])
    x = torch.from_numpy(rng.standard_normal((2, k)).astype(np.float32)).cuda().half()
    dense = (codes.reshape(-1, 128) * scales.astype(np.float16).astype(np.float32)[:, None]).reshape(n, k).astype(np.float64)
    y = w.gemv(x, out_dtype=torch.float32).cpu().numpy()
    assert O.rel_l2(y, x.float().cpu().numpy().astype(np.float64) @ dense.T) < 1e-3


def test_symbols_and_packed_codes_already_on_the_device():
    """``eoq_b200_weight_from_device_symbols`` (what ``QuantizedLinear`` uses for its packed buffer on the first forward):
    same tiles as the host encoder, also from an address that is not 4-byte aligned."""
    rng = np.random.default_rng(8)
    n, k = 700, 1024
    sym = rng.integers(0, 15, (n, k)).astype(np.uint8)
    scales = (rng.random(n * k // 128) * 0.01 + 0.001).astype(np.float16)
    host = _host_tiles(sym, L.KIND_INT4_ABSMAX, 128)
    d = torch.from_numpy(sym).cuda()
    w = EOQWeight.from_device_symbols(d, scales)
    assert np.array_equal(_read(w, 0), host["stream"]) and np.array_equal(_read(w, 1), host["tiles"])
    odd = torch.zeros(n * k + 8, dtype=torch.uint8, device="cuda")
    odd[1:1 + n * k] = d.reshape(-1)
    w2 = EOQWeight.from_device_symbols(odd[1:1 + n * k].view(n, k), scales)
    assert np.array_equal(_read(w2, 0), host["stream"])
    packed = torch.from_numpy((sym[:, 0::2] | (sym[:, 1::2] << 4)).astype(np.uint8)).cuda()
    w3 = EOQWeight.from_packed(packed, torch.from_numpy(scales).cuda(), k, 4)
    assert np.array_equal(_read(w3, 0), host["stream"])
    assert np.array_equal(w3.decode_symbols().cpu().numpy(), sym)
