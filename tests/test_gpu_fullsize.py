"""The benchmark configurations at full size, checked against what the imported reference made of the same seeded
inputs (tests/golden/ref_fullsize.npz, written by tests/golden/make_golden.py; tests/golden/recipes.py regenerates
the inputs).  Hashes pin the quantised inputs to the reference's quantisers bit for bit; outputs are compared with
the reference's dequantise-then-linear results: decoded symbols and dequantised matrices bit-exact, products within
rel-L2 <= 1e-3 (fp32 accumulation; outputs rounded to fp16 where stated)."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.core import rans_bitpacked as RBP
from eoq_quantization_b200.core import rans_blocked as RB
from eoq_quantization_b200.core.polar_quant import _ensure_centroids, polar_dequantize, polar_quantize
from eoq_quantization_b200.fused import EOQWeight
from oracle import oracle as O

sys.path.insert(0, GOLDEN)
import recipes as RC  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.fixture(scope="module")
def ref():
    return np.load(os.path.join(GOLDEN, "ref_fullsize.npz"), allow_pickle=False)


def _int4(name, ref):
    """Seeded weight -> (codes int8 [n, k], scales fp16 [n*k/128]) through the oracle's quantiser, proven equal to the
    reference's output on the same weight by hash."""
    n, k, seed, sigma = RC.INT4_SHAPES[name]
    codes, scales = O.quantize_absmax(RC.weight(n, k, seed, sigma).numpy(), 4, 128)
    codes = codes.reshape(n, k).astype(np.int8)
    s16 = scales.astype(np.float16)
    assert RC.sha(codes) == str(ref[name + "/sha_codes"]), "quantised codes differ from the reference's"
    assert RC.sha(s16) == str(ref[name + "/sha_scales16"]), "scales differ from the reference's"
    return n, k, seed, codes, s16


def test_config1_wire_format_at_full_size(ref):
    """4096 x 4096, blocks of 4096 symbols, 12-bit table, through the reference-facing entry points."""
    name = "square_4096x4096"
    n, k, seed, codes, s16 = _int4(name, ref)
    sym = (codes.astype(np.int64) + 7).ravel()
    data = RB.BlockedRANSEncoder(block_size=4096, precision_bits=12).encode(sym, 15)
    ser = RB.serialize_blocked_rans(data)
    assert len(ser) == int(ref[name + "/rans_len"])
    assert RC.sha(np.frombuffer(ser, np.uint8)) == str(ref[name + "/sha_rans"]), "container differs from the reference encoder's"
    # BlockedRANSDecoder.decode_all: every block on the GPU, symbols bit-exact
    got = RB.BlockedRANSDecoder().decode_all(RB.deserialize_blocked_rans(ser))
    assert got.dtype == np.int64 and np.array_equal(got, sym)
    assert np.array_equal(RB.decode_quantized_tensor(RB.deserialize_blocked_rans(ser), 4), codes.ravel().astype(np.int64))
    # the dequantised fp16 matrix from the same container, bit-exact with the reference's dequantize()
    w = EOQWeight.from_rans(ser, s16, (n, k))
    assert torch.equal(w.decode_symbols().cpu(), torch.from_numpy((codes + 7).astype(np.uint8)))
    assert RC.sha(w.dequantize(torch.float16)) == str(ref[name + "/sha_dequant16"])
    # eoq_parallel_decode over 64-row tasks (C payloads, byte symbols)
    lib = L.lib()
    rows_per_task = 64
    ntasks = n // rows_per_task
    tasks = (L.DecodeTask * ntasks)()
    keep = []
    for i in range(ntasks):
        chunk = sym[i * rows_per_task * k:(i + 1) * rows_per_task * k]
        hdr, payload = O.make_c_payload(O.encode_blocked(chunk, 15, 4096, 12))
        h = L.TensorHeader(*[int(v) for v in hdr])
        buf = (C.c_ubyte * len(payload)).from_buffer_copy(payload)
        out = np.full(chunk.size, 255, np.uint8)
        keep.append((h, buf, out))
        tasks[i].header = C.pointer(h)
        tasks[i].compressed_data = C.cast(buf, C.c_void_p)
        tasks[i].compressed_size = len(payload)
        tasks[i].output = out.ctypes.data
        tasks[i].output_capacity = out.size
    assert lib.eoq_parallel_decode(tasks, ntasks, None) == 0
    for i, (_, _, out) in enumerate(keep):
        assert tasks[i].result == 0
        assert np.array_equal(out, sym[i * rows_per_task * k:(i + 1) * rows_per_task * k].astype(np.uint8)), i


def test_config1_tensor_bridge_reads_the_reference_bytes(ref):
    """decompress_tensor_rans on bytes the reference's compress_tensor_rans wrote (block 256, 14-bit table)."""
    name = "square_4096x4096"
    n, k, seed, codes, s16 = _int4(name, ref)
    rows = RC.BRIDGE_ROWS
    rans, scales = ref[name + "/bridge_rans"].tobytes(), ref[name + "/bridge_scales"].tobytes()
    ct = RBP.CompressedTensorData(name="w", shape=(rows, k), bits=4, block_size=128, scales_bytes=scales, rans_bytes=rans,
                                  n_elements=rows * k, original_size=rows * k * 2, compressed_size=len(rans) + len(scales))
    got_codes, got_scales = RBP.decompress_tensor_rans(ct)
    assert got_codes.dtype == torch.int8 and got_scales.dtype == torch.float32
    assert np.array_equal(got_codes.cpu().numpy().ravel(), codes[:rows].ravel())
    assert np.array_equal(got_scales.cpu().numpy(), s16[: rows * k // 128].astype(np.float32))


@pytest.mark.parametrize("name", ["up_11008x4096", "down_4096x11008"])
def test_config2_fused_gemv_against_the_reference_outputs(ref, name):
    n, k, seed, codes, s16 = _int4(name, ref)
    w = EOQWeight.from_symbols((codes + 7).astype(np.uint8), s16)
    assert torch.equal(w.decode_symbols().cpu(), torch.from_numpy((codes + 7).astype(np.uint8)))
    for batch in (1, 4):
        x = RC.activations(batch, k, seed * 10 + batch).cuda()
        y = w.gemv(x)
        assert y.dtype == torch.float16 and y.shape == (batch, n)
        got = y.float().cpu().numpy()
        assert O.rel_l2(got, ref[f"{name}/y_fp32_b{batch}"]) < TOL            # fp32 accumulation, fp16 output
        assert O.rel_l2(got, ref[f"{name}/y_fp16_b{batch}"]) < 2e-3           # the reference's own fp16 composition
        y32 = w.gemv(x, out_dtype=torch.float32).cpu().numpy()
        assert O.rel_l2(y32, ref[f"{name}/y_fp32_b{batch}"]) < 1e-5
        assert torch.equal(w.gemv(x), y)
    assert w.status() == 0


def test_config3_polar_q5_against_the_reference_slice(ref):
    name, n, k, seed, sigma = RC.POLAR_SHAPE
    wt = RC.polar_weight(n, k, seed, sigma)
    rows = RC.SLICE_ROWS
    # first rows on the host, where the quantiser's arithmetic is the reference's bit for bit
    head = polar_quantize(wt[:rows], bits=5, block_size=64, use_qjl=False)
    assert RC.sha(head.codes) == str(ref[name + "/sha_codes_slice"])
    assert RC.sha(head.norms) == str(ref[name + "/sha_norms_slice"])
    # the whole matrix on the GPU (the same operations in another summation order: a value that sits on a decision
    # boundary may fall the other way, nothing else)
    full = polar_quantize(wt.cuda(), bits=5, block_size=64, use_qjl=False, chunk_blocks=1 << 14)
    codes = full.codes.view(n, k).clone()
    differ = (codes[:rows].cpu() != head.codes.view(rows, k)).float().mean().item()
    assert differ < 1e-4
    codes[:rows] = head.codes.view(rows, k).cuda()
    norms = full.norms.clone()
    norms[: rows * k // 64] = head.norms.cuda()
    cent = _ensure_centroids(5)
    w = EOQWeight.from_symbols(codes.to(torch.uint8), norms, kind=L.KIND_Q5_POLAR, group=64, centroids=cent.tolist())
    assert torch.equal(w.decode_symbols(), codes.to(torch.uint8))
    res = type(full)(codes=codes.flatten(), norms=norms, bits=5, block_size=64, shape=(n, k), n_elements=n * k, use_qjl=False)
    dense = torch.cat([polar_dequantize(type(full)(codes=codes[lo:lo + 1024].flatten(), norms=norms[lo * k // 64:(lo + 1024) * k // 64],
                                                  bits=5, block_size=64, shape=(min(1024, n - lo), k),
                                                  n_elements=min(1024, n - lo) * k, use_qjl=False)).float()
                       for lo in range(0, n, 1024)])
    del res
    for batch in (1, 4, 8):
        x = RC.activations(batch, k, seed * 10 + batch).cuda()
        y = w.gemv(x, out_dtype=torch.float32)
        assert O.rel_l2(y[:, :rows].cpu().numpy(), ref[f"{name}/y_slice_b{batch}"]) < TOL      # the reference's rows
        assert O.rel_l2(y.cpu().numpy(), (x.float() @ dense.T).cpu().numpy()) < TOL            # every row, same device
    assert w.status() == 0


@pytest.mark.parametrize("name", ["gate_shard_3584x8192", "down_shard_1024x28672"])
def test_config5_prefill_shapes_against_the_reference_outputs(ref, name):
    n, k, seed, codes, s16 = _int4(name, ref)
    w = EOQWeight.from_symbols((codes + 7).astype(np.uint8), s16)
    stride = int(ref[name + "/stride"])
    for m in (16, 64, 256, 2048):
        x = RC.activations(m, k, seed * 10 + m, torch.bfloat16).cuda()
        y = w.gemm(x, out_dtype=torch.float32)
        assert y.shape == (m, n)
        assert O.rel_l2(y[:, ::stride].cpu().numpy(), ref[f"{name}/y_m{m}"]) < TOL, m
    assert w.status() == 0
