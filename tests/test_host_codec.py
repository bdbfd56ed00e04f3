"""CPU-side checks of the product library: it loads, exports every declared symbol,
validates arguments like the reference, and its host encoders reproduce the reference's
bytes.  No compute call needs a GPU here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import GOLDEN, ROOT
from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.core import rans as PR
from eoq_quantization_b200.core import rans_blocked as RB
from oracle import oracle as O


def _z(name):
    return np.load(f"{GOLDEN}/{name}.npz", allow_pickle=False)


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    hdr = open(os.path.join(ROOT, "include", "eoq_b200.h")).read()
    declared = set(re.findall(r"\b(eoq_(?:b200_|cuda_)?[a-z0-9_]+)\s*\(", hdr))
    declared -= {"eoq_progress_fn", "eoq_parallel_progress_fn"}
    declared -= {"eoq_parallel_decode_auto"}        # a static inline wrapper in the header, as in the reference's header
    assert declared == set(L.EXPORTS), declared ^ set(L.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_error_strings_and_header_validation():
    lib = L.lib()
    assert lib.eoq_error_string(0) == b"success"
    assert lib.eoq_error_string(-3) == b"corrupt compressed stream"
    assert lib.eoq_error_string(-99) == b"unknown error"
    assert lib.eoq_validate_header(None) == L.EOQ_ERR_NULL_PTR
    good = L.TensorHeader(0, 4, 15, 12, 256, 15 * 2 + 16 + 100, 1000)
    assert lib.eoq_validate_header(C.byref(good)) == 0
    for field, value in (("freq_table_size", 0), ("freq_table_size", 4097), ("precision_bits", 0),
                         ("precision_bits", 17), ("rans_block_size", 0), ("compressed_size", 10)):
        h = L.TensorHeader(0, 4, 15, 12, 256, 146, 1000)
        setattr(h, field, value)
        assert lib.eoq_validate_header(C.byref(h)) == L.EOQ_ERR_INVALID_HEADER, field
    assert lib.eoq_detect_num_threads() >= 1


def _payload(n=1000, a=15, p=12, bs=256, seed=0):
    sym = np.random.default_rng(seed).integers(0, a, n)
    hdr, body = O.make_c_payload(O.encode_blocked(sym, a, bs, p))
    return sym, L.TensorHeader(*[int(v) for v in hdr]), np.frombuffer(body, np.uint8).copy()


def test_decode_tensor_v2_argument_checks_match_reference_order():
    lib = L.lib()
    sym, h, body = _payload()
    out = np.zeros(1000, np.uint8)
    f = lib.eoq_decode_tensor_v2
    assert f(None, body.ctypes.data, body.size, out.ctypes.data, out.size, None) == L.EOQ_ERR_NULL_PTR
    assert f(C.byref(h), None, body.size, out.ctypes.data, out.size, None) == L.EOQ_ERR_NULL_PTR
    assert f(C.byref(h), body.ctypes.data, body.size, None, out.size, None) == L.EOQ_ERR_NULL_PTR
    z = L.TensorHeader(0, 0, 0, 0, 0, 0, 0)                      # zero length wins over a bad header
    assert f(C.byref(z), body.ctypes.data, body.size, out.ctypes.data, out.size, None) == 0
    assert f(C.byref(h), body.ctypes.data, body.size, out.ctypes.data, 10, None) == L.EOQ_ERR_BUFFER_TOO_SMALL
    assert f(C.byref(h), body.ctypes.data, body.size - 1, out.ctypes.data, out.size, None) == L.EOQ_ERR_CORRUPT_STREAM
    bad = L.TensorHeader(0, 4, 15, 17, 256, h.compressed_size, 1000)
    assert f(C.byref(bad), body.ctypes.data, body.size, out.ctypes.data, out.size, None) == L.EOQ_ERR_INVALID_HEADER
    # corrupt offset table: second block starts past the end of the stream
    broken = body.copy()
    broken[15 * 2 + 4:15 * 2 + 8] = np.frombuffer(np.uint32(10 ** 6).tobytes(), np.uint8)
    assert f(C.byref(h), broken.ctypes.data, broken.size, out.ctypes.data, out.size, None) == L.EOQ_ERR_CORRUPT_STREAM
    # state length byte larger than the block
    broken = body.copy()
    broken[15 * 2 + 16] = 250
    rc = f(C.byref(h), broken.ctypes.data, broken.size, out.ctypes.data, out.size, None)
    assert rc in (L.EOQ_ERR_CORRUPT_STREAM,)


def test_parallel_decode_host_semantics_without_device():
    lib = L.lib()
    assert lib.eoq_parallel_decode(None, 0, None) == 0
    assert lib.eoq_parallel_decode(None, 3, None) == L.EOQ_ERR_NULL_PTR
    assert lib.eoq_parallel_decode(None, -1, None) == 0
    sym, h, body = _payload()
    out = np.zeros(1000, np.uint8)
    tasks = (L.DecodeTask * 3)()
    for t in tasks:
        t.header, t.compressed_data, t.compressed_size = C.pointer(h), body.ctypes.data, body.size
        t.output, t.output_capacity = out.ctypes.data, out.size
    tasks[1].output_capacity = 5
    rc = lib.eoq_parallel_decode(tasks, 3, None)
    assert tasks[1].result == L.EOQ_ERR_BUFFER_TOO_SMALL
    assert [t.task_index for t in tasks] == [0, 1, 2]
    import torch
    if not torch.cuda.is_available():
        assert tasks[0].result == L.EOQ_ERR_CUDA and rc == L.EOQ_ERR_CUDA   # first error in task order; no CPU fallback


def test_host_encoder_reproduces_reference_bytes():
    z = _z("ref_blocked")
    for name in z["names"]:
        a, bs, p = (int(v) for v in z[f"{name}/params"])
        data = RB.BlockedRANSEncoder(block_size=bs, precision_bits=p).encode(z[f"{name}/symbols"], a)
        assert RB.serialize_blocked_rans(data) == z[f"{name}/rans"].tobytes(), name
        back = RB.deserialize_blocked_rans(z[f"{name}/rans"].tobytes())
        assert back.block_offsets == data.block_offsets and back.num_blocks == data.num_blocks
        assert np.array_equal(back.freq_table, data.freq_table)
    x = _z("xval_vectors")
    for name in x["names"]:
        n, a, p, _ = (int(v) for v in x[f"{name}/meta"])
        assert PR.RANSEncoder(x[f"{name}/freq"], precision_bits=p).encode(x[f"{name}/expected"]) == x[f"{name}/comp"].tobytes(), name


def test_python_normaliser_matches_reference():
    z = _z("ref_normalise")
    for i in range(int(z["count"])):
        f, c = PR._normalize_frequencies(z[f"{i}/raw"], int(z[f"{i}/p"]))
        assert np.array_equal(f, z[f"{i}/freq"]) and np.array_equal(c, z[f"{i}/cdf"]), i


def test_container_and_index_errors():
    z = _z("ref_blocked")
    raw = z["exact_block/rans"].tobytes()
    with pytest.raises(ValueError):
        RB.deserialize_blocked_rans(b"NOPE" + raw[4:])
    with pytest.raises(ValueError):
        RB.deserialize_blocked_rans(raw[:4] + b"\x07\x00\x00\x00" + raw[8:])
    d = RB.deserialize_blocked_rans(raw)
    with pytest.raises(IndexError):
        RB.BlockedRANSDecoder().decode_block(d, d.num_blocks)
    with pytest.raises(IndexError):
        RB.BlockedRANSDecoder().decode_block(d, -1)
    with pytest.raises(ValueError):
        PR.compute_frequency_table(np.array([0, 16]), 16)
    with pytest.raises(ValueError):
        PR.RANSEncoder(np.ones(4), precision_bits=21)
    assert d.total_size_bytes() == len(d.compressed_blocks) + d.num_blocks * 4 + d.alphabet_size * 4 + 32
    assert RB.BlockedRANSDecoder().decode_all(RB.BlockedRANSEncoder().encode(np.empty(0, np.int64), 15)).size == 0


def _tiles(sym, kind, group, g=0, p=0, target=0):
    lib = L.lib()
    cent = (C.c_float * 32)(*np.linspace(-2, 2, 32))
    o = L.WeightOpts(kind, sym.shape[0], sym.shape[1], group, g, p, target, cent)
    h = C.c_void_p()
    s = np.ascontiguousarray(sym, np.uint8)
    rc = lib.eoq_b200_tiles_build(s.ctypes.data, C.byref(o), C.byref(h))
    if rc != 0:
        return rc, None
    v = L.TilesView()
    assert lib.eoq_b200_tiles_view(h, C.byref(v)) == 0
    got = dict(table=np.ctypeslib.as_array(v.table, (1 << v.precision_bits,)).copy(),
               desc=np.ctypeslib.as_array(v.tiles, (v.num_tiles * 6,)).copy(),
               stream=np.ctypeslib.as_array(v.stream, (v.stream_bytes,)).copy(),
               G=v.symbols_per_step, p=v.precision_bits, bits=v.bits, nseg=v.num_col_segments, ntiles=v.num_tiles,
               npad=v.padded_rows, head=v.head_bytes)
    lib.eoq_b200_tiles_free(h)
    return 0, got


def test_default_int4_layout_keeps_tiles_short_enough_to_stage_two_per_warp():
    """The fused GEMV stages two whole tiles per warp in shared memory, which holds tiles of up to 7 x 16 columns:
    the default layout of an INT4 weight (three symbols per step) must respect that for wide matrices too, and still
    decode back to the symbols it was built from."""
    rng = np.random.default_rng(5)
    n = 4608
    codes, _ = O.quantize_absmax((rng.standard_normal((n, 4096)) * 0.02).astype(np.float32), 4, 128)
    sym = (codes + 7).astype(np.uint8)
    rc, t = _tiles(sym, L.KIND_INT4_ABSMAX, 128)
    assert rc == 0 and t["G"] == 3
    desc = t["desc"].reshape(-1, 6)
    assert desc[:, 2].max() <= 112 and desc[:, 2].min() >= 64 and (desc[:, 2] % 16 == 0).all()
    assert (desc[:, 5].astype(np.int64) * 64).max() + 64 <= 8192          # eight one-kilobyte chunks per tile
    assert np.array_equal(O.decode_tiles(t["table"], t["p"], t["G"], t["bits"], t["desc"], t["stream"], n, 4096, t["head"]), sym)
    # every tile of this layout is longer than two kilobytes, so two kilobytes of each sit at the fixed stride
    assert t["head"] == 2048 and (desc[:, 4].astype(np.int64) * 64 >= t["ntiles"] * 2048).all()
    # a matrix so small that tile pairs of 32 columns still fit one wave of warps gets those (one kilobyte at the stride)
    rc, t = _tiles(sym[:1152], L.KIND_INT4_ABSMAX, 128)
    desc = t["desc"].reshape(-1, 6)
    assert rc == 0 and (desc[:, 2] == 32).all() and t["head"] == 1024 and t["ntiles"] == 12 * 128
    assert np.array_equal(O.decode_tiles(t["table"], t["p"], t["G"], t["bits"], t["desc"], t["stream"], 1152, 4096, t["head"]), sym[:1152])


@pytest.mark.parametrize("n,k,g", [(24, 256, 3), (100, 512, 2), (33, 128, 1), (97, 384, 3), (1, 128, 3), (96, 128, 3)])
def test_tile_encoder_round_trips_through_oracle(n, k, g):
    rng = np.random.default_rng(n * 1000 + k)
    codes, _ = O.quantize_absmax((rng.standard_normal((n, k)) * 0.02).astype(np.float32), 4, 128)
    sym = (codes + 7).astype(np.uint8)
    rc, t = _tiles(sym, L.KIND_INT4_ABSMAX, 128, g)
    assert rc == 0 and t["G"] == g
    assert t["npad"] % (32 * g) == 0 and t["ntiles"] == t["nseg"] * (t["npad"] // (32 * g))
    desc = t["desc"].reshape(-1, 6)
    assert (desc[:, 2] % 16 == 0).all() and desc[:, 2].min() > 0
    out = O.decode_tiles(t["table"], t["p"], t["G"], t["bits"], t["desc"], t["stream"], n, k, t["head"])
    assert np.array_equal(out, sym)
    # table: every entry has 1 <= freq <= 511 and bias < freq
    e = t["table"]
    freq, bias = e >> 23, e & ((1 << (23 - g * 4)) - 1)
    assert freq.min() >= 1 and freq.max() <= 511 and (bias < freq).all()


def test_tile_encoder_degenerate_distributions_and_q5():
    rc, t = _tiles(np.full((40, 128), 7, np.uint8), L.KIND_INT4_ABSMAX, 128, 2)      # one symbol only: freq capped at 511
    assert rc == 0
    assert (O.decode_tiles(t["table"], t["p"], t["G"], t["bits"], t["desc"], t["stream"], 40, 128, t["head"]) == 7).all()
    sym = np.clip(np.random.default_rng(3).normal(16, 5, (64, 256)), 0, 31).astype(np.uint8)
    rc, t = _tiles(sym, L.KIND_Q5_POLAR, 64)
    assert rc == 0 and t["bits"] == 5 and t["G"] == 2
    assert np.array_equal(O.decode_tiles(t["table"], t["p"], t["G"], t["bits"], t["desc"], t["stream"], 64, 256, t["head"]), sym)


def test_tile_builder_rejects_what_it_cannot_tile():
    sym = np.zeros((8, 100), np.uint8)
    assert _tiles(sym, L.KIND_INT4_ABSMAX, 128)[0] == L.EOQ_ERR_UNSUPPORTED          # K not a multiple of 16
    assert _tiles(np.zeros((8, 128), np.uint8), 7, 128)[0] == L.EOQ_ERR_UNSUPPORTED  # unknown kind
    assert _tiles(np.zeros((8, 128), np.uint8), L.KIND_INT4_ABSMAX, 128, 3, 15)[0] == L.EOQ_ERR_UNSUPPORTED


def test_bitpacked_bridge_bytes_match_reference():
    import torch
    from eoq_quantization_b200.core import rans_bitpacked as RBP
    from eoq_quantization_b200.core import utils as U
    z = _z("ref_tensor")
    for k in z["names"]:
        bits = int(str(k)[4:])
        w = torch.from_numpy(z[f"{k}/w"])
        qt = U.quantize_absmax(w, bits, 128)
        assert np.array_equal(qt.data.numpy(), z[f"{k}/codes"])
        ct = RBP.compress_tensor_rans(str(k), qt.data, qt.scale, bits, 128, tuple(w.shape))
        assert ct.rans_bytes == z[f"{k}/rans"].tobytes(), k
        assert ct.scales_bytes == z[f"{k}/scales_bytes"].tobytes(), k
        assert ct.original_size == w.numel() * 2 and ct.compressed_size == len(ct.rans_bytes) + len(ct.scales_bytes)
    s = RBP.estimate_savings({"a": ct})
    assert s["total_compression_ratio"] > 1.0


def test_quantized_linear_host_packing_matches_reference():
    import torch
    from eoq_quantization_b200.core.quantized_linear import QuantizedLinear, replace_linear_with_quantized, get_model_memory
    z = _z("ref_linear")
    for name in z["names"]:
        w = torch.from_numpy(z[f"{name}/weight"])
        lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=f"{name}/bias" in z)
        with torch.no_grad():
            lin.weight.copy_(w)
            if lin.bias is not None:
                lin.bias.copy_(torch.from_numpy(z[f"{name}/bias"]))
        ql = QuantizedLinear.from_float(lin, bits=4, block_size=128)
        assert np.array_equal(ql.packed_weight.numpy(), z[f"{name}/packed"]), name
        assert np.array_equal(ql.scales.numpy(), z[f"{name}/scales"]), name
        with pytest.raises(RuntimeError):
            ql(torch.from_numpy(z[f"{name}/x"]))          # CPU tensors: no CPU path, fail loudly
    codes = torch.randint(-7, 8, (37,))
    assert torch.equal(QuantizedLinear.unpack_4bit(QuantizedLinear.pack_4bit(codes), 37), codes.to(torch.int8))
    codes = torch.randint(-1, 2, (41,))
    assert torch.equal(QuantizedLinear.unpack_2bit(QuantizedLinear.pack_2bit(codes), 41), codes.to(torch.int8))
    m = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4), torch.nn.Linear(8, 8))
    assert replace_linear_with_quantized(m, min_size=100) == 2
    mem = get_model_memory(m)
    assert mem["quantized_layers"] == 2 and mem["regular_layers"] == 1 and mem["compression_ratio"] > 1


def test_eoq_container_reader_parses_reference_file(tmp_path):
    from eoq_quantization_b200 import eoq_file as EF
    path = f"{GOLDEN}/sample.eoq"
    header, recs = EF.read_eoq(path)
    assert header["config"] == {"bits": 4, "block_size": 128, "rans_block_size": 256, "precision_bits": 14}
    assert [r.name for r in recs] == ["layers.0.mlp.up.weight", "layers.0.mlp.down.weight", "layers.0.norm.weight", "embed.weight"]
    assert recs[0].shape == (48, 256) and recs[0].bits == 4 and recs[0].quant_block_size == 128
    assert len(recs[0].scales) == 48 * 256 // 128 * 2 and recs[0].rans_data[:4] == b"RANS"
    assert [EF.fusable(r) for r in recs] == [True, True, False, False]
    # the symbols inside decode (with the oracle) to what the reference's own loader reconstructs
    z = _z("ref_eoq_file")
    for r in recs:
        d = O.deserialize_rans_v1(r.rans_data)
        codes = O.decode_blocked(d) - 7
        sc = np.frombuffer(r.scales, np.float16).astype(np.float32)
        assert np.array_equal(O.dequantize(codes.reshape(r.shape), sc, 128), z[r.name]), r.name
    raw = bytearray(open(path, "rb").read())
    raw[40] ^= 0xFF
    bad = tmp_path / "bad.eoq"
    bad.write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="Checksum"):
        EF.read_eoq(bad)
    import struct, zlib
    body = b"NOPE" + bytes(raw[4:-4])
    bad.write_bytes(body + struct.pack("<I", zlib.crc32(body) & 0xFFFFFFFF))
    with pytest.raises(ValueError, match="magic"):
        EF.read_eoq(bad)


def test_polar_quantize_on_the_host_is_the_reference_bit_for_bit():
    """core/polar_quant.py:141-264: codes, fp16 norms, centroids, the Hadamard matrix and the dequantised matrix
    equal what the imported reference produced from the same weight."""
    import torch
    from eoq_quantization_b200.core import polar_quant as PQ
    z = _z("ref_polar")
    r = PQ.polar_quantize(torch.from_numpy(z["w"]), bits=5, block_size=64, use_qjl=False)
    assert r.codes.dtype == torch.int8 and r.norms.dtype == torch.float16 and r.shape == (16, 256) and r.n_elements == 4096
    assert np.array_equal(r.codes.numpy(), z["codes"]) and np.array_equal(r.norms.numpy(), z["norms"])
    assert np.array_equal(PQ._ensure_centroids(5).numpy(), z["centroids5"])
    assert np.array_equal(PQ.hadamard_matrix(64).numpy(), z["hadamard64"])
    deq = PQ.polar_dequantize(r)
    assert deq.dtype == torch.float16 and np.array_equal(deq.float().numpy(), z["dequant"])
    # chunking the nearest-centroid search does not change a single code
    r2 = PQ.polar_quantize(torch.from_numpy(z["w"]), bits=5, block_size=64, use_qjl=False, chunk_blocks=7)
    assert torch.equal(r2.codes, r.codes)
    with pytest.raises(ValueError):
        PQ.hadamard_matrix(48)
