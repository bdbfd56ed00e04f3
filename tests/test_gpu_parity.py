"""GPU parity tests: every result of the CUDA path is compared with the CPU oracle or the
committed golden fixtures, through the C ABI.  Integer work is bit-exact; GEMV outputs are
within rel-L2 <= 1e-3 of dequantise-then-matmul (fp32 accumulation, output in x.dtype)."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from eoq_quantization_b200 import _lib as L
from eoq_quantization_b200.core import rans as PR
from eoq_quantization_b200.core import rans_blocked as RB
from eoq_quantization_b200.fused import EOQWeight
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _z(name):
    return np.load(f"{GOLDEN}/{name}.npz", allow_pickle=False)


def _payload(sym, a, p, bs):
    hdr, body = O.make_c_payload(O.encode_blocked(sym, a, bs, p))
    return L.TensorHeader(*[int(v) for v in hdr]), np.frombuffer(body, np.uint8).copy()


# ---------------------------------------------------------------- wire-format decode
def test_known_answer_vectors_decode_bit_exact():
    x = _z("xval_vectors")
    for name in x["names"]:
        n, a, p, _ = (int(v) for v in x[f"{name}/meta"])
        got = PR.RANSDecoder(x[f"{name}/freq"], precision_bits=p).decode(x[f"{name}/comp"].tobytes(), n)
        assert np.array_equal(got, x[f"{name}/expected"]), name


@pytest.mark.parametrize("n", [1, 2, 3, 127, 255, 256, 257, 1000, 4097, 70000])
def test_decode_tensor_v2_matches_oracle(n):
    lib = L.lib()
    rng = np.random.default_rng(n)
    for a, p, bs in ((15, 12, 4096), (256, 16, 256), (31, 14, 256), (2, 8, 64)):
        sym = np.clip(rng.normal(a / 2, max(a / 6, 0.7), n), 0, a - 1).astype(np.int64)
        h, body = _payload(sym, a, p, bs)
        out = np.full(n + 8, 0xEE, np.uint8)                       # canary bytes after the output
        rc = lib.eoq_decode_tensor_v2(C.byref(h), body.ctypes.data, body.size, out.ctypes.data, n, None)
        assert rc == 0
        assert np.array_equal(out[:n], sym.astype(np.uint8)), (n, a, p, bs)
        assert (out[n:] == 0xEE).all()
        rc2, ref = O.decode_c_payload(np.array([getattr(h, f) for f, _ in L.TensorHeader._fields_], np.uint32), body.tobytes())
        assert rc2 == 0 and np.array_equal(ref, out[:n])
        out2 = np.zeros(n, np.uint8)
        assert lib.eoq_decode_tensor(C.byref(h), body.ctypes.data, out2.ctypes.data) == 0 and np.array_equal(out2, out[:n])
        assert lib.eoq_cuda_decode_tensor(C.byref(h), body.ctypes.data, out2.ctypes.data, None) == 0


@pytest.mark.parametrize("alphabet,p,block,n", [
    (2, 8, 8, 100), (2, 9, 7, 1000), (3, 8, 50, 333), (5, 8, 33, 5000), (15, 12, 4096, 9000), (16, 14, 256, 70001),
    (31, 14, 100, 12345), (200, 12, 1000, 40000), (256, 16, 256, 66000), (256, 12, 31, 3000), (1000, 16, 512, 50000),
    (4096, 16, 2048, 100000), (4096, 13, 300, 30000), (5000, 16, 256, 20000)])
def test_blocked_decoder_over_alphabets_precisions_and_block_sizes(alphabet, p, block, n):
    """Streams from the oracle's encoder, decoded on the GPU: both table forms of the lane kernel (one packed word per
    slot; slot -> symbol -> {freq, cum}), 8- and 16-bit symbols, blocks that end inside a group of eight steps or inside a
    32-byte sector of the output, short last blocks, and the one-thread-per-block kernel (alphabets above 4096).

    Both sides get a table that already sums to 2**p: normalising it again is the identity, so the test does not depend
    on how ties are ordered when a residual is dealt out (numpy's argsort leaves that open above 16 symbols; the oracle
    breaks ties by symbol index like the reference's C decoders)."""
    rng = np.random.default_rng(alphabet * 31 + p)
    sym = np.clip(rng.normal(alphabet / 2, max(alphabet / 7, 0.6), n), 0, alphabet - 1).astype(np.int64)
    if alphabet > 2:
        sym[rng.integers(0, n, n // 50)] = rng.integers(0, alphabet, n // 50)      # rare symbols get frequency 1
    freq, _ = O.normalize(np.bincount(sym, minlength=alphabet), p)
    t = O.Table(freq, p)
    assert np.array_equal(t.freq, freq)
    parts, offs, at = [], [], 0
    for b in range(0, n, block):
        enc = t.encode(sym[b:b + block])
        assert np.array_equal(t.decode(enc, len(sym[b:b + block])), sym[b:b + block])   # the oracle round-trips its own stream
        offs.append(at); parts.append(enc); at += len(enc)
    stream = b"".join(parts)
    nb = len(offs)
    data = RB.BlockedRANSData(compressed_blocks=stream, block_offsets=offs, freq_table=freq.astype(np.int64),
                              num_symbols=n, block_size=block, num_blocks=nb, alphabet_size=alphabet, precision_bits=p)
    dec = RB.BlockedRANSDecoder()
    assert np.array_equal(dec.decode_all(data), sym)
    for b in (0, nb // 2, nb - 1):
        assert np.array_equal(dec.decode_block(data, b), sym[b * block:(b + 1) * block])
    data_ours, offs_ours = RB.encode_blocks(freq.astype(np.int64), p, sym, block)   # and our encoder writes the same bytes
    assert bytes(data_ours) == stream and list(offs_ours) == offs


def test_corrupt_stream_stays_in_bounds():
    """Garbage inside a block is not detected (as in the reference) but decoding terminates
    and never writes outside the output."""
    lib = L.lib()
    rng = np.random.default_rng(1)
    sym = rng.integers(0, 15, 5000)
    h, body = _payload(sym, 15, 12, 256)
    meta = 15 * 2 + 4 * 20
    offs = body[15 * 2:meta].view(np.uint32)
    for b in (0, 3, 7):                                                   # overwrite the payload of three blocks, keeping
        lo, hi = int(offs[b]) + 5, int(offs[b + 1])                       # their state-length prefix and state intact
        body[meta + lo:meta + hi] = rng.integers(0, 256, hi - lo).astype(np.uint8)
    out = np.full(5000 + 16, 0xEE, np.uint8)
    rc = lib.eoq_decode_tensor_v2(C.byref(h), body.ctypes.data, body.size, out.ctypes.data, 5000, None)
    assert rc == 0
    assert (out[5000:] == 0xEE).all() and out[:5000].max() < 15
    good = [b for b in range(20) if b not in (0, 3, 7)]
    for b in good:
        assert np.array_equal(out[b * 256:(b + 1) * 256][:5000 - b * 256], sym[b * 256:(b + 1) * 256].astype(np.uint8))


def test_progress_callback_of_single_tensor():
    lib = L.lib()
    sym = np.random.default_rng(2).integers(0, 15, 3000)
    h, body = _payload(sym, 15, 12, 256)
    seen = []
    cb = L.PROGRESS_FN(lambda done, total, ud: seen.append((done, total)) or 0)
    opts = L.DecodeOpts(4, cb, None)
    out = np.zeros(3000, np.uint8)
    assert lib.eoq_decode_tensor_v2(C.byref(h), body.ctypes.data, body.size, out.ctypes.data, 3000, C.byref(opts)) == 0
    assert seen == [(3000, 3000)] and np.array_equal(out, sym)


def _tasks(n_tasks, sizes=None, seed=0):
    rng = np.random.default_rng(seed)
    keep, tasks = [], (L.DecodeTask * n_tasks)()
    for i in range(n_tasks):
        n = int(sizes[i]) if sizes is not None else int(rng.integers(1, 6000))
        sym = rng.integers(0, 200, n)
        h, body = _payload(sym, 256, 16, 256)
        out = np.zeros(max(n, 1), np.uint8)
        keep.append((sym, h, body, out))
        tasks[i].header, tasks[i].compressed_data, tasks[i].compressed_size = C.pointer(h), body.ctypes.data, body.size
        tasks[i].output, tasks[i].output_capacity = out.ctypes.data, n
    return tasks, keep


def test_parallel_decode_many_tensors_progress_and_results():
    lib = L.lib()
    tasks, keep = _tasks(23)
    seen = []
    cb = L.PARALLEL_PROGRESS_FN(lambda d, t, ud: seen.append((d, t)) or 0)
    for threads in (0, 1, 3, 64):
        seen.clear()
        for sym, h, body, out in keep:
            out[:] = 0
        opts = L.ParallelOpts(threads, cb, None)
        assert lib.eoq_parallel_decode(tasks, 23, C.byref(opts)) == 0
        assert seen == [(i + 1, 23) for i in range(23)]              # monotonic, serialised
        for i, (sym, h, body, out) in enumerate(keep):
            assert tasks[i].result == 0 and tasks[i].task_index == i
            assert np.array_equal(out, sym.astype(np.uint8))
    assert lib.eoq_parallel_decode(tasks, 23, None) == 0                  # NULL opts = defaults


def test_parallel_decode_error_propagation_and_cancel():
    lib = L.lib()
    tasks, keep = _tasks(12, seed=3)
    tasks[4].output_capacity = 0 if keep[4][0].size == 0 else keep[4][0].size - 1
    tasks[7].compressed_size = 3
    rc = lib.eoq_parallel_decode(tasks, 12, None)
    assert rc == L.EOQ_ERR_BUFFER_TOO_SMALL                               # first error in task order
    assert tasks[4].result == L.EOQ_ERR_BUFFER_TOO_SMALL and tasks[7].result == L.EOQ_ERR_CORRUPT_STREAM
    assert all(tasks[i].result == 0 for i in range(12) if i not in (4, 7))
    tasks, keep = _tasks(20, seed=4)
    calls = []
    cb = L.PARALLEL_PROGRESS_FN(lambda d, t, ud: calls.append(d) or (1 if d >= 3 else 0))
    opts = L.ParallelOpts(2, cb, None)
    rc = lib.eoq_parallel_decode(tasks, 20, C.byref(opts))
    assert rc == L.EOQ_ERR_THREAD
    results = [tasks[i].result for i in range(20)]
    assert results[:3] == [0, 0, 0] and results[-1] == L.EOQ_ERR_THREAD
    assert calls[-1] == 3 and set(results) == {0, L.EOQ_ERR_THREAD}
    done = [i for i, r in enumerate(results) if r == 0]
    assert done == list(range(len(done)))                                 # cancelled tasks form a suffix
    for i in done:
        assert np.array_equal(keep[i][3], keep[i][0].astype(np.uint8))
    tasks, keep = _tasks(3, sizes=[0, 10, 0])                              # zero-length tensors are OK
    assert lib.eoq_parallel_decode(tasks, 3, None) == 0


def test_incremental_block_decoder():
    lib = L.lib()
    rng = np.random.default_rng(9)
    sym = rng.integers(0, 100, 700)
    t = O.Table(np.bincount(sym, minlength=256), 16)
    block = np.frombuffer(t.encode(sym), np.uint8).copy()
    f16 = t.freq.astype(np.uint16)
    dec = L.Decoder()
    assert lib.eoq_decoder_init(C.byref(dec), f16.ctypes.data, 256, 16, block.ctypes.data, block.size) == 0
    got = []
    for count in (1, 99, 250, 350):
        out = np.zeros(count, np.uint8)
        assert lib.eoq_decoder_decode(C.byref(dec), out.ctypes.data, count) == 0
        got.append(out)
    assert np.array_equal(np.concatenate(got), sym.astype(np.uint8))
    assert dec.stream_pos == dec.stream_end and dec.state == 1 << 24       # stream consumed, state back at its lower bound
    lib.eoq_decoder_free(C.byref(dec))
    assert dec.sym_info is None
    assert lib.eoq_decoder_init(C.byref(dec), f16.ctypes.data, 0, 16, block.ctypes.data, block.size) == L.EOQ_ERR_INVALID_HEADER
    bad = block[:8].copy(); bad[0] = 200                                  # state length runs past the block
    assert lib.eoq_decoder_init(C.byref(dec), f16.ctypes.data, 256, 16, bad.ctypes.data, bad.size) == L.EOQ_ERR_CORRUPT_STREAM


def test_cuda_device_entry_points_and_batch():
    lib = L.lib()
    rng = np.random.default_rng(11)
    sym = rng.integers(0, 256, 9000)
    blocked = O.encode_blocked(sym, 256, 256, 16)
    t = O.Table(blocked.freq_table, 16)
    info = np.zeros((1 << 16, 4), np.uint16)
    for s in range(256):
        info[t.cdf[s]:t.cdf[s + 1]] = (s, t.freq[s], t.cdf[s], 0)
    offs = np.asarray(blocked.block_offsets, np.uint32)
    sizes = np.diff(np.append(offs, len(blocked.compressed_blocks))).astype(np.uint32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).cuda()
    d_stream, d_offs, d_sizes, d_info = dev(np.frombuffer(blocked.compressed_blocks, np.uint8)), dev(offs), dev(sizes), dev(info)
    d_out = torch.zeros(9000, dtype=torch.uint8, device="cuda")
    rc = lib.eoq_cuda_decode_tensor_device(d_stream.data_ptr(), d_offs.data_ptr(), d_sizes.data_ptr(), d_info.data_ptr(),
                                           d_out.data_ptr(), blocked.num_blocks, 256, 9000, 16, None)
    torch.cuda.synchronize()
    assert rc == 0 and np.array_equal(d_out.cpu().numpy(), sym.astype(np.uint8))
    ctx = lib.eoq_cuda_batch_create(None)
    outs, syms, keep = [], [], []
    for i in range(5):
        s = rng.integers(0, 50, 1000 + 317 * i)
        h, body = _payload(s, 256, 16, 256)
        o = torch.zeros(s.size, dtype=torch.uint8, device="cuda")
        assert lib.eoq_cuda_batch_prepare_tensor(ctx, C.byref(h), body.ctypes.data, o.data_ptr()) == 0
        outs.append(o); syms.append(s); keep.append((h, body))
    assert lib.eoq_cuda_batch_launch(ctx) == 0 and lib.eoq_cuda_batch_sync_and_free(ctx) == 0
    for o, s in zip(outs, syms):
        assert np.array_equal(o.cpu().numpy(), s.astype(np.uint8))
    lib.eoq_cuda_batch_destroy(ctx)


# ---------------------------------------------------------------- Python decode entry points
def test_blocked_decoder_matches_reference_fixtures():
    z = _z("ref_blocked")
    for name in z["names"]:
        d = RB.deserialize_blocked_rans(z[f"{name}/rans"].tobytes())
        got = RB.BlockedRANSDecoder().decode_all(d)
        assert got.dtype == np.int64 and np.array_equal(got, z[f"{name}/symbols"]), name
        assert np.array_equal(RB.BlockedRANSDecoder().decode_block(d, d.num_blocks - 1), z[f"{name}/last_block"]), name
        assert np.array_equal(RB.BlockedRANSDecoder().decode_block(d, 0), z[f"{name}/symbols"][:d.block_size]), name


def test_quantized_tensor_round_trip_and_bridge():
    from eoq_quantization_b200.core import rans_bitpacked as RBP
    from eoq_quantization_b200.core import utils as U
    z = _z("ref_tensor")
    comp = {}
    for k in z["names"]:
        bits = int(str(k)[4:])
        w = torch.from_numpy(z[f"{k}/w"])
        ct = RBP.CompressedTensorData(str(k), tuple(w.shape), bits, 128, z[f"{k}/scales_bytes"].tobytes(),
                                      z[f"{k}/rans"].tobytes(), w.numel(), w.numel() * 2, 0)
        codes, scales = RBP.decompress_tensor_rans(ct)
        assert codes.dtype == torch.int8 and scales.dtype == torch.float32
        assert np.array_equal(codes.numpy(), z[f"{k}/dec_codes"]) and np.array_equal(scales.numpy(), z[f"{k}/dec_scales"])
        comp[str(k)] = ct
        data = RB.encode_quantized_tensor(z[f"{k}/codes"], bits)
        assert np.array_equal(RB.decode_quantized_tensor(data, bits), z[f"{k}/codes"].ravel())
    sd = RBP.decompress_model_rans(comp, {})
    for k in z["names"]:
        assert sd[str(k)].dtype == torch.float16
        assert np.array_equal(sd[str(k)].float().numpy(), z[f"{k}/dequant"].astype(np.float16).astype(np.float32))


# ---------------------------------------------------------------- tiled layout on the device
def _int4_case(n, k, seed, sigma=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * sigma).astype(np.float32)
    codes, scales = O.quantize_absmax(w, 4, 128)
    s16 = scales.astype(np.float16)
    return (codes + 7).astype(np.uint8), s16, O.pack_int4_rows(codes)


@pytest.mark.parametrize("n,k,g", [(24, 256, 3), (100, 512, 2), (33, 128, 1), (200, 1408, 3), (96, 4096, 3), (257, 1024, 2)])
def test_tile_decode_bit_exact_and_dequant(n, k, g):
    sym, s16, packed = _int4_case(n, k, n + k)
    w = EOQWeight.from_symbols(sym, s16, symbols_per_step=g)
    assert np.array_equal(w.decode_symbols().cpu().numpy(), sym)
    assert np.array_equal(w.decode_symbols(packed=True).cpu().numpy(), packed)
    ref = O.int4_dequant_matrix(packed, s16.astype(np.float32), n, k, 128)
    assert np.array_equal(w.dequantize(torch.float32).cpu().numpy(), ref)
    assert np.array_equal(w.dequantize(torch.float16).cpu().numpy(), ref.astype(np.float16))
    assert w.info.padded_rows % (32 * g) == 0 and w.info.symbols_per_step == g


def test_weight_from_reference_container():
    sym, s16, packed = _int4_case(48, 512, 5)
    ser = O.serialize_rans_v1(O.encode_blocked(sym.ravel().astype(np.int64), 15, 4096, 12))
    w = EOQWeight.from_rans(ser, s16, (48, 512))
    assert np.array_equal(w.decode_symbols().cpu().numpy(), sym)
    with pytest.raises(L.EOQError):
        EOQWeight.from_rans(b"XXXX" + ser[4:], s16, (48, 512))
    with pytest.raises(L.EOQError):
        EOQWeight.from_rans(ser, s16, (48, 256))


# ---------------------------------------------------------------- fused GEMV
@pytest.mark.parametrize("n,k,g", [(24, 256, 3), (100, 512, 2), (33, 128, 1), (200, 1408, 3), (300, 4096, 3), (257, 1024, 2)])
@pytest.mark.parametrize("batch", [1, 2, 3, 5, 8])
def test_fused_gemv_matches_dequant_then_matmul(n, k, g, batch):
    sym, s16, packed = _int4_case(n, k, 7 * n + k)
    w = EOQWeight.from_symbols(sym, s16, symbols_per_step=g)
    rng = np.random.default_rng(batch)
    x = rng.standard_normal((batch, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    ref = O.int4_linear(packed, s16.astype(np.float32), n, k, 128, x, bias)
    y = w.gemv(torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda())
    assert y.shape == (batch, n) and y.dtype == torch.float32
    assert O.rel_l2(y.cpu().numpy(), ref) < 2e-5                       # fp32 in, fp32 accumulate, fp32 out
    for dt in (torch.float16, torch.bfloat16):
        xh = torch.from_numpy(x).cuda().to(dt)
        refh = O.int4_linear(packed, s16.astype(np.float32), n, k, 128, xh.float().cpu().numpy(), bias)
        yh = w.gemv(xh, torch.from_numpy(bias).cuda())
        assert yh.dtype == dt
        # the output is rounded to x.dtype; bf16 rounding alone is ~1.1e-3 rel-L2, so compare like with like
        want = torch.from_numpy(refh).to(dt).float().numpy()
        assert O.rel_l2(yh.float().cpu().numpy(), want) < TOL
    y2 = w.gemv(torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda())
    assert torch.equal(y, y2)                                          # same input, same bits
    yh = w.gemv_host(x.astype(np.float16), bias)
    assert O.rel_l2(yh.astype(np.float32), O.int4_linear(packed, s16.astype(np.float32), n, k, 128,
                                                         x.astype(np.float16).astype(np.float32), bias)) < TOL


def test_gemv_input_shapes_and_errors():
    sym, s16, packed = _int4_case(64, 256, 3)
    w = EOQWeight.from_symbols(sym, s16)
    x = torch.randn(2, 2, 256, device="cuda")
    assert w.gemv(x).shape == (2, 2, 64)
    assert w.gemv(torch.randn(256, device="cuda")).shape == (64,)
    assert w.gemv(torch.randn(19, 256, device="cuda")).shape == (19, 64)     # more than 8 rows: chunks of 8
    with pytest.raises(ValueError):
        w.gemv(torch.randn(2, 255, device="cuda"))
    with pytest.raises(RuntimeError):
        w.gemv(torch.randn(2, 256))
    lib = L.lib()
    y = torch.empty(9, 64, device="cuda")
    assert lib.eoq_b200_gemv(w._h, x.data_ptr(), L.F32, 9, y.data_ptr(), L.F32, None, None) == L.EOQ_ERR_UNSUPPORTED
    assert lib.eoq_b200_gemv(w._h, None, L.F32, 1, y.data_ptr(), L.F32, None, None) == L.EOQ_ERR_NULL_PTR
    assert lib.eoq_b200_gemv(w._h, x.data_ptr(), 7, 1, y.data_ptr(), L.F32, None, None) == L.EOQ_ERR_UNSUPPORTED


def test_quantized_linear_forward_matches_reference_outputs():
    from eoq_quantization_b200.core.quantized_linear import QuantizedLinear
    from eoq_quantization_b200.core.quantized_matmul import QuantizedLinearFast, quantized_matmul
    from eoq_quantization_b200.core.fast_dequant import dequantize_weight_fast, unpack_4bit_fast
    z = _z("ref_linear")
    for name in z["names"]:
        w = torch.from_numpy(z[f"{name}/weight"])
        n, k = w.shape
        lin = torch.nn.Linear(k, n, bias=f"{name}/bias" in z)
        with torch.no_grad():
            lin.weight.copy_(w)
            if lin.bias is not None:
                lin.bias.copy_(torch.from_numpy(z[f"{name}/bias"]))
        ql = QuantizedLinear.from_float(lin).cuda()
        x = torch.from_numpy(z[f"{name}/x"]).cuda()
        y = ql(x)
        assert y.dtype == x.dtype and O.rel_l2(y.cpu().numpy(), z[f"{name}/y"]) < 1e-4, name
        assert np.array_equal(ql._dequantize_weight().cpu().numpy(), z[f"{name}/dequant"]), name
        assert np.array_equal(dequantize_weight_fast(ql.packed_weight, ql.scales, n, k).cpu().numpy(), z[f"{name}/dequant"])
        codes = unpack_4bit_fast(ql.packed_weight, n, k)
        assert codes.dtype == torch.int8 and np.array_equal(codes.cpu().numpy(), O.unpack_int4_rows(z[f"{name}/packed"], k))
        for strategy in ("blocked", "vectorized", "auto"):
            ym = quantized_matmul(x, ql.packed_weight, ql.scales, n, k, strategy=strategy, chunk_rows=5)
            assert O.rel_l2(ym.cpu().numpy(), z[f"{name}/y_matmul_blocked"]) < 1e-4
        with pytest.raises(ValueError):
            quantized_matmul(x, ql.packed_weight, ql.scales, n, k, strategy="nope")
        fast = QuantizedLinearFast.from_quantized_linear(ql)
        assert fast.packed_weight.data_ptr() == ql.packed_weight.data_ptr()
        assert O.rel_l2(fast(x).cpu().numpy(), z[f"{name}/y"]) < 1e-4
        for shape in ((k,), (2, k), (2, 3, k), (1, 2, 2, k), (11, k)):      # 1-D .. 4-D inputs, and > 8 rows
            xi = torch.randn(*shape, device="cuda")
            yi = ql(xi)
            assert yi.shape == (*shape[:-1], n)
            assert O.rel_l2(yi.cpu().numpy(), O.int4_linear(z[f"{name}/packed"], z[f"{name}/scales"].astype(np.float32), n, k, 128,
                                                            xi.cpu().numpy(), z[f"{name}/bias"] if lin.bias is not None else None)) < 1e-4
        yh = ql(x.half())
        assert yh.dtype == torch.float16 and O.rel_l2(yh.float().cpu().numpy(), z[f"{name}/y"]) < 2e-3


def test_polar_q5_gemv_matches_reference_dequant():
    z = _z("ref_polar")
    codes = z["codes"].reshape(16, 256).astype(np.uint8)
    w = EOQWeight.from_symbols(codes, z["norms"], kind=L.KIND_Q5_POLAR, group=64, centroids=z["centroids5"])
    assert np.array_equal(w.decode_symbols().cpu().numpy(), codes)
    rng = np.random.default_rng(0)
    for batch in (1, 4, 8):
        x = rng.standard_normal((batch, 256)).astype(np.float32)
        ref = x.astype(np.float64) @ z["dequant"].astype(np.float64).T       # the reference's fp16 dequantised weight
        y = w.gemv(torch.from_numpy(x).cuda())
        assert O.rel_l2(y.cpu().numpy(), ref) < TOL


# ---------------------------------------------------------------- full-size properties
def test_full_size_gate_projection_round_trip_and_gemv():
    """Headline shape 11008 x 4096: decode == original symbols (bit-exact, 45 M symbols) and the fused
    GEMV agrees with dequantise-then-matmul computed by torch on the same device."""
    n, k = 11008, 4096
    g = torch.Generator(device="cuda").manual_seed(0)
    wt = torch.randn(n, k, device="cuda", generator=g) * 0.02
    blocks = wt.view(-1, 128)
    scale = (blocks.abs().amax(dim=1) / 7).clamp(min=1e-10)
    codes = (blocks / scale[:, None]).round().clamp(-7, 7).to(torch.int8).view(n, k)
    s16 = scale.half()
    sym = (codes + 7).to(torch.uint8)
    w = EOQWeight.from_symbols(sym, s16)
    assert torch.equal(w.decode_symbols(), sym)
    assert 3.3 < w.info.bits_per_weight < 3.8
    dense = (codes.float().view(-1, 128) * s16.float()[:, None]).view(n, k)
    assert torch.equal(w.dequantize(torch.float32), dense)
    x = torch.randn(1, k, device="cuda", generator=g).half()
    ref = x.float() @ dense.T
    y = w.gemv(x)
    assert O.rel_l2(y.float().cpu().numpy(), ref.cpu().numpy()) < TOL
    ref16 = x @ dense.half().T                                          # the reference's own fp16 composition
    assert O.rel_l2(y.float().cpu().numpy(), ref16.float().cpu().numpy()) < 2e-3


@pytest.mark.parametrize("dt,batch", [(torch.float16, 4), (torch.bfloat16, 3), (torch.float32, 4), (torch.float16, 7)])
def test_fused_gemv_four_rows_on_a_wide_layer(dt, batch):
    """11008 x 4096 has 112-column tiles, beside which four fp32 activation segments per warp do not fit: fp16 and
    bf16 activations are kept as 16-bit values in shared memory instead, fp32 ones run two rows per launch, and seven
    rows are two launches.  All must agree with dequantise-then-matmul."""
    n, k = 11008, 4096
    g = torch.Generator(device="cuda").manual_seed(batch)
    wt = torch.randn(n, k, device="cuda", generator=g) * 0.02
    blocks = wt.view(-1, 128)
    scale = (blocks.abs().amax(dim=1) / 7).clamp(min=1e-10)
    codes = (blocks / scale[:, None]).round().clamp(-7, 7).to(torch.int8).view(n, k)
    s16 = scale.half()
    w = EOQWeight.from_symbols((codes + 7).to(torch.uint8), s16)
    dense = (codes.float().view(-1, 128) * s16.float()[:, None]).view(n, k)
    x = torch.randn(batch, k, device="cuda", generator=g).to(dt)
    bias = torch.randn(n, device="cuda", generator=g)
    ref = (x.float() @ dense.T + bias).cpu().numpy()
    y = w.gemv(x, bias=bias, out_dtype=torch.float32)
    assert O.rel_l2(y.cpu().numpy(), ref) < TOL
    assert torch.equal(w.gemv(x, bias=bias, out_dtype=torch.float32), y)
    for r in range(batch):                                   # every row equals the same row run on its own
        assert O.rel_l2(w.gemv(x[r:r + 1], bias=bias, out_dtype=torch.float32).cpu().numpy(), ref[r:r + 1]) < TOL


@pytest.mark.parametrize("n,k,batch", [(2752, 4096, 1), (1024, 11008, 1), (1376, 4096, 2), (512, 11008, 1), (512, 11008, 4), (96, 8192, 1)])
def test_fused_gemv_on_row_shards_much_wider_than_tall(n, k, batch):
    """The row shards of the Llama-7B MLP pair over four and eight GPUs.  The segments of one pair of row blocks are
    spread over dozens of CTAs here, so the warp elected to add their partial rows up has the whole CTA help it; the
    result must match dequantise-then-matmul and be the same from run to run."""
    g = torch.Generator(device="cuda").manual_seed(n + k + batch)
    wt = torch.randn(n, k, device="cuda", generator=g) * 0.02
    blocks = wt.view(-1, 128)
    scale = (blocks.abs().amax(dim=1) / 7).clamp(min=1e-10)
    codes = (blocks / scale[:, None]).round().clamp(-7, 7).to(torch.int8).view(n, k)
    s16 = scale.half()
    w = EOQWeight.from_symbols((codes + 7).to(torch.uint8), s16)
    dense = (codes.float().view(-1, 128) * s16.float()[:, None]).view(n, k)
    x = torch.randn(batch, k, device="cuda", generator=g).half()
    bias = torch.randn(n, device="cuda", generator=g)
    ref = (x.float() @ dense.T + bias).cpu().numpy()
    y0 = w.gemv(x, bias=bias, out_dtype=torch.float32)
    assert O.rel_l2(y0.cpu().numpy(), ref) < 1e-5
    for _ in range(5):
        assert torch.equal(w.gemv(x, bias=bias, out_dtype=torch.float32), y0)
    assert w.status() == 0


@pytest.mark.parametrize("n,k,batch", [(22016, 4096, 1), (32000, 4096, 2), (7680, 2048, 4)])
def test_fused_gemv_over_several_waves_of_tile_pairs(n, k, batch):
    """Shapes whose tile pairs outnumber the resident warps (the gate/up projection and the vocabulary head of the
    Llama-7B shape): the kernel makes several passes with chunks of unequal length, so some warps sit out a pass
    and re-arm their copy barriers later.  Results must still match dequantise-then-matmul, run to run."""
    g = torch.Generator(device="cuda").manual_seed(n + batch)
    wt = torch.randn(n, k, device="cuda", generator=g) * 0.02
    blocks = wt.view(-1, 128)
    scale = (blocks.abs().amax(dim=1) / 7).clamp(min=1e-10)
    codes = (blocks / scale[:, None]).round().clamp(-7, 7).to(torch.int8).view(n, k)
    s16 = scale.half()
    w = EOQWeight.from_symbols((codes + 7).to(torch.uint8), s16)
    dense = (codes.float().view(-1, 128) * s16.float()[:, None]).view(n, k)
    x = torch.randn(batch, k, device="cuda", generator=g).half()
    ref = (x.float() @ dense.T).cpu().numpy()
    y0 = w.gemv(x)
    assert O.rel_l2(y0.float().cpu().numpy(), ref) < TOL
    for _ in range(3):
        assert torch.equal(w.gemv(x), y0)


def test_full_size_polar_q5_gemv_batches():
    """Benchmark shape 14336 x 4096, N(0, 0.015) with 0.1 % outliers at 8 sigma, PolarQuant Q5 with
    per-64 norms (core/polar_quant.py:138-264 restated in torch on the GPU as the checker): symbols
    round-trip bit-exactly and the fused GEMV matches the reference's fp16 dequantised weight."""
    z = _z("ref_polar")
    n, k, d = 14336, 4096, 64
    cent = torch.from_numpy(z["centroids5"]).cuda()
    H = torch.from_numpy(z["hadamard64"]).cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.015
    out = torch.rand(n, k, device="cuda", generator=g) < 1e-3
    sign = torch.where(torch.rand(n, k, device="cuda", generator=g) < 0.5, -1.0, 1.0)
    w = torch.where(out, sign * 8 * 0.015, w)
    codes = torch.empty(n, k, dtype=torch.uint8, device="cuda")
    norms = torch.empty(n * k // d, dtype=torch.float16, device="cuda")
    dense = torch.empty(n, k, dtype=torch.float16, device="cuda")
    rows = 512
    for lo in range(0, n, rows):                                           # per-block independent, so chunking is exact
        blk = w[lo:lo + rows].reshape(-1, d)
        nr = blk.norm(dim=1, keepdim=True).clamp(min=1e-10)
        scaled = (blk / nr) @ H * (d ** 0.5)
        c = (scaled.unsqueeze(-1) - cent).abs().argmin(dim=-1)
        codes[lo:lo + rows] = c.reshape(rows, k).to(torch.uint8)
        n16 = nr.squeeze(1).half()
        norms[lo * k // d:(lo + rows) * k // d] = n16
        dense[lo:lo + rows] = ((cent[c] / (d ** 0.5)) @ H * n16.float().unsqueeze(1)).reshape(rows, k).half()
    ew = EOQWeight.from_symbols(codes, norms, kind=L.KIND_Q5_POLAR, group=64, centroids=z["centroids5"])
    assert torch.equal(ew.decode_symbols(), codes)
    assert 4.4 < ew.info.bits_per_weight < 5.0
    for batch in (1, 4, 8):
        x = torch.randn(batch, k, device="cuda", generator=g).half()
        ref = x.float() @ dense.float().T
        y = ew.gemv(x)
        assert O.rel_l2(y.float().cpu().numpy(), ref.cpu().numpy()) < TOL, batch
    assert L.lib().eoq_b200_weight_status(ew._h, None) == 0


def test_eoq_file_loads_straight_to_device():
    from eoq_quantization_b200 import eoq_file as EF
    z = _z("ref_eoq_file")
    loaded = EF.load_eoq_to_device(f"{GOLDEN}/sample.eoq", dense_dtype=torch.float32)
    assert set(loaded) == set(z.files)
    for name in z.files:
        ref = z[name]
        got = loaded[name]
        if isinstance(got, EOQWeight):
            assert ref.ndim == 2 and (got.rows, got.cols) == ref.shape
            assert np.array_equal(got.dequantize(torch.float32).cpu().numpy(), ref), name
            x = torch.randn(2, ref.shape[1], device="cuda")
            assert O.rel_l2(got.gemv(x).cpu().numpy(), x.cpu().numpy() @ ref.T) < 1e-4
        else:
            assert got.is_cuda and np.array_equal(got.cpu().numpy(), ref), name


def test_host_buffer_gemv_async_two_weights_one_sync():
    """eoq_b200_gemv_host_async: two weights queued from pinned host buffers, one synchronisation."""
    lib = L.lib()
    cases = []
    for seed, (n, k) in enumerate(((192, 512), (100, 1024))):
        sym, s16, packed = _int4_case(n, k, 40 + seed)
        w = EOQWeight.from_symbols(sym, s16)
        x = torch.randn(2, k).half().pin_memory()
        y = torch.empty(2, n).half().pin_memory()
        cases.append((w, x, y, packed, s16, n, k))
    for w, x, y, *_ in cases:
        L.check(lib.eoq_b200_gemv_host_async(w._h, x.data_ptr(), L.F16, 2, y.data_ptr(), L.F16, None, None), "async")
    for w, *_ in cases:
        assert lib.eoq_b200_weight_status(w._h, None) == 0
    for w, x, y, packed, s16, n, k in cases:
        ref = O.int4_linear(packed, s16.astype(np.float32), n, k, 128, x.float().numpy())
        assert O.rel_l2(y.float().numpy(), ref) < TOL


@pytest.mark.parametrize("n,k", [(96, 256), (500, 1536), (1000, 11008), (4096, 4096), (193, 4096)])
def test_dequantised_matrix_in_every_dtype_is_the_reference_product(n, k):
    """``EOQWeight.dequantize`` (the two-tiles-per-warp kernel for the default 4-bit layout; odd numbers of row blocks,
    ragged last rows, 96- and 112-column tiles): fp32 equals code * scale bit for bit (core/utils.py:130-161), and the
    16-bit outputs are that product rounded once."""
    rng = np.random.default_rng(n + k)
    wt = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    codes, scales = O.quantize_absmax(wt, 4, 128)
    s16 = scales.astype(np.float16)
    w = EOQWeight.from_symbols((codes + 7).astype(np.uint8), s16)
    dense = (codes.reshape(-1, 128).astype(np.float32) * s16.astype(np.float32)[:, None]).reshape(n, k)
    got = w.dequantize(torch.float32)
    assert np.array_equal(got.cpu().numpy(), dense)
    ref = torch.from_numpy(dense)
    assert torch.equal(w.dequantize(torch.float16).cpu(), ref.half())
    assert torch.equal(w.dequantize(torch.bfloat16).cpu(), ref.bfloat16())
    assert w.status() == 0


@pytest.mark.parametrize("rows", [1, 2, 4, 8])
def test_fused_gemv_on_short_tiles_of_wide_short_matrices(rows):
    """Low-entropy codes make tiles much shorter than the buffers' later use (the warp's sums, its share of a cooperative
    meeting: 3 KB at four activation rows), and a matrix much wider than tall takes the cooperative meeting: the buffers
    have a floor that covers both.  Checked against the oracle's dequantise-then-matmul."""
    rng = np.random.default_rng(rows)
    n, k = 150, 8192
    codes = np.where(rng.random((n, k)) < 0.9, 0, rng.integers(-7, 8, (n, k))).astype(np.int64)       # nine codes in ten are zero
    scales = (rng.random(n * k // 128) * 0.01 + 0.001).astype(np.float16)
    w = EOQWeight.from_symbols((codes + 7).astype(np.uint8), scales)
    assert w.info.bits_per_weight < 3.0              # tiles of about a kilobyte
    dense = (codes.reshape(-1, 128).astype(np.float32) * scales.astype(np.float32)[:, None]).reshape(n, k).astype(np.float64)
    for dt in (torch.float16, torch.float32):
        x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda().to(dt)
        y = w.gemv(x, out_dtype=torch.float32).cpu().numpy()
        assert O.rel_l2(y, x.float().cpu().numpy().astype(np.float64) @ dense.T) < 1e-3
        assert np.array_equal(y, w.gemv(x, out_dtype=torch.float32).cpu().numpy())              # and the same bits again
    assert w.status() == 0
