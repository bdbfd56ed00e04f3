#!/usr/bin/env python3
"""Generate the committed golden fixtures from the reference itself.

Run in a container that has the reference checkout:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [/path/to/reference]

It imports the reference's Python modules (never copies them), runs them on
seeded synthetic inputs and stores inputs + outputs as small ``.npz`` files
beside this script.  It also re-packs the nine known-answer vectors of the
reference's cross-validation suite (``llamacpp/test_vectors/*.bin``, layout in
``llamacpp/test_cross_validate.py:8-15``) into one ``.npz``.  The tests read only
the ``.npz`` files, so they run where the reference is absent.
"""
from __future__ import annotations

import os
import struct
import sys

import numpy as np

OUT = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: the argument, else $EOQ_REFERENCE_DIR, else a directory named `reference` beside this repository
REF = (sys.argv[1] if len(sys.argv) > 1 else os.environ.get("EOQ_REFERENCE_DIR")
       or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(OUT))), "reference"))
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from core import rans as R  # noqa: E402
from core import rans_blocked as RB  # noqa: E402
from core import rans_bitpacked as RBP  # noqa: E402
from core import utils as U  # noqa: E402
from core import quantized_linear as QL  # noqa: E402
from core import quantized_matmul as QM  # noqa: E402
from core import fast_dequant as FD  # noqa: E402
from core import polar_quant as PQ  # noqa: E402


def xval_vectors():
    d = {}
    vdir = os.path.join(REF, "llamacpp", "test_vectors")
    names = sorted(f[:-4] for f in os.listdir(vdir) if f.endswith(".bin"))
    for name in names:
        raw = open(os.path.join(vdir, name + ".bin"), "rb").read()
        n, a, p, csz = struct.unpack_from("<4I", raw, 0)
        at = 16
        freq = np.frombuffer(raw, "<u4", a, at); at += 4 * a
        comp = np.frombuffer(raw, np.uint8, csz, at); at += csz
        exp = np.frombuffer(raw, "<u4", n, at)
        # the vectors must decode with the reference's own decoder before they are trusted
        got = R.RANSDecoder(freq.astype(np.int64), precision_bits=p).decode(comp.tobytes(), n)
        assert np.array_equal(got, exp.astype(np.int64)), name
        d[name + "/meta"] = np.array([n, a, p, csz], np.int64)
        d[name + "/freq"] = freq.astype(np.int64)
        d[name + "/comp"] = comp.copy()
        d[name + "/expected"] = exp.astype(np.int64)
    d["names"] = np.array(names)
    np.savez_compressed(os.path.join(OUT, "xval_vectors.npz"), **d)
    print("xval_vectors:", names)


def normalisation():
    rng = np.random.default_rng(7)
    d = {}
    cases = []
    for i, (a, p) in enumerate([(15, 12), (15, 14), (16, 16), (4, 8), (2, 16), (1, 16), (8, 12), (3, 10), (16, 8)]):
        raw = rng.integers(0, 5000, size=a)
        if i % 3 == 0:
            raw[rng.integers(0, a)] = 0
        if i == 4:
            raw = np.array([1, 10 ** 6])
        cases.append((raw, p))
    # ties among the largest buckets, alphabets <= 16 (numpy's argsort is an insertion sort there)
    cases.append((np.array([100, 100, 100, 100, 3, 3, 3]), 12))
    cases.append((np.array([7] * 15), 12))
    cases.append((np.array([1, 0, 0, 0, 0, 0, 0, 0]), 8))
    # wider alphabets with all-distinct counts (no tie can straddle the cut)
    cases.append((np.arange(1, 33) * 37 + np.arange(32) ** 2, 12))
    cases.append((np.arange(1, 257) * 3 + (np.arange(256) % 7) * 1000 + np.arange(256), 16))
    for i, (raw, p) in enumerate(cases):
        f, c = R._normalize_frequencies(np.asarray(raw, np.int64), p)
        d[f"{i}/raw"] = np.asarray(raw, np.int64)
        d[f"{i}/p"] = np.array(p)
        d[f"{i}/freq"] = f
        d[f"{i}/cdf"] = c
    d["count"] = np.array(len(cases))
    np.savez_compressed(os.path.join(OUT, "ref_normalise.npz"), **d)
    print("ref_normalise:", len(cases))


def blocked():
    rng = np.random.default_rng(2024)
    torch.manual_seed(1)
    d = {}
    cases = {}
    w = torch.randn(13, 1024) * 0.02
    q4 = U.quantize_absmax(w, 4, 128)
    cases["int4_p12_b4096"] = ((q4.data.flatten().numpy() + 7).astype(np.int64), 15, 4096, 12)
    cases["int4_p14_b256"] = ((q4.data.flatten().numpy()[:1000] + 7).astype(np.int64), 15, 256, 14)
    q5 = U.quantize_absmax(w[:4], 5, 64)
    cases["q5abs_p14_b256"] = ((q5.data.flatten().numpy() + 15).astype(np.int64), 31, 256, 14)
    q2 = U.quantize_absmax(w[:2], 2, 128)
    cases["q2_p14_b256"] = ((q2.data.flatten().numpy() + 1).astype(np.int64), 3, 256, 14)
    cases["bytes_p16_b256"] = (np.clip(rng.normal(128, 20, 3000), 0, 255).astype(np.int64), 256, 256, 16)
    cases["one_symbol"] = (np.array([5], np.int64), 8, 256, 14)
    cases["exact_block"] = (rng.integers(0, 15, 512).astype(np.int64), 15, 256, 12)
    cases["block_plus_one"] = (rng.integers(0, 15, 513).astype(np.int64), 15, 256, 12)
    cases["all_same"] = (np.full(700, 3, np.int64), 8, 256, 12)
    cases["p8_small_alphabet"] = (rng.integers(0, 4, 600).astype(np.int64), 4, 128, 8)
    for name, (sym, a, bs, p) in cases.items():
        data = RB.BlockedRANSEncoder(block_size=bs, precision_bits=p).encode(sym, a)
        ser = RB.serialize_blocked_rans(data)
        back = RB.BlockedRANSDecoder().decode_all(RB.deserialize_blocked_rans(ser))
        assert np.array_equal(back, sym), name
        blk = RB.BlockedRANSDecoder().decode_block(data, data.num_blocks - 1)
        d[name + "/symbols"] = sym
        d[name + "/params"] = np.array([a, bs, p], np.int64)
        d[name + "/rans"] = np.frombuffer(ser, np.uint8).copy()
        d[name + "/last_block"] = blk
    d["names"] = np.array(list(cases))
    np.savez_compressed(os.path.join(OUT, "ref_blocked.npz"), **d)
    print("ref_blocked:", list(cases))


def tensors():
    torch.manual_seed(3)
    d = {}
    names = []
    for bits in (2, 3, 4, 5, 8):
        w = torch.randn(24, 256) * 0.02
        qt = U.quantize_absmax(w, bits, 128)
        ct = RBP.compress_tensor_rans(f"t{bits}", qt.data, qt.scale, bits, 128, tuple(w.shape))
        codes, scales = RBP.decompress_tensor_rans(ct)
        qt2 = U.QuantizedTensor(data=codes.reshape(w.shape).to(torch.int32), scale=scales,
                                zero_point=torch.zeros(len(scales)), bits=bits, shape=tuple(w.shape), block_size=128)
        deq = U.dequantize(qt2)
        k = f"bits{bits}"
        names.append(k)
        d[k + "/w"] = w.numpy()
        d[k + "/codes"] = qt.data.numpy().astype(np.int32)
        d[k + "/scales_fp32"] = qt.scale.numpy()
        d[k + "/rans"] = np.frombuffer(ct.rans_bytes, np.uint8).copy()
        d[k + "/scales_bytes"] = np.frombuffer(ct.scales_bytes, np.uint8).copy()
        d[k + "/dec_codes"] = codes.numpy()
        d[k + "/dec_scales"] = scales.numpy()
        d[k + "/dequant"] = deq.numpy()
    d["names"] = np.array(names)
    np.savez_compressed(os.path.join(OUT, "ref_tensor.npz"), **d)
    print("ref_tensor:", names)


def linears():
    torch.manual_seed(5)
    d = {}
    names = []
    for name, (n, k, bias) in {"24x256_bias": (24, 256, True), "40x512": (40, 512, False),
                               "13x100_ragged": (13, 100, True), "7x130_ragged": (7, 130, False)}.items():
        lin = torch.nn.Linear(k, n, bias=bias)
        with torch.no_grad():
            lin.weight.mul_(0.5)
        ql = QL.QuantizedLinear.from_float(lin, bits=4, block_size=128)
        x = torch.randn(3, k)
        y = ql(x)
        ym = QM.quantized_matmul(x, ql.packed_weight, ql.scales, n, k, bits=4, block_size=128, strategy="blocked")
        deq = FD.dequantize_weight_fast(ql.packed_weight, ql.scales, n, k, 4, 128)
        assert torch.allclose(deq, ql._dequantize_weight())
        names.append(name)
        d[name + "/weight"] = lin.weight.detach().numpy()
        d[name + "/packed"] = ql.packed_weight.numpy()
        d[name + "/scales"] = ql.scales.numpy()
        if bias:
            d[name + "/bias"] = ql.bias_param.numpy()
        d[name + "/x"] = x.numpy()
        d[name + "/y"] = y.detach().numpy()
        d[name + "/y_matmul_blocked"] = ym.detach().numpy()
        d[name + "/dequant"] = deq.numpy()
    d["names"] = np.array(names)
    np.savez_compressed(os.path.join(OUT, "ref_linear.npz"), **d)
    print("ref_linear:", names)


def polar():
    torch.manual_seed(11)
    w = torch.randn(16, 256) * 0.015
    mask = torch.rand_like(w) < 0.01
    w = torch.where(mask, torch.sign(torch.randn_like(w)) * 8 * 0.015, w)
    r = PQ.polar_quantize(w, bits=5, block_size=64, use_qjl=False)
    deq = PQ.polar_dequantize(r)
    d = {"w": w.numpy(), "codes": r.codes.numpy(), "norms": r.norms.numpy(), "dequant": deq.float().numpy(),
         "centroids5": PQ._ensure_centroids(5).numpy(), "hadamard64": PQ.hadamard_matrix(64).numpy(),
         "gauss_freq_5_14": PQ.get_gaussian_freq_table(5, 14)}
    np.savez_compressed(os.path.join(OUT, "ref_polar.npz"), **d)
    print("ref_polar: codes", r.codes.shape)


def eoq_container():
    """A small .eoq file written by the reference's own writer (core/eoq_format.py:117-184)."""
    from core import eoq as E
    from core import eoq_format as EF
    torch.manual_seed(21)
    comp = E.EOQCompressor(E.EOQConfig(bits=4, block_size=128, rans_block_size=256, precision_bits=14))
    model = E.EOQCompressedModel(config=comp.config, metadata={"model_name": "synthetic"})
    tensors = {"layers.0.mlp.up.weight": torch.randn(48, 256) * 0.02,
               "layers.0.mlp.down.weight": torch.randn(32, 384) * 0.02,
               "layers.0.norm.weight": torch.randn(100) * 0.1 + 1.0,
               "embed.weight": torch.randn(10, 30) * 0.02}
    for name, t in tensors.items():
        model.tensors[name] = comp.compress_tensor(name, t)
    path = os.path.join(OUT, "sample.eoq")
    EF.save_eoq(model, path)
    back = E.EOQDecompressor().decompress_model(EF.load_eoq(path))
    np.savez_compressed(os.path.join(OUT, "ref_eoq_file.npz"), **{k: v.numpy() for k, v in back.items()})
    print("sample.eoq:", os.path.getsize(path), "bytes,", list(tensors))


def fullsize():
    """The benchmark shapes at full size.  The matrices are too large to commit, so the fixture holds what pins them:
    hashes of what the reference's quantisers make of the seeded weights (recipes.py regenerates the weights), the
    hash and length of the reference-encoded config-1 container, and the reference's own dequantise-then-linear
    outputs (whole vectors for the GEMV shapes, 32 evenly spaced output columns for the prefill shapes)."""
    import recipes as RC
    d = {}
    for name, (n, k, seed, sigma) in RC.INT4_SHAPES.items():
        w = RC.weight(n, k, seed, sigma)
        qt = U.quantize_absmax(w, 4, 128)
        codes = qt.data.to(torch.int8).reshape(n, k)
        s16 = qt.scale.to(torch.float16)
        d[name + "/sha_codes"] = np.array(RC.sha(codes))
        d[name + "/sha_scales16"] = np.array(RC.sha(s16))
        qt16 = U.QuantizedTensor(data=qt.data, scale=s16.float(), zero_point=qt.zero_point, bits=4, shape=qt.shape, block_size=128)
        deq = U.dequantize(qt16).reshape(n, k)                     # what a loader sees: scales went through fp16
        if name.startswith(("up_", "down_4096")):
            for batch in (1, 4):
                x = RC.activations(batch, k, seed * 10 + batch)
                d[f"{name}/y_fp32_b{batch}"] = F.linear(x.float(), deq).numpy()          # fp32 accumulate, the parity bar
                d[f"{name}/y_fp16_b{batch}"] = F.linear(x, deq.half()).float().numpy()   # the reference's own composition
        if "shard" in name:
            stride = n // 32
            for m in (16, 64, 256, 2048):
                x = RC.activations(m, k, seed * 10 + m, torch.bfloat16)
                d[f"{name}/y_m{m}"] = F.linear(x.float(), deq[::stride]).numpy()
            d[name + "/stride"] = np.array(stride)
        if name.startswith("square"):
            sym = (codes.flatten().numpy().astype(np.int64) + 7)
            data = RB.BlockedRANSEncoder(block_size=4096, precision_bits=12).encode(sym, 15)
            ser = RB.serialize_blocked_rans(data)
            d[name + "/rans_len"] = np.array(len(ser))
            d[name + "/sha_rans"] = np.array(RC.sha(np.frombuffer(ser, np.uint8)))
            d[name + "/sha_dequant16"] = np.array(RC.sha(deq.half()))
            # the bridge of core/rans_bitpacked.py (block 256, p 14) on the first SLICE_ROWS rows
            rows = RC.BRIDGE_ROWS
            ct = RBP.compress_tensor_rans("w", qt.data.flatten()[: rows * k], qt.scale.flatten()[: rows * k // 128], 4, 128, (rows, k))
            d[name + "/bridge_rans"] = np.frombuffer(ct.rans_bytes, np.uint8).copy()
            d[name + "/bridge_scales"] = np.frombuffer(ct.scales_bytes, np.uint8).copy()
        print("fullsize:", name)
    name, n, k, seed, sigma = RC.POLAR_SHAPE
    w = RC.polar_weight(n, k, seed, sigma)
    rows = RC.SLICE_ROWS
    r = PQ.polar_quantize(w[:rows], bits=5, block_size=64, use_qjl=False)
    deq = PQ.polar_dequantize(r).float()
    d[name + "/sha_codes_slice"] = np.array(RC.sha(r.codes))
    d[name + "/sha_norms_slice"] = np.array(RC.sha(r.norms))
    for batch in (1, 4, 8):
        x = RC.activations(batch, k, seed * 10 + batch)
        d[f"{name}/y_slice_b{batch}"] = F.linear(x.float(), deq).numpy()
    np.savez_compressed(os.path.join(OUT, "ref_fullsize.npz"), **d)
    print("ref_fullsize:", os.path.getsize(os.path.join(OUT, "ref_fullsize.npz")), "bytes")


if __name__ == "__main__":
    sys.path.insert(0, OUT)
    if len(sys.argv) > 2 and sys.argv[2] == "fullsize":
        fullsize()
        raise SystemExit(0)
    eoq_container()
    xval_vectors()
    normalisation()
    blocked()
    tensors()
    linears()
    polar()
    fullsize()
