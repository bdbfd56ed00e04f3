/*
 * eoq_oracle.c -- CPU restatement of the EOQ rANS hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA implementation.  Nothing in the
 * product package links, imports or executes it; only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: PINNED.  The functions below are checked (tests/test_oracle.py)
 * against the nine known-answer vectors of the reference's cross-validation
 * suite (llamacpp/test_cross_validate.py:65-153), against fixtures produced by
 * importing the reference's Python modules, and against the reference's own C
 * decoders compiled from source (oracle/Makefile, target `ref`).
 *
 * Each function names the reference lines whose behaviour it restates.
 * Plain C99, no dependencies beyond libc.
 */

#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define ORC_OK                0
#define ORC_ERR_NULL_PTR     -1
#define ORC_ERR_TOO_SMALL    -2
#define ORC_ERR_CORRUPT      -3
#define ORC_ERR_HEADER       -4
#define ORC_ERR_ALLOC        -5

/* ------------------------------------------------------------------------
 * Frequency normalisation.
 * Restates core/rans.py:85-153 (C twins: llamacpp/eoq_rans.c:56-125,
 * llamacpp_integration/eoq_rans_v2.c:78-141).
 *
 *   raw' = max(raw, 1); scaled = trunc(raw' / sum * 2^p) in float64;
 *   scaled = max(scaled, 1); the residual 2^p - sum(scaled) is handed out one
 *   unit at a time, round-robin over symbols in descending order of scaled
 *   frequency, never letting a frequency fall below 1.
 *
 * Ties in the descending order are resolved by ascending symbol index (a
 * stable sort), which is what the C references do and what numpy's argsort
 * does for alphabets of at most 16 symbols.
 * ---------------------------------------------------------------------- */
int orc_normalize(const uint64_t *raw, uint32_t alphabet, uint32_t precision_bits,
                  uint32_t *freq, uint32_t *cdf /* alphabet+1 */)
{
    if (!raw || !freq || !cdf) return ORC_ERR_NULL_PTR;
    if (alphabet == 0 || precision_bits == 0 || precision_bits > 20) return ORC_ERR_HEADER;
    const uint64_t M = 1ull << precision_bits;
    if (alphabet > M) return ORC_ERR_HEADER;

    double total = 0.0;
    uint64_t itotal = 0;
    for (uint32_t s = 0; s < alphabet; s++) itotal += raw[s] ? raw[s] : 1;
    total = (double)itotal;

    int64_t assigned = 0;
    for (uint32_t s = 0; s < alphabet; s++) {
        double r = (double)(raw[s] ? raw[s] : 1);
        int64_t v = (int64_t)(r / total * (double)M);
        if (v < 1) v = 1;
        freq[s] = (uint32_t)v;
        assigned += v;
    }

    int64_t residual = (int64_t)M - assigned;
    if (residual != 0) {
        uint32_t *order = (uint32_t *)malloc(sizeof(uint32_t) * alphabet);
        if (!order) return ORC_ERR_ALLOC;
        for (uint32_t s = 0; s < alphabet; s++) order[s] = s;
        /* stable, descending by freq */
        for (uint32_t i = 1; i < alphabet; i++) {
            uint32_t k = order[i];
            int64_t j = (int64_t)i - 1;
            while (j >= 0 && freq[order[j]] < freq[k]) { order[j + 1] = order[j]; j--; }
            order[j + 1] = k;
        }
        uint32_t at = 0;
        while (residual != 0) {
            int step = residual > 0 ? 1 : -1;
            if ((int64_t)freq[order[at]] + step >= 1) {
                freq[order[at]] = (uint32_t)((int64_t)freq[order[at]] + step);
                residual -= step;
            }
            at = (at + 1) % alphabet;
        }
        free(order);
    }

    cdf[0] = 0;
    for (uint32_t s = 0; s < alphabet; s++) cdf[s + 1] = cdf[s] + freq[s];
    return cdf[alphabet] == M ? ORC_OK : ORC_ERR_HEADER;
}

/* slot -> symbol table, 2^p entries.  core/rans.py:356-364. */
int orc_build_lut(const uint32_t *cdf, uint32_t alphabet, uint32_t precision_bits, uint16_t *lut)
{
    if (!cdf || !lut) return ORC_ERR_NULL_PTR;
    for (uint32_t s = 0; s < alphabet; s++)
        for (uint32_t k = cdf[s]; k < cdf[s + 1]; k++) lut[k] = (uint16_t)s;
    (void)precision_bits;
    return ORC_OK;
}

/* ------------------------------------------------------------------------
 * Decode one block of the reference byte-renormalised wire format
 *   [1 B state_len][state, big-endian][renormalisation bytes]
 * Restates core/rans.py:368-419 (eoq_rans_v2.c:307-351 for p <= 16).
 * The state is 64-bit so precision up to 20 bits behaves as in Python.
 * An empty block or n == 0 decodes to nothing (rans.py:378-379).
 * ---------------------------------------------------------------------- */
int orc_decode_block(const uint32_t *freq, const uint32_t *cdf, const uint16_t *lut,
                     uint32_t precision_bits, const uint8_t *data, size_t len,
                     uint32_t n, uint32_t *out)
{
    if (n == 0 || len == 0) return ORC_OK;
    if (!freq || !cdf || !lut || !data || !out) return ORC_ERR_NULL_PTR;
    uint32_t state_len = data[0];
    if ((size_t)1 + state_len > len) return ORC_ERR_CORRUPT;   /* eoq_rans_v2.c:392 */
    uint64_t x = 0;
    for (uint32_t i = 0; i < state_len; i++) x = (x << 8) | data[1 + i];
    const uint8_t *stream = data + 1 + state_len;
    size_t pos = 0, end = len - 1 - state_len;
    const uint64_t mask = (1ull << precision_bits) - 1;
    const uint64_t low = 1ull << (precision_bits + 8);
    for (uint32_t i = 0; i < n; i++) {
        uint64_t slot = x & mask;
        uint32_t s = lut[slot];
        x = (uint64_t)freq[s] * (x >> precision_bits) + slot - cdf[s];
        while (x < low && pos < end) x = (x << 8) | stream[pos++];
        out[i] = s;
    }
    return ORC_OK;
}

/* ------------------------------------------------------------------------
 * Encode one block.  Restates core/rans.py:210-276: symbols visited last to
 * first, state starts at 2^(p+8), bytes pushed while x >= freq << 16, final
 * state written big-endian with exactly the bytes it needs behind a length
 * byte, pushed bytes reversed.  Returns the encoded length, or a negative
 * error.  `cap` must be at least 9 + 3*n bytes to be safe.
 * ---------------------------------------------------------------------- */
long orc_encode_block(const uint32_t *freq, const uint32_t *cdf, uint32_t precision_bits,
                      const uint32_t *syms, uint32_t n, uint8_t *out, size_t cap)
{
    if (n == 0) return 0;                                   /* rans.py:226-227 */
    if (!freq || !cdf || !syms || !out) return ORC_ERR_NULL_PTR;
    size_t tmp_cap = (size_t)n * 3 + 16, tmp_len = 0;
    uint8_t *tmp = (uint8_t *)malloc(tmp_cap);
    if (!tmp) return ORC_ERR_ALLOC;
    uint64_t x = 1ull << (precision_bits + 8);
    for (uint32_t i = n; i-- > 0;) {
        uint32_t s = syms[i];
        uint64_t f = freq[s], c = cdf[s];
        uint64_t x_max = f << 16;
        while (x >= x_max) {
            if (tmp_len == tmp_cap) { free(tmp); return ORC_ERR_TOO_SMALL; }
            tmp[tmp_len++] = (uint8_t)(x & 0xFF);
            x >>= 8;
        }
        x = (x / f << precision_bits) + (x % f) + c;
    }
    uint8_t st[8];
    uint32_t st_len = 0;
    for (uint64_t v = x; v > 0; v >>= 8) st[st_len++] = (uint8_t)(v & 0xFF);
    size_t total = 1 + st_len + tmp_len;
    if (total > cap) { free(tmp); return ORC_ERR_TOO_SMALL; }
    out[0] = (uint8_t)st_len;
    for (uint32_t i = 0; i < st_len; i++) out[1 + i] = st[st_len - 1 - i];
    for (size_t i = 0; i < tmp_len; i++) out[1 + st_len + i] = tmp[tmp_len - 1 - i];
    free(tmp);
    return (long)total;
}

/* ------------------------------------------------------------------------
 * Blocked decode over an offset table.  Restates
 * core/rans_blocked.py:124-145: block i holds symbols
 * [i*block, min((i+1)*block, n)) and bytes [offsets[i], offsets[i+1]) -- the
 * last block runs to the end of the data.  `raw_freq` is the un-normalised
 * table carried by BlockedRANSData; it is normalised here as the decoder's
 * constructor does (rans.py:349).
 * ---------------------------------------------------------------------- */
int orc_decode_blocked(const uint64_t *raw_freq, uint32_t alphabet, uint32_t precision_bits,
                       const uint8_t *data, size_t data_len,
                       const uint32_t *offsets, uint32_t num_blocks,
                       uint32_t block_size, uint32_t n, uint32_t *out)
{
    if (n == 0) return ORC_OK;
    if (!raw_freq || !data || !offsets || !out) return ORC_ERR_NULL_PTR;
    uint32_t *freq = (uint32_t *)malloc(sizeof(uint32_t) * alphabet);
    uint32_t *cdf = (uint32_t *)malloc(sizeof(uint32_t) * (alphabet + 1));
    uint16_t *lut = (uint16_t *)malloc(sizeof(uint16_t) << precision_bits);
    int rc = ORC_ERR_ALLOC;
    if (freq && cdf && lut) {
        rc = orc_normalize(raw_freq, alphabet, precision_bits, freq, cdf);
        if (rc == ORC_OK) rc = orc_build_lut(cdf, alphabet, precision_bits, lut);
        for (uint32_t b = 0; rc == ORC_OK && b < num_blocks; b++) {
            size_t lo = offsets[b];
            size_t hi = (b + 1 < num_blocks) ? offsets[b + 1] : data_len;
            if (hi < lo || hi > data_len) { rc = ORC_ERR_CORRUPT; break; }
            uint32_t first = b * block_size;
            uint32_t cnt = n - first < block_size ? n - first : block_size;
            rc = orc_decode_block(freq, cdf, lut, precision_bits, data + lo, hi - lo, cnt, out + first);
        }
    }
    free(freq); free(cdf); free(lut);
    return rc;
}

/* ------------------------------------------------------------------------
 * Tensor-level decode of the C payload
 *   [u16 freq x A][u32 block_offsets x B][blocks]
 * with the checks and error codes of eoq_rans_v2.c:577-782 and :482-498.
 * header[7] = {original_type, num_blocks, freq_table_size, precision_bits,
 *              rans_block_size, compressed_size, uncompressed_size}.
 * Output is one byte per symbol (eoq_rans_v2.c:343).
 * ---------------------------------------------------------------------- */
int orc_decode_c_payload(const uint32_t *header, const uint8_t *compressed, size_t comp_size,
                         uint8_t *output, size_t out_cap)
{
    if (!header || !compressed || !output) return ORC_ERR_NULL_PTR;
    uint32_t alphabet = header[2], p = header[3], block = header[4];
    uint32_t csize = header[5], usize = header[6];
    if (usize == 0) return ORC_OK;
    if (alphabet == 0 || alphabet > 4096) return ORC_ERR_HEADER;
    if (p == 0 || p > 16) return ORC_ERR_HEADER;
    if (block == 0) return ORC_ERR_HEADER;
    if ((uint64_t)csize < (uint64_t)alphabet * 2 + 4) return ORC_ERR_HEADER;
    if (out_cap < usize) return ORC_ERR_TOO_SMALL;
    if (comp_size < csize) return ORC_ERR_CORRUPT;
    uint32_t nb = (usize + block - 1) / block;
    uint64_t meta = (uint64_t)alphabet * 2 + (uint64_t)nb * 4;
    if (meta > csize) return ORC_ERR_CORRUPT;

    uint64_t *raw = (uint64_t *)malloc(sizeof(uint64_t) * alphabet);
    uint32_t *offs = (uint32_t *)malloc(sizeof(uint32_t) * nb);
    uint32_t *sym = (uint32_t *)malloc(sizeof(uint32_t) * usize);
    int rc = ORC_ERR_ALLOC;
    if (raw && offs && sym) {
        for (uint32_t s = 0; s < alphabet; s++) {
            uint16_t v; memcpy(&v, compressed + 2 * (size_t)s, 2); raw[s] = v;
        }
        memcpy(offs, compressed + (size_t)alphabet * 2, (size_t)nb * 4);
        rc = orc_decode_blocked(raw, alphabet, p, compressed + meta, csize - (uint32_t)meta,
                                offs, nb, block, usize, sym);
        if (rc == ORC_OK) for (uint32_t i = 0; i < usize; i++) output[i] = (uint8_t)sym[i];
    }
    free(raw); free(offs); free(sym);
    return rc;
}

/* ------------------------------------------------------------------------
 * INT4 dequantise + linear, the composition the fused GPU kernel replaces:
 * core/quantized_linear.py:189-228 (unpack low nibble first, value-7, scale
 * indexed over the FLATTENED weight, i // group) followed by F.linear.
 * Accumulates in double; returns float.  x is [batch, K], y is [batch, N].
 * ---------------------------------------------------------------------- */
void orc_int4_linear(const uint8_t *packed /* [N, ceil(K/2)] */, const float *scales,
                     uint32_t N, uint32_t K, uint32_t group,
                     const float *x, uint32_t batch, const float *bias, float *y)
{
    size_t row_bytes = ((size_t)K + 1) / 2;
    for (uint32_t b = 0; b < batch; b++) {
        for (uint32_t r = 0; r < N; r++) {
            double acc = 0.0;
            for (uint32_t c = 0; c < K; c++) {
                uint8_t byte = packed[r * row_bytes + c / 2];
                int code = (int)((c & 1) ? (byte >> 4) : (byte & 0x0F)) - 7;
                size_t flat = (size_t)r * K + c;
                acc += (double)((float)code * scales[flat / group]) * (double)x[(size_t)b * K + c];
            }
            if (bias) acc += bias[r];
            y[(size_t)b * N + r] = (float)acc;
        }
    }
}

/* ------------------------------------------------------------------------
 * Scalar decode of the product's tiled device layout (the checker for the
 * host-side tile encoder and for the GPU tile decoder).  No reference
 * counterpart: the layout is this project's own; what it must reproduce is the
 * symbol matrix, which the reference decoders pin.
 *
 * Tile bytes: 32 x u32 initial states, then rows of 32 x u16 words; lane l owns
 * G consecutive rows row0 + l*G + j and reads column l of the word rows.  Step:
 *   e = table[x & (2^p - 1)];  x = (e >> 23) * (x >> p) + (e & bias_mask);
 *   symbols = (e >> (23 - G*bits)) fields;  if x < 2^16: x = x << 16 | next word.
 * desc[t] = {row0, col0, ncols, seg, off64, len64}.  Byte b of tile t is at
 * stream[t * head_bytes + b] for b < head_bytes and at
 * stream[64 * off64 + b - head_bytes] from there on.  out is [rows, cols] bytes.
 * ---------------------------------------------------------------------- */
int orc_decode_tiles(const uint32_t *table, uint32_t p, uint32_t G, uint32_t bits,
                     const uint32_t *desc, uint32_t ntiles, const uint8_t *stream, size_t stream_bytes,
                     uint32_t head_bytes, uint32_t rows, uint32_t cols, uint8_t *out)
{
    if (!table || !desc || !stream || !out) return ORC_ERR_NULL_PTR;
    const uint32_t shift = 23 - G * bits, bias_mask = (1u << shift) - 1, fmask = (1u << bits) - 1;
    const uint32_t mask = (1u << p) - 1;
    for (uint32_t t = 0; t < ntiles; t++) {
        const uint32_t *d = desc + 6 * (size_t)t;
        const size_t head = (size_t)t * head_bytes, tail = ((size_t)d[4] << 6) - head_bytes;
#define ORC_TILE_AT(b) ((b) < head_bytes ? head + (b) : tail + (b))
        if (ORC_TILE_AT((size_t)0) + 128 > stream_bytes) return ORC_ERR_CORRUPT;
        for (uint32_t l = 0; l < 32; l++) {
            uint32_t x;
            memcpy(&x, stream + ORC_TILE_AT((size_t)4 * l), 4);
            size_t k = 0;
            for (uint32_t c = 0; c < d[2]; c++) {
                uint32_t e = table[x & mask];
                x = (e >> 23) * (x >> p) + (e & bias_mask);
                for (uint32_t j = 0; j < G; j++) {
                    uint32_t r = d[0] + l * G + j;
                    if (r < rows) out[(size_t)r * cols + d[1] + c] = (uint8_t)((e >> (shift + bits * j)) & fmask);
                }
                if (x < 65536u) {
                    size_t at = ORC_TILE_AT(128 + (k * 32 + l) * 2);
                    if (at + 2 > stream_bytes) return ORC_ERR_CORRUPT;
                    uint16_t w;
                    memcpy(&w, stream + at, 2);
                    x = (x << 16) | w;
                    k++;
                }
            }
        }
#undef ORC_TILE_AT
    }
    return ORC_OK;
}
