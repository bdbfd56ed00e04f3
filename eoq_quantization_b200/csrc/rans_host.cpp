// Host side of the codec: table normalisation, the wire-format block encoder and
// the load-time re-tiling of a weight matrix into the device layout.  Nothing
// here decodes: decoding happens on the GPU only.
#include "eoq_internal.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <functional>
#include <queue>
#include <thread>

namespace eoq {

// ---------------------------------------------------------------------------
// Reference normalisation.  Behaviour of core/rans.py:85-153: zero counts are
// raised to 1, counts are scaled by 2^p/total in double precision and truncated,
// raised to 1 again, and the residual is dealt out one unit at a time over the
// symbols in descending order of scaled frequency (ties: lower symbol first,
// as the C decoders do, eoq_rans_v2.c:108-121), never going below 1.
// ---------------------------------------------------------------------------
eoq_error_t normalize_reference(const uint32_t *raw, uint32_t alphabet, uint32_t p,
                                std::vector<uint32_t> &freq, std::vector<uint32_t> &cdf)
{
    if (!raw) return EOQ_ERR_NULL_PTR;
    if (alphabet == 0 || p == 0 || p > 16) return EOQ_ERR_INVALID_HEADER;
    const uint64_t M = 1ull << p;
    if (alphabet > M) return EOQ_ERR_INVALID_HEADER;
    freq.assign(alphabet, 0);
    cdf.assign(alphabet + 1, 0);

    uint64_t total = 0;
    for (uint32_t s = 0; s < alphabet; s++) total += raw[s] ? raw[s] : 1;
    const double dtotal = (double)total, dM = (double)M;
    int64_t sum = 0;
    for (uint32_t s = 0; s < alphabet; s++) {
        int64_t v = (int64_t)((double)(raw[s] ? raw[s] : 1) / dtotal * dM);
        freq[s] = (uint32_t)std::max<int64_t>(v, 1);
        sum += freq[s];
    }
    int64_t residual = (int64_t)M - sum;
    if (residual != 0) {
        std::vector<uint32_t> order(alphabet);
        for (uint32_t s = 0; s < alphabet; s++) order[s] = s;
        std::stable_sort(order.begin(), order.end(),
                         [&](uint32_t a, uint32_t b) { return freq[a] > freq[b]; });
        uint32_t at = 0;
        while (residual != 0) {
            const int step = residual > 0 ? 1 : -1;
            uint32_t &f = freq[order[at]];
            if ((int64_t)f + step >= 1) { f = (uint32_t)((int64_t)f + step); residual -= step; }
            at = (at + 1) % alphabet;
        }
    }
    for (uint32_t s = 0; s < alphabet; s++) cdf[s + 1] = cdf[s] + freq[s];
    return cdf[alphabet] == M ? EOQ_OK : EOQ_ERR_INVALID_HEADER;
}

// ---------------------------------------------------------------------------
// Wire-format block encoder: [1 B state_len][state big-endian][bytes].
// Symbols last to first; state starts at 2^(p+8); a byte is pushed while
// x >= freq << 16; pushed bytes are reversed (core/rans.py:229-276).
// ---------------------------------------------------------------------------
void encode_block_v1(const uint32_t *freq, const uint32_t *cdf, uint32_t p,
                     const uint32_t *syms, uint32_t n, std::vector<uint8_t> &out)
{
    out.clear();
    if (n == 0) return;
    std::vector<uint8_t> pushed;
    pushed.reserve(n);
    uint64_t x = 1ull << (p + 8);
    for (uint32_t i = n; i-- > 0;) {
        const uint64_t f = freq[syms[i]], c = cdf[syms[i]];
        const uint64_t limit = f << 16;
        while (x >= limit) { pushed.push_back((uint8_t)x); x >>= 8; }
        x = ((x / f) << p) + (x % f) + c;
    }
    uint8_t st[8];
    uint32_t len = 0;
    for (uint64_t v = x; v; v >>= 8) st[len++] = (uint8_t)v;
    out.reserve(1 + len + pushed.size());
    out.push_back((uint8_t)len);
    for (uint32_t i = len; i-- > 0;) out.push_back(st[i]);
    out.insert(out.end(), pushed.rbegin(), pushed.rend());
}

// ---------------------------------------------------------------------------
// Frequencies for the joint-symbol table of the tiled layout.  Only symbols
// that occur get a slot; each frequency is capped at kMaxFreq so it fits the
// 9-bit field of the table entry; the residual goes where it saves most bits.
// If the cap leaves slots unused they stay unreachable (filled by the caller).
// ---------------------------------------------------------------------------
static eoq_error_t normalize_joint(const std::vector<uint64_t> &count, uint32_t p, std::vector<uint32_t> &freq)
{
    const uint64_t M = 1ull << p;
    const size_t A = count.size();
    freq.assign(A, 0);
    uint64_t total = 0, present = 0;
    for (uint64_t c : count) { total += c; present += c != 0; }
    if (present == 0) return EOQ_OK;
    if (present > M) return EOQ_ERR_UNSUPPORTED;
    uint64_t sum = 0;
    for (size_t s = 0; s < A; s++) {
        if (!count[s]) continue;
        uint64_t f = (uint64_t)((long double)count[s] * (long double)M / (long double)total);
        f = std::min<uint64_t>(std::max<uint64_t>(f, 1), kMaxFreq);
        freq[s] = (uint32_t)f;
        sum += f;
    }
    typedef std::pair<double, uint32_t> Item;
    if (sum < M) {
        std::priority_queue<Item> gain;   // bits saved by one more slot
        for (size_t s = 0; s < A; s++)
            if (count[s] && freq[s] < kMaxFreq)
                gain.push({(double)count[s] * std::log2((freq[s] + 1.0) / freq[s]), (uint32_t)s});
        while (sum < M && !gain.empty()) {
            const uint32_t s = gain.top().second;
            gain.pop();
            freq[s]++; sum++;
            if (freq[s] < kMaxFreq) gain.push({(double)count[s] * std::log2((freq[s] + 1.0) / freq[s]), s});
        }
    } else if (sum > M) {
        std::priority_queue<Item, std::vector<Item>, std::greater<Item>> cost;   // bits lost by one slot fewer
        for (size_t s = 0; s < A; s++)
            if (freq[s] > 1) cost.push({(double)count[s] * std::log2(freq[s] / (freq[s] - 1.0)), (uint32_t)s});
        while (sum > M && !cost.empty()) {
            const uint32_t s = cost.top().second;
            cost.pop();
            freq[s]--; sum--;
            if (freq[s] > 1) cost.push({(double)count[s] * std::log2(freq[s] / (freq[s] - 1.0)), s});
        }
        if (sum > M) return EOQ_ERR_UNSUPPORTED;
    }
    return EOQ_OK;
}

void parallel_for(size_t n, const std::function<void(size_t)> &fn)
{
    unsigned hw = std::thread::hardware_concurrency();
    size_t nt = std::min<size_t>(hw ? hw : 4, std::max<size_t>(n, 1));
    nt = std::min<size_t>(nt, 64);
    if (nt <= 1) { for (size_t i = 0; i < n; i++) fn(i); return; }
    std::atomic<size_t> next(0);
    std::vector<std::thread> pool;
    for (size_t t = 0; t < nt; t++)
        pool.emplace_back([&] { for (size_t i; (i = next.fetch_add(1)) < n;) fn(i); });
    for (auto &t : pool) t.join();
}

// Geometry of the tiled layout: padded rows, row blocks, column segments.
eoq_error_t tiled_geometry(uint32_t N, uint32_t K, uint32_t bits, uint32_t G, uint32_t p, uint32_t group, uint32_t kind,
                           uint32_t target_tiles, TiledWeights &out)
{
    if (N == 0 || K == 0) return EOQ_ERR_INVALID_HEADER;
    if (G < 1 || G > 3 || bits < 1 || bits * G > 12 || p < bits * G || p > 16) return EOQ_ERR_UNSUPPORTED;
    if (K % kColGranule || group == 0 || K % group || group % kColGranule) return EOQ_ERR_UNSUPPORTED;
    if ((uint64_t)N * K > (1ull << 34)) return EOQ_ERR_OVERFLOW;

    const uint32_t rows_per_tile = 32 * G;
    const uint32_t Npad = (N + rows_per_tile - 1) / rows_per_tile * rows_per_tile;
    const uint32_t nrb = Npad / rows_per_tile;
    const uint32_t units = K / kColGranule;
    uint32_t nseg = target_tiles / nrb;
    nseg = std::max<uint32_t>(1, std::min<uint32_t>(nseg, std::max<uint32_t>(1, units / 2)));      // tiles of at least 32 columns

    out = TiledWeights();
    out.N = N; out.K = K; out.Npad = Npad; out.G = G; out.bits = bits; out.p = p; out.group = group; out.kind = kind;
    out.alphabet = 1u << (bits * G);
    out.nrb = nrb; out.nseg = nseg;
    out.seg_start.resize(nseg + 1);
    for (uint32_t s = 0; s <= nseg; s++) out.seg_start[s] = (uint32_t)((uint64_t)s * units / nseg) * kColGranule;
    out.tiles.resize((size_t)nrb * nseg);
    for (size_t t = 0; t < out.tiles.size(); t++) {
        const uint32_t rb = (uint32_t)(t / nseg), seg = (uint32_t)(t % nseg);
        TileDesc &d = out.tiles[t];
        d.row0 = rb * rows_per_tile; d.col0 = out.seg_start[seg]; d.ncols = out.seg_start[seg + 1] - d.col0; d.seg = seg; d.off64 = 0; d.len64 = 0;
    }
    return EOQ_OK;
}

// Joint-symbol frequencies and the decode table from the counts of the joint symbols.
eoq_error_t tiled_table(const std::vector<uint64_t> &count, TiledWeights &out, std::vector<uint32_t> &freq, std::vector<uint32_t> &cum)
{
    eoq_error_t rc = normalize_joint(count, out.p, freq);
    if (rc != EOQ_OK) return rc;
    cum.assign(out.alphabet + 1, 0);
    for (uint32_t s = 0; s < out.alphabet; s++) cum[s + 1] = cum[s] + freq[s];
    const uint32_t M = 1u << out.p, sym_shift = 23 - out.bits * out.G;
    out.table.assign(M, (1u << 23));   // unreachable slots: freq 1, symbol 0, bias 0
    for (uint32_t s = 0; s < out.alphabet; s++)
        for (uint32_t k = 0; k < freq[s]; k++)
            out.table[cum[s] + k] = (freq[s] << 23) | (s << sym_shift) | k;
    return EOQ_OK;
}

// Stream layout from the tiles' byte counts (len64 set): [heads: ntiles x head_bytes][tails][padding].  The first
// head_bytes of every tile sit at a fixed stride, so a kernel can request them from the tile index alone, without a
// descriptor fetch in front; the rest of a tile (its tail) is packed behind and found through the descriptor.
// head_bytes is a whole number of kilobytes no longer than the shortest tile (two at most: enough to cover the
// descriptor's round trip).  Sets head_bytes and every off64; `total` is the stream's size with its 4096 bytes of padding.
eoq_error_t tiled_layout(TiledWeights &out, size_t &total)
{
    const size_t ntiles = out.tiles.size();
    size_t shortest = ~(size_t)0;
    for (size_t t = 0; t < ntiles; t++) shortest = std::min(shortest, (size_t)out.tiles[t].len64 << 6);
    const uint32_t H = shortest >= 2048 ? 2048u : shortest >= 1024 ? 1024u : 0u;
    out.head_bytes = H;
    total = ntiles * (size_t)H;
    for (size_t t = 0; t < ntiles; t++) {
        if ((total >> 6) > 0xFFFFFFFFull) return EOQ_ERR_OVERFLOW;
        out.tiles[t].off64 = (uint32_t)(total >> 6);
        total += ((size_t)out.tiles[t].len64 << 6) - H;
    }
    total += 4096;
    return EOQ_OK;
}

eoq_error_t build_tiled(const uint8_t *symbols, uint32_t N, uint32_t K, uint32_t bits, uint32_t G,
                        uint32_t p, uint32_t group, uint32_t kind, uint32_t target_tiles,
                        uint8_t pad_symbol, TiledWeights &out)
{
    (void)pad_symbol;
    if (!symbols) return EOQ_ERR_NULL_PTR;
    eoq_error_t rc = tiled_geometry(N, K, bits, G, p, group, kind, target_tiles, out);
    if (rc != EOQ_OK) return rc;
    const uint32_t Npad = out.Npad, nseg = out.nseg;

    // joint symbols, [Npad/G][K]
    const size_t njoint = (size_t)(Npad / G) * K;
    std::vector<uint16_t> joint(njoint);
    const uint32_t sym_mask = (1u << bits) - 1;
    parallel_for(Npad / G, [&](size_t rg) {
        uint16_t *dst = joint.data() + rg * K;
        for (uint32_t c = 0; c < K; c++) {
            uint32_t v = 0;
            for (uint32_t j = 0; j < G; j++) {
                const size_t r = rg * G + j;
                // rows past the end are never written back; they repeat real rows so that their lanes
                // consume words at the same rate as their neighbours
                const uint32_t n = symbols[(r < N ? r : r % N) * K + c] & sym_mask;
                v |= n << (bits * j);
            }
            dst[c] = (uint16_t)v;
        }
    });

    std::vector<uint64_t> count(out.alphabet, 0);
    {
        const size_t nchunks = 64;
        std::vector<std::vector<uint64_t>> part(nchunks, std::vector<uint64_t>(out.alphabet, 0));
        parallel_for(nchunks, [&](size_t ch) {
            const size_t lo = njoint * ch / nchunks, hi = njoint * (ch + 1) / nchunks;
            for (size_t i = lo; i < hi; i++) part[ch][joint[i]]++;
        });
        for (auto &pc : part) for (uint32_t s = 0; s < out.alphabet; s++) count[s] += pc[s];
    }
    std::vector<uint32_t> freq, cum;
    rc = tiled_table(count, out, freq, cum);
    if (rc != EOQ_OK) return rc;

    // encode every tile: 32 independent lane streams each
    const size_t ntiles = out.tiles.size();
    std::vector<std::vector<uint8_t>> tile_bytes(ntiles);
    std::vector<uint32_t> tile_drift(ntiles, 0);
    parallel_for(ntiles, [&](size_t t) {
        const uint32_t rb = (uint32_t)(t / nseg);
        const uint32_t col0 = out.tiles[t].col0, ncols = out.tiles[t].ncols;
        std::vector<uint16_t> words[32];
        std::vector<uint8_t> took(32 * (size_t)ncols, 0);    // took[l*ncols + c] = lane l reads a word after step c
        uint32_t state[32];
        size_t longest = 0;
        for (uint32_t l = 0; l < 32; l++) {
            const uint16_t *src = joint.data() + ((size_t)rb * 32 + l) * K + col0;
            uint64_t x = 1ull << 16;
            auto &w = words[l];
            w.reserve(ncols);
            for (uint32_t c = ncols; c-- > 0;) {
                const uint64_t f = freq[src[c]], cm = cum[src[c]];
                if (x >= (f << (32 - p))) { w.push_back((uint16_t)x); x >>= 16; took[l * (size_t)ncols + c] = 1; }
                x = ((x / f) << p) + (x % f) + cm;
            }
            state[l] = (uint32_t)x;
            longest = std::max(longest, w.size());
        }
        longest = (longest + 1) & ~(size_t)1;
        auto &tb = tile_bytes[t];
        tb.assign(128 + longest * 64, 0);
        std::memcpy(tb.data(), state, 128);
        uint16_t *rows = reinterpret_cast<uint16_t *>(tb.data() + 128);
        for (uint32_t l = 0; l < 32; l++) {
            const auto &w = words[l];
            for (size_t k = 0; k < w.size(); k++) rows[k * 32 + l] = w[w.size() - 1 - k];
        }
        // how far apart the lanes' read positions get; beyond the bound the tile is read without the ring
        uint32_t pos[32] = {0}, drift = 0;
        for (uint32_t c = 0; c < ncols; c++) {
            uint32_t lo = ~0u, hi = 0;
            for (uint32_t l = 0; l < 32; l++) {
                pos[l] += took[l * (size_t)ncols + c];
                lo = std::min(lo, pos[l]); hi = std::max(hi, pos[l]);
            }
            drift = std::max(drift, hi - lo);
        }
        tile_drift[t] = drift;
        if (drift > kMaxRingDrift) out.tiles[t].seg |= kTileDirectFlag;
        out.tiles[t].len64 = (uint32_t)(tb.size() >> 6);
    });
    for (uint32_t v : tile_drift) out.max_drift = std::max(out.max_drift, v);
    size_t total = 0;
    rc = tiled_layout(out, total);
    if (rc != EOQ_OK) return rc;
    const uint32_t H = out.head_bytes;
    out.stream.assign(total, 0);
    parallel_for(ntiles, [&](size_t t) {
        if (H) std::memcpy(out.stream.data() + t * (size_t)H, tile_bytes[t].data(), H);
        std::memcpy(out.stream.data() + ((size_t)out.tiles[t].off64 << 6), tile_bytes[t].data() + H, tile_bytes[t].size() - H);
    });
    return EOQ_OK;
}

}  // namespace eoq
