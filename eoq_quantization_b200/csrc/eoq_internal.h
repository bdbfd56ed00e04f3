// Internal declarations shared by the host codec, the kernels and the C ABI.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <functional>
#include <vector>

#include <vector_types.h>

#include "../../include/eoq_b200.h"

// Exported for this project's own benchmarks and tests, not part of the public interface:
// eoq_b200_tune sets a diagnostic knob and returns 0 if the key is known --
//   "gemv_ctas_per_sm" (0 = as many CTAs of the one-tile-per-warp GEMV kernel as fit on an SM),
//   "gemv_pairs" (1 = 4-bit weights with three symbols per step run through the kernel that decodes two tiles per
//                 warp, the default; 0 = always the one-tile-per-warp kernel),
//   "gemm_warps" (warps per CTA of the tensor-core kernel, 2..16; 0 = as many as fit),
//   "pdl" (1 = programmatic stream serialisation for the fused kernels, the default; 0 = plain launches),
//   "v1_lanes" (1 = the lane-per-block wire-format decoder, the default; 0 = the one-thread-per-block kernel);
// eoq_b200_launch_count is the number of kernels this library has launched since it was loaded.
extern "C" int eoq_b200_tune(const char *key, int value);
extern "C" uint64_t eoq_b200_launch_count(void);
struct eoq_b200_weight;
extern "C" uint64_t eoq_b200_weight_read(eoq_b200_weight *w, int what, void *host, uint64_t capacity);   // test hook, see abi.cu

namespace eoq {

// ---------------------------------------------------------------------------
// Tiled device layout ("v2").
//
// A weight matrix [N, K] is cut into tiles of (32*G rows) x (ncols columns).
// One warp decodes one tile; lane l owns rows row0 + l*G .. row0 + l*G + G-1
// and walks the tile's columns left to right.  Each rANS step decodes ONE joint
// symbol holding the G weights of the lane's rows at the current column:
//     sym = n_0 | n_1 << bits | ... | n_{G-1} << (G-1)*bits.
// Every lane has its own rANS stream: 32-bit state in [2^16, 2^32), 16-bit
// renormalisation words, at most one word per step (precision <= 16).
//
// Stream: [heads: tile t's first head_bytes at t * head_bytes][tails, packed][padding]; head_bytes is 0, 1024
// or 2048 and never more than the shortest tile, so the start of every tile is addressable from its index
// alone and only the tail needs the descriptor.
//
// Tile bytes:  [32 x u32 initial states][rows of 32 x u16]
// where row k holds, for lane l, that lane's k-th renormalisation word; lanes
// that need fewer words than the longest lane are padded with zeros, and the
// row count is even so every tile starts on a 128-byte boundary.
//
// Table entry (one 32-bit word per slot, 2^p slots):
//     [31:23] freq (1..511)   [22:23-G*bits] sym   [low bits] slot - cum(sym)
// so that one shared-memory load yields everything a step needs, and the INT4
// fields sit in float mantissa bits (see kernels.cu).
// ---------------------------------------------------------------------------
struct TileDesc {
    uint32_t row0;    // first row of the tile (multiple of 32*G)
    uint32_t col0;    // first column
    uint32_t ncols;   // columns (= rANS steps per lane), multiple of 16
    uint32_t seg;     // column-segment index (same for all row blocks); top bit: kTileDirectFlag
    uint32_t off64;   // byte offset in the stream of the tile's tail (its bytes past head_bytes), divided by 64
    uint32_t len64;   // bytes of the whole tile (head + tail), divided by 64
};

constexpr uint32_t kMaxFreq = 511;
constexpr uint32_t kMaxRingDrift = 31;           // rows the lanes of a ring-mode tile may be apart at any step
constexpr uint32_t kTileDirectFlag = 0x80000000u; // set in TileDesc::seg when the tile breaks that bound
constexpr uint32_t kColGranule = 16;   // tile column boundaries are multiples of this

struct TiledWeights {
    uint32_t N = 0, K = 0, Npad = 0, G = 0, bits = 0, p = 0, group = 0, kind = 0;
    uint32_t alphabet = 0;       // (1 << bits*G) slots in the joint symbol space
    uint32_t nrb = 0, nseg = 0;
    uint32_t max_drift = 0;      // largest distance (rows) between lanes' read positions in any tile
    uint32_t head_bytes = 0;     // bytes of every tile kept in the fixed-stride head region of the stream
    std::vector<uint32_t> table;     // 1 << p entries
    std::vector<TileDesc> tiles;     // nrb * nseg
    std::vector<uint32_t> seg_start; // nseg + 1 column boundaries
    std::vector<uint8_t>  stream;    // heads, tails, then 4096 bytes of padding (read-ahead never leaves it)
};

// Host codec (rans_host.cpp) -------------------------------------------------

// Reference normalisation (core/rans.py:85-153; stable descending order as
// eoq_rans_v2.c:78-141).  raw has `alphabet` entries; freq/cdf are resized.
eoq_error_t normalize_reference(const uint32_t *raw, uint32_t alphabet, uint32_t p,
                                std::vector<uint32_t> &freq, std::vector<uint32_t> &cdf);

// Wire-format ("v1") block encoder, byte-identical to core/rans.py:210-276.
void encode_block_v1(const uint32_t *freq, const uint32_t *cdf, uint32_t p,
                     const uint32_t *syms, uint32_t n, std::vector<uint8_t> &out);

// fn(0) ... fn(n - 1) on the host's cores (at most 64 threads, joined before it returns).
void parallel_for(size_t n, const std::function<void(size_t)> &fn);

// The pieces of build_tiled that do not touch the symbols, shared with the device-side tile encoder: geometry
// (padded rows, row blocks, column segments, tile descriptors without sizes), joint-symbol frequencies and decode table
// from the joint symbols' counts, and the stream layout (head_bytes, every off64, total bytes) from the tiles' len64.
eoq_error_t tiled_geometry(uint32_t N, uint32_t K, uint32_t bits, uint32_t G, uint32_t p, uint32_t group, uint32_t kind,
                           uint32_t target_tiles, TiledWeights &out);
eoq_error_t tiled_table(const std::vector<uint64_t> &count, TiledWeights &out, std::vector<uint32_t> &freq, std::vector<uint32_t> &cum);
eoq_error_t tiled_layout(TiledWeights &out, size_t &total);

// Build the tiled layout from one symbol per byte, row-major [N, K].
eoq_error_t build_tiled(const uint8_t *symbols, uint32_t N, uint32_t K, uint32_t bits, uint32_t G,
                        uint32_t p, uint32_t group, uint32_t kind, uint32_t target_tiles,
                        uint8_t pad_symbol, TiledWeights &out);

// Kernels (kernels.cu) --------------------------------------------------------

struct V1Table {          // wire-format decode table entry, one per slot
    uint32_t freq;        // 1..65536
    uint32_t sym_bias;    // sym << 16 | (slot - cum)
};

constexpr uint32_t kMaxPeers = 8;

struct GemvArgs {
    const uint32_t *table;
    const TileDesc *tiles;
    const uint8_t  *stream;
    const uint16_t *scales;     // fp16 bits, [N * K/group]
    const float    *centroids;  // polar: 32 floats, else null
    const void     *x;          // [batch, K]
    void           *y;          // [batch, N]
    const float    *bias;       // [N] or null
    float          *partials;   // [nseg][Npad][BT]
    uint32_t       *counters;   // [nrb], zero on entry, zero on exit
    uint32_t       *status;     // one word, set nonzero if a bounded wait expired
    uint32_t N, K, Npad, group, p, ntiles, nseg, batch;
    int x_dtype, y_dtype;
    // Pair kernel: row blocks, bytes of one staged-tile buffer (longest tile + one row, rounded to 128) and the
    // widest column segment; zero if the caller has not worked them out (the ring kernel is used then).
    uint32_t nrb, stage_bytes, max_ncols;
    uint32_t head_bytes;        // bytes of every tile in the fixed-stride head region of the stream (TiledWeights::head_bytes)
    float *pair_partials;       // pair kernel: partial rows [slots][Npad][BT], every word 0xFFFFFFFF between launches; null: meet through `partials` with a fence
    const uint2 *scales_t;      // [K/group][Npad/3] words {s0 | s1 << 16, s2}: the fp16 scales of rows 3i..3i+2, zero past N; or null
    // Fused all-gather of row-sharded outputs (world > 1): a lane's finished rows go into this rank's own full-size
    // output and, as 8-byte words, into every peer's receive buffer (plain stores over NVLink; an aligned 8-byte store
    // arrives whole, so the epoch inside the word is the flag).  16-bit outputs: one word carries the `gather_g` rows of a
    // lane, {v0 | v1 << 16, v2 | (epoch & 0xFFFF) << 16}; fp32 outputs: one word per value, {bits, epoch}.  Word index in a
    // receive buffer: (b * world + sender) * words_per_rank + (local row / gather_g, or local row for fp32), with
    // words_per_rank = Npad / gather_g (N for fp32).  The same kernel then waits, bounded by gather_limit clock ticks,
    // for the words of the other ranks and unpacks them into its output, so the full vector is complete when the
    // kernel is; the CTA that finishes last advances the slot's epoch.
    uint32_t world, rank;        // world <= 1: plain output into y
    uint32_t row_offset, n_total;// this shard's first row and the full row count: y index = b * n_total + row_offset + r
    uint64_t *peer_ll[kMaxPeers];      // the slot's receive buffer on each rank, 8-byte words ([rank]: this rank's own)
    uint32_t *gather_epoch;            // local: gathers this slot has completed; this launch sends epoch + 1
    uint32_t *gather_done;             // local: CTAs of this launch that have finished unpacking
    uint32_t *gather_status;           // local: set nonzero when the wait for a peer gave up
    uint32_t gather_g;                 // rows per lane of this weight's layout
    long long gather_limit;            // clock ticks the wait for the peers may take
};

struct DecodeArgs {
    const uint32_t *table;
    const TileDesc *tiles;
    const uint8_t  *stream;
    const uint16_t *scales;
    const float    *centroids;  // unused for INT4
    uint32_t       *status;
    uint8_t        *out_sym;    // packed nibbles [N, K/2] or bytes [N, K], or null
    void           *out_deq;    // [N, K] or null
    uint32_t N, K, group, p, ntiles;
    uint32_t head_bytes;
    int packed, out_dtype;
    // the pair layout's extras (4-bit weights, three codes per step): set, they let the dequantised matrix come from
    // the two-tiles-per-warp kernel
    const uint2 *scales_t = nullptr;      // [K / group][Npad / 3] {s0 | s1 << 16, s2}
    uint32_t nseg = 0, nrb = 0, Npad = 0, stage_bytes = 0;
};

int  device_sm_count();
// Each returns a cudaError_t as int; launches are asynchronous on `stream`.
int launch_gemv(const GemvArgs &a, uint32_t G, uint32_t bits, uint32_t kind, void *stream);
int launch_decode_tiles(const DecodeArgs &a, uint32_t G, uint32_t bits, uint32_t kind, void *stream);
int launch_decode_v1(const uint8_t *d_stream, const uint32_t *d_offsets, const uint32_t *d_sizes,
                     const V1Table *d_table, void *d_out, int out_elem_bytes, uint32_t nblocks,
                     uint32_t block_size, uint32_t total, uint32_t p, uint32_t alphabet, void *stream);
void set_v1_lanes(int v);
bool v1_lanes_enabled();

// One tensor of a batched wire-format decode (decode_v1_lanes_kernel); lives in device memory during the launch.
// All pointers are device pointers.  Either `freq` (normalised frequencies, u32 x alphabet: the kernel builds its
// table from them) or `table` (a caller's slot table in the reference's {symbol, freq, cum} form) is set.
struct V1Task {
    const uint8_t  *stream;
    const uint32_t *offsets, *sizes;   // per block: first byte in `stream`, byte count
    const uint32_t *freq;
    const void     *table;
    void           *out;
    uint32_t nblocks, block_size, total, p, alphabet, out_elem_bytes;
    uint32_t sym_bits, packed, first_cta, pad_;   // filled by v1_task_prepare / v1_plan_ctas
};
static_assert(sizeof(V1Task) % 4 == 0 && sizeof(V1Task) <= 256 * 4, "copied into shared memory one word per thread");
bool   v1_task_prepare(V1Task &t);
size_t v1_task_smem(const V1Task &t, uint32_t warps);
uint32_t v1_plan_ctas(V1Task *tasks, uint32_t ntasks, uint32_t &warps_per_cta, size_t &smem);
int launch_decode_v1_lanes(const V1Task *d_tasks, const uint32_t *d_cta_task, uint32_t grid, uint32_t warps_per_cta, size_t smem,
                           void *stream);
int launch_decode_v1_syminfo(const uint8_t *d_stream, const uint32_t *d_offsets, const uint32_t *d_sizes,
                             const eoq_sym_info_packed *d_info, uint8_t *d_out, uint32_t nblocks,
                             uint32_t block_size, uint32_t total, uint32_t p, void *stream);
int launch_decode_v1_resume(const uint8_t *d_block, uint32_t stream_end, const V1Table *d_table,
                            uint32_t *d_state_pos /* [2]: state, pos */, uint8_t *d_out, uint32_t count,
                            uint32_t p, void *stream);
// GEMV on QuantizedLinear's in-memory form (packed codes, fp16 scales): see gemv_packed_kernel.
struct PackedGemvArgs {
    const uint8_t *packed;      // [N][row_bytes]
    const uint16_t *scales;     // fp16 bits, [N][K / group]
    const void *x;              // [batch][K]
    const uint16_t *xsplit;     // fp32 activations on the tensor cores: fp16 bits [2][batch][K], the nearest fp16 and the nearest to the remainder
    void *y;                    // [batch][N]
    const float *bias;          // [N] or null
    uint32_t N, K, group, row_bytes, batch, bits;
    int x_dtype, y_dtype;
};
struct PolarCodesArgs {
    const uint8_t *codes;       // [N][K], one centroid index per byte
    const uint16_t *norms;      // fp16 bits, [N][K / block]
    const float *centroids;     // [entries]
    const float *xrot;          // [batch][K]: activations rotated per block and divided by sqrt(block)
    const uint16_t *xsplit;     // or (tensor-core form) fp16 bits [2][batch][K]: the fp16 nearest to each rotated activation, then the remainder
    void *y;                    // [batch][N]
    const float *bias;          // [N] or null
    uint32_t N, K, block_shift, batch, entries;
    int y_dtype;
};
int launch_gemv_polar_codes(const PolarCodesArgs &a, void *stream);
int launch_polar_rotate(const void *x, int x_dtype, uint32_t K, uint32_t block_shift, uint32_t batch, float *out32, uint16_t *out_split, void *stream);
uint32_t gemv_packed_rows(const PackedGemvArgs &a);
void set_packed_warps(int v);
void set_dequant_vec(int v);
int launch_gemv_packed(const PackedGemvArgs &a, void *stream);
int launch_dequant_packed(const uint8_t *packed, const uint16_t *scales, uint32_t K, uint32_t row_bytes, uint32_t bits,
                          uint32_t group, uint32_t row_lo, uint32_t row_hi, void *out, int out_dtype, void *stream);
int launch_gemm_tc(const uint32_t *table, const TileDesc *tiles, const uint8_t *stream, const uint2 *scales_t, const void *x,
                   void *xhalf, float *partials, uint32_t *counters, void *y, const float *bias, uint32_t *status, uint32_t N,
                   uint32_t K, uint32_t group, uint32_t p, uint32_t nseg, uint32_t nrb, uint32_t head_bytes, uint32_t M, int x_dtype, int y_dtype,
                   void *stream_);
uint32_t gemm_grid(uint32_t nrb, uint32_t nseg);
size_t gemm_partial_bytes(uint32_t grid, uint32_t m);
constexpr uint32_t kGemmRowsPerPass = 512;      // activation rows one launch of the tensor-core kernel takes
size_t gemv_smem_bytes(uint32_t K, uint32_t p, uint32_t bt, uint32_t kind);
uint64_t launch_counter();
void set_gemv_ctas_per_sm(int v);
void set_gemm_warps(int v);
void set_pdl(int v);
void set_gemv_pairs(int v);
uint32_t pair_partial_slots(uint32_t nrb, uint32_t nseg);
bool gemv_takes_pairs(const GemvArgs &a, uint32_t G, uint32_t bits, uint32_t kind);
int launch_gather_wait(const GemvArgs &a, void *stream);

// Device-side tile encoder (kernels.cu): joint-symbol counts; per-tile encode into a scratch of max_ncols x 32 words
// per tile; scatter into the laid-out stream.  `sym` is one symbol per byte, row-major [N, K], K a multiple of 16.
struct TileEncodeArgs {
    const uint8_t *sym;
    const TileDesc *tiles;        // row0, col0, ncols of every tile
    const uint2 *freq_cum;        // per joint symbol {freq, cum}
    uint32_t *scratch;            // [ntiles][max_ncols][32] {word | step << 16}
    uint32_t *state, *count;      // [ntiles][32]
    uint2 *info;                  // [ntiles] {rows of 32 words (even), drift}
    uint32_t N, K, G, bits, p, ntiles, max_ncols;
};
struct TileScatterArgs {
    const TileDesc *tiles;        // with off64 and len64
    const uint32_t *scratch, *state, *count;
    uint8_t *stream;              // zero-filled
    uint32_t head_bytes, ntiles, max_ncols;
};
int launch_tile_hist(const uint8_t *sym, uint32_t N, uint32_t K, uint32_t Npad, uint32_t G, uint32_t bits, unsigned long long *counts,
                     void *stream);
int launch_tile_encode(const TileEncodeArgs &a, void *stream);
int launch_tile_scatter(const TileScatterArgs &a, void *stream);

}  // namespace eoq
