// sm_100a kernels of the EOQ hot path.
//
//   gemv_pairs_kernel     fused rANS decode -> unpack -> scale -> GEMV, INT4, 1..4 rows: two tiles per warp, staged whole
//   gemv_tiles_kernel     the same for every kind and 1..8 rows: one tile per warp through a word ring
//   gemm_tiles_kernel     fused rANS decode -> fp16 pieces -> tcgen05 MMA (TMEM accumulator), 9..128 rows
//   decode_tiles_kernel   rANS decode of the tiled layout to packed INT4 / bytes / dequantised matrix
//   decode_v1_kernel      decode of the reference wire format (one thread per independent block)
//
// The decode and GEMV kernels are integer/byte streaming kernels bounded by the SM's integer and
// shared-memory pipes and by HBM, not by tensor throughput; only the many-row case is a contraction.
#include "eoq_internal.h"

#include <algorithm>
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

namespace eoq {

static std::atomic<uint64_t> g_launches{0};
uint64_t launch_counter() { return g_launches.load(); }

int device_sm_count()
{
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

// Build-time tuning (defaults are what the committed measurements use).
#ifndef EOQ_GEMV_THREADS
#define EOQ_GEMV_THREADS 512
#endif
#ifndef EOQ_SHIFT_BY_MULHI
#define EOQ_SHIFT_BY_MULHI 0     // 1: do the two right shifts of a step as IMAD.HI (FMA pipe) instead of SHF (ALU pipe)
#endif
constexpr int kThreads = EOQ_GEMV_THREADS;

// ---------------------------------------------------------------------------
// Table-entry geometry for G weights of BITS bits per rANS step.
// ---------------------------------------------------------------------------
template <int G, int BITS>
struct Fmt {
    static constexpr int kSymBits = G * BITS;
    static constexpr int kSymShift = 23 - kSymBits;
    static constexpr uint32_t kBiasMask = (1u << kSymShift) - 1u;
    static constexpr uint32_t kFieldMask = (1u << BITS) - 1u;
    __host__ __device__ static constexpr int field_bit(int j) { return kSymShift + BITS * j; }
};

// INT4 weights are turned into floats without an integer->float conversion:
// the 4-bit field of the table entry sits in mantissa bits [b, b+4) of a float
// whose exponent is chosen so that the float equals 2^(23-b) + n exactly.
//   b >= 15: accumulate (2^(23-b) + n) * x and subtract (2^(23-b) + 7) * sum(x)
//            once per scale group (the product is exact in fp32, and the sums
//            cancel to ~2^-15 relative);
//   b <  15: the constant would swamp the sum, so subtract it first (exact).
// The same holds for fields of any width (2-, 3-, 8-bit symmetric codes: symbol = code + qmax, qmax = 2^(bits-1) - 1).
template <int B, int BITS = 4>
struct Int4Field {
    static constexpr uint32_t kMask = ((1u << BITS) - 1u) << B;
    static constexpr uint32_t kMagic = (uint32_t)(150 - B) << 23;       // exponent of 2^(23-B)
    static constexpr float kBase = (float)(1u << (23 - B));
    static constexpr float kQmax = (float)((1u << (BITS - 1)) - 1u);
    static constexpr float kOffset = kBase + kQmax;                     // the float that stands for code 0
    static constexpr bool kPreSubtract = B < 15;
    static constexpr float kCorr = kPreSubtract ? 0.0f : kOffset;
    // `magic` is kMagic held in a register: the mask is the instruction's one immediate, so with the
    // exponent in a register the extraction stays a single LOP3
    __device__ __forceinline__ static float value(uint32_t e, uint32_t magic)
    {
        float m = __uint_as_float((e & kMask) | magic);
        if (kPreSubtract) m -= kOffset;
        return m;
    }
    __device__ __forceinline__ static uint32_t magic_reg()
    {
        uint32_t m;
        asm volatile("mov.b32 %0, %1;" : "=r"(m) : "n"(kMagic));   // opaque to constant propagation
        return m;
    }
};

template <typename T> __device__ __forceinline__ float load_as_float(const void *p, size_t i);
template <> __device__ __forceinline__ float load_as_float<__half>(const void *p, size_t i) { return __half2float(reinterpret_cast<const __half *>(p)[i]); }
template <> __device__ __forceinline__ float load_as_float<__nv_bfloat16>(const void *p, size_t i) { return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]); }
template <> __device__ __forceinline__ float load_as_float<float>(const void *p, size_t i) { return reinterpret_cast<const float *>(p)[i]; }

__device__ __forceinline__ float load_x(const void *p, size_t i, int dtype)
{
    if (dtype == EOQ_B200_F16) return load_as_float<__half>(p, i);
    if (dtype == EOQ_B200_BF16) return load_as_float<__nv_bfloat16>(p, i);
    return load_as_float<float>(p, i);
}

__device__ __forceinline__ void store_y(void *p, size_t i, float v, int dtype)
{
    if (dtype == EOQ_B200_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else if (dtype == EOQ_B200_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float *>(p)[i] = v;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// A read-only global load that stays where it is written (volatile asm), for prefetching into registers.
__device__ __forceinline__ uint16_t ldg_u16_pinned(const uint16_t *p)
{
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint2 ldg_u32x2_pinned(const uint2 *p)
{
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// Geometry of the per-warp word ring (see "Streaming a tile's renormalisation words" below): rows of 32 x u16,
// filled in chunks, checked every kSync steps.  64 rows in four chunks is the least that covers the encoder's drift
// bound.
template <uint32_t ROWS, uint32_t CHUNK_ROWS, uint32_t SYNC>
struct RingGeom {
    static constexpr uint32_t kRows = ROWS, kChunkRows = CHUNK_ROWS, kChunks = ROWS / CHUNK_ROWS, kSync = SYNC;
    static constexpr uint32_t kBytes = ROWS * 64, kChunkBytes = CHUNK_ROWS * 64;
    static_assert(kMaxRingDrift + SYNC + 1 + CHUNK_ROWS <= ROWS, "ring too small for the drift bound");
    static_assert((ROWS & (ROWS - 1)) == 0, "ring positions are taken modulo a power of two");
};
using RingSmall = RingGeom<64, 16, 16>;

template <typename R>
__host__ __device__ inline size_t ring_smem_bytes(uint32_t warps) { return (size_t)warps * (R::kBytes + R::kChunks * 8) + R::kBytes; }

// Shared-memory carve-up of the fused kernel (bytes).
__host__ __device__ inline size_t smem_table_bytes(uint32_t p) { return (size_t)4 << p; }
template <typename R>
static size_t gemv_smem_bytes_for(uint32_t K, uint32_t p, uint32_t bt, uint32_t kind, uint32_t threads)
{
    size_t b = smem_table_bytes(p) + 16 + (size_t)K * bt * 4;      // table, its arrival barrier, x
    b += kind == EOQ_B200_KIND_Q5_POLAR ? 32 * 32 * 4 : (size_t)(K / 16) * bt * 4;
    return b + ring_smem_bytes<R>(threads / 32);
}
size_t gemv_smem_bytes(uint32_t K, uint32_t p, uint32_t bt, uint32_t kind) { return gemv_smem_bytes_for<RingSmall>(K, p, bt, kind, kThreads); }

// One rANS step: table lookup, state update; returns the entry.
__device__ __forceinline__ uint32_t rans_step(const uint32_t *tab, uint32_t &x, uint32_t mask, uint32_t p, uint32_t bias_mask)
{
    const uint32_t e = tab[x & mask];
#if EOQ_SHIFT_BY_MULHI
    x = __umulhi(e, 1u << 9) * __umulhi(x, 1u << (32 - p)) + (e & bias_mask);
#else
    x = (e >> 23) * (x >> p) + (e & bias_mask);
#endif
    return e;
}

// The same step with the INT4 fields of the entry turned into float bit patterns, written out
// instruction by instruction so that a step is exactly: AND, IMAD (address), LDS, 2 x SHR, AND, IMAD
// (state), and one LOP3 per field ((e & mask) | exponent, exponent in a register).
template <uint32_t MASK0, uint32_t MASK1, uint32_t MASK2>
__device__ __forceinline__ void rans_step_int4(uint32_t tab_addr, uint32_t &x, uint32_t mask, uint32_t p, uint32_t bias_mask,
                                               uint32_t mg0, uint32_t mg1, uint32_t mg2, uint32_t &m0, uint32_t &m1, uint32_t &m2)
{
    asm("{\n\t.reg .b32 s, e, q, f, b;\n\t"
        "and.b32 s, %0, %4;\n\t"
        "mad.lo.u32 s, s, 4, %5;\n\t"
        "ld.shared.u32 e, [s];\n\t"
#if EOQ_SHIFT_BY_MULHI
        "mul.hi.u32 q, %0, %14;\n\t"
        "mul.hi.u32 f, e, 512;\n\t"
#else
        "shr.u32 q, %0, %6;\n\t"
        "shr.u32 f, e, 23;\n\t"
#endif
        "and.b32 b, e, %7;\n\t"
        "mad.lo.u32 %0, f, q, b;\n\t"
        "lop3.b32 %1, e, %8, %11, 0xEA;\n\t"
        "lop3.b32 %2, e, %9, %12, 0xEA;\n\t"
        "lop3.b32 %3, e, %10, %13, 0xEA;\n\t}"
        : "+r"(x), "=r"(m0), "=r"(m1), "=r"(m2)
        : "r"(mask), "r"(tab_addr), "r"(p), "r"(bias_mask), "n"(MASK0), "n"(MASK1), "n"(MASK2), "r"(mg0), "r"(mg1), "r"(mg2), "r"(1u << (32u - p)));
}

// ---------------------------------------------------------------------------
// Streaming a tile's renormalisation words.
//
// Ring mode (the normal case): each warp owns a ring in shared memory (RingGeom: 64 or 128 rows
// of 32 x u16) filled by bulk asynchronous copies (cp.async.bulk, the 1-D TMA path) of four
// chunks, each completing on its own mbarrier.  Lane l reads column l; `koff` is 64 x the row
// of the word the lane currently holds in `w`, counted from the warp's first chunk so that
// ring position = koff mod ring bytes across tiles.  Every kSync steps the warp takes the min and
// max of koff over its lanes: chunks wholly below the min are refilled, and the chunk the
// fastest lane can reach before the next check is waited for.  The host encoder guarantees that
// lanes of a ring-mode tile never drift more than kMaxRingDrift rows apart, which is what makes
// four chunks enough; tiles that break the bound are flagged and read their words straight from
// global memory instead (direct mode).  Waits are bounded: on expiry a status word is set and
// the kernel carries on with whatever the ring holds, so it always terminates.
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t *status)
{
    for (uint32_t i = 0; i < (1u << 22); i++)
        if (mbar_test(bar, parity)) return;
    *status = 1u;   // gave up; the host turns this into an error
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
    return v;
}

// Where the bytes of one tile are: its first `hbytes` in the fixed-stride head region of the stream, the rest in
// its tail; `tail` is biased by -hbytes so that byte b of the tile is head[b] below hbytes and tail[b] from there on.
struct TileSrc {
    const uint8_t *head, *tail;
    uint32_t hbytes;
    __device__ __forceinline__ const uint8_t *at(uint32_t b) const { return b < hbytes ? head + b : tail + b; }
};
__device__ __forceinline__ TileSrc tile_src(const uint8_t *stream, uint32_t head_bytes, uint32_t t, const TileDesc &d)
{
    TileSrc s;
    s.head = stream + (size_t)t * head_bytes;
    s.tail = stream + ((size_t)d.off64 << 6) - head_bytes;
    s.hbytes = head_bytes;
    return s;
}

struct WordState {            // per lane
    uint32_t w;               // the lane's next unread word
    const uint16_t *ptr;      // direct mode: where w came from
    const uint16_t *head_end, *tail_row;   // direct mode: first address past the lane's head rows, and where its rows go on
    uint32_t koff, ring_lane; // ring mode: see above; ring_lane = shared address of the ring | lane*2
    uint32_t c64, c1;         // the constants 64 and 1 in registers the compiler cannot see through
};

template <typename R>
struct RingCtlT {             // per warp (all fields warp-uniform)
    using Geom = R;
    uint32_t ring_base, bar0; // shared addresses
    uint32_t issued, ready;   // chunks issued / known complete since the kernel started
    uint32_t tile_first, tile_last, tile_bytes;  // chunk range [first, last) and byte length of the open tile
    TileSrc src;              // global addresses of the open tile
    uint32_t *status;
};

template <typename R>
__device__ __forceinline__ void ring_setup(RingCtlT<R> &r, uint8_t *ring_area, uint32_t warp, uint32_t nwarps, uint32_t lane, uint32_t *status)
{
    const uint32_t base = (smem_addr(ring_area) + R::kBytes - 1) & ~(R::kBytes - 1);
    r.ring_base = base + warp * R::kBytes;
    r.bar0 = base + nwarps * R::kBytes + warp * R::kChunks * 8;
    r.issued = r.ready = 0;
    r.status = status;
    if (lane == 0) {
#pragma unroll
        for (uint32_t i = 0; i < R::kChunks; i++) mbar_init(r.bar0 + i * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// Start copies for every chunk of the current tile below `limit` that has not been started yet.
template <typename R>
__device__ __forceinline__ void ring_issue(RingCtlT<R> &r, uint32_t limit, uint32_t lane)
{
    while (r.issued < limit) {
        if (lane == 0) {
            const uint32_t c = r.issued - r.tile_first, slot = r.issued % R::kChunks;
            const uint32_t bytes = min(R::kChunkBytes, r.tile_bytes - c * R::kChunkBytes);
            mbar_expect_tx(r.bar0 + slot * 8, bytes);
            bulk_copy_g2s(r.ring_base + slot * R::kChunkBytes, r.src.at(c * R::kChunkBytes), bytes, r.bar0 + slot * 8);
        }
        r.issued++;
    }
}

// Keep the ring ahead of the readers.  Two warp votes against warp-uniform thresholds: a chunk is
// refilled once every lane has left the chunk it replaces, and the next chunk is waited for as soon as
// any lane could reach it within kSync steps.
template <typename R>
__device__ __forceinline__ void ring_sync(RingCtlT<R> &r, const WordState &s, uint32_t lane)
{
    // chunk numbers count from the warp's first chunk of the kernel; koff is in the same frame
    while (r.issued < r.tile_last && __all_sync(0xffffffffu, s.koff >= (r.issued + 1 - R::kChunks) * R::kChunkBytes))
        ring_issue(r, r.issued + 1, lane);
    while (r.ready < r.issued && __any_sync(0xffffffffu, s.koff + (R::kSync + 1) * 64 >= r.ready * R::kChunkBytes)) {
        mbar_wait_bounded(r.bar0 + (r.ready % R::kChunks) * 8, (r.ready / R::kChunks) & 1u, r.status);
        r.ready++;
    }
}

// The same between two checks at most kSync = one chunk of steps apart: lanes consume at most one row per step,
// so at most one chunk is freed and at most one more is needed -- one vote each instead of a loop.
template <typename R>
__device__ __forceinline__ void ring_sync_step(RingCtlT<R> &r, const WordState &s, uint32_t lane)
{
    static_assert(R::kSync <= R::kChunkRows, "a check period may not span more than one chunk");
    if (r.issued < r.tile_last && __all_sync(0xffffffffu, s.koff >= (r.issued + 1 - R::kChunks) * R::kChunkBytes))
        ring_issue(r, r.issued + 1, lane);
    if (r.ready < r.issued && __any_sync(0xffffffffu, s.koff + (R::kSync + 1) * 64 >= r.ready * R::kChunkBytes)) {
        mbar_wait_bounded(r.bar0 + (r.ready % R::kChunks) * 8, (r.ready / R::kChunks) & 1u, r.status);
        r.ready++;
    }
}

// Open a tile: ask L2 for all of it and, in ring mode, start its first copies.  Waits for nothing, so it
// can run well before the tile is decoded (before the kernel's prologue, or while the previous tile's
// results are being written).  The whole tile goes through the ring, its 128-byte state header included.
template <typename R>
__device__ __forceinline__ void tile_open(RingCtlT<R> &r, const TileDesc &d, const TileSrc &base, uint32_t lane)
{
    static_assert(1024u % R::kChunkBytes == 0, "a ring chunk may not straddle the end of a tile's head");
    const uint32_t bytes = d.len64 << 6;
    uint32_t ahead = 0;        // bytes already on their way through the ring
    if ((d.seg & kTileDirectFlag) == 0) {
        r.tile_first = r.issued;
        r.tile_bytes = bytes;
        r.tile_last = r.tile_first + (r.tile_bytes + R::kChunkBytes - 1) / R::kChunkBytes;
        r.src = base;
        ring_issue(r, min(r.tile_last, r.tile_first + R::kChunks), lane);
        ahead = min(bytes, R::kBytes);
    }
    // The rest of the tile is only asked into L2, and after the ring copies: when every warp of the grid opens its
    // tile at the same moment, the copies that are needed first must not queue behind megabytes of prefetch.
    if (lane == 0 && bytes > ahead) {
        if (ahead < base.hbytes) {
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base.head + ahead), "r"(base.hbytes - ahead) : "memory");
            ahead = base.hbytes;
        }
        if (bytes > ahead)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base.tail + ahead), "r"(bytes - ahead) : "memory");
    }
}

// Begin decoding an opened tile: wait for its first chunk, read the lane's state and first word.
// Returns true if the tile runs in ring mode.
template <typename R>
__device__ __forceinline__ bool tile_begin(RingCtlT<R> &r, WordState &s, const TileDesc &d, const TileSrc &base, uint32_t lane, uint32_t &x)
{
    const bool ring = (d.seg & kTileDirectFlag) == 0;
    if (ring) {
        const uint32_t start = r.tile_first * R::kChunkBytes;
        s.koff = start + 128;                                   // word row 0 sits behind the two header rows
        s.ring_lane = r.ring_base | (lane * 2);
        asm volatile("mov.b32 %0, 64;\n\tmov.b32 %1, 1;" : "=r"(s.c64), "=r"(s.c1));
        ring_sync(r, s, lane);
        x = lds_u32(r.ring_base + (start & (R::kBytes - 1)) + lane * 4);
        s.w = lds_u16((s.koff & (R::kBytes - 1)) | s.ring_lane);
    } else {
        // states and word rows straight from global memory; a lane's rows continue in the tail after the head
        x = __ldg(reinterpret_cast<const uint32_t *>(base.at(0)) + lane);
        s.head_end = reinterpret_cast<const uint16_t *>(base.head + base.hbytes) + lane;
        s.tail_row = reinterpret_cast<const uint16_t *>(base.tail + base.hbytes) + lane;
        s.ptr = base.hbytes > 128u ? reinterpret_cast<const uint16_t *>(base.head + 128) + lane
                                   : reinterpret_cast<const uint16_t *>(base.tail + 128) + lane;
        if (base.hbytes <= 128u) s.head_end = nullptr;
        s.w = __ldg(s.ptr);
    }
    return ring;
}

template <typename R>
__device__ __forceinline__ void tile_end(RingCtlT<R> &r, bool ring)
{
    if (!ring) return;
    while (r.ready < r.issued) {       // nothing of this tile may still be in flight when the next one starts
        mbar_wait_bounded(r.bar0 + (r.ready % R::kChunks) * 8, (r.ready / R::kChunks) & 1u, r.status);
        r.ready++;
    }
}

// Renormalise: at most one 16-bit word per step, since p <= 16.
template <bool RING, uint32_t RING_BYTES = RingSmall::kBytes>
__device__ __forceinline__ void rans_renorm(uint32_t &x, WordState &s)
{
    if (RING) {
        // predicated, branch-free: x = x * 65536 + w; koff += 64; w = ring[(koff mod ring) | lane*2].  A plain C++
        // conditional and a select-based form with an unconditional reload were measured: all three within 2 %.
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t"
                     "setp.lt.u32 p, %0, 65536;\n\t"
                     "@p mad.lo.u32 %0, %0, 65536, %1;\n\t"
                     "@p mad.lo.u32 %2, %5, %6, %2;\n\t"     // koff += 64 as a multiply-add: keeps it off the ALU pipe
                     "@p lop3.b32 t, %2, %4, %3, 0xEA;\n\t"
                     "@p ld.shared.u16 %1, [t];\n\t}"
                     : "+r"(x), "+r"(s.w), "+r"(s.koff)
                     : "r"(s.ring_lane), "n"(RING_BYTES - 1), "r"(s.c64), "r"(s.c1));
    } else if (x < 65536u) {
        x = (x << 16) | s.w;
        s.ptr += 32;
        if (s.ptr == s.head_end) s.ptr = s.tail_row;
        s.w = __ldg(s.ptr);
    }
}

// ---------------------------------------------------------------------------
// Fused decode + dequantise + GEMV.
//
// Grid: persistent, a multiple of the SM count; 16 warps per CTA; warp w of CTA
// c owns tiles c + gridDim.x * (w + 16*i).  Shared memory: the decode table,
// x converted to fp32 as [K][BT], and either per-16-column sums of x (INT4) or
// the centroid table replicated per lane (polar).  Each lane accumulates G rows
// x BT batch entries in registers; per scale group the accumulators are folded
// into the row sums with the group's fp16 scale.  Tiles of one row block that
// cover different column segments meet through `partials`; the last warp to
// arrive (a ticket on `counters`) adds them up in segment order, so results do
// not depend on scheduling.
// ---------------------------------------------------------------------------
template <int G, int BT>
__device__ __forceinline__ void write_rows(const GemvArgs &a, uint32_t row, const float (&y)[G][BT]);
__device__ __forceinline__ void gather_finish(const GemvArgs &a);

// The column loop of one tile: decode, unpack, multiply-accumulate, fold per scale group.
template <int G, int BITS, int BT, int KIND, bool RING, int UNROLL, typename R>
__device__ __forceinline__ void gemv_tile_columns(const GemvArgs &a, const TileDesc &d, const uint32_t *tab, const float *xs,
                                                  const float *aux, uint32_t lane, uint32_t row, uint32_t mask, uint32_t p,
                                                  uint32_t sgroups, uint32_t &x, WordState &ws, RingCtlT<R> &ring, float (&y)[G][BT])
{
    using F = Fmt<G, BITS>;
    constexpr int kFB = KIND == EOQ_B200_KIND_INT4_ABSMAX ? BITS : 4;      // field width of the integer kinds
    const uint32_t magic0 = Int4Field<F::field_bit(0), kFB>::magic_reg();
    const uint32_t magic1 = Int4Field<F::field_bit(G > 1 ? 1 : 0), kFB>::magic_reg();
    const uint32_t magic2 = Int4Field<F::field_bit(G > 2 ? 2 : 0), kFB>::magic_reg();
    const uint32_t tab_addr = smem_addr(tab);
        uint32_t c = d.col0;
        const uint32_t cend = c + d.ncols;
        // The group scales are fetched one run ahead with loads the compiler may not move: left to itself it
        // sinks them to their use at the end of the run, where each costs a full memory round trip.
        uint16_t sc_next[G];
#pragma unroll
        for (int j = 0; j < G; j++) sc_next[j] = ldg_u16_pinned(a.scales + (size_t)min(row + j, a.N - 1) * sgroups + c / a.group);
        while (c < cend) {
            const uint32_t g = c / a.group;
            const uint32_t rstart = c, rend = min(cend, (g + 1) * a.group);
            uint16_t sc_bits[G];
#pragma unroll
            for (int j = 0; j < G; j++) sc_bits[j] = sc_next[j];
            if (rend < cend) {
#pragma unroll
                for (int j = 0; j < G; j++) sc_next[j] = ldg_u16_pinned(a.scales + (size_t)min(row + j, a.N - 1) * sgroups + g + 1);
            }
            float acc[G][BT];
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) acc[j][b] = 0.0f;

#pragma unroll UNROLL
            for (; c < rend; c += 4) {
                // runs start on multiples of 16 columns, so this fires at least every kSync (16 or 32) steps
                if (RING && (c & (R::kSync - 4u)) == 0) ring_sync_step(ring, ws, lane);
                float xv[4][BT];
                if (BT == 1) {
                    const float4 v = *reinterpret_cast<const float4 *>(xs + c);
                    xv[0][0] = v.x; xv[1][0] = v.y; xv[2][0] = v.z; xv[3][0] = v.w;
                } else if (BT == 2) {
                    const float4 v0 = *reinterpret_cast<const float4 *>(xs + c * 2);
                    const float4 v1 = *reinterpret_cast<const float4 *>(xs + c * 2 + 4);
                    xv[0][0] = v0.x; xv[0][BT - 1] = v0.y; xv[1][0] = v0.z; xv[1][BT - 1] = v0.w;
                    xv[2][0] = v1.x; xv[2][BT - 1] = v1.y; xv[3][0] = v1.z; xv[3][BT - 1] = v1.w;
                }
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    if (BT > 2) {
#pragma unroll
                        for (int q = 0; q < BT / 4; q++) {
                            const float4 v = *reinterpret_cast<const float4 *>(xs + (size_t)(c + s) * BT + q * 4);
                            xv[s][(q * 4 + 0) % BT] = v.x; xv[s][(q * 4 + 1) % BT] = v.y;
                            xv[s][(q * 4 + 2) % BT] = v.z; xv[s][(q * 4 + 3) % BT] = v.w;
                        }
                    }
                    if (KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                        using F0 = Int4Field<F::field_bit(0), kFB>;
                        using F1 = Int4Field<F::field_bit(G > 1 ? 1 : 0), kFB>;
                        using F2 = Int4Field<F::field_bit(G > 2 ? 2 : 0), kFB>;
                        constexpr uint32_t kM1 = (G > 1) ? F1::kMask : 0u, kM2 = (G > 2) ? F2::kMask : 0u;
                        uint32_t u0, u1, u2;
                        rans_step_int4<F0::kMask, kM1, kM2>(tab_addr, x, mask, p, F::kBiasMask, magic0, magic1, magic2, u0, u1, u2);
                        {
                            float m = __uint_as_float(u0);
                            if (F0::kPreSubtract) m -= F0::kOffset;
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[0][b] = fmaf(m, xv[s][b], acc[0][b]);
                        }
                        if (G > 1) {
                            float m = __uint_as_float(u1);
                            if (F1::kPreSubtract) m -= F1::kOffset;
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[G > 1 ? 1 : 0][b] = fmaf(m, xv[s][b], acc[G > 1 ? 1 : 0][b]);
                        }
                        if (G > 2) {
                            float m = __uint_as_float(u2);
                            if (F2::kPreSubtract) m -= F2::kOffset;
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[G > 2 ? 2 : 0][b] = fmaf(m, xv[s][b], acc[G > 2 ? 2 : 0][b]);
                        }
                    } else {
                        const uint32_t e = rans_step(tab, x, mask, p, F::kBiasMask);
#pragma unroll
                        for (int j = 0; j < G; j++) {
                            const uint32_t code = (e >> F::field_bit(j)) & F::kFieldMask;
                            const float m = aux[code * 32 + lane];
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[j][b] = fmaf(m, xv[s][b], acc[j][b]);
                        }
                    }
                    rans_renorm<RING, R::kBytes>(x, ws);
                }
            }

            float sc[G];
#pragma unroll
            for (int j = 0; j < G; j++) sc[j] = row + j < a.N ? half_bits_to_float(sc_bits[j]) : 0.0f;
            if (KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                float rs[BT];
#pragma unroll
                for (int b = 0; b < BT; b++) rs[b] = 0.0f;
                for (uint32_t u = rstart / 16; u < rend / 16; u++)
#pragma unroll
                    for (int b = 0; b < BT; b++) rs[b] += aux[u * BT + b];
                const float corr[3] = {Int4Field<F::field_bit(0), kFB>::kCorr,
                                       Int4Field<F::field_bit(G > 1 ? 1 : 0), kFB>::kCorr,
                                       Int4Field<F::field_bit(G > 2 ? 2 : 0), kFB>::kCorr};
#pragma unroll
                for (int j = 0; j < G; j++)
#pragma unroll
                    for (int b = 0; b < BT; b++) y[j][b] = fmaf(sc[j], acc[j][b] - corr[j] * rs[b], y[j][b]);
            } else {
#pragma unroll
                for (int j = 0; j < G; j++)
#pragma unroll
                    for (int b = 0; b < BT; b++) y[j][b] = fmaf(sc[j], acc[j][b], y[j][b]);
            }
        }

}

template <int G, int BITS, int BT, int KIND, int THREADS, typename R>
__global__ void __launch_bounds__(THREADS, 1) gemv_tiles_kernel(const GemvArgs a)
{
    constexpr int kThreads = THREADS, kWarps = THREADS / 32;
    constexpr int kUnroll = THREADS <= 512 ? 4 : THREADS <= 768 ? 2 : 1;   // fewer registers per thread as the CTA grows
    using F = Fmt<G, BITS>;
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tab = reinterpret_cast<uint32_t *>(smem);
    float *xs = reinterpret_cast<float *>(smem + smem_table_bytes(a.p) + 16);
    float *aux = xs + (size_t)a.K * BT;   // INT4: [K/16][BT] sums; polar: [32][32] centroids
    uint8_t *ring_area = reinterpret_cast<uint8_t *>(aux + (KIND == EOQ_B200_KIND_Q5_POLAR ? 32 * 32 : (size_t)(a.K / 16) * BT));

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t K = a.K, M = 1u << a.p;
    // Prologue: everything that has to come from global memory is requested before anything is waited for --
    // the decode table (one bulk copy onto a barrier), x (vector loads into registers) and this warp's first tile
    // (descriptor, L2 prefetch, first ring chunks) -- so the prologue costs about one memory round trip.
    // The launch may be programmatic (see launch_with_pdl): this grid can start while the previous kernel of the
    // stream is still finishing.  Everything up to griddepcontrol.wait (barrier set-up, the table copy, the first
    // tile descriptor) touches only this weight's read-only data; x, bias and all global writes come after it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t tab_bar = smem_addr(smem + smem_table_bytes(a.p));
    if (tid == 0) {
        mbar_init(tab_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(tab_bar, 4u << a.p);
        for (uint32_t off = 0; off < (4u << a.p); off += 16384u)
            bulk_copy_g2s(smem_addr(tab) + off, reinterpret_cast<const uint8_t *>(a.table) + off, min(16384u, (4u << a.p) - off), tab_bar);
    }
    RingCtlT<R> ring;
    ring_setup(ring, ring_area, warp, kWarps, lane, a.status);
    uint32_t t = blockIdx.x + gridDim.x * warp;
    bool have = t < a.ntiles;
    TileDesc d;
    if (have) d = a.tiles[t];                    // requested here, needed by tile_open below
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const bool x_vec = a.x_dtype != EOQ_B200_F32 && K % 16 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0;
    const uint32_t vec_per_row = K / 8, nvec = vec_per_row * a.batch;
    constexpr int kXV = 3;                       // 16-byte x loads in flight per thread
    uint4 xq[kXV];
    if (x_vec) {
#pragma unroll
        for (int u = 0; u < kXV; u++)
            if (tid + u * kThreads < nvec) xq[u] = __ldg(reinterpret_cast<const uint4 *>(a.x) + tid + u * kThreads);
    }
    if (have) tile_open(ring, d, tile_src(a.stream, a.head_bytes, t, d), lane);

    if (x_vec) {
        // 8 columns per vector: convert, store as fp32 [K][BT], and (INT4) add up 16-column sums with the neighbour lane
        for (uint32_t v0 = 0; v0 < nvec; v0 += kThreads * kXV) {
            if (v0 > 0) {
#pragma unroll
                for (int u = 0; u < kXV; u++)
                    if (v0 + tid + u * kThreads < nvec) xq[u] = __ldg(reinterpret_cast<const uint4 *>(a.x) + v0 + tid + u * kThreads);
            }
#pragma unroll
            for (int u = 0; u < kXV; u++) {
                const uint32_t v = v0 + tid + u * kThreads;
                const bool on = v < nvec;
                const uint32_t b = on ? v / vec_per_row : 0, c0 = on ? (v % vec_per_row) * 8 : 0;
                const uint32_t wds[4] = {xq[u].x, xq[u].y, xq[u].z, xq[u].w};
                float sum = 0.0f;
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    float lo, hi;
                    if (a.x_dtype == EOQ_B200_F16) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&wds[h]));
                        lo = f.x; hi = f.y;
                    } else {
                        lo = __uint_as_float(wds[h] << 16); hi = __uint_as_float(wds[h] & 0xFFFF0000u);
                    }
                    if (on) {
                        xs[(c0 + 2 * h) * BT + b] = lo;
                        xs[(c0 + 2 * h + 1) * BT + b] = hi;
                        sum += lo + hi;
                    }
                }
                if (KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                    // vectors v and v^1 are the two halves of one 16-column unit (same row: K is a multiple of 16)
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    if (on && (v & 1u) == 0) aux[(c0 / 16) * BT + b] = sum;
                }
            }
        }
        if (BT > 1) {
            for (uint32_t i = tid; i < K * BT; i += kThreads)
                if (i % BT >= a.batch) xs[i] = 0.0f;
            if (KIND == EOQ_B200_KIND_INT4_ABSMAX)
                for (uint32_t i = tid; i < K / 16 * BT; i += kThreads)
                    if (i % BT >= a.batch) aux[i] = 0.0f;
        }
    } else {
        for (uint32_t i0 = tid; i0 < K * BT; i0 += kThreads * 8) {      // eight independent loads in flight per thread
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const uint32_t i = i0 + u * kThreads, c = i / BT, b = i % BT;
                v[u] = (i < K * BT && b < a.batch) ? load_x(a.x, (size_t)b * K + c, a.x_dtype) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (i0 + u * kThreads < K * BT) xs[i0 + u * kThreads] = v[u];
        }
    }
    if (KIND == EOQ_B200_KIND_Q5_POLAR)
        for (uint32_t i = tid; i < 32 * 32; i += kThreads) aux[i] = __ldg(a.centroids + (i >> 5));
    __syncthreads();
    if (KIND == EOQ_B200_KIND_Q5_POLAR) {
        // x'' = H64 x / 64 per 64-column block (unnormalised Sylvester butterflies), so that
        // W_block . x_block = norm * sum_j centroid[code_j] * x''_j   (core/polar_quant.py:242-262)
        for (uint32_t h = 1; h < 64; h <<= 1) {
            for (uint32_t q = tid; q < K / 2 * BT; q += kThreads) {
                const uint32_t b = q % BT, pr = q / BT;
                const uint32_t c = 2 * (pr - (pr % h)) + (pr % h);
                const float u = xs[c * BT + b], v = xs[(c + h) * BT + b];
                const float sc = h == 32 ? 1.0f / 64.0f : 1.0f;
                xs[c * BT + b] = (u + v) * sc;
                xs[(c + h) * BT + b] = (u - v) * sc;
            }
            __syncthreads();
        }
    } else if (!x_vec) {
        for (uint32_t i = tid; i < K / 16 * BT; i += kThreads) {
            const uint32_t u = i / BT, b = i % BT;
            float sm = 0.0f;
#pragma unroll
            for (int k = 0; k < 16; k++) sm += xs[(u * 16 + k) * BT + b];
            aux[i] = sm;
        }
        __syncthreads();
    }

    mbar_wait_bounded(tab_bar, 0u, a.status);
    const uint32_t mask = M - 1u, p = a.p;
    const uint32_t sgroups = K / a.group;
    while (have) {
        const TileDesc cur = d;
        uint32_t x;
        WordState ws;
        const bool ring_mode = tile_begin(ring, ws, cur, tile_src(a.stream, a.head_bytes, t, cur), lane, x);
        const uint32_t row = cur.row0 + lane * G;
        const uint32_t rb = cur.row0 / (32u * G);
        const uint32_t seg = cur.seg & ~kTileDirectFlag;

        float y[G][BT];
#pragma unroll
        for (int j = 0; j < G; j++)
#pragma unroll
            for (int b = 0; b < BT; b++) y[j][b] = 0.0f;

        if (ring_mode) gemv_tile_columns<G, BITS, BT, KIND, true, kUnroll>(a, cur, tab, xs, aux, lane, row, mask, p, sgroups, x, ws, ring, y);
        else gemv_tile_columns<G, BITS, BT, KIND, false, 1>(a, cur, tab, xs, aux, lane, row, mask, p, sgroups, x, ws, ring, y);
        tile_end(ring, ring_mode);

        // the next tile's copies start now and overlap the write-back of this one
        t += gridDim.x * kWarps;
        have = t < a.ntiles;
        if (have) {
            d = a.tiles[t];
            tile_open(ring, d, tile_src(a.stream, a.head_bytes, t, d), lane);
        }

        bool write_out = true;
        if (a.nseg > 1) {
            float *mine = a.partials + ((size_t)seg * a.Npad + row) * BT;
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) __stcg(mine + j * BT + b, y[j][b]);
            __threadfence();
            __syncwarp();
            uint32_t ticket = 0;
            if (lane == 0) ticket = atomicAdd(a.counters + rb, 1u);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            write_out = ticket == a.nseg - 1;
            if (write_out) {
                // last warp of the row block: add the segments' partial sums, always in segment order;
                // loads are issued kU segments at a time so their latencies overlap
                __threadfence();
                constexpr int kU = G * BT <= 3 ? 16 : G * BT <= 6 ? 8 : G * BT <= 12 ? 4 : 2;
#pragma unroll
                for (int j = 0; j < G; j++)
#pragma unroll
                    for (int b = 0; b < BT; b++) y[j][b] = 0.0f;
                for (uint32_t s0 = 0; s0 < a.nseg; s0 += kU) {
                    float v[kU][G][BT];
#pragma unroll
                    for (int u = 0; u < kU; u++) {
                        const uint32_t sidx = min(s0 + u, a.nseg - 1);
                        const float *src = a.partials + ((size_t)sidx * a.Npad + row) * BT;
#pragma unroll
                        for (int j = 0; j < G; j++)
#pragma unroll
                            for (int b = 0; b < BT; b++) v[u][j][b] = __ldcg(src + j * BT + b);
                    }
#pragma unroll
                    for (int u = 0; u < kU; u++)
                        if (s0 + u < a.nseg)
#pragma unroll
                            for (int j = 0; j < G; j++)
#pragma unroll
                                for (int b = 0; b < BT; b++) y[j][b] += v[u][j][b];
                }
                if (lane == 0) a.counters[rb] = 0u;
            }
        }
        if (write_out) write_rows<G, BT>(a, row, y);     // bias, output type and, in row-sharded runs, the stores into the peers' buffers
    }
    gather_finish(a);          // row-sharded runs: wait for the other ranks' rows and unpack them
}

// Programmatic dependent launch: the grid may be scheduled as soon as the previous kernel of the stream lets go of
// SMs (its CTAs exit one by one while the last ones still reduce), so that this kernel's table copy and first tile
// fetch overlap the other's tail.  The kernels order themselves with griddepcontrol.wait before they read an
// input or write anything.  "pdl" = 0 in eoq_b200_tune falls back to plain launches.
static std::atomic<int> g_pdl{1};
void set_pdl(int v) { g_pdl.store(v != 0); }

template <typename Kern, typename... Args>
static cudaError_t launch_with_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Launch configuration is resolved once per (kernel, device, shared-memory size) and cached,
// so that a steady-state launch is nothing but the launch itself (and can be stream-captured).
static std::atomic<int> g_gemv_ctas_per_sm{0};   // 0 = as many as fit
void set_gemv_ctas_per_sm(int v) { g_gemv_ctas_per_sm.store(v < 0 ? 0 : v); }

template <int G, int BITS, int BT, int KIND, int THREADS, typename R>
static int launch_gemv_cfg(const GemvArgs &a, cudaStream_t st)
{
    struct Cfg { size_t smem = 0; int per_sm = 0, sms = 0; };
    static Cfg cfg[16];
    static std::mutex mu;
    auto kern = gemv_tiles_kernel<G, BITS, BT, KIND, THREADS, R>;
    const size_t smem = gemv_smem_bytes_for<R>(a.K, a.p, BT, KIND, THREADS);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    Cfg c;
    {
        std::lock_guard<std::mutex> lock(mu);
        Cfg &slot = cfg[dev & 15];
        if (slot.smem != smem || slot.per_sm == 0) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            int per_sm = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem);
            if (e != cudaSuccess) return (int)e;
            if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
            slot.smem = smem; slot.per_sm = per_sm; slot.sms = device_sm_count();
        }
        c = slot;
    }
    int per_sm = c.per_sm;
    const int want = g_gemv_ctas_per_sm.load();
    if (want > 0) per_sm = std::min(per_sm, want);
    uint32_t grid = (uint32_t)(c.sms * per_sm);
    grid = max(1u, min(grid, a.ntiles));
    e = launch_with_pdl(kern, dim3(grid), dim3(THREADS), smem, st, a);
    g_launches++;
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// 16 warps per CTA, one CTA per SM.  CTAs of 24 and 32 warps (with proportionally more, shorter tiles) were
// measured and are no faster: the step rate is bounded by the SM's shared-memory and ALU pipes, not by the
// number of resident warps, and shorter tiles pay the per-tile costs more often.
template <int G, int BITS, int BT, int KIND>
static int launch_gemv_one(const GemvArgs &a, cudaStream_t st)
{
    // A 128-row ring checked every 32 steps (RingGeom<128, 32, 32>) was measured for batch 1: within 1 % on
    // 11008x4096 and 8 % slower on 4096x11008, so every launch uses the 64-row ring.
    return launch_gemv_cfg<G, BITS, BT, KIND, kThreads, RingSmall>(a, st);
}

template <int G, int BITS, int KIND>
static int launch_gemv_bt(const GemvArgs &a, cudaStream_t st)
{
    if (a.batch <= 1) return launch_gemv_one<G, BITS, 1, KIND>(a, st);
    if (a.batch <= 2) return launch_gemv_one<G, BITS, 2, KIND>(a, st);
    if (a.batch <= 4) return launch_gemv_one<G, BITS, 4, KIND>(a, st);
    return launch_gemv_one<G, BITS, 8, KIND>(a, st);
}

// ---------------------------------------------------------------------------
// Fused decode + dequantise + GEMV, two tiles per warp, tiles staged whole ("pair kernel").
//
// The column loop of gemv_tiles_kernel is bound by the latency of one dependent chain per warp (table look-up ->
// state update -> renormalisation) and by the integer pipe, a fifth of which goes into keeping the word ring ahead
// of its readers.  This kernel removes both: a warp decodes TWO tiles at once -- the same column segment of two
// adjacent row blocks, so that the activations of a step are loaded once and two independent chains are in flight
// per lane -- and each tile is copied whole into its own shared-memory buffer by bulk asynchronous copies
// (cp.async.bulk, the 1-D TMA path) of one kilobyte each, every kilobyte completing on its own mbarrier.  All copies
// of a tile are requested when it is opened; kilobyte j (word rows 16 j - 2 .. 16 j + 13) is waited for eight steps
// before column 16 j, by which time no lane can have read past row 16 j - 8.  No ring, no warp votes, no wrap-around
// of the read address.
//
// x is not staged for the whole CTA: each warp converts only the columns of its own segment to fp32 (at most a few
// hundred values), so the kernel has no CTA-wide prologue besides the table copy.
//
// Pair q = (row-block pair q / nseg, segment q % nseg).  The pairs are cut into runs of at most sixteen consecutive
// pairs; a CTA takes one run per pass, one pair per warp, adds the results of a run up in shared memory and only
// then meets the other CTAs that hold segments of the same rows (partial rows + a ticket, summed in run order by
// the last to arrive).  With an odd number of row blocks the last pair decodes its one tile twice and drops the
// second result.  Output and the fused all-gather are those of gemv_tiles_kernel.
// ---------------------------------------------------------------------------
__host__ __device__ inline uint32_t pair_region_bytes(uint32_t stage, uint32_t max_ncols, uint32_t bt, uint32_t xbytes = 4)
{
    // two stage buffers, 128 bytes of barriers, the warp's x segment [max_ncols][bt] (fp32, or the caller's 16-bit values as
    // they are) and its 16-column sums
    return 2u * stage + 128u + ((max_ncols * bt * xbytes + (max_ncols / 16u) * bt * 4u + 127u) & ~127u);
}
constexpr uint32_t kPairJobBytes = 512;    // sixteen 32-byte notices "this warp adds up a pair of row blocks and wants help"
static size_t pair_smem_bytes(uint32_t p, uint32_t bt, uint32_t stage, uint32_t max_ncols, uint32_t warps, uint32_t xbytes = 4)
{
    return ((size_t)4 << p) + 128 + kPairJobBytes + (size_t)warps * pair_region_bytes(stage, max_ncols, bt, xbytes);
}

// Bounded wait on try_wait: the warp is suspended by the hardware between polls instead of spinning through issue
// slots.  A poll may sleep for a system-dependent time, so the bound is on elapsed time (about a second), not on polls.
__device__ __forceinline__ void mbar_wait_suspended(uint32_t bar, uint32_t parity, uint32_t *status)
{
    long long t0 = 0;
    for (uint32_t i = 0;; i++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
        if (i == 0) t0 = clock64();
        else if (clock64() - t0 > (1ll << 31)) break;      // ~1 s at 2 GHz
    }
    *status = 1u;   // gave up; the host turns this into an error
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

// Renormalise from a staged tile: x = x * 65536 + w; addr += 64; w = [addr]  (predicated, branch-free).
__device__ __forceinline__ void staged_renorm(uint32_t &x, uint32_t &w, uint32_t &addr, uint32_t c64, uint32_t c1)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.lt.u32 p, %0, 65536;\n\t"
                 "@p mad.lo.u32 %0, %0, 65536, %1;\n\t"
                 "@p mad.lo.u32 %2, %3, %4, %2;\n\t"
                 "@p ld.shared.u16 %1, [%2];\n\t}"
                 : "+r"(x), "+r"(w), "+r"(addr)
                 : "r"(c64), "r"(c1));
}

// Sum the partial results of all column segments for G rows of one lane, in segment order.
template <int G, int BT>
__device__ __forceinline__ void reduce_segments(const GemvArgs &a, uint32_t row, float (&y)[G][BT])
{
    constexpr int kU = G * BT <= 3 ? 16 : G * BT <= 6 ? 8 : G * BT <= 12 ? 4 : 2;
#pragma unroll
    for (int j = 0; j < G; j++)
#pragma unroll
        for (int b = 0; b < BT; b++) y[j][b] = 0.0f;
    for (uint32_t s0 = 0; s0 < a.nseg; s0 += kU) {
        float v[kU][G][BT];
#pragma unroll
        for (int u = 0; u < kU; u++) {
            const uint32_t sidx = min(s0 + u, a.nseg - 1);
            const float *src = a.partials + ((size_t)sidx * a.Npad + row) * BT;
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) v[u][j][b] = __ldcg(src + j * BT + b);
        }
#pragma unroll
        for (int u = 0; u < kU; u++)
            if (s0 + u < a.nseg)
#pragma unroll
                for (int j = 0; j < G; j++)
#pragma unroll
                    for (int b = 0; b < BT; b++) y[j][b] += v[u][j][b];
    }
}

// Final values of G rows of one lane: bias, output type, and (row-sharded runs) the stores into the peers' buffers.
template <int G, int BT>
__device__ __forceinline__ void write_rows(const GemvArgs &a, uint32_t row, const float (&y)[G][BT])
{
    if (a.world > 1) {
        if (row >= a.N) return;
        const uint32_t epoch = __ldcg(a.gather_epoch) + 1u;
        const bool f32 = a.y_dtype == EOQ_B200_F32;
        const uint32_t wpr = f32 ? a.N : a.Npad / G;
        float bv[G];
#pragma unroll
        for (int j = 0; j < G; j++) bv[j] = (a.bias && row + j < a.N) ? __ldg(a.bias + row + j) : 0.0f;
#pragma unroll
        for (int b = 0; b < BT; b++)
            if ((uint32_t)b < a.batch) {
                uint32_t bits[3] = {0u, 0u, 0u};
#pragma unroll
                for (int j = 0; j < G; j++)
                    if (row + j < a.N) {
                        const float v = y[j][b] + bv[j];
                        store_y(a.y, (size_t)b * a.n_total + a.row_offset + row + j, v, a.y_dtype);
                        bits[j] = a.y_dtype == EOQ_B200_F16 ? (uint32_t)__half_as_ushort(__float2half_rn(v))
                                : a.y_dtype == EOQ_B200_BF16 ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v))
                                : __float_as_uint(v);
                    }
                const size_t base = (size_t)(b * a.world + a.rank) * wpr;
                if (f32) {
#pragma unroll
                    for (int j = 0; j < G; j++)
                        if (row + j < a.N)
                            for (uint32_t pr = 0; pr < a.world; pr++)
                                if (pr != a.rank)
                                    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(a.peer_ll[pr] + base + row + j), "r"(bits[j]), "r"(epoch) : "memory");
                } else {
                    const uint32_t lo = bits[0] | (bits[1] << 16), hi = bits[2] | (epoch << 16);
                    for (uint32_t pr = 0; pr < a.world; pr++)
                        if (pr != a.rank)
                            asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(a.peer_ll[pr] + base + row / G), "r"(lo), "r"(hi) : "memory");
                }
            }
    } else {
#pragma unroll
        for (int j = 0; j < G; j++) {
            const uint32_t r = row + j;
            if (r < a.N) {
                const float bv = a.bias ? __ldg(a.bias + r) : 0.0f;
#pragma unroll
                for (int b = 0; b < BT; b++)
                    if ((uint32_t)b < a.batch) store_y(a.y, (size_t)b * a.N + r, y[j][b] + bv, a.y_dtype);
            }
        }
    }
}

struct PairChain {            // per lane, one per decoded tile
    uint32_t x, w, addr;      // rANS state, next unread word, shared address that word came from
};

// Four columns of both chains: one activation load, then per column a step and a renormalisation of each chain.
// XH: how the x segment is kept in shared memory -- 0: fp32; 1 / 2: the caller's fp16 / bf16 values, converted here
// (four activation rows only; halves the segment so that four rows fit beside 112-column tiles).
template <int XH>
__device__ __forceinline__ void x16_pair_to_float(uint32_t w, float &lo, float &hi)
{
    if (XH == 1) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
        lo = f.x; hi = f.y;
    } else {
        lo = __uint_as_float(w << 16); hi = __uint_as_float(w & 0xFFFF0000u);
    }
}

template <int G, int BT, int XH>
__device__ __forceinline__ void pair_steps4(const void *xptr, uint32_t tab_addr, uint32_t mask, uint32_t p, uint32_t magic0, uint32_t magic1,
                                            uint32_t magic2, uint32_t c64, uint32_t c1, PairChain &ca, PairChain &cb,
                                            float (&acc)[2][G][BT])
{
    using F = Fmt<G, 4>;
    using F0 = Int4Field<F::field_bit(0)>;
    using F1 = Int4Field<F::field_bit(G > 1 ? 1 : 0)>;
    using F2 = Int4Field<F::field_bit(G > 2 ? 2 : 0)>;
    constexpr uint32_t kM1 = (G > 1) ? F1::kMask : 0u, kM2 = (G > 2) ? F2::kMask : 0u;
    float xv[4][BT];
    const float *xp = reinterpret_cast<const float *>(xptr);
    if (XH != 0) {
        static_assert(XH == 0 || BT == 4, "16-bit x segments are built for four activation rows");
        const uint4 v0 = reinterpret_cast<const uint4 *>(xptr)[0], v1 = reinterpret_cast<const uint4 *>(xptr)[1];
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};       // column s: words 2 s, 2 s + 1
#pragma unroll
        for (int s = 0; s < 4; s++) {
            x16_pair_to_float<XH>(w[2 * s], xv[s][0], xv[s][1 % BT]);
            x16_pair_to_float<XH>(w[2 * s + 1], xv[s][2 % BT], xv[s][3 % BT]);
        }
    } else if (BT == 1) {
        const float4 v = *reinterpret_cast<const float4 *>(xp);
        xv[0][0] = v.x; xv[1][0] = v.y; xv[2][0] = v.z; xv[3][0] = v.w;
    } else if (BT == 2) {
        const float4 v0 = *reinterpret_cast<const float4 *>(xp);
        const float4 v1 = *reinterpret_cast<const float4 *>(xp + 4);
        xv[0][0] = v0.x; xv[0][BT - 1] = v0.y; xv[1][0] = v0.z; xv[1][BT - 1] = v0.w;
        xv[2][0] = v1.x; xv[2][BT - 1] = v1.y; xv[3][0] = v1.z; xv[3][BT - 1] = v1.w;
    } else {
#pragma unroll
        for (int s = 0; s < 4; s++)
#pragma unroll
            for (int q = 0; q < BT / 4; q++) {
                const float4 v = *reinterpret_cast<const float4 *>(xp + s * BT + q * 4);
                xv[s][(q * 4 + 0) % BT] = v.x; xv[s][(q * 4 + 1) % BT] = v.y;
                xv[s][(q * 4 + 2) % BT] = v.z; xv[s][(q * 4 + 3) % BT] = v.w;
            }
    }
#pragma unroll
    for (int s = 0; s < 4; s++) {
        uint32_t u[2][3];
        rans_step_int4<F0::kMask, kM1, kM2>(tab_addr, ca.x, mask, p, F::kBiasMask, magic0, magic1, magic2, u[0][0], u[0][1], u[0][2]);
        rans_step_int4<F0::kMask, kM1, kM2>(tab_addr, cb.x, mask, p, F::kBiasMask, magic0, magic1, magic2, u[1][0], u[1][1], u[1][2]);
#pragma unroll
        for (int ch = 0; ch < 2; ch++) {
            {
                float m = __uint_as_float(u[ch][0]);
                if (F0::kPreSubtract) m -= F0::kBase + 7.0f;
#pragma unroll
                for (int b = 0; b < BT; b++) acc[ch][0][b] = fmaf(m, xv[s][b], acc[ch][0][b]);
            }
            if (G > 1) {
                float m = __uint_as_float(u[ch][1]);
                if (F1::kPreSubtract) m -= F1::kBase + 7.0f;
#pragma unroll
                for (int b = 0; b < BT; b++) acc[ch][G > 1 ? 1 : 0][b] = fmaf(m, xv[s][b], acc[ch][G > 1 ? 1 : 0][b]);
            }
            if (G > 2) {
                float m = __uint_as_float(u[ch][2]);
                if (F2::kPreSubtract) m -= F2::kBase + 7.0f;
#pragma unroll
                for (int b = 0; b < BT; b++) acc[ch][G > 2 ? 2 : 0][b] = fmaf(m, xv[s][b], acc[ch][G > 2 ? 2 : 0][b]);
            }
        }
        staged_renorm(ca.x, ca.w, ca.addr, c64, c1);
        staged_renorm(cb.x, cb.w, cb.addr, c64, c1);
    }
}

template <int G, int BT, int THREADS, int XH = 0>
__global__ void __launch_bounds__(THREADS, 1) gemv_pairs_kernel(const GemvArgs a)
{
    constexpr int kWarps = THREADS / 32;
    constexpr uint32_t kChunk = 1024, kMaxChunks = 8;   // a tile arrives in kilobytes, each on its own barrier (the first: states + 14 rows of words)
    using F = Fmt<G, 4>;
    extern __shared__ __align__(128) uint8_t pair_smem[];
    uint8_t *smem = pair_smem;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t tab_bytes = 4u << a.p;
    const uint32_t tab_addr = smem_addr(smem), tab_bar = tab_addr + tab_bytes;
    constexpr uint32_t kXBytes = XH ? 2u : 4u;
    const uint32_t region = pair_region_bytes(a.stage_bytes, a.max_ncols, BT, kXBytes);
    uint32_t *jobs = reinterpret_cast<uint32_t *>(smem + tab_bytes + 128);        // [warp][8]: valid, count, slot, row0 a, row0 b, has b
    uint8_t *mine = smem + tab_bytes + 128 + kPairJobBytes + (size_t)warp * region;
    const uint32_t stage[2] = {smem_addr(mine), smem_addr(mine) + a.stage_bytes};
    const uint32_t bars = stage[0] + 2u * a.stage_bytes;       // [chain][chunk], 8 bytes each
    float *xs = reinterpret_cast<float *>(mine + 2u * a.stage_bytes + 128);
    uint16_t *xs16 = reinterpret_cast<uint16_t *>(xs);
    float *aux = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(xs) + (size_t)a.max_ncols * BT * kXBytes);

    if (tid == 0) {
        mbar_init(tab_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(tab_bar, tab_bytes);
        for (uint32_t off = 0; off < tab_bytes; off += 16384u)
            bulk_copy_g2s(tab_addr + off, reinterpret_cast<const uint8_t *>(a.table) + off, min(16384u, tab_bytes - off), tab_bar);
    }
    if (lane < 2 * kMaxChunks) {
        mbar_init(bars + lane * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const uint32_t nrbp = (a.nrb + 1u) / 2u, npairs = nrbp * a.nseg;
    const uint32_t mask = (1u << a.p) - 1u, p = a.p;
    const uint32_t magic0 = Int4Field<F::field_bit(0)>::magic_reg();
    const uint32_t magic1 = Int4Field<F::field_bit(G > 1 ? 1 : 0)>::magic_reg();
    const uint32_t magic2 = Int4Field<F::field_bit(G > 2 ? 2 : 0)>::magic_reg();
    uint32_t c64, c1;
    asm volatile("mov.b32 %0, 64;\n\tmov.b32 %1, 1;" : "=r"(c64), "=r"(c1));

    // Geometry of the warp's pair.  Rows and columns follow from the pair's index alone (column boundaries are those of
    // the host encoder: segment s starts at column floor(s * K/16 / nseg) * 16), and so do the addresses of the tiles'
    // heads; only the tails need the descriptor ({off64, len64}, requested here and first used after the x loads).
    struct PairGeo {
        uint32_t t[2];        // tile indices (equal when the pair has no second row block)
        uint32_t row0[2];     // first rows
        uint32_t col0, ncols;
        bool has_b;
    } geo = {};
    uint2 dl = make_uint2(0u, 0u);    // lanes 0..15: {off64, len64} of tile lane / 8
    const uint32_t head_chunks = a.head_bytes / kChunk;
    // Read-only data of this weight only.  Lane k * 8 + j owns chunk j of tile k, so copies are issued side by side.
    auto open_pair = [&](uint32_t qq) {
        const uint32_t rbp = qq / a.nseg, seg = qq - rbp * a.nseg, units = a.K / kColGranule;
        geo.has_b = 2u * rbp + 1u < a.nrb;
        geo.t[0] = (2u * rbp) * a.nseg + seg;
        geo.t[1] = geo.has_b ? geo.t[0] + a.nseg : geo.t[0];
        geo.row0[0] = 2u * rbp * (32u * G);
        geo.row0[1] = geo.has_b ? geo.row0[0] + 32u * G : geo.row0[0];
        // (64-bit division is a long software routine: it is kept for matrices so large that the products overflow)
        if (((uint64_t)units * (a.nseg + 1u)) >> 32 == 0) {
            geo.col0 = (seg * units / a.nseg) * kColGranule;
            geo.ncols = ((seg + 1u) * units / a.nseg) * kColGranule - geo.col0;
        } else {
            geo.col0 = (uint32_t)((uint64_t)seg * units / a.nseg) * kColGranule;
            geo.ncols = (uint32_t)(((uint64_t)seg + 1u) * units / a.nseg) * kColGranule - geo.col0;
        }
        if (lane < 2 * kMaxChunks) {
            const uint32_t k = lane >> 3, j = lane & 7u, tk = k ? geo.t[1] : geo.t[0];
            if (j < head_chunks) {
                const uint32_t bar = bars + lane * 8;
                mbar_expect_tx(bar, kChunk);
                bulk_copy_g2s((k ? stage[1] : stage[0]) + j * kChunk, a.stream + (size_t)tk * a.head_bytes + j * kChunk, kChunk, bar);
            }
            dl = ldg_u32x2_pinned(reinterpret_cast<const uint2 *>(&a.tiles[tk].off64));
        }
    };
    // The chunks behind the heads: their place in the stream comes from the descriptor.
    auto tail_copy = [&]() {
        if (lane < 2 * kMaxChunks) {
            const uint32_t k = lane >> 3, j = lane & 7u;
            if (j >= head_chunks) {
                uint32_t bytes = dl.y << 6;
                if (bytes + 64u > a.stage_bytes) { *a.status = 2u; bytes = a.stage_bytes - 64u; }   // cannot happen with a host-computed stage size
                const uint32_t bar = bars + lane * 8, off = j * kChunk;
                if (off < bytes) {
                    const uint32_t n = min(kChunk, bytes - off);
                    mbar_expect_tx(bar, n);
                    bulk_copy_g2s((k ? stage[1] : stage[0]) + off, a.stream + ((size_t)dl.x << 6) + (off - a.head_bytes), n, bar);
                } else {
                    mbar_arrive(bar);                   // nothing to copy: complete the phase by hand
                }
            }
        }
    };
    // The pair's columns of x: loaded into registers (four columns per lane and batch row, up to 256 columns), then
    // converted to fp32 [ncols][BT] in shared memory together with the 16-column sums the INT4 unpack needs.
    const bool x_vec = a.x_dtype != EOQ_B200_F32 && (reinterpret_cast<uintptr_t>(a.x) & 7u) == 0;
    auto load_x_segment = [&](bool then_rest) {
        const uint32_t col0 = geo.col0, ncols = geo.ncols;
        for (uint32_t base = 0; base < ncols; base += 128u) {
            const uint32_t c = base + lane * 4u;
            const bool on = c < ncols;
            float v[BT][4];
            uint32_t raw[BT][2];          // XH: the same four values as the caller's 16-bit patterns
#pragma unroll
            for (int b = 0; b < BT; b++) {
#pragma unroll
                for (int i = 0; i < 4; i++) v[b][i] = 0.0f;
                raw[b][0] = raw[b][1] = 0u;
                if (on && (uint32_t)b < a.batch) {
                    const size_t i0 = (size_t)b * a.K + col0 + c;
                    if (x_vec) {
                        const uint2 r = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(a.x) + i0));
                        raw[b][0] = r.x; raw[b][1] = r.y;
                        if (a.x_dtype == EOQ_B200_F16) {
                            const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
                            const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
                            v[b][0] = f0.x; v[b][1] = f0.y; v[b][2] = f1.x; v[b][3] = f1.y;
                        } else {
                            v[b][0] = __uint_as_float(r.x << 16); v[b][1] = __uint_as_float(r.x & 0xFFFF0000u);
                            v[b][2] = __uint_as_float(r.y << 16); v[b][3] = __uint_as_float(r.y & 0xFFFF0000u);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) v[b][i] = load_x(a.x, i0 + i, a.x_dtype);
                        if (XH != 0) {
                            const uint16_t *h = reinterpret_cast<const uint16_t *>(a.x) + i0;
                            raw[b][0] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
                            raw[b][1] = (uint32_t)h[2] | ((uint32_t)h[3] << 16);
                        }
                    }
                }
            }
            // the bulk of the tiles is requested behind the first x loads, so that these do not queue behind megabytes
            if (then_rest && base == 0) tail_copy();
#pragma unroll
            for (int b = 0; b < BT; b++) {
                float sum = (v[b][0] + v[b][1]) + (v[b][2] + v[b][3]);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (on) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (XH != 0) xs16[(c + i) * BT + b] = (uint16_t)(raw[b][i >> 1] >> ((i & 1) * 16));
                        else xs[(c + i) * BT + b] = v[b][i];
                    }
                    if ((lane & 3u) == 0) aux[(c / 16u) * BT + b] = sum;
                }
            }
        }
        __syncwarp();
    };

    // The pairs are cut into nchunks = waves x gridDim.x runs of consecutive pairs, as equal as possible and at most
    // sixteen long; CTA c takes chunks c, c + gridDim.x, ...  A chunk holds neighbouring column segments of (mostly)
    // one pair of row blocks, whose results the CTA adds up in shared memory before anything goes to global memory.
    const uint32_t nchunks = ((npairs + kWarps * gridDim.x - 1u) / (kWarps * gridDim.x)) * gridDim.x;
    const bool narrow = ((uint64_t)(npairs + 1u) * (nchunks + 1u)) >> 32 == 0;      // the products below fit 32 bits
    // Matrices much wider than tall: the segments of a pair of row blocks are spread over many CTAs (more than six
    // partial rows to add up).  Then the elected warp does not poll them alone: it posts a notice and all warps of its CTA
    // take a share of the slots (see below).  The condition is the same for every CTA of the grid.
    const bool coop = a.pair_partials && (uint64_t)a.nseg * nchunks > 6ull * npairs;
    auto chunk_lo = [&](uint32_t t) { return narrow ? t * npairs / nchunks : (uint32_t)((uint64_t)t * npairs / nchunks); };
    auto chunk_of = [&](uint32_t qq) {
        return narrow ? ((qq + 1u) * nchunks - 1u) / npairs : (uint32_t)((((uint64_t)qq + 1u) * nchunks - 1u) / npairs);
    };
    uint32_t t = blockIdx.x;
    uint32_t cs = chunk_lo(t + 1) - chunk_lo(t);
    uint32_t q = chunk_lo(t) + warp;
    bool have = warp < cs;
    if (have) open_pair(q);
    __syncthreads();                                   // the table barrier is initialised before anyone polls it
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (have) load_x_segment(true);
    mbar_wait_suspended(tab_bar, 0u, a.status);

    // `uses` counts the pairs this warp has opened: a warp that sits out a short chunk does not arm its barriers,
    // so their phase follows its own count, not the CTA's trip count
    for (uint32_t uses = 0; t < nchunks;) {
        const uint32_t parity = uses & 1u;
        const PairGeo cur = geo;
        const bool cur_b = cur.has_b, cur_have = have;
        if (coop && lane == 0) jobs[warp * 8] = 0u;
        const uint32_t row[2] = {cur.row0[0] + lane * G, cur.row0[1] + lane * G};
        const uint32_t len_a = __shfl_sync(0xffffffffu, dl.y, 0) << 6, len_b = __shfl_sync(0xffffffffu, dl.y, 8) << 6;   // tile bytes
        float y[2][G][BT];
#pragma unroll
        for (int k = 0; k < 2; k++)
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) y[k][j][b] = 0.0f;

        if (cur_have) {
            uses++;
            // group scales of the first two runs: requested before anything is waited for, used at the end of a run
            // (transposed copy of the scales: one 8-byte word holds the three scales of a lane's rows for one group, and the
            // words of a warp's 32 lanes are contiguous, so a run's scales are one coalesced load per tile)
            const uint32_t sc_stride = a.Npad / G;
            const uint2 *sc_ptr[2];
            uint2 sc_cur[2], sc_next[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                sc_ptr[k] = a.scales_t + row[k] / G;
                sc_cur[k] = ldg_u32x2_pinned(sc_ptr[k] + (size_t)(cur.col0 / a.group) * sc_stride);
                sc_next[k] = make_uint2(0u, 0u);
            }
            if ((cur.col0 / a.group + 1) * a.group < cur.col0 + cur.ncols) {
#pragma unroll
                for (int k = 0; k < 2; k++) sc_next[k] = ldg_u32x2_pinned(sc_ptr[k] + (size_t)(cur.col0 / a.group + 1) * sc_stride);
            }
            PairChain ch[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                mbar_wait_suspended(bars + k * 64, parity, a.status);
                ch[k].x = lds_u32(stage[k] + lane * 4u);
                ch[k].addr = stage[k] + 128u + lane * 2u;
                ch[k].w = lds_u16(ch[k].addr);
            }
            uint32_t c = cur.col0;
            const uint32_t col0 = cur.col0, cend = cur.col0 + cur.ncols;
            const uint32_t nchunks0 = min(kMaxChunks, (len_a + kChunk - 1) / kChunk), nchunks1 = min(kMaxChunks, (len_b + kChunk - 1) / kChunk);
            while (c < cend) {
                const uint32_t g = c / a.group;
                const uint32_t rstart = c, rend = min(cend, (g + 1) * a.group);
                float acc[2][G][BT];
#pragma unroll
                for (int k = 0; k < 2; k++)
#pragma unroll
                    for (int j = 0; j < G; j++)
#pragma unroll
                        for (int b = 0; b < BT; b++) acc[k][j][b] = 0.0f;

                // Eight columns per trip.  After s steps no lane has read past word row s, and chunk j holds rows
                // 16 j - 2 .. 16 j + 13: waiting for chunk j eight steps before column 16 j is always early enough.
#pragma unroll 1
                for (; c < rend; c += 8) {
                    const uint8_t *xp = reinterpret_cast<const uint8_t *>(xs) + (size_t)(c - col0) * BT * kXBytes;
                    pair_steps4<G, BT, XH>(xp, tab_addr, mask, p, magic0, magic1, magic2, c64, c1, ch[0], ch[1], acc);
                    pair_steps4<G, BT, XH>(xp + 4 * BT * kXBytes, tab_addr, mask, p, magic0, magic1, magic2, c64, c1, ch[0], ch[1], acc);
                    if (((c - col0) & 8u) == 0) {
                        const uint32_t j = (c - col0) / 16u + 1u;
                        if (j < nchunks0) mbar_wait_suspended(bars + j * 8, parity, a.status);
                        if (j < nchunks1) mbar_wait_suspended(bars + 64 + j * 8, parity, a.status);
                    }
                }

                float rs[BT];
#pragma unroll
                for (int b = 0; b < BT; b++) rs[b] = 0.0f;
                for (uint32_t u = (rstart - col0) / 16; u < (rend - col0) / 16; u++)
#pragma unroll
                    for (int b = 0; b < BT; b++) rs[b] += aux[u * BT + b];
                const float corr[3] = {Int4Field<F::field_bit(0)>::kCorr,
                                       Int4Field<F::field_bit(G > 1 ? 1 : 0)>::kCorr,
                                       Int4Field<F::field_bit(G > 2 ? 2 : 0)>::kCorr};
#pragma unroll
                for (int k = 0; k < 2; k++)
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        // rows past the matrix have scale 0 in the transposed copy
                        const float sc = half_bits_to_float((uint16_t)(j == 0 ? sc_cur[k].x : j == 1 ? sc_cur[k].x >> 16 : sc_cur[k].y));
#pragma unroll
                        for (int b = 0; b < BT; b++) y[k][j][b] = fmaf(sc, acc[k][j][b] - corr[j] * rs[b], y[k][j][b]);
                    }
                // rotate the scales at the end of the run, when the loads issued a run ago have long landed
#pragma unroll
                for (int k = 0; k < 2; k++) sc_cur[k] = sc_next[k];
                if ((g + 2) * a.group < cend) {
#pragma unroll
                    for (int k = 0; k < 2; k++) sc_next[k] = ldg_u32x2_pinned(sc_ptr[k] + (size_t)(g + 2) * sc_stride);
                }
            }
            __syncwarp();
            // this warp's sums go into its first stage buffer, which nothing reads any more: [tile][row j][batch][lane]
            float *red = reinterpret_cast<float *>(mine);
#pragma unroll
            for (int k = 0; k < 2; k++)
#pragma unroll
                for (int j = 0; j < G; j++)
#pragma unroll
                    for (int b = 0; b < BT; b++) red[((k * G + j) * BT + b) * 32 + lane] = y[k][j][b];
        }
        // The first warp of each run of pairs that share a row-block pair adds the run up, in warp order.
        const uint32_t rbp = q / a.nseg, seg = q - rbp * a.nseg;
        const bool leader = cur_have && (warp == 0 || seg == 0);
        // A leader that will meet other CTAs through the empty-slot scheme takes its ticket now: the ticket only elects
        // who adds up (the last to take one; every other contributor is then at least this far and needs nothing from
        // the elected one to deliver its row), so its round trip can overlap the barrier and the sums below.
        uint32_t early_ticket = 0;
        const uint32_t first_q = rbp * a.nseg;
        const uint32_t count = leader ? chunk_of(first_q + a.nseg - 1u) - chunk_of(first_q) + 1u : 1u;
        if (leader && count > 1 && a.pair_partials && lane == 0) early_ticket = atomicAdd(a.counters + cur.row0[0] / (32u * G), 1u);
        __syncthreads();

        if (leader) {
            const uint32_t run = min(cs - warp, a.nseg - seg);
            for (uint32_t w = 1; w < run; w++) {
                const float *red = reinterpret_cast<const float *>(mine + (size_t)w * region);
#pragma unroll
                for (int k = 0; k < 2; k++)
#pragma unroll
                    for (int j = 0; j < G; j++)
#pragma unroll
                        for (int b = 0; b < BT; b++) y[k][j][b] += red[((k * G + j) * BT + b) * 32 + lane];
            }
            // runs of this row-block pair are numbered by the chunk they fall in
            const uint32_t slot = t - chunk_of(first_q);
            bool last = true;
            if (count > 1 && a.pair_partials) {
                // Partial rows meet without a fence: an empty slot holds the pattern kEmpty; whoever took the last ticket
                // keeps its row in registers and polls the others' slots until every value has arrived (the others are
                // past their tickets and on their way to these stores, so this ends within their own remaining work;
                // bounded all the same), adds the rows in run order and leaves the slots empty for the next launch.
                constexpr uint32_t kEmpty = 0xFFFFFFFFu;
                uint32_t *slots = reinterpret_cast<uint32_t *>(a.pair_partials);
                const uint32_t ticket = __shfl_sync(0xffffffffu, early_ticket, 0);
                last = ticket == count - 1u;
                if (!last) {
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        if (k == 1 && !cur_b) continue;
                        uint32_t *dst = slots + ((size_t)slot * a.Npad + row[k]) * BT;
#pragma unroll
                        for (int j = 0; j < G; j++)
#pragma unroll
                            for (int b = 0; b < BT; b++) {
                                const uint32_t bits = __float_as_uint(y[k][j][b]);
                                __stcg(dst + j * BT + b, bits == kEmpty ? 0x7FC00000u : bits);     // a NaN stays a NaN
                            }
                    }
                } else if (coop) {
                    // post the notice; the CTA adds the runs' rows up together below, this warp writes the result.  Its own
                    // row goes into its slot like everyone else's, so that the order of the additions does not depend on who
                    // was elected.
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        if (k == 1 && !cur_b) continue;
                        uint32_t *dst = slots + ((size_t)slot * a.Npad + row[k]) * BT;
#pragma unroll
                        for (int j = 0; j < G; j++)
#pragma unroll
                            for (int b = 0; b < BT; b++) {
                                const uint32_t bits = __float_as_uint(y[k][j][b]);
                                __stcg(dst + j * BT + b, bits == kEmpty ? 0x7FC00000u : bits);
                                y[k][j][b] = 0.0f;
                            }
                    }
                    if (lane == 0) {
                        jobs[warp * 8 + 1] = count; jobs[warp * 8 + 2] = slot; jobs[warp * 8 + 3] = cur.row0[0];
                        jobs[warp * 8 + 4] = cur.row0[1]; jobs[warp * 8 + 5] = cur_b ? 1u : 0u;
                        jobs[warp * 8] = 1u;
                    }
                    last = false;
                } else {
                    float own[2][G][BT];
#pragma unroll
                    for (int k = 0; k < 2; k++)
#pragma unroll
                        for (int j = 0; j < G; j++)
#pragma unroll
                            for (int b = 0; b < BT; b++) { own[k][j][b] = y[k][j][b]; y[k][j][b] = 0.0f; }
                    // Up to kP slots are polled together: the loads of every slot still missing are issued before any of them
                    // is tested, so a round costs one trip to the L2 however many slots it covers; the rows are added in
                    // slot order all the same.
                    constexpr int kP = G * BT <= 3 ? 4 : G * BT <= 6 ? 2 : 1;
                    const long long t0 = clock64();
                    for (uint32_t s0 = 0; s0 < count; s0 += kP) {
                        uint32_t v[kP][2][G][BT];
                        uint32_t pending = 0;
#pragma unroll
                        for (int u = 0; u < kP; u++)
                            if (s0 + u < count && s0 + u != slot) pending |= 1u << u;
                        while (pending) {
#pragma unroll
                            for (int u = 0; u < kP; u++)
                                if (pending >> u & 1u) {
#pragma unroll
                                    for (int k = 0; k < 2; k++)
#pragma unroll
                                        for (int j = 0; j < G; j++)
#pragma unroll
                                            for (int b = 0; b < BT; b++) {
                                                v[u][k][j][b] = 0u;
                                                if (k == 0 || cur_b)
                                                    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v[u][k][j][b])
                                                                 : "l"(slots + ((size_t)(s0 + u) * a.Npad + row[k]) * BT + j * BT + b) : "memory");
                                            }
                                }
#pragma unroll
                            for (int u = 0; u < kP; u++)
                                if (pending >> u & 1u) {
                                    bool all = true;
#pragma unroll
                                    for (int k = 0; k < 2; k++)
#pragma unroll
                                        for (int j = 0; j < G; j++)
#pragma unroll
                                            for (int b = 0; b < BT; b++) all = all && v[u][k][j][b] != kEmpty;
                                    if (all) pending &= ~(1u << u);
                                }
                            if (pending && clock64() - t0 > (1ll << 31)) { *a.status = 3u; pending = 0; }   // ~1 s: give up, the host reports it
                        }
#pragma unroll
                        for (int u = 0; u < kP; u++)
                            if (s0 + u < count)
#pragma unroll
                                for (int k = 0; k < 2; k++)
#pragma unroll
                                    for (int j = 0; j < G; j++)
#pragma unroll
                                        for (int b = 0; b < BT; b++) y[k][j][b] += s0 + u == slot ? own[k][j][b] : __uint_as_float(v[u][k][j][b]);
                    }
                    for (uint32_t s = 0; s < count; s++)
#pragma unroll
                        for (int k = 0; k < 2; k++) {
                            if (k == 1 && !cur_b) continue;
#pragma unroll
                            for (int j = 0; j < G; j++)
#pragma unroll
                                for (int b = 0; b < BT; b++) __stcg(slots + ((size_t)s * a.Npad + row[k]) * BT + j * BT + b, kEmpty);
                        }
                    if (lane == 0) a.counters[cur.row0[0] / (32u * G)] = 0u;
                }
            } else if (count > 1) {
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    if (k == 1 && !cur_b) continue;
                    float *dst = a.partials + ((size_t)slot * a.Npad + row[k]) * BT;
#pragma unroll
                    for (int j = 0; j < G; j++)
#pragma unroll
                        for (int b = 0; b < BT; b++) __stcg(dst + j * BT + b, y[k][j][b]);
                }
                __threadfence();
                __syncwarp();
                uint32_t ticket = 0;
                if (lane == 0) ticket = atomicAdd(a.counters + cur.row0[0] / (32u * G), 1u);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                last = ticket == count - 1u;
                if (last) {
                    __threadfence();
#pragma unroll
                    for (int k = 0; k < 2; k++)
#pragma unroll
                        for (int j = 0; j < G; j++)
#pragma unroll
                            for (int b = 0; b < BT; b++) y[k][j][b] = 0.0f;
                    constexpr int kU = BT <= 2 ? 4 : 2;     // runs whose loads are in flight together
                    for (uint32_t s0 = 0; s0 < count; s0 += kU) {
                        float v[kU][2][G][BT];
#pragma unroll
                        for (int u = 0; u < kU; u++)
#pragma unroll
                            for (int k = 0; k < 2; k++) {
                                const float *src = a.partials + ((size_t)min(s0 + u, count - 1u) * a.Npad + row[k]) * BT;
#pragma unroll
                                for (int j = 0; j < G; j++)
#pragma unroll
                                    for (int b = 0; b < BT; b++) v[u][k][j][b] = (k == 0 || cur_b) ? __ldcg(src + j * BT + b) : 0.0f;
                            }
#pragma unroll
                        for (int u = 0; u < kU; u++)
                            if (s0 + u < count)
#pragma unroll
                                for (int k = 0; k < 2; k++)
#pragma unroll
                                    for (int j = 0; j < G; j++)
#pragma unroll
                                        for (int b = 0; b < BT; b++) y[k][j][b] += v[u][k][j][b];
                    }
                    if (lane == 0) a.counters[cur.row0[0] / (32u * G)] = 0u;
                }
            }
            if (last) {
                write_rows<G, BT>(a, row[0], y[0]);
                if (cur_b) write_rows<G, BT>(a, row[1], y[1]);
            }
        }
        if (coop) {
            // Every notice is served by the whole CTA: warp w polls slots w, w + 16, ... (all its loads of a round in
            // flight together), empties them, and leaves its share of the sum in its second stage buffer; the warp that
            // posted the notice adds the shares in warp order to its own row and writes the result.  Which warp takes which
            // slot is fixed by the geometry, so results are the same from run to run.
            constexpr uint32_t kEmpty = 0xFFFFFFFFu;
            uint32_t *slots = reinterpret_cast<uint32_t *>(a.pair_partials);
            __syncthreads();
            for (uint32_t jw = 0; jw < (uint32_t)kWarps; jw++) {
                if (jobs[jw * 8] == 0u) continue;              // same answer in every warp
                const uint32_t jcount = jobs[jw * 8 + 1];
                const uint32_t jrow[2] = {jobs[jw * 8 + 3] + lane * G, jobs[jw * 8 + 4] + lane * G};
                const bool jb = jobs[jw * 8 + 5] != 0u;
                float share[2][G][BT];
#pragma unroll
                for (int k = 0; k < 2; k++)
#pragma unroll
                    for (int j = 0; j < G; j++)
#pragma unroll
                        for (int b = 0; b < BT; b++) share[k][j][b] = 0.0f;
                const long long t0 = clock64();
                for (uint32_t sl = warp; sl < jcount; sl += kWarps) {
                    uint32_t v[2][G][BT];
                    bool all = false;
                    while (!all) {
                        all = true;
#pragma unroll
                        for (int k = 0; k < 2; k++)
#pragma unroll
                            for (int j = 0; j < G; j++)
#pragma unroll
                                for (int b = 0; b < BT; b++) {
                                    v[k][j][b] = 0u;
                                    if (k == 0 || jb)
                                        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v[k][j][b])
                                                     : "l"(slots + ((size_t)sl * a.Npad + jrow[k]) * BT + j * BT + b) : "memory");
                                }
#pragma unroll
                        for (int k = 0; k < 2; k++)
#pragma unroll
                            for (int j = 0; j < G; j++)
#pragma unroll
                                for (int b = 0; b < BT; b++)
                                    if (k == 0 || jb) all = all && v[k][j][b] != kEmpty;
                        if (!all && clock64() - t0 > (1ll << 31)) { *a.status = 3u; all = true; }   // ~1 s: give up, the host reports it
                    }
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        if (k == 1 && !jb) continue;
#pragma unroll
                        for (int j = 0; j < G; j++)
#pragma unroll
                            for (int b = 0; b < BT; b++) {
                                share[k][j][b] += __uint_as_float(v[k][j][b]);
                                __stcg(slots + ((size_t)sl * a.Npad + jrow[k]) * BT + j * BT + b, kEmpty);
                            }
                    }
                }
                float *help = reinterpret_cast<float *>(mine + a.stage_bytes);
#pragma unroll
                for (int k = 0; k < 2; k++)
#pragma unroll
                    for (int j = 0; j < G; j++)
#pragma unroll
                        for (int b = 0; b < BT; b++) help[((k * G + j) * BT + b) * 32 + lane] = share[k][j][b];
                __syncthreads();
                if (warp == jw) {
                    for (uint32_t w = 0; w < (uint32_t)kWarps; w++) {
                        const float *hw = reinterpret_cast<const float *>(smem + tab_bytes + 128 + kPairJobBytes + (size_t)w * region + a.stage_bytes);
#pragma unroll
                        for (int k = 0; k < 2; k++)
#pragma unroll
                            for (int j = 0; j < G; j++)
#pragma unroll
                                for (int b = 0; b < BT; b++) y[k][j][b] += hw[((k * G + j) * BT + b) * 32 + lane];
                    }
                    // every slot is empty again; the counter goes back to zero for the next launch
                    if (lane == 0) a.counters[jobs[jw * 8 + 3] / (32u * G)] = 0u;
                    write_rows<G, BT>(a, jrow[0], y[0]);
                    if (jb) write_rows<G, BT>(a, jrow[1], y[1]);
                }
                __syncthreads();
            }
        }

        t += gridDim.x;
        if (t < nchunks) {
            __syncthreads();                           // every leader has read the sums before the buffers are refilled
            cs = chunk_lo(t + 1) - chunk_lo(t);
            q = chunk_lo(t) + warp;
            have = warp < cs;
            if (have) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the copies overwrite buffers read through ordinary loads
                open_pair(q);
                load_x_segment(true);
            }
        }
    }
    gather_finish(a);          // row-sharded runs: wait for the other ranks' rows and unpack them
}

static std::atomic<int> g_gemv_pairs{1};
void set_gemv_pairs(int v) { g_gemv_pairs.store(v != 0); }

// Rows of partial sums a row-block pair can need: the most runs any pair's segments are cut into on this device.
uint32_t pair_partial_slots(uint32_t nrb, uint32_t nseg)
{
    const uint32_t sms = (uint32_t)std::max(1, device_sm_count());
    const uint32_t nrbp = (nrb + 1u) / 2u, npairs = nrbp * nseg;
    if (npairs == 0) return 0;
    const uint32_t grid = std::max(1u, std::min(sms, npairs));
    const uint32_t nchunks = ((npairs + 16u * grid - 1u) / (16u * grid)) * grid;
    auto chunk_of = [&](uint32_t q) { return (uint32_t)((((uint64_t)q + 1u) * nchunks - 1u) / npairs); };
    uint32_t most = 1;
    for (uint32_t r = 0; r < nrbp; r++) most = std::max(most, chunk_of(r * nseg + nseg - 1u) - chunk_of(r * nseg) + 1u);
    return most;
}

// Activation rows one launch of the pair kernel can take: 4 if the staging buffers leave room for four fp32 x
// segments, or for four 16-bit ones when x is fp16 / bf16; else 2; 0 if even two do not fit.
static uint32_t pair_rows_per_launch(const GemvArgs &a)
{
    if (pair_smem_bytes(a.p, 4, a.stage_bytes, a.max_ncols, 16) <= 227 * 1024) return 4;
    if (a.x_dtype != EOQ_B200_F32 && pair_smem_bytes(a.p, 4, a.stage_bytes, a.max_ncols, 16, 2) <= 227 * 1024) return 4;
    return pair_smem_bytes(a.p, 2, a.stage_bytes, a.max_ncols, 16) <= 227 * 1024 ? 2u : 0u;
}

// Whether launch_gemv would take the pair kernel for these arguments (the ring kernel needs a.partials instead).
bool gemv_takes_pairs(const GemvArgs &a, uint32_t G, uint32_t bits, uint32_t kind)
{
    if (!(kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4 && G == 3 && g_gemv_pairs.load() && a.stage_bytes && a.scales_t)) return false;
    const uint32_t per = pair_rows_per_launch(a);
    return per && a.stage_bytes <= 8192u && (a.batch <= per || a.world <= 1);
}

// Returns -1 if the pair kernel does not apply (shared memory), else a cudaError_t.
template <int G, int BT, int XH = 0>
static int launch_gemv_pairs(const GemvArgs &a, cudaStream_t st)
{
    struct Cfg { size_t smem = 0; int sms = 0; };
    static Cfg cfg[16];
    static std::mutex mu;
    constexpr int THREADS = 512;
    auto kern = gemv_pairs_kernel<G, BT, THREADS, XH>;
    if (a.stage_bytes == 0 || a.stage_bytes > 8192u || a.max_ncols == 0 || a.nrb == 0 || !a.scales_t) return -1;   // eight 1 KB chunks per tile
    if (a.stage_bytes < 2u * G * BT * 128u) return -1;      // a tile buffer also holds the warp's sums after the loop: [2][G][BT][32] floats
    const size_t smem = pair_smem_bytes(a.p, BT, a.stage_bytes, a.max_ncols, THREADS / 32, XH ? 2 : 4);
    if (smem > 227 * 1024) return -1;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    Cfg c;
    {
        std::lock_guard<std::mutex> lock(mu);
        Cfg &slot = cfg[dev & 15];
        if (slot.smem < smem || slot.sms == 0) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            slot.smem = smem; slot.sms = device_sm_count();
        }
        c = slot;
    }
    const uint32_t npairs = ((a.nrb + 1u) / 2u) * a.nseg;
    const uint32_t grid = max(1u, min((uint32_t)c.sms, npairs));   // the kernel cuts the pairs into equal runs per CTA
    e = launch_with_pdl(kern, dim3(grid), dim3(THREADS), smem, st, a);
    g_launches++;
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_gemv(const GemvArgs &a, uint32_t G, uint32_t bits, uint32_t kind, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (gemv_takes_pairs(a, G, bits, kind)) {
        // The pair kernel takes as many activation rows per launch as leave room for its staging buffers (4, else 2);
        // more rows run as consecutive launches over row slices, which is still faster than one launch of the ring kernel.
        const uint32_t per = pair_rows_per_launch(a);
        const bool x16 = per == 4 && pair_smem_bytes(a.p, 4, a.stage_bytes, a.max_ncols, 16) > 227 * 1024;   // four rows only as 16-bit segments
        static const size_t esz[3] = {2, 2, 4};
        for (uint32_t b0 = 0; b0 < a.batch; b0 += per) {
            GemvArgs s = a;
            s.batch = min(per, a.batch - b0);
            s.x = static_cast<const uint8_t *>(a.x) + (size_t)b0 * a.K * esz[a.x_dtype];
            s.y = static_cast<uint8_t *>(a.y) + (size_t)b0 * a.N * esz[a.y_dtype];
            const int r = s.batch <= 1 ? launch_gemv_pairs<3, 1>(s, st) : s.batch <= 2 ? launch_gemv_pairs<3, 2>(s, st)
                        : !x16 ? launch_gemv_pairs<3, 4>(s, st)
                        : a.x_dtype == EOQ_B200_F16 ? launch_gemv_pairs<3, 4, 1>(s, st) : launch_gemv_pairs<3, 4, 2>(s, st);
            if (r != 0) return r == -1 ? (int)cudaErrorInvalidValue : r;
        }
        return 0;
    }
    if (a.nseg > 1 && !a.partials) return (int)cudaErrorInvalidValue;      // the ring kernel has no scratch to meet in
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4) {
        if (G == 1) return launch_gemv_bt<1, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 2) return launch_gemv_bt<2, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 3) return launch_gemv_bt<3, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    }
    // the other symmetric integer codes (kernels are templated on the field width; the kind tag is the integer family's)
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 2 && G == 3) return launch_gemv_bt<3, 2, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 3 && G == 3) return launch_gemv_bt<3, 3, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 8 && G == 1) return launch_gemv_bt<1, 8, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    if (kind == EOQ_B200_KIND_Q5_POLAR && bits == 5) {
        if (G == 1) return launch_gemv_bt<1, 5, EOQ_B200_KIND_Q5_POLAR>(a, st);
        if (G == 2) return launch_gemv_bt<2, 5, EOQ_B200_KIND_Q5_POLAR>(a, st);
    }
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// Second half of the fused all-gather: unpack what the other ranks sent (GemvArgs describes the words).  Every
// word of the slot's receive buffer that another rank owns is polled until it carries this gather's epoch, and its
// values are written into the full output vector.  The wait is bounded by a.gather_limit clock ticks, after which the
// status word is set and the kernel carries on.  The CTA that finishes last advances the slot's epoch.  Called by all
// threads of every CTA at the end of the fused GEMV kernels, and by gather_wait_kernel on its own.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void gather_finish(const GemvArgs &a)
{
    if (a.world <= 1) return;
    const uint32_t G = a.gather_g;
    const uint32_t epoch = __ldcg(a.gather_epoch) + 1u;
    const bool f32 = a.y_dtype == EOQ_B200_F32;
    const uint32_t wpr = f32 ? a.N : a.Npad / G, used = f32 ? a.N : (a.N + G - 1u) / G;
    const uint32_t per_b = (a.world - 1u) * used, total = a.batch * per_b;
    const uint64_t *ll = a.peer_ll[a.rank];
    const long long t0 = clock64();
    bool gave_up = false;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t b = i / per_b, rem = i - b * per_b, pi = rem / used, wi = rem - pi * used;
        const uint32_t pr = pi + (pi >= a.rank ? 1u : 0u);
        const uint64_t *src = ll + (size_t)(b * a.world + pr) * wpr + wi;
        uint32_t lo = 0, hi = 0;
        while (!gave_up) {
            asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "l"(src) : "memory");
            if (f32 ? hi == epoch : (hi >> 16) == (epoch & 0xFFFFu)) break;
            if (clock64() - t0 > a.gather_limit) gave_up = true;
        }
        if (gave_up) continue;
        const size_t at = (size_t)b * a.n_total + (size_t)pr * a.N;
        if (f32) {
            reinterpret_cast<uint32_t *>(a.y)[at + wi] = lo;
        } else {
            uint16_t *dst = reinterpret_cast<uint16_t *>(a.y) + at;
            const uint32_t r = wi * G;
            dst[r] = (uint16_t)lo;
            if (G > 1 && r + 1 < a.N) dst[r + 1] = (uint16_t)(lo >> 16);
            if (G > 2 && r + 2 < a.N) dst[r + 2] = (uint16_t)hi;
        }
    }
    if (gave_up) *a.gather_status = 4u;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(a.gather_done, 1u) == gridDim.x - 1u) {
            *a.gather_done = 0u;
            *a.gather_epoch = epoch;
        }
    }
}

// The wait on its own: for receive buffers filled by something other than the GEMV of this launch.
__global__ void __launch_bounds__(256) gather_wait_kernel(const GemvArgs a)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    gather_finish(a);
}

int launch_gather_wait(const GemvArgs &a, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const uint32_t total = a.batch * a.n_total;
    const uint32_t grid = max(1u, min(64u, (total + 255u) / 256u));
    cudaError_t e = launch_with_pdl(gather_wait_kernel, dim3(grid), dim3(256), 0, st, a);
    g_launches++;
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Decode the tiled layout back to memory: symbols (packed two per byte as
// QuantizedLinear.packed_weight, or one per byte) and/or the dequantised
// matrix (INT4 only; w = (n - 7) * scale).  One warp per tile; a lane buffers
// eight columns of each of its rows and writes them with one store per row.
// ---------------------------------------------------------------------------
template <int G, int BITS, int KIND>
__global__ void __launch_bounds__(256) decode_tiles_kernel(const DecodeArgs a)
{
    using F = Fmt<G, BITS>;
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tab = reinterpret_cast<uint32_t *>(smem);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const uint32_t K = a.K, M = 1u << a.p;
    for (uint32_t i = tid * 4; i < M; i += blockDim.x * 4)
        *reinterpret_cast<uint4 *>(tab + i) = __ldg(reinterpret_cast<const uint4 *>(a.table + i));
    RingCtlT<RingSmall> ring;
    ring_setup(ring, smem + smem_table_bytes(a.p), warp, nwarps, lane, a.status);
    __syncthreads();

    const uint32_t mask = M - 1u, p = a.p, sgroups = K / a.group;
    for (uint32_t t = blockIdx.x + gridDim.x * warp; t < a.ntiles; t += gridDim.x * nwarps) {
        const TileDesc d = a.tiles[t];
        const TileSrc base = tile_src(a.stream, a.head_bytes, t, d);
        uint32_t x;
        WordState ws;
        tile_open(ring, d, base, lane);
        const bool ring_mode = tile_begin(ring, ws, d, base, lane, x);
        const uint32_t row = d.row0 + lane * G;
        // sixteen columns at a time: a lane's fp16 / bf16 output for one row is then a whole 32-byte sector
        for (uint32_t c = d.col0; c < d.col0 + d.ncols; c += 16) {
            uint32_t sym[G][16];
            if (ring_mode) {
                ring_sync_step(ring, ws, lane);
#pragma unroll
                for (int s = 0; s < 16; s++) {
                    const uint32_t e = rans_step(tab, x, mask, p, F::kBiasMask);
#pragma unroll
                    for (int j = 0; j < G; j++) sym[j][s] = (e >> F::field_bit(j)) & F::kFieldMask;
                    rans_renorm<true>(x, ws);
                }
            } else {
#pragma unroll
                for (int s = 0; s < 16; s++) {
                    const uint32_t e = rans_step(tab, x, mask, p, F::kBiasMask);
#pragma unroll
                    for (int j = 0; j < G; j++) sym[j][s] = (e >> F::field_bit(j)) & F::kFieldMask;
                    rans_renorm<false>(x, ws);
                }
            }
#pragma unroll
            for (int j = 0; j < G; j++) {
                const uint32_t r = row + j;
                if (r >= a.N) continue;
                if (a.out_sym) {
                    if (a.packed) {
                        uint2 v = make_uint2(0, 0);
#pragma unroll
                        for (int s = 0; s < 8; s++) { v.x |= sym[j][s] << (4 * s); v.y |= sym[j][s + 8] << (4 * s); }
                        *reinterpret_cast<uint2 *>(a.out_sym + (size_t)r * (K / 2) + c / 2) = v;
                    } else {
                        uint4 v = make_uint4(0, 0, 0, 0);
#pragma unroll
                        for (int s = 0; s < 4; s++) {
                            v.x |= sym[j][s] << (8 * s); v.y |= sym[j][s + 4] << (8 * s);
                            v.z |= sym[j][s + 8] << (8 * s); v.w |= sym[j][s + 12] << (8 * s);
                        }
                        *reinterpret_cast<uint4 *>(a.out_sym + (size_t)r * K + c) = v;
                    }
                }
                if (a.out_deq && KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                    // group is a multiple of 16 and so is c, so the sixteen columns share one scale
                    const float sc = half_bits_to_float(__ldg(a.scales + (size_t)r * sgroups + c / a.group));
                    float v[16];
#pragma unroll
                    for (int s = 0; s < 16; s++) v[s] = (float)((int)sym[j][s] - (int)((1u << (BITS - 1)) - 1u)) * sc;
                    const size_t o = (size_t)r * K + c;
                    if (a.out_dtype == EOQ_B200_F32) {
                        float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.out_deq) + o);
#pragma unroll
                        for (int q = 0; q < 4; q++) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else if (a.out_dtype == EOQ_B200_F16) {
                        __half2 h[8];
#pragma unroll
                        for (int s = 0; s < 8; s++) h[s] = __floats2half2_rn(v[2 * s], v[2 * s + 1]);
                        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(a.out_deq) + o);
                        dst[0] = reinterpret_cast<uint4 *>(h)[0];
                        dst[1] = reinterpret_cast<uint4 *>(h)[1];
                    } else {
                        __nv_bfloat162 h[8];
#pragma unroll
                        for (int s = 0; s < 8; s++) h[s] = __floats2bfloat162_rn(v[2 * s], v[2 * s + 1]);
                        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(a.out_deq) + o);
                        dst[0] = reinterpret_cast<uint4 *>(h)[0];
                        dst[1] = reinterpret_cast<uint4 *>(h)[1];
                    }
                }
            }
        }
        tile_end(ring, ring_mode);
    }
}

// ---------------------------------------------------------------------------
// The dequantised matrix of a 4-bit weight in the pair layout (three codes per step, tiles that fit the staging
// buffers): the structure of the fused GEMV without the product.  One 16-warp CTA per SM; a warp takes two
// vertically adjacent tiles, stages them whole (kilobyte chunks on their own mbarriers) and runs their two rANS chains
// side by side; a code becomes a float with one logic instruction (the field sits in mantissa bits), (code - 7) * scale
// is one exact subtraction and one multiplication, and a lane's sixteen columns of a row leave as one 32-byte sector.
// About half the instructions per weight of the one-tile-per-warp kernel above, which is bound by instruction issue.
// ---------------------------------------------------------------------------
// One 32-byte store (a whole sector, one request) to a 32-byte aligned address.
__device__ __forceinline__ void stg_256(void *p, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4, uint32_t a5, uint32_t a6, uint32_t a7)
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(a4), "r"(a5), "r"(a6), "r"(a7)
                 : "memory");
}

template <int OUT>
__global__ void __launch_bounds__(512, 1) dequant_pairs_kernel(const DecodeArgs a)
{
    constexpr int G = 3, kWarps = 16;
    constexpr uint32_t kChunk = 1024, kMaxChunks = 8;
    using F = Fmt<G, 4>;
    using F0 = Int4Field<F::field_bit(0)>;
    using F1 = Int4Field<F::field_bit(1)>;
    using F2 = Int4Field<F::field_bit(2)>;
    extern __shared__ __align__(128) uint8_t dq_smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t tab_bytes = 4u << a.p;
    const uint32_t tab_addr = smem_addr(dq_smem), tab_bar = tab_addr + tab_bytes;
    const uint32_t region = 2u * a.stage_bytes + 128u;
    const uint32_t stage[2] = {tab_addr + tab_bytes + 128u + warp * region, tab_addr + tab_bytes + 128u + warp * region + a.stage_bytes};
    const uint32_t bars = stage[0] + 2u * a.stage_bytes;       // [chain][chunk], 8 bytes each
    if (tid == 0) {
        mbar_init(tab_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(tab_bar, tab_bytes);
        for (uint32_t off = 0; off < tab_bytes; off += 16384u)
            bulk_copy_g2s(tab_addr + off, reinterpret_cast<const uint8_t *>(a.table) + off, min(16384u, tab_bytes - off), tab_bar);
    }
    if (lane < 2 * kMaxChunks) {
        mbar_init(bars + lane * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const uint32_t nrbp = (a.nrb + 1u) / 2u, npairs = nrbp * a.nseg;
    const uint32_t mask = (1u << a.p) - 1u, p = a.p;
    const uint32_t magic0 = F0::magic_reg(), magic1 = F1::magic_reg(), magic2 = F2::magic_reg();
    uint32_t c64, c1;
    asm volatile("mov.b32 %0, 64;\n\tmov.b32 %1, 1;" : "=r"(c64), "=r"(c1));
    const uint32_t head_chunks = a.head_bytes / kChunk, sc_stride = a.Npad / G;
    constexpr uint32_t kEsz = OUT == EOQ_B200_F32 ? 4u : 2u;
    mbar_wait_suspended(tab_bar, 0u, a.status);

    uint32_t uses = 0;
    // pair q goes to CTA q mod grid: every SM gets its share even when there are fewer pairs than warps
    for (uint32_t q = blockIdx.x + gridDim.x * warp; q < npairs; q += gridDim.x * kWarps, uses++) {
        const uint32_t parity = uses & 1u;
        const uint32_t rbp = q / a.nseg, seg = q - rbp * a.nseg;
        const bool has_b = 2u * rbp + 1u < a.nrb;
        const uint32_t t0 = 2u * rbp * a.nseg + seg, t1 = has_b ? t0 + a.nseg : t0;
        // lane k * 8 + j owns chunk j of tile k: descriptor, then the copy (head region or tail)
        uint2 cols = make_uint2(0u, 0u), dl = make_uint2(0u, 0u);
        if (lane < 2 * kMaxChunks) {
            const uint32_t k = lane >> 3, j = lane & 7u, tk = k ? t1 : t0;
            cols = make_uint2(__ldg(&a.tiles[tk].col0), __ldg(&a.tiles[tk].ncols));      // (the pair starts 4 bytes into a 24-byte record: two loads)
            dl = ldg_u32x2_pinned(reinterpret_cast<const uint2 *>(&a.tiles[tk].off64));
            uint32_t bytes = dl.y << 6;
            if (bytes + 64u > a.stage_bytes) { *a.status = 2u; bytes = a.stage_bytes - 64u; }   // cannot happen with a host-computed stage size
            const uint32_t bar = bars + lane * 8, off = j * kChunk;
            if (off < bytes) {
                const uint32_t n = min(kChunk, bytes - off);
                mbar_expect_tx(bar, n);
                const uint8_t *src = j < head_chunks ? a.stream + (size_t)tk * a.head_bytes + off
                                                     : a.stream + ((size_t)dl.x << 6) + (off - a.head_bytes);
                bulk_copy_g2s((k ? stage[1] : stage[0]) + off, src, n, bar);
            } else {
                mbar_arrive(bar);                       // nothing to copy: complete the phase by hand
            }
        }
        const uint32_t col0 = __shfl_sync(0xffffffffu, cols.x, 0), ncols = __shfl_sync(0xffffffffu, cols.y, 0);
        const uint32_t len_a = __shfl_sync(0xffffffffu, dl.y, 0) << 6, len_b = __shfl_sync(0xffffffffu, dl.y, 8) << 6;
        const uint32_t nch[2] = {min(kMaxChunks, (len_a + kChunk - 1) / kChunk), min(kMaxChunks, (len_b + kChunk - 1) / kChunk)};
        const uint32_t row[2] = {2u * rbp * (32u * G) + lane * G, (2u * rbp + (has_b ? 1u : 0u)) * (32u * G) + lane * G};
        // transposed scales: one 8-byte word holds the three scales of a lane's rows for one group (zero past row N)
        const uint2 *sc_ptr[2] = {a.scales_t + row[0] / G, a.scales_t + row[1] / G};
        uint2 sc_next[2];
        float sc[2][G];
#pragma unroll
        for (int k = 0; k < 2; k++) sc_next[k] = ldg_u32x2_pinned(sc_ptr[k] + (size_t)(col0 / a.group) * sc_stride);
        PairChain ch[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            mbar_wait_suspended(bars + k * 64, parity, a.status);
            ch[k].x = lds_u32(stage[k] + lane * 4u);
            ch[k].addr = stage[k] + 128u + lane * 2u;
            ch[k].w = lds_u16(ch[k].addr);
        }
        const uint32_t cend = col0 + ncols;
        for (uint32_t c = col0; c < cend; c += 16) {
            if (c == col0 || c % a.group == 0) {
                // a new scale group: take the scales requested a group ago, request the next
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    sc[k][0] = half_bits_to_float((uint16_t)sc_next[k].x);
                    sc[k][1] = half_bits_to_float((uint16_t)(sc_next[k].x >> 16));
                    sc[k][2] = half_bits_to_float((uint16_t)sc_next[k].y);
                }
                const uint32_t g = c / a.group;
                if ((g + 1) * a.group < cend) {
#pragma unroll
                    for (int k = 0; k < 2; k++) sc_next[k] = ldg_u32x2_pinned(sc_ptr[k] + (size_t)(g + 1) * sc_stride);
                }
            }
            uint32_t held[2][G][4];                                  // 16-bit outputs: the first eight columns, packed
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float v[2][G][8];
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    uint32_t u[2][3];
                    rans_step_int4<F0::kMask, F1::kMask, F2::kMask>(tab_addr, ch[0].x, mask, p, F::kBiasMask, magic0, magic1, magic2, u[0][0], u[0][1], u[0][2]);
                    rans_step_int4<F0::kMask, F1::kMask, F2::kMask>(tab_addr, ch[1].x, mask, p, F::kBiasMask, magic0, magic1, magic2, u[1][0], u[1][1], u[1][2]);
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        v[k][0][s] = (__uint_as_float(u[k][0]) - F0::kOffset) * sc[k][0];
                        v[k][1][s] = (__uint_as_float(u[k][1]) - F1::kOffset) * sc[k][1];
                        v[k][2][s] = (__uint_as_float(u[k][2]) - F2::kOffset) * sc[k][2];
                    }
                    staged_renorm(ch[0].x, ch[0].w, ch[0].addr, c64, c1);
                    staged_renorm(ch[1].x, ch[1].w, ch[1].addr, c64, c1);
                }
                if (half == 0) {
                    // After s steps no lane has read past word row s, and chunk j holds rows 16 j - 2 .. 16 j + 13:
                    // waiting for chunk j eight steps before column 16 j is always early enough.
                    const uint32_t j = (c - col0) / 16u + 1u;
                    if (j < nch[0]) mbar_wait_suspended(bars + j * 8, parity, a.status);
                    if (j < nch[1]) mbar_wait_suspended(bars + 64 + j * 8, parity, a.status);
                }
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    if (k == 1 && !has_b) continue;
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        const uint32_t r = row[k] + j;
                        if (OUT == EOQ_B200_F32) {
                            if (r < a.N)
                                stg_256(reinterpret_cast<float *>(a.out_deq) + (size_t)r * a.K + c + half * 8,
                                        __float_as_uint(v[k][j][0]), __float_as_uint(v[k][j][1]), __float_as_uint(v[k][j][2]), __float_as_uint(v[k][j][3]),
                                        __float_as_uint(v[k][j][4]), __float_as_uint(v[k][j][5]), __float_as_uint(v[k][j][6]), __float_as_uint(v[k][j][7]));
                        } else {
                            uint32_t pk[4];
#pragma unroll
                            for (int s = 0; s < 4; s++) {
                                if (OUT == EOQ_B200_F16) {
                                    const __half2 h = __floats2half2_rn(v[k][j][2 * s], v[k][j][2 * s + 1]);
                                    pk[s] = *reinterpret_cast<const uint32_t *>(&h);
                                } else {
                                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[k][j][2 * s], v[k][j][2 * s + 1]);
                                    pk[s] = *reinterpret_cast<const uint32_t *>(&h);
                                }
                            }
                            if (half == 0) {
#pragma unroll
                                for (int s = 0; s < 4; s++) held[k][j][s] = pk[s];
                            } else if (r < a.N) {
                                stg_256(reinterpret_cast<uint8_t *>(a.out_deq) + ((size_t)r * a.K + c) * kEsz,
                                        held[k][j][0], held[k][j][1], held[k][j][2], held[k][j][3], pk[0], pk[1], pk[2], pk[3]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Whether the pair form serves this call: the dequantised matrix alone, of a weight laid out for the pair kernel.
static bool dequant_takes_pairs(const DecodeArgs &a, uint32_t G, uint32_t bits, uint32_t kind)
{
    if (!(kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4 && G == 3) || !a.out_deq || a.out_sym || !a.scales_t || a.stage_bytes == 0) return false;
    if (a.group % 16u != 0 || a.K % 16u != 0) return false;
    const size_t smem = ((size_t)4 << a.p) + 128 + (size_t)16 * (2u * a.stage_bytes + 128u);
    return smem <= 227 * 1024 && (size_t)8 * 1024 >= a.stage_bytes;
}

static int launch_dequant_pairs(const DecodeArgs &a, cudaStream_t st)
{
    const size_t smem = ((size_t)4 << a.p) + 128 + (size_t)16 * (2u * a.stage_bytes + 128u);
    const uint32_t npairs = ((a.nrb + 1u) / 2u) * a.nseg;
    const uint32_t grid = max(1u, min((uint32_t)device_sm_count(), npairs));
    cudaError_t e = cudaSuccess;
#define EOQ_LAUNCH_DQ(O)                                                                                          \
    do {                                                                                                          \
        e = cudaFuncSetAttribute(dequant_pairs_kernel<O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess) dequant_pairs_kernel<O><<<grid, 512, smem, st>>>(a);                                \
    } while (0)
    if (a.out_dtype == EOQ_B200_F16) EOQ_LAUNCH_DQ(EOQ_B200_F16);
    else if (a.out_dtype == EOQ_B200_BF16) EOQ_LAUNCH_DQ(EOQ_B200_BF16);
    else EOQ_LAUNCH_DQ(EOQ_B200_F32);
#undef EOQ_LAUNCH_DQ
    if (e != cudaSuccess) return (int)e;
    g_launches++;
    return (int)cudaGetLastError();
}

template <int G, int BITS, int KIND>
static int launch_decode_tiles_t(const DecodeArgs &a, cudaStream_t st)
{
    const size_t smem = smem_table_bytes(a.p) + ring_smem_bytes<RingSmall>(256 / 32);
    auto kern = decode_tiles_kernel<G, BITS, KIND>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
    uint32_t grid = max(1u, min((uint32_t)(device_sm_count() * per_sm), a.ntiles));
    kern<<<grid, 256, smem, st>>>(a);
    g_launches++;
    return (int)cudaGetLastError();
}

int launch_decode_tiles(const DecodeArgs &a, uint32_t G, uint32_t bits, uint32_t kind, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dequant_takes_pairs(a, G, bits, kind)) return launch_dequant_pairs(a, st);
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4) {
        if (G == 1) return launch_decode_tiles_t<1, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 2) return launch_decode_tiles_t<2, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 3) return launch_decode_tiles_t<3, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    }
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 2 && G == 3) return launch_decode_tiles_t<3, 2, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 3 && G == 3) return launch_decode_tiles_t<3, 3, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 8 && G == 1) return launch_decode_tiles_t<1, 8, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    if (kind == EOQ_B200_KIND_Q5_POLAR && bits == 5) {
        if (G == 1) return launch_decode_tiles_t<1, 5, EOQ_B200_KIND_Q5_POLAR>(a, st);
        if (G == 2) return launch_decode_tiles_t<2, 5, EOQ_B200_KIND_Q5_POLAR>(a, st);
    }
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// Reference wire format: independent blocks `[1 B state_len][state BE][bytes]`,
// byte-wise renormalisation with lower bound 2^(p+8) (core/rans.py:368-419,
// eoq_rans_v2.c:307-351).  One thread per block; the table (8 bytes per slot)
// is staged in shared memory when it fits.  Every stream read is bounded by the
// block's end and every loop by the symbol count, so a corrupt stream produces
// wrong symbols but never an out-of-range access.
// ---------------------------------------------------------------------------
template <typename OutT, bool kShared>
__global__ void __launch_bounds__(128) decode_v1_kernel(const uint8_t *__restrict__ stream, const uint32_t *__restrict__ offsets,
                                                       const uint32_t *__restrict__ sizes, const V1Table *__restrict__ table,
                                                       OutT *__restrict__ out, uint32_t nblocks, uint32_t block_size,
                                                       uint32_t total, uint32_t p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint2 *tab = reinterpret_cast<const uint2 *>(table);
    if (kShared) {
        uint2 *s = reinterpret_cast<uint2 *>(smem);
        for (uint32_t i = threadIdx.x; i < (1u << p); i += blockDim.x) s[i] = __ldg(tab + i);
        __syncthreads();
        tab = s;
    }
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint32_t first = b * block_size;
    const uint32_t n = min(block_size, total - first);
    const uint32_t bytes = sizes[b];
    if (bytes == 0) return;
    const uint8_t *blk = stream + offsets[b];
    const uint32_t state_len = blk[0];
    if (1u + state_len > bytes) return;              // rejected on the host before launch
    uint32_t x = 0;
    for (uint32_t i = 0; i < state_len; i++) x = (x << 8) | blk[1 + i];
    const uint8_t *s = blk + 1 + state_len;
    uint32_t pos = 0;
    const uint32_t end = bytes - 1 - state_len;
    const uint32_t mask = (1u << p) - 1u, low = 1u << (p + 8);
    OutT *dst = out + first;
    for (uint32_t i = 0; i < n; i++) {
        const uint2 e = tab[x & mask];
        x = e.x * (x >> p) + (e.y & 0xFFFFu);
        while (x < low && pos < end) x = (x << 8) | s[pos++];
        dst[i] = (OutT)(e.y >> 16);
    }
}

static std::atomic<int> g_v1_lanes{1};
void set_v1_lanes(int v) { g_v1_lanes.store(v != 0); }
bool v1_lanes_enabled() { return g_v1_lanes.load() != 0; }
int launch_decode_v1_lanes_single(V1Task t, void *stream);

int launch_decode_v1(const uint8_t *d_stream, const uint32_t *d_offsets, const uint32_t *d_sizes,
                     const V1Table *d_table, void *d_out, int out_elem_bytes, uint32_t nblocks,
                     uint32_t block_size, uint32_t total, uint32_t p, uint32_t alphabet, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (nblocks == 0) return 0;
    (void)alphabet;
    const uint32_t grid = (nblocks + 127) / 128;
    const size_t tbytes = (size_t)8 << p;
    const bool shared = tbytes <= 128 * 1024 && nblocks >= 1024;
    cudaError_t e = cudaSuccess;
#define EOQ_LAUNCH_V1(T, S)                                                                                   \
    do {                                                                                                      \
        auto k = decode_v1_kernel<T, S>;                                                                      \
        if (S) e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tbytes);         \
        if (e == cudaSuccess)                                                                                 \
            k<<<grid, 128, S ? tbytes : 0, st>>>(d_stream, d_offsets, d_sizes, d_table,                       \
                                                 reinterpret_cast<T *>(d_out), nblocks, block_size, total, p); \
    } while (0)
    if (out_elem_bytes == 1) { if (shared) EOQ_LAUNCH_V1(uint8_t, true); else EOQ_LAUNCH_V1(uint8_t, false); }
    else if (out_elem_bytes == 2) { if (shared) EOQ_LAUNCH_V1(uint16_t, true); else EOQ_LAUNCH_V1(uint16_t, false); }
    else return (int)cudaErrorInvalidValue;
#undef EOQ_LAUNCH_V1
    if (e != cudaSuccess) return (int)e;
    g_launches++;
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Wire-format decode, one independent rANS block per LANE.
//
// A warp takes 32 consecutive blocks.  Everything a step touches is in shared memory:
//   * the decode table, in one of two forms chosen by the host: PACKED, one 32-bit entry per slot
//     {freq - 1 : p bits | symbol | slot - cum : p bits} when 2 p + symbol bits <= 32 (16 KB at p = 12, 64 KB at
//     p = 14), else TWO-LEVEL, slot -> symbol (u16) and symbol -> {freq, cum};
//   * the bytes of the 32 streams: each lane owns a 128-byte ring, stored word-interleaved ([word][lane], so lane l
//     only ever touches bank l and reads never conflict) and filled 32 bytes at a time by asynchronous 4-byte
//     copies (cp.async) issued two chunks ahead of the read position.
// Decoded symbols are collected in registers and leave as whole 32-byte sectors.  Every global read stays inside
// [chunk of the block's first byte, block end): whole words by plain copies, the block's last partial word by a copy
// with a source size.
// ---------------------------------------------------------------------------
constexpr uint32_t kV1RingBytes = 128, kV1ChunkBytes = 32;

__device__ __forceinline__ uint32_t v1_ring_addr(uint32_t ring, uint32_t lane, uint32_t pos)
{
    // byte `pos` of the lane's stream: word (pos / 4) mod 32 of the ring, column `lane`
    return ring + (((pos >> 2) & (kV1RingBytes / 4 - 1)) << 7) + (lane << 2) + (pos & 3u);
}

__device__ __forceinline__ uint32_t lds_u8(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ uint2 lds_v2(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t msb_index(uint32_t v)      // 31 - clz(v); 0xFFFFFFFF for 0
{
    uint32_t m;
    asm("bfind.u32 %0, %1;" : "=r"(m) : "r"(v));
    return m;
}

// Request chunk `c` (stream bytes [32 c, 32 c + 32)) of a lane's block into its ring.  Words wholly below `end` are
// copied whole, the block's last, partial word with a source size (the rest of the ring word is zero-filled), words at
// or past `end` not at all; a chunk may begin before the block does (never before the stream: offsets are >= 0).
__device__ __forceinline__ void v1_issue_chunk_edge(const uint8_t *stream, uint32_t lane_col, uint32_t c, uint32_t end)
{
    const uint32_t dst = lane_col + ((c & 3u) << 10);
    const uint8_t *src = stream + (size_t)c * kV1ChunkBytes;
#pragma unroll
    for (uint32_t i = 0; i < kV1ChunkBytes / 4; i++) {
        const uint32_t w = c * kV1ChunkBytes + i * 4u;
        if (w < end) {
            const uint32_t sz = min(4u, end - w);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + i * 128u), "l"(src + i * 4u), "r"(sz) : "memory");
        }
    }
}
// The same for a chunk that lies wholly inside the block's words: eight copies at constant offsets.
__device__ __forceinline__ void v1_issue_chunk_inner(const uint8_t *stream, uint32_t lane_col, uint32_t c)
{
    const uint32_t dst = lane_col + ((c & 3u) << 10);
    const uint8_t *src = stream + (size_t)c * kV1ChunkBytes;
#pragma unroll
    for (uint32_t i = 0; i < kV1ChunkBytes / 4; i++)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + i * 128u), "l"(src + i * 4u) : "memory");
}

// The block of one lane: decode, collect, store.  `tab` is the CTA's table in shared memory, `live` the lanes of the
// warp that have a block (they vote together).
//
// Read position: the stream bytes around it live in two registers, words wi and wi + 1 of the stream, and the byte
// offset k inside that window is kept as the selector of the byte permute that extracts the next two bytes into the
// top half of a register: sel = k * 0x1100 + 0x0100 (result byte 3 = window byte k, byte 2 = k + 1).
//
// A step in the common case is straight-line code: table look-up, state update, the number of bytes to take from the
// position of the state's highest set bit, one funnel shift that moves them in, one multiply-add that advances the
// selector; every second step the window moves on by a word if the offset has passed 4.  That form is exact while
// the state is in [2^(p+8), 2^(p+16)) at the top of a step and two bytes are left: both hold for a group of eight
// steps if they hold at its start with sixteen bytes left (a state in range comes out of the update at 2^8 or more,
// so two bytes bring it back in range).  The warp votes once per group; near the end of the blocks, and for streams
// that are not well-formed, the group runs the careful form of the step instead, which counts bytes against the end
// of the block and reads on byte by byte when two bytes were not enough, like the reference decoder.
template <typename OutT, bool PACKED>
__device__ __forceinline__ void v1_decode_lane(const V1Task &a, uint8_t *tab, uint32_t ring, uint32_t lane, uint32_t b, uint32_t live)
{
    const uint32_t p = a.p, mask = (1u << p) - 1u, low = 1u << (p + 8);
    const uint32_t tab_addr = smem_addr(tab);                                  // packed: [1 << p] words; two-level: [alphabet] {freq, cum}
    const uint32_t symtab_addr = tab_addr + a.alphabet * 8u;                   // two-level: [1 << p] u16
    const uint32_t bytes = a.sizes[b];
    const uint32_t start = a.offsets[b], end = start + bytes;
    const uint32_t first = b * a.block_size;
    uint32_t n = min(a.block_size, a.total - first);
    const uint32_t lane_col = ring + (lane << 2);
    auto ring_word = [&](uint32_t w) { return lds_u32(lane_col + ((w & (kV1RingBytes / 4 - 1)) << 7)); };

    // the first three chunks, then the header: one byte of state length, the state big-endian
    uint32_t c_next = start / kV1ChunkBytes;
    for (int i = 0; i < 3; i++) {
        v1_issue_chunk_edge(a.stream, lane_col, c_next++, end);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const uint32_t state_len = bytes ? lds_u8(v1_ring_addr(ring, lane, start)) : 0u;
    if (bytes == 0 || 1u + state_len > bytes || state_len > 4u) n = 0;      // rejected on the host before launch; takes no step that counts
    uint32_t x = 0;
    for (uint32_t i = 0; i < state_len && n; i++) x = (x << 8) | lds_u8(v1_ring_addr(ring, lane, start + 1u + i));
    const uint32_t pos0 = n ? start + 1u + state_len : end;
    uint32_t wi = pos0 >> 2, sel = (pos0 & 3u) * 0x1100u + 0x0100u, cur = ring_word(wi), nxt = ring_word(wi + 1u);

    constexpr uint32_t kPer = 32u / sizeof(OutT);                // symbols per 32-byte sector
    OutT *dst = reinterpret_cast<OutT *>(a.out) + first;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(dst) & 31u) == 0;
    const uint32_t symmask = (1u << a.sym_bits) - 1u, fshift = 32u - p, top = p + 15u, last_sym = a.alphabet - 1u;

    auto look_up = [&]() -> uint32_t {                          // x <- freq * (x >> p) + slot - cum; returns the symbol
        const uint32_t xs = x >> p;
        if (PACKED) {
            const uint32_t e = lds_u32(tab_addr + ((x & mask) << 2));      // {freq - 1 | symbol | slot - cum}
            x = (e >> fshift) * xs + ((e & mask) + xs);
            return (e >> p) & symmask;
        }
        const uint32_t slot = x & mask;
        const uint32_t sym = lds_u16(symtab_addr + (slot << 1));
        const uint2 fc = lds_v2(tab_addr + (min(sym, last_sym) << 3));     // a caller's table may name symbols past the alphabet: stay in the array
        x = fc.x * xs + (slot - fc.y);
        return sym;
    };
    auto move_window = [&]() {
        if (sel >= 0x4500u) { sel -= 0x4400u; cur = nxt; wi++; nxt = ring_word(wi + 1u); }
    };
    auto step = [&]() -> uint32_t {                             // exact under the conditions voted on per group
        const uint32_t sym = look_up();
        const uint32_t two = __byte_perm(cur, nxt, sel);
        const uint32_t t8 = (top - msb_index(x)) & 0x18u;      // 0, 8 or 16 bits to take
        x = __funnelshift_l(two, x, t8);
        sel += t8 * 0x220u;
        return sym;
    };
    auto careful_step = [&](bool counts) -> uint32_t {
        const uint32_t pos = wi * 4u + (sel >> 12);
        const uint32_t sym = look_up();
        // bytes pos and pos + 1, first one in the higher half; 0, 1 or 2 of them are taken (p <= 16), never past the block
        const uint32_t two = __byte_perm(cur, nxt, sel) >> 16;
        uint32_t take = (x < low ? 1u : 0u) + (x < (low >> 8) ? 1u : 0u);
        take = min(take, end - pos);
        x = (x << (8u * take)) | (two >> (16u - 8u * take));
        sel += take * 0x1100u;
        move_window();
        uint32_t at = pos + take;
        if (counts && x < low && at < end) {
            // only a corrupt stream gets here: read on like the reference decoder, byte by byte and inside the block
            while (x < low && at < end) { x = (x << 8) | a.stream[at]; at++; }
            wi = at >> 2;
            sel = (at & 3u) * 0x1100u + 0x0100u;
            cur = nxt = 0u;
            for (uint32_t k = 0; k < 8u; k++) {
                const uint32_t q = wi * 4u + k;
                const uint32_t byte = q >= start && q < end ? a.stream[q] : 0u;
                if (k < 4u) cur |= byte << (8u * k); else nxt |= byte << (8u * (k - 4u));
            }
        }
        return sym;
    };

    const uint32_t n_warp = __reduce_max_sync(live, n);
    const uint32_t end4 = end & ~3u;
    for (uint32_t i = 0; i < n_warp; i += kPer) {
        uint32_t w[8];
#pragma unroll
        for (uint32_t g = 0; g < kPer / 8u; g++) {
            // Every 8 steps (<= 16 bytes).  Here the chunk under the position and the next one are complete; a chunk is
            // requested as soon as the position is within two chunks of it, and every group of steps closes one copy group,
            // so that "all but the two latest groups" is exactly "everything requested two groups ago", the latest moment it
            // is needed.
            const uint32_t pos = wi * 4u + (sel >> 12);
            const bool counts = i + g * 8u < n;                 // a lane past its block only keeps the warp company
            if (counts && (pos / kV1ChunkBytes) + 3u > c_next) {
                if (c_next * kV1ChunkBytes + kV1ChunkBytes <= end4) v1_issue_chunk_inner(a.stream, lane_col, c_next);
                else v1_issue_chunk_edge(a.stream, lane_col, c_next, end);
                c_next++;
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 2;" ::: "memory");
            const bool plain = !counts || (end - pos >= 16u && pos <= end && (x >> (p + 8u)) - 1u < 255u);
            if (__all_sync(live, plain)) {
#pragma unroll
                for (uint32_t k = 0; k < 8u; k++) {
                    const uint32_t sym = step();
                    if (k & 1u) move_window();
                    const uint32_t idx = g * 8u + k;
                    if (sizeof(OutT) == 1) {
                        if ((idx & 3u) == 0) w[idx >> 2] = sym; else w[idx >> 2] |= sym << (8u * (idx & 3u));
                    } else {
                        if ((idx & 1u) == 0) w[idx >> 1] = sym; else w[idx >> 1] |= sym << 16;
                    }
                }
            } else {
#pragma unroll
                for (uint32_t k = 0; k < 8u; k++) {
                    const uint32_t sym = careful_step(counts);
                    const uint32_t idx = g * 8u + k;
                    if (sizeof(OutT) == 1) {
                        if ((idx & 3u) == 0) w[idx >> 2] = sym; else w[idx >> 2] |= sym << (8u * (idx & 3u));
                    } else {
                        if ((idx & 1u) == 0) w[idx >> 1] = sym; else w[idx >> 1] |= sym << 16;
                    }
                }
            }
        }
        if (vec_ok && i + kPer <= n) {
            uint4 *o = reinterpret_cast<uint4 *>(dst + i);
            o[0] = make_uint4(w[0], w[1], w[2], w[3]);
            o[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else if (i < n) {
            // the tail of a tensor's last block, or an output that does not start on a sector
#pragma unroll
            for (uint32_t k = 0; k < kPer; k++)
                if (i + k < n) dst[i + k] = (OutT)(w[k * sizeof(OutT) / 4u] >> (8u * sizeof(OutT) * (k % (4u / sizeof(OutT)))));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Grid: the CTAs of all tasks back to back; cta_task[blockIdx.x] says whose blocks a CTA decodes.  Each CTA builds its
// task's table in shared memory: from the normalised frequencies (a warp-wide prefix sum, then every warp fills the
// slot ranges of its share of the symbols, lanes side by side), or from a caller's slot table in the reference's
// {symbol, freq, cum} form.
__device__ __forceinline__ void v1_lanes_body(const V1Task &a, uint8_t *v1_smem)
{
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const uint32_t p = a.p, M = 1u << p;
    // shared memory: [rings: nwarps x 4 KB][table][cdf: alphabet + 1 words]
    const uint32_t ring = smem_addr(v1_smem) + warp * (kV1RingBytes * 32u);
    uint8_t *tab = v1_smem + (size_t)nwarps * kV1RingBytes * 32u;
    uint32_t *packed = reinterpret_cast<uint32_t *>(tab);
    uint2 *info = reinterpret_cast<uint2 *>(tab);
    uint16_t *symtab = reinterpret_cast<uint16_t *>(tab + (size_t)a.alphabet * 8u);
    const size_t tab_bytes = a.packed ? ((size_t)4 << p) : ((size_t)a.alphabet * 8u + ((size_t)2 << p));
    uint32_t *cdf = reinterpret_cast<uint32_t *>(tab + ((tab_bytes + 15u) & ~(size_t)15u));
    if (a.freq) {
        if (warp == 0) {
            // exclusive prefix sum of the frequencies: each lane sums a run of symbols, the runs are scanned by shuffles
            const uint32_t per = (a.alphabet + 31u) / 32u, lo = min(a.alphabet, lane * per), hi = min(a.alphabet, lo + per);
            uint32_t sum = 0;
            for (uint32_t s = lo; s < hi; s++) sum += a.freq[s];
            uint32_t incl = sum;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t o = __shfl_up_sync(0xffffffffu, incl, d);
                if ((int)lane >= d) incl += o;
            }
            uint32_t run = incl - sum;
            for (uint32_t s = lo; s < hi; s++) { cdf[s] = run; run += a.freq[s]; }
            if (lane == 31) cdf[a.alphabet] = incl;
        }
        __syncthreads();
        for (uint32_t s = warp; s < a.alphabet; s += nwarps) {
            const uint32_t c = cdf[s], f = cdf[s + 1] - c;
            if (!a.packed && lane == 0) info[s] = make_uint2(f, c);
            for (uint32_t k = lane; k < f && c + k < M; k += 32u) {
                if (a.packed) packed[c + k] = ((f - 1u) << (32u - p)) | (s << p) | k;
                else symtab[c + k] = (uint16_t)s;
            }
        }
    } else {
        // The caller's slot table, {symbol | freq << 16, cum} per slot: every CTA reads all of it once (from L2 after the
        // first), so what matters is bytes in flight: sixteen independent 16-byte loads (two slots each) per thread and
        // round, 64 KB per round and 256-thread CTA.
        auto put = [&](uint32_t slot, uint32_t e0, uint32_t e1) {
            const uint32_t sym = e0 & 0xFFFFu, freq = e0 >> 16, cum = e1 & 0xFFFFu;
            if (a.packed) {
                packed[slot] = ((freq - 1u) << (32u - p)) | ((sym & ((1u << a.sym_bits) - 1u)) << p) | ((slot - cum) & (M - 1u));
            } else {
                symtab[slot] = (uint16_t)sym;
                if (sym < a.alphabet && slot == cum) info[sym] = make_uint2(freq, cum);       // a symbol's first slot speaks for it
            }
        };
        if ((reinterpret_cast<uintptr_t>(a.table) & 15u) == 0 && M >= 2u) {
            const uint4 *src = reinterpret_cast<const uint4 *>(a.table);
            const uint32_t pairs = M >> 1;
            constexpr uint32_t kInFlight = 16;
            for (uint32_t q0 = tid; q0 < pairs; q0 += blockDim.x * kInFlight) {
                uint4 e[kInFlight];
#pragma unroll
                for (uint32_t u = 0; u < kInFlight; u++)
                    if (q0 + u * blockDim.x < pairs) e[u] = __ldg(src + q0 + u * blockDim.x);
#pragma unroll
                for (uint32_t u = 0; u < kInFlight; u++) {
                    const uint32_t q = q0 + u * blockDim.x;
                    if (q >= pairs) continue;
                    put(2u * q, e[u].x, e[u].y);
                    put(2u * q + 1u, e[u].z, e[u].w);
                }
            }
        } else {
            const uint2 *src = reinterpret_cast<const uint2 *>(a.table);
            for (uint32_t slot = tid; slot < M; slot += blockDim.x) {
                const uint2 e = __ldg(src + slot);
                put(slot, e.x, e.y);
            }
        }
    }
    __syncthreads();

    const uint32_t b = ((blockIdx.x - a.first_cta) * nwarps + warp) * 32u + lane;
    const uint32_t live = __ballot_sync(0xffffffffu, b < a.nblocks);
    if (b >= a.nblocks) return;
    if (a.out_elem_bytes == 1) {
        if (a.packed) v1_decode_lane<uint8_t, true>(a, tab, ring, lane, b, live); else v1_decode_lane<uint8_t, false>(a, tab, ring, lane, b, live);
    } else {
        if (a.packed) v1_decode_lane<uint16_t, true>(a, tab, ring, lane, b, live); else v1_decode_lane<uint16_t, false>(a, tab, ring, lane, b, live);
    }
}

__global__ void __launch_bounds__(256, 2) decode_v1_lanes_kernel(const V1Task *__restrict__ tasks, const uint32_t *__restrict__ cta_task)
{
    extern __shared__ __align__(128) uint8_t v1_smem[];
    __shared__ V1Task a;
    if (threadIdx.x < sizeof(V1Task) / 4)
        reinterpret_cast<uint32_t *>(&a)[threadIdx.x] = reinterpret_cast<const uint32_t *>(tasks + cta_task[blockIdx.x])[threadIdx.x];
    __syncthreads();
    v1_lanes_body(a, v1_smem);
}

// One tensor, its description passed by value: for entry points that may neither allocate nor copy (device pointers in,
// asynchronous launch out).
__global__ void __launch_bounds__(256, 2) decode_v1_lanes_single_kernel(const V1Task a)
{
    extern __shared__ __align__(128) uint8_t v1_smem[];
    v1_lanes_body(a, v1_smem);
}

// Fill in what the kernel derives from a task's parameters; false if the lane kernel does not take it (stream not
// 4-byte aligned, alphabet above 4096, table too large for shared memory): the caller then uses the one-thread-per-
// block kernel.
bool v1_task_prepare(V1Task &t)
{
    if ((reinterpret_cast<uintptr_t>(t.stream) & 3u) != 0 || t.p == 0 || t.p > 16 || t.alphabet == 0 || t.alphabet > 4096u) return false;
    if (t.out_elem_bytes != 1 && t.out_elem_bytes != 2) return false;
    t.sym_bits = 1;
    while ((1u << t.sym_bits) < t.alphabet) t.sym_bits++;
    t.packed = 2u * t.p + t.sym_bits <= 32u ? 1u : 0u;
    return v1_task_smem(t, 8) != 0;
}

size_t v1_task_smem(const V1Task &t, uint32_t warps)
{
    const size_t table = t.packed ? ((size_t)4 << t.p) : ((size_t)t.alphabet * 8u + ((size_t)2 << t.p));
    const size_t total = (size_t)warps * kV1RingBytes * 32u + ((table + 15u) & ~(size_t)15u) + ((size_t)t.alphabet + 1u) * 4u;
    return total <= 200 * 1024 ? total : 0;
}

// Launch the lane kernel over `ntasks` prepared tasks.  `d_tasks` / `d_cta_task` are device copies the caller has
// already queued on `stream` (host arrays given for sizing): tasks[i].first_cta must be set from v1_plan_ctas.
uint32_t v1_plan_ctas(V1Task *tasks, uint32_t ntasks, uint32_t &warps_per_cta, size_t &smem)
{
    uint64_t total_warps = 0;
    for (uint32_t i = 0; i < ntasks; i++) total_warps += (tasks[i].nblocks + 31u) / 32u;
    const uint32_t sms = (uint32_t)std::max(1, device_sm_count());
    warps_per_cta = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(8, (total_warps + sms - 1u) / sms));   // spread over the SMs first
    uint32_t cta = 0;
    smem = 0;
    for (uint32_t i = 0; i < ntasks; i++) {
        tasks[i].first_cta = cta;
        cta += ((tasks[i].nblocks + 31u) / 32u + warps_per_cta - 1u) / warps_per_cta;
        smem = std::max(smem, v1_task_smem(tasks[i], warps_per_cta));
    }
    return cta;
}

int launch_decode_v1_lanes_single(V1Task t, void *stream)
{
    static std::mutex mu;
    static bool attr_set[16] = {false};
    uint32_t warps = 1;
    size_t smem = 0;
    const uint32_t grid = v1_plan_ctas(&t, 1, warps, smem);
    if (grid == 0) return 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev & 15]) {
            e = cudaFuncSetAttribute(decode_v1_lanes_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return (int)e;
            attr_set[dev & 15] = true;
        }
    }
    decode_v1_lanes_single_kernel<<<grid, warps * 32u, smem, reinterpret_cast<cudaStream_t>(stream)>>>(t);
    g_launches++;
    return (int)cudaGetLastError();
}

int launch_decode_v1_lanes(const V1Task *d_tasks, const uint32_t *d_cta_task, uint32_t grid, uint32_t warps_per_cta, size_t smem, void *stream)
{
    static std::mutex mu;
    static bool attr_set[16] = {false};
    if (grid == 0) return 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev & 15]) {
            e = cudaFuncSetAttribute(decode_v1_lanes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return (int)e;
            attr_set[dev & 15] = true;
        }
    }
    decode_v1_lanes_kernel<<<grid, warps_per_cta * 32u, smem, reinterpret_cast<cudaStream_t>(stream)>>>(d_tasks, d_cta_task);
    g_launches++;
    return (int)cudaGetLastError();
}

// Same decode, reading the reference's 8-byte {symbol, freq, cum} device table
// (eoq_cuda_decompress.cu:116-121) that callers of the _device entry point build.
__global__ void __launch_bounds__(128) decode_v1_syminfo_kernel(const uint8_t *__restrict__ stream, const uint32_t *__restrict__ offsets,
                                                               const uint32_t *__restrict__ sizes,
                                                               const eoq_sym_info_packed *__restrict__ info,
                                                               uint8_t *__restrict__ out, uint32_t nblocks, uint32_t block_size,
                                                               uint32_t total, uint32_t p)
{
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint32_t first = b * block_size;
    const uint32_t n = min(block_size, total - first);
    const uint32_t bytes = sizes[b];
    if (bytes == 0) return;
    const uint8_t *blk = stream + offsets[b];
    const uint32_t state_len = blk[0];
    if (1u + state_len > bytes) return;
    uint32_t x = 0;
    for (uint32_t i = 0; i < state_len; i++) x = (x << 8) | blk[1 + i];
    const uint8_t *s = blk + 1 + state_len;
    uint32_t pos = 0;
    const uint32_t end = bytes - 1 - state_len;
    const uint32_t mask = (1u << p) - 1u, low = 1u << (p + 8);
    const uint2 *tab = reinterpret_cast<const uint2 *>(info);
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t slot = x & mask;
        const uint2 e = __ldg(tab + slot);                 // x: symbol | freq << 16, y: cum
        x = (e.x >> 16) * (x >> p) + slot - (e.y & 0xFFFFu);
        while (x < low && pos < end) x = (x << 8) | s[pos++];
        out[first + i] = (uint8_t)e.x;
    }
}

int launch_decode_v1_syminfo(const uint8_t *d_stream, const uint32_t *d_offsets, const uint32_t *d_sizes,
                             const eoq_sym_info_packed *d_info, uint8_t *d_out, uint32_t nblocks,
                             uint32_t block_size, uint32_t total, uint32_t p, void *stream)
{
    if (nblocks == 0) return 0;
    if (g_v1_lanes.load()) {
        // the reference's entry point does not say how many symbols the table has: bytes are written, so at most 256
        V1Task t = {};
        t.stream = d_stream; t.offsets = d_offsets; t.sizes = d_sizes; t.freq = nullptr; t.table = d_info; t.out = d_out;
        t.nblocks = nblocks; t.block_size = block_size; t.total = total; t.p = p; t.alphabet = 256; t.out_elem_bytes = 1;
        if (v1_task_prepare(t)) return launch_decode_v1_lanes_single(t, stream);
    }
    decode_v1_syminfo_kernel<<<(nblocks + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        d_stream, d_offsets, d_sizes, d_info, d_out, nblocks, block_size, total, p);
    g_launches++;
    return (int)cudaGetLastError();
}

// Continue one wire-format block from a saved (state, position): the
// incremental decoder object of eoq_rans_v2.h:187-208.
__global__ void decode_v1_resume_kernel(const uint8_t *__restrict__ s, uint32_t end, const V1Table *__restrict__ table,
                                        uint32_t *state_pos, uint8_t *__restrict__ out, uint32_t count, uint32_t p)
{
    if (blockIdx.x || threadIdx.x) return;
    const uint2 *tab = reinterpret_cast<const uint2 *>(table);
    uint32_t x = state_pos[0], pos = state_pos[1];
    const uint32_t mask = (1u << p) - 1u, low = 1u << (p + 8);
    for (uint32_t i = 0; i < count; i++) {
        const uint2 e = __ldg(tab + (x & mask));
        x = e.x * (x >> p) + (e.y & 0xFFFFu);
        while (x < low && pos < end) x = (x << 8) | s[pos++];
        out[i] = (uint8_t)(e.y >> 16);
    }
    state_pos[0] = x;
    state_pos[1] = pos;
}

int launch_decode_v1_resume(const uint8_t *d_block, uint32_t stream_end, const V1Table *d_table,
                            uint32_t *d_state_pos, uint8_t *d_out, uint32_t count, uint32_t p, void *stream)
{
    decode_v1_resume_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(d_block, stream_end, d_table,
                                                                                   d_state_pos, d_out, count, p);
    g_launches++;
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// General dequantisation of QuantizedLinear's in-memory form, any shape:
// rows of packed codes (2 per byte for 4-bit, 4 per byte for 2-bit, one int8
// otherwise) and scales indexed over the FLATTENED matrix, scale[i / group]
// (core/quantized_linear.py:189-217, core/fast_dequant.py:47-87).  Rows
// [row_lo, row_hi) are written to `out` as a dense [row_hi-row_lo, K] matrix.
// ---------------------------------------------------------------------------
__global__ void dequant_packed_kernel(const uint8_t *__restrict__ packed, const uint16_t *__restrict__ scales,
                                      uint32_t K, uint32_t row_bytes, uint32_t bits, uint32_t group,
                                      uint32_t row_lo, uint64_t count, void *__restrict__ out, int out_dtype)
{
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = row_lo + (uint32_t)(i / K), c = (uint32_t)(i % K);
        const uint8_t *rowp = packed + (size_t)r * row_bytes;
        int code;
        if (bits == 4) code = (int)((rowp[c >> 1] >> ((c & 1) * 4)) & 0xF) - 7;
        else if (bits == 2) code = (int)((rowp[c >> 2] >> ((c & 3) * 2)) & 0x3) - 1;
        else code = (int)(int8_t)rowp[c];
        const uint64_t flat = (uint64_t)r * K + c;
        if (out_dtype == EOQ_B200_I8) reinterpret_cast<int8_t *>(out)[i] = (int8_t)code;          // the codes themselves, no scale
        else store_y(out, i, (float)code * half_bits_to_float(__ldg(scales + flat / group)), out_dtype);
    }
}

static std::atomic<int> g_dequant_vec{1};               // "dequant_vec" = 0 in eoq_b200_tune: the general kernel for every shape
void set_dequant_vec(int v) { g_dequant_vec.store(v != 0); }

// The same for float outputs when K and the group are multiples of 8 and the buffers are aligned: a thread takes the
// eight columns of one 4-byte word of nibbles (2 bytes of 2-bit codes, 8 signed bytes), which share a scale, and writes
// them with one 16-byte store (two for fp32), so a warp reads 128 contiguous bytes and writes 512.  A code becomes a
// float by one logic operation and one exact subtraction (the code in the low mantissa bits of 2^23); the product
// with the scale is the reference's fp32 product, rounded once to the output type.
template <int BITS>
__global__ void __launch_bounds__(256) dequant_packed_vec_kernel(const uint8_t *__restrict__ packed, const uint16_t *__restrict__ scales,
                                                                 uint32_t K, uint32_t row_bytes, uint32_t group, uint32_t row_lo,
                                                                 uint32_t nrows, void *__restrict__ out, int out_dtype)
{
    // blockIdx.x, threadIdx.x: the eight-column piece of the row; blockIdx.y (strided): the row.  No division but the
    // one that finds the scale (the groups run over the flattened matrix; whole groups per row in the common case).
    const uint32_t kpieces = K >> 3, piece = blockIdx.x * blockDim.x + threadIdx.x, c = piece << 3;
    if (piece >= kpieces) return;
    const uint32_t per_row = K % group == 0 ? K / group : 0u, cg = c / group;
    constexpr int kR = 4;                                          // rows per trip: their loads are in flight together
    for (uint32_t r0 = blockIdx.y * kR; r0 < nrows; r0 += gridDim.y * kR) {
        uint32_t w[kR][2];
        uint16_t sb[kR];
#pragma unroll
        for (int j = 0; j < kR; j++) {
            if (r0 + j < nrows) {
                const uint32_t r = row_lo + r0 + j;
                const uint8_t *src = packed + (size_t)r * row_bytes;
                const uint64_t si = per_row ? (uint64_t)r * per_row + cg : ((uint64_t)r * K + c) / group;
                sb[j] = __ldg(scales + si);
                if (BITS == 4) w[j][0] = __ldg(reinterpret_cast<const uint32_t *>(src + (c >> 1)));
                else if (BITS == 2) w[j][0] = __ldg(reinterpret_cast<const uint16_t *>(src + (c >> 2)));
                else { const uint2 v2 = __ldg(reinterpret_cast<const uint2 *>(src + c)); w[j][0] = v2.x; w[j][1] = v2.y; }
            }
        }
#pragma unroll
        for (int j = 0; j < kR; j++) {
            if (r0 + j >= nrows) break;
            const uint64_t p = (uint64_t)(r0 + j) * kpieces + piece;
            const float s = half_bits_to_float(sb[j]);
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                // the code in the low mantissa bits of 2^23, minus 2^23 + its offset (7, 1; signed bytes: code + 128 after the XOR)
                if (BITS == 4) v[i] = (__uint_as_float(0x4B000000u | ((w[j][0] >> (4 * i)) & 15u)) - 8388615.0f) * s;
                else if (BITS == 2) v[i] = (__uint_as_float(0x4B000000u | ((w[j][0] >> (2 * i)) & 3u)) - 8388609.0f) * s;
                else v[i] = (__uint_as_float(0x4B000000u | ((((i < 4 ? w[j][0] : w[j][1]) >> (8 * (i & 3))) & 255u) ^ 128u)) - 8388736.0f) * s;
            }
            if (out_dtype == EOQ_B200_F32) {
                float4 *dst = reinterpret_cast<float4 *>(out) + 2 * p;
                dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            } else {
                uint4 o;
                uint32_t *q = &o.x;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (out_dtype == EOQ_B200_F16) {
                        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                        q[i] = *reinterpret_cast<const uint32_t *>(&h);
                    } else {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                        q[i] = *reinterpret_cast<const uint32_t *>(&h);
                    }
                }
                reinterpret_cast<uint4 *>(out)[p] = o;
            }
        }
    }
}

int launch_dequant_packed(const uint8_t *packed, const uint16_t *scales, uint32_t K, uint32_t row_bytes, uint32_t bits,
                          uint32_t group, uint32_t row_lo, uint32_t row_hi, void *out, int out_dtype, void *stream)
{
    const uint64_t count = (uint64_t)(row_hi - row_lo) * K;
    if (count == 0) return 0;
    const uint32_t word = bits == 4 ? 4u : bits == 2 ? 2u : 8u;                  // bytes that hold eight codes
    if (g_dequant_vec.load() && out_dtype != EOQ_B200_I8 && K % 8u == 0 && group % 8u == 0 && row_bytes % word == 0 &&
        (reinterpret_cast<uintptr_t>(packed) & (word - 1u)) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
        const uint32_t nrows = row_hi - row_lo;
        const dim3 vgrid((K / 8u + 255u) / 256u, std::min((nrows + 3u) / 4u, 65535u));
        cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
        if (bits == 4) dequant_packed_vec_kernel<4><<<vgrid, 256, 0, st>>>(packed, scales, K, row_bytes, group, row_lo, nrows, out, out_dtype);
        else if (bits == 2) dequant_packed_vec_kernel<2><<<vgrid, 256, 0, st>>>(packed, scales, K, row_bytes, group, row_lo, nrows, out, out_dtype);
        else dequant_packed_vec_kernel<8><<<vgrid, 256, 0, st>>>(packed, scales, K, row_bytes, group, row_lo, nrows, out, out_dtype);
        g_launches++;
        return (int)cudaGetLastError();
    }
    const uint32_t grid = (uint32_t)std::min<uint64_t>((count + 255) / 256, (uint64_t)device_sm_count() * 16);
    dequant_packed_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(packed, scales, K, row_bytes, bits, group,
                                                                                     row_lo, count, out, out_dtype);
    g_launches++;
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// GEMV straight from QuantizedLinear's in-memory form (packed codes + fp16 scales, no entropy coding): the module's
// forward for up to eight activation rows (core/quantized_linear.py:219-228 dequantises the whole matrix and calls a
// GEMM).  General form (any float activations, groups that are multiples of 8 columns): every weight byte is read once,
// coalesced; a warp takes kPackedRows output rows, a lane sixteen bytes of each per trip (the next trip's requested
// before this one's are consumed), in pieces of eight columns whose activations come through L1 (the same eight serve
// all the warp's rows).  A code becomes a float by a shift and one logic instruction: it is placed in the top mantissa
// bits of 128.0 (nibbles, 2-bit) or assembled by a byte permute into 32768.0 + u (byte codes), and one exact
// subtraction leaves the signed code; products and sums in fp32, the group's scale applied once per eight columns.
// ---------------------------------------------------------------------------
constexpr int kPackedRows = 2, kPackedWarps = 8;

template <int BITS, int BT>
__global__ void __launch_bounds__(kPackedWarps * 32) gemv_packed_kernel(const PackedGemvArgs a)
{
    constexpr uint32_t kCols = BITS == 4 ? 32u : BITS == 2 ? 64u : 16u;      // columns in a lane's 16-byte load
    constexpr uint32_t kSub = kCols / 8u, kSpan = 32u * kCols;               // eight-column pieces per load; columns a warp covers per trip
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row0 = (blockIdx.x * kPackedWarps + warp) * kPackedRows;
    if (row0 >= a.N) return;
    const uint32_t sgroups = a.K / a.group;
    // the float that stands for code 0: 128 + qmax for codes stored as code + qmax; 32768 + 128 for signed bytes (u = code ^ 0x80)
    const float offset = BITS == 8 ? 32768.0f + 128.0f : 128.0f + (float)((1u << (BITS - 1)) - 1u);
    uint32_t magic;
    asm volatile("mov.b32 %0, %1;" : "=r"(magic) : "n"(0x43000000));      // 128.0f; in a register so that the mask stays the immediate
    const bool x_vec = a.x_dtype != EOQ_B200_F32 && (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0;
    const uint8_t *src[kPackedRows];
    const uint16_t *srow[kPackedRows];
#pragma unroll
    for (int r = 0; r < kPackedRows; r++) {
        const uint32_t row = min(row0 + r, a.N - 1u);
        src[r] = a.packed + (size_t)row * a.row_bytes;
        srow[r] = a.scales + (size_t)row * sgroups;
    }
    float acc[kPackedRows][BT];
#pragma unroll
    for (int r = 0; r < kPackedRows; r++)
#pragma unroll
        for (int b = 0; b < BT; b++) acc[r][b] = 0.0f;

    // the weights are what comes from DRAM: a lane's sixteen bytes of the next trip are requested before this trip's
    // are consumed
    uint32_t wc[kPackedRows][4], wn[kPackedRows][4];
    auto load_w = [&](uint32_t c, uint32_t (&w)[kPackedRows][4]) {
#pragma unroll
        for (int r = 0; r < kPackedRows; r++) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c < a.K) v = __ldg(reinterpret_cast<const uint4 *>(src[r] + (size_t)c * BITS / 8u));
            w[r][0] = v.x; w[r][1] = v.y; w[r][2] = v.z; w[r][3] = v.w;
        }
    };
    uint32_t c = lane * kCols;
    load_w(c, wc);
    for (; c < a.K; c += kSpan) {
        load_w(c + kSpan, wn);
#pragma unroll
        for (uint32_t sub = 0; sub < kSub; sub++) {
            const uint32_t cc = c + sub * 8u;
            float xv[BT][8];
#pragma unroll
            for (int b = 0; b < BT; b++) {
                if ((uint32_t)b < a.batch) {
                    const size_t i0 = (size_t)b * a.K + cc;
                    if (x_vec) {
                        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(a.x) + i0));
                        const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int h = 0; h < 4; h++) {
                            if (a.x_dtype == EOQ_B200_F16) {
                                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&q[h]));
                                xv[b][2 * h] = f.x; xv[b][2 * h + 1] = f.y;
                            } else {
                                xv[b][2 * h] = __uint_as_float(q[h] << 16); xv[b][2 * h + 1] = __uint_as_float(q[h] & 0xFFFF0000u);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; i++) xv[b][i] = load_x(a.x, i0 + i, a.x_dtype);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++) xv[b][i] = 0.0f;
                }
            }
#pragma unroll
            for (int r = 0; r < kPackedRows; r++) {
                const float s = half_bits_to_float(__ldg(srow[r] + cc / a.group));
                // the eight codes of this piece: one word of nibbles, half a word of 2-bit codes, two words of bytes
                const uint32_t w0 = BITS == 4 ? wc[r][sub] : BITS == 2 ? wc[r][sub >> 1] >> (16u * (sub & 1u)) : wc[r][2 * sub] ^ 0x80808080u;
                const uint32_t w1 = BITS == 8 ? wc[r][(2 * sub + 1) & 3] ^ 0x80808080u : 0u;
                float p[BT];
#pragma unroll
                for (int b = 0; b < BT; b++) p[b] = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    uint32_t t;
                    if (BITS == 4) {
                        const uint32_t sh = i < 4 ? w0 << (16 - 4 * i) : w0 >> (4 * i - 16);
                        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(sh), "n"(0x000F0000), "r"(magic));       // (sh & mask) | 128.0f
                    } else if (BITS == 2) {
                        const uint32_t sh = w0 << (16 - 2 * i);
                        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(sh), "n"(0x00030000), "r"(magic));
                    } else {
                        // {0x47, 0x00, byte i, 0x00} = 32768.0f + u
                        t = __byte_perm(i < 4 ? w0 : w1, 0x47000000u, 0x7404u | ((uint32_t)(i & 3) << 4));
                    }
                    const float m = __uint_as_float(t) - offset;              // exact: the signed code
#pragma unroll
                    for (int b = 0; b < BT; b++) p[b] = fmaf(m, xv[b][i], p[b]);
                }
#pragma unroll
                for (int b = 0; b < BT; b++) acc[r][b] = fmaf(s, p[b], acc[r][b]);
            }
        }
#pragma unroll
        for (int r = 0; r < kPackedRows; r++)
#pragma unroll
            for (int q = 0; q < 4; q++) wc[r][q] = wn[r][q];
    }
#pragma unroll
    for (int r = 0; r < kPackedRows; r++)
#pragma unroll
        for (int b = 0; b < BT; b++) {
            float v = acc[r][b];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            const uint32_t row = row0 + r;
            if (lane == 0 && row < a.N && (uint32_t)b < a.batch)
                store_y(a.y, (size_t)b * a.N + row, v + (a.bias ? __ldg(a.bias + row) : 0.0f), a.y_dtype);
        }
}

// The same product on the warp-level tensor-core path, for 16-bit activations and scale groups that are multiples
// of 128 columns: D[16 weight rows x 8 activation rows] += A[16 x 16] * B[16 x 8] (mma.sync m16n8k16, fp32
// accumulate).  The contraction index is a dummy, so the sixteen "k" positions of one instruction need not be
// sixteen adjacent columns: lane (g, t) takes 32 adjacent columns of weight rows g and g + 8 (sixteen bytes of
// nibbles: whole sectors per row across a quad) and the same 32 columns of activation row g, and feeds them in the
// order in which the codes come out of the words cheapest: (word >> 4i) & 0x000F000F puts codes i and i + 4 into
// the two halves of a register, OR with 0x6400 (fp16 1024) or 0x4300 (bf16 128) makes them the exact values
// 1024 + code or 128 + code, one packed subtraction the exact signed code.  The activations are paired the same
// way with one byte permute per register.  A quad of lanes covers 128 columns per trip (a "span"); the spans of a
// 16-row tile are dealt to the 8 or 16 warps of the CTA, each folds its per-span accumulator into the total with the
// rows' fp16 scales (fp32), and the warps' totals meet in shared memory.
constexpr int kMmaMaxWarps = 16;

template <bool BF16>
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// the first instruction of a chain: D = A * B + 0 (the zeros are operands, not four registers to clear)
template <bool BF16>
__device__ __forceinline__ void mma_m16n8k16_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// two codes, already sitting in the low bits of the two halves of v, to two exact signed 16-bit floats
template <bool BF16>
__device__ __forceinline__ uint32_t codes_to_pair(uint32_t v, uint32_t mask, uint32_t q)
{
    const uint32_t magic = BF16 ? 0x43004300u : 0x64006400u;
    const uint32_t biased = (v & mask) | magic, off = magic | q | (q << 16);
    uint32_t r;
    if (BF16) asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(biased), "r"(off));
    else asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(biased), "r"(off));
    return r;
}

// For fp16 the odd positions of a word are taken without a shift: (w & 0x00F000F0) | 0x6400 is 1024 + 16 code, one
// fused multiply-add (x 1/16, - 71) the signed code; the 2-bit codes likewise with 1/4, 1/16, 1/64.
template <bool BF16>
__device__ __forceinline__ uint32_t scaled_pair(uint32_t v, uint32_t mask, uint32_t mul, uint32_t sub)
{
    static_assert(!BF16, "a bf16 mantissa has no room above bit 6");
    const uint32_t biased = (v & mask) | 0x64006400u;
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(biased), "r"(mul | (mul << 16)), "r"(sub | (sub << 16)));
    return r;
}

// the 16 registers of signed 16-bit float pairs of a lane's 32 columns of one row, in the order the words give them
template <int BITS, bool BF16>
__device__ __forceinline__ void unpack_span(const uint32_t (&w)[BITS], uint32_t (&h)[16])
{
#pragma unroll
    for (int j = 0; j < BITS; j++) {
        if (BITS == 4) {                // register 4j + i: columns 8j + i and 8j + i + 4
            if (BF16) {
#pragma unroll
                for (int i = 0; i < 4; i++) h[4 * j + i] = codes_to_pair<BF16>(w[j] >> (4 * i), 0x000F000Fu, 7u);
            } else {
                const uint32_t u = w[j] >> 8;
                h[4 * j + 0] = codes_to_pair<false>(w[j], 0x000F000Fu, 7u);
                h[4 * j + 1] = scaled_pair<false>(w[j], 0x00F000F0u, 0x2C00u, 0xD470u);       // (1024 + 16 c) / 16 - 71
                h[4 * j + 2] = codes_to_pair<false>(u, 0x000F000Fu, 7u);
                h[4 * j + 3] = scaled_pair<false>(u, 0x00F000F0u, 0x2C00u, 0xD470u);
            }
        } else if (BITS == 2) {         // register 8j + i: columns 16j + i and 16j + i + 8
            if (BF16) {
#pragma unroll
                for (int i = 0; i < 8; i++) h[8 * j + i] = codes_to_pair<BF16>(w[j] >> (2 * i), 0x00030003u, 1u);
            } else {
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const uint32_t u = w[j] >> (8 * half);
                    h[8 * j + 4 * half + 0] = codes_to_pair<false>(u, 0x00030003u, 1u);
                    h[8 * j + 4 * half + 1] = scaled_pair<false>(u, 0x000C000Cu, 0x3400u, 0xDC04u);   // / 4 - 257
                    h[8 * j + 4 * half + 2] = scaled_pair<false>(u, 0x00300030u, 0x2C00u, 0xD410u);   // / 16 - 65
                    h[8 * j + 4 * half + 3] = scaled_pair<false>(u, 0x00C000C0u, 0x2400u, 0xCC40u);   // / 64 - 17
                }
            }
        } else if (!BF16) {             // signed bytes: u = code + 128 under 0x64 is 1024 + u; register 2j + i: columns 4j + 2i, + 1
#pragma unroll
            for (int i = 0; i < 2; i++)
                h[2 * j + i] = codes_to_pair<false>(__byte_perm(w[j] ^ 0x80808080u, 0u, i ? 0x4342u : 0x4140u), 0x00FF00FFu, 128u);
        } else {
            // 128 + u needs nine significant bits, a bf16 has eight: the byte goes under 0x4B (2^23 + u as an fp32), one
            // exact subtraction gives the code, and two codes are packed into a bf16 pair (|code| <= 128: exact)
            const uint32_t u = w[j] ^ 0x80808080u;
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540u | (2 * i))) - 8388736.0f;
                const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540u | (2 * i + 1))) - 8388736.0f;
                const __nv_bfloat162 b = __floats2bfloat162_rn(f0, f1);
                h[2 * j + i] = *reinterpret_cast<const uint32_t *>(&b);
            }
        }
    }
}

// The weights and scales of the next kDepth - 1 spans are requested before this span's are consumed (register sets in
// rotation).  Lanes whose activation row does not exist read zeros from a constant block instead of branching.
__device__ const uint4 kZeroBlock[4] = {};

template <int BITS, bool BF16, int NB, bool SPLIT = false>
__global__ void __launch_bounds__(BITS == 8 ? 256 : 512, NB > 1 || SPLIT ? 1 : BITS == 8 ? 3 : 2) gemv_packed_mma_kernel(const PackedGemvArgs a)
{
    static_assert(BITS == 2 || BITS == 4 || BITS == 8, "two or four bits packed, or one code per byte");
    static_assert(!(SPLIT && BF16), "the two halves of an fp32 activation are fp16");
    constexpr int kRows = 2;                                       // a lane's weight rows: g and g + 8 of the tile
    constexpr int kDepth = 2;                                      // register sets of weights: kDepth - 1 spans requested ahead
    __shared__ float red[kMmaMaxWarps][NB][16][8];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, g = lane >> 2, t = lane & 3u;
    const uint32_t row0 = blockIdx.x * 16u;
    const uint32_t sgroups = a.K / a.group, nspans = a.K >> 7, gspans = a.group >> 7;
    const uint8_t *pw[kRows];
    const uint16_t *ps[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        const uint32_t row = min(row0 + r * 8u + g, a.N - 1u);
        pw[r] = a.packed + (size_t)row * a.row_bytes + t * (4u * BITS);
        ps[r] = a.scales + (size_t)row * sgroups;
    }
    // a lane's 64 bytes of activation row 8n + g per span, or the zero block with no stride where that row does not exist
    const uint16_t *xr[NB];
    uint32_t xstep[NB];
#pragma unroll
    for (int n = 0; n < NB; n++) {
        const bool has = 8u * n + g < a.batch;
        xr[n] = has ? (SPLIT ? a.xsplit : reinterpret_cast<const uint16_t *>(a.x)) + (size_t)(8u * n + g) * a.K + t * 32u : reinterpret_cast<const uint16_t *>(kZeroBlock);
        xstep[n] = has ? 128u : 0u;
    }
    float tot[NB][4];
#pragma unroll
    for (int n = 0; n < NB; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[n][i] = 0.0f;

    auto load_span = [&](uint32_t s, uint32_t (&w)[kRows][BITS], uint16_t (&sc)[kRows]) {
        if (s >= nspans) return;
        const uint32_t off = s * (16u * BITS), gi = gspans == 1u ? s : s / gspans;
#pragma unroll
        for (int r = 0; r < kRows; r++) {
            if (BITS == 2) {
                const uint2 v = __ldg(reinterpret_cast<const uint2 *>(pw[r] + off));
                w[r][0] = v.x; w[r][1] = v.y;
            } else {
#pragma unroll
                for (int h = 0; h < BITS / 4; h++) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(pw[r] + off) + h);
                    w[r][4 * h] = v.x; w[r][4 * h + 1] = v.y; w[r][4 * h + 2] = v.z; w[r][4 * h + 3] = v.w;
                }
            }
            sc[r] = __ldg(ps[r] + gi);
        }
    };
    auto compute_span = [&](uint32_t s, const uint32_t (&w)[kRows][BITS], const uint16_t (&sc)[kRows]) {
        uint32_t h0[16], h1[16];
        unpack_span<BITS, BF16>(w[0], h0);
        unpack_span<BITS, BF16>(w[1], h1);
        // the activations in the weights' order: register r of the 16 holds the two columns that h0[r] holds
        auto load_xp = [&](const uint16_t *src, uint32_t (&xp)[16]) {
            uint32_t q[16];
#pragma unroll
            for (int h = 0; h < 4; h++) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src) + h);
                q[4 * h] = v.x; q[4 * h + 1] = v.y; q[4 * h + 2] = v.z; q[4 * h + 3] = v.w;
            }
#pragma unroll
            for (int r = 0; r < 16; r++) {
                if (BITS == 4) {            // j = r / 4, columns 8j + (r & 3) and + 4: halves of q[4j + (r & 3) / 2] and q[4j + 2 + (r & 3) / 2]
                    const int j = r >> 2, k = (r & 3) >> 1;
                    xp[r] = __byte_perm(q[4 * j + k], q[4 * j + 2 + k], (r & 1) ? 0x7632u : 0x5410u);
                } else if (BITS == 2) {     // j = r / 8, columns 16j + (r & 7) and + 8
                    const int j = r >> 3, k = (r & 7) >> 1;
                    xp[r] = __byte_perm(q[8 * j + k], q[8 * j + 4 + k], (r & 1) ? 0x7632u : 0x5410u);
                } else {
                    xp[r] = q[r];
                }
            }
        };
#pragma unroll
        for (int n = 0; n < NB; n++) {
            uint32_t xp[16];
            float c[4], d[4];
            load_xp(xr[n] + s * xstep[n], xp);
            if (!SPLIT) {
                // two accumulators: consecutive instructions do not wait for one another
                mma_m16n8k16_first<BF16>(c, h0[0], h1[0], h0[1], h1[1], xp[0], xp[1]);
                mma_m16n8k16_first<BF16>(d, h0[2], h1[2], h0[3], h1[3], xp[2], xp[3]);
#pragma unroll
                for (int m = 2; m < 8; m += 2) {
                    mma_m16n8k16<BF16>(c, h0[2 * m], h1[2 * m], h0[2 * m + 1], h1[2 * m + 1], xp[2 * m], xp[2 * m + 1]);
                    mma_m16n8k16<BF16>(d, h0[2 * m + 2], h1[2 * m + 2], h0[2 * m + 3], h1[2 * m + 3], xp[2 * m + 2], xp[2 * m + 3]);
                }
            } else {
                // fp32 activations as two fp16 halves (the nearest fp16, then the nearest to the remainder): the codes are
                // exact, so code * hi + code * lo is the fp32 product to about 2^-22; one accumulator per half
                mma_m16n8k16_first<false>(c, h0[0], h1[0], h0[1], h1[1], xp[0], xp[1]);
#pragma unroll
                for (int m = 1; m < 8; m++) mma_m16n8k16<false>(c, h0[2 * m], h1[2 * m], h0[2 * m + 1], h1[2 * m + 1], xp[2 * m], xp[2 * m + 1]);
                load_xp(xr[n] + (xstep[n] ? (size_t)a.batch * a.K : 0u) + s * xstep[n], xp);
                mma_m16n8k16_first<false>(d, h0[0], h1[0], h0[1], h1[1], xp[0], xp[1]);
#pragma unroll
                for (int m = 1; m < 8; m++) mma_m16n8k16<false>(d, h0[2 * m], h1[2 * m], h0[2 * m + 1], h1[2 * m + 1], xp[2 * m], xp[2 * m + 1]);
            }
            const float fa = half_bits_to_float(sc[0]), fb = half_bits_to_float(sc[1]);
            tot[n][0] = fmaf(fa, c[0] + d[0], tot[n][0]); tot[n][1] = fmaf(fa, c[1] + d[1], tot[n][1]);
            tot[n][2] = fmaf(fb, c[2] + d[2], tot[n][2]); tot[n][3] = fmaf(fb, c[3] + d[3], tot[n][3]);
        }
    };

    // The weights and scales do not depend on the kernel before this one in the stream, the activations may: the
    // first span's weight loads are in flight before the dependency wait (programmatic dependent launch).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t wbuf[kDepth][kRows][BITS];
    uint16_t sbuf[kDepth][kRows];
#pragma unroll
    for (int d = 0; d < kDepth - 1; d++) load_span(warp + d * nwarps, wbuf[d], sbuf[d]);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t s = warp; s < nspans; s += kDepth * nwarps) {
#pragma unroll
        for (int d = 0; d < kDepth; d++) {                          // register sets in rotation: every index below is static
            const uint32_t sd = s + d * nwarps;
            if (sd >= nspans) break;
            load_span(sd + (kDepth - 1) * nwarps, wbuf[(d + kDepth - 1) % kDepth], sbuf[(d + kDepth - 1) % kDepth]);
            compute_span(sd, wbuf[d], sbuf[d]);
        }
    }
#pragma unroll
    for (int n = 0; n < NB; n++) {
        red[warp][n][g][2 * t] = tot[n][0]; red[warp][n][g][2 * t + 1] = tot[n][1];
        red[warp][n][g + 8][2 * t] = tot[n][2]; red[warp][n][g + 8][2 * t + 1] = tot[n][3];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < NB * 128u; i += blockDim.x) {
        const uint32_t n = i >> 7, r = (i >> 3) & 15u, b = 8u * n + (i & 7u), row = row0 + r;
        float v = 0.0f;
        for (uint32_t w = 0; w < nwarps; w++) v += red[w][n][r][i & 7u];
        if (row < a.N && b < a.batch) store_y(a.y, (size_t)b * a.N + row, v + (a.bias ? __ldg(a.bias + row) : 0.0f), a.y_dtype);
    }
}

// bits: 2 and 4 as packed by QuantizedLinear (low bits first, code + qmax), anything else one signed code per byte.
// K a multiple of the group and of the columns in sixteen bytes (32 nibbles, 64 two-bit codes, 16 bytes), the group a
// multiple of 8, packed rows 16-byte aligned: checked by the caller.
// Activation rows one launch takes: 32 on the tensor-core form (16-bit activations, 16-byte aligned, or fp32 ones with a
// split copy, against scale groups of whole 128-column spans), 8 otherwise.
static std::atomic<int> g_packed_warps{0};              // 0 = by shape; "packed_warps" in eoq_b200_tune
void set_packed_warps(int v) { g_packed_warps.store(v >= 1 && v <= 16 ? v : 0); }

// Warps per CTA of the tensor-core form (they share a tile's spans).  The CTAs are short, so a grid that needs a second,
// partly filled round of CTAs loses that fraction of the machine: take the most warps per CTA with which the whole
// grid is resident at once (given the registers the compiler gave this instantiation) and every warp still has two
// spans; when no choice fits, the one with the most resident warps per SM.
template <typename Kern, typename Args>
static cudaError_t launch_packed_mma(Kern kern, uint32_t fixed_warps, uint32_t tiles, uint32_t nspans, cudaStream_t st, const Args &a, size_t smem = 0)
{
    // byte codes and more than eight activation rows (more registers, longer spans of work per warp): 8 warps measured best
    if (fixed_warps) {
        const uint32_t w = g_packed_warps.load() ? std::min((uint32_t)g_packed_warps.load(), fixed_warps) : nspans >= 16u ? fixed_warps : 4u;
        return launch_with_pdl(kern, dim3(tiles), dim3(w * 32u), smem, st, a);
    }
    const uint32_t max_warps = 16;
    // registers per kernel, asked once (kernels of one signature share this function: the key is the kernel, not its type)
    static std::mutex mu;
    static std::vector<std::pair<const void *, int>> known;
    int regs = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const auto &kv : known)
            if (kv.first == reinterpret_cast<const void *>(kern)) regs = kv.second;
        if (regs == 0) {
            cudaFuncAttributes fa;
            cudaError_t e = cudaFuncGetAttributes(&fa, kern);
            if (e != cudaSuccess) return e;
            regs = std::max(fa.numRegs, 16);
            known.emplace_back(reinterpret_cast<const void *>(kern), regs);
        }
    }
    const uint32_t per_thread = ((uint32_t)regs + 7u) & ~7u, sms = (uint32_t)device_sm_count();
    static const uint32_t kChoices[] = {16, 12, 10, 8, 6, 5, 4};
    uint32_t warps = 0, best_resident = 0, fallback = 4;
    for (uint32_t w : kChoices) {
        if (w > max_warps || (2u * w > nspans && w > 4u)) continue;
        const uint32_t ctas = std::min(64u / w, 65536u / (per_thread * 32u * w));
        if (ctas == 0) continue;
        if (!warps && tiles <= sms * ctas) warps = w;
        if (w * ctas > best_resident) { best_resident = w * ctas; fallback = w; }
    }
    if (!warps) warps = fallback;
    if (g_packed_warps.load()) warps = std::min((uint32_t)g_packed_warps.load(), max_warps);
    return launch_with_pdl(kern, dim3(tiles), dim3(warps * 32u), smem, st, a);
}

uint32_t gemv_packed_rows(const PackedGemvArgs &a)
{
    const bool tensor = a.K % 128u == 0 && a.group % 128u == 0 &&
                        (a.x_dtype == EOQ_B200_F32 ? a.xsplit != nullptr : (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0);
    return tensor ? 32u : 8u;
}

int launch_gemv_packed(const PackedGemvArgs &a, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (gemv_packed_rows(a) > 8u) {
        const uint32_t tiles = (a.N + 15u) / 16u, nspans = a.K >> 7;
        cudaError_t e = cudaSuccess;
#define EOQ_LAUNCH_MMA(B, H)                                                                                             \
    do {                                                                                                                 \
        if (a.batch <= 8) e = launch_packed_mma(gemv_packed_mma_kernel<B, H, 1>, B == 8 ? 8u : 0u, tiles, nspans, st, a);  \
        else if (a.batch <= 16) e = launch_packed_mma(gemv_packed_mma_kernel<B, H, 2>, 8u, tiles, nspans, st, a);        \
        else e = launch_packed_mma(gemv_packed_mma_kernel<B, H, 4>, 8u, tiles, nspans, st, a);                           \
    } while (0)
        const bool bf = a.x_dtype == EOQ_B200_BF16;
        if (a.x_dtype == EOQ_B200_F32) {
#define EOQ_LAUNCH_SPLIT(B)                                                                                              \
    do {                                                                                                                 \
        if (a.batch <= 8) e = launch_packed_mma(gemv_packed_mma_kernel<B, false, 1, true>, 8u, tiles, nspans, st, a);    \
        else if (a.batch <= 16) e = launch_packed_mma(gemv_packed_mma_kernel<B, false, 2, true>, 8u, tiles, nspans, st, a); \
        else e = launch_packed_mma(gemv_packed_mma_kernel<B, false, 4, true>, 8u, tiles, nspans, st, a);                 \
    } while (0)
            if (a.bits == 4) EOQ_LAUNCH_SPLIT(4);
            else if (a.bits == 2) EOQ_LAUNCH_SPLIT(2);
            else EOQ_LAUNCH_SPLIT(8);
#undef EOQ_LAUNCH_SPLIT
        } else
        if (a.bits == 4) { if (bf) EOQ_LAUNCH_MMA(4, true); else EOQ_LAUNCH_MMA(4, false); }
        else if (a.bits == 2) { if (bf) EOQ_LAUNCH_MMA(2, true); else EOQ_LAUNCH_MMA(2, false); }
        else { if (bf) EOQ_LAUNCH_MMA(8, true); else EOQ_LAUNCH_MMA(8, false); }
#undef EOQ_LAUNCH_MMA
        g_launches++;
        return (int)e;
    }
    if (a.batch > 8) return (int)cudaErrorInvalidValue;
    const uint32_t grid = (a.N + kPackedWarps * kPackedRows - 1u) / (kPackedWarps * kPackedRows);
    const uint32_t bt = a.batch <= 1 ? 1u : a.batch <= 2 ? 2u : a.batch <= 4 ? 4u : 8u;
#define EOQ_LAUNCH_PACKED(B)                                                                                             \
    do {                                                                                                                 \
        if (bt == 1) gemv_packed_kernel<B, 1><<<grid, kPackedWarps * 32, 0, st>>>(a);                                    \
        else if (bt == 2) gemv_packed_kernel<B, 2><<<grid, kPackedWarps * 32, 0, st>>>(a);                               \
        else if (bt == 4) gemv_packed_kernel<B, 4><<<grid, kPackedWarps * 32, 0, st>>>(a);                               \
        else gemv_packed_kernel<B, 8><<<grid, kPackedWarps * 32, 0, st>>>(a);                                            \
    } while (0)
    if (a.bits == 4) EOQ_LAUNCH_PACKED(4);
    else if (a.bits == 2) EOQ_LAUNCH_PACKED(2);
    else EOQ_LAUNCH_PACKED(8);
#undef EOQ_LAUNCH_PACKED
    g_launches++;
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// GEMV straight from PolarLinear's in-memory form (kernels/polar_engine.py:144-360: one code per byte, fp16 norm per
// block, a table of 2^bits centroids), for up to eight activation rows:
//   y[n] = sum over blocks b of norm[n, b] * sum_j centroid[code[n, b, j]] * xr[b, j]
// where xr is the caller's activation block rotated by the block's Hadamard matrix and divided by sqrt(block) (H is
// symmetric, so x . (c H) = (x H) . c: the rotation is done once per call on the activations, never on the weights).
// A warp takes two rows, a lane sixteen codes of each per trip (one 16-byte load, the next trip's requested before
// this one's are consumed); the centroid table sits in shared memory once per lane (entry e of lane l at word
// 32 e + l), so the 32 look-ups of a step hit 32 different banks whatever the codes are; a code becomes a table
// offset by one shift and one mask.  fp32 throughout.
// ---------------------------------------------------------------------------
// The rotation of the activations: every block of 2^shift columns of x times the normalised Hadamard matrix of that
// order (Sylvester construction, core/polar_quant.py:104-120) and divided by sqrt(block), i.e. a fast Walsh-Hadamard
// transform in shared memory scaled by 1 / block.  One CTA per activation row and stretch of columns.  Output: fp32
// [batch][K], or with `split` two fp16 planes [2][batch][K] (the fp16 nearest to the value, then to the remainder).
__global__ void __launch_bounds__(1024) polar_rotate_kernel(const void *__restrict__ x, int x_dtype, uint32_t K, uint32_t shift, uint32_t batch,
                                                           float *__restrict__ out32, uint16_t *__restrict__ out_split)
{
    extern __shared__ float rot[];
    const uint32_t b = blockIdx.y, width = blockDim.x * 4u, c0 = blockIdx.x * width;      // width: a multiple of the block
    const uint32_t count = min(width, K - c0);
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) rot[i] = load_x(x, (size_t)b * K + c0 + i, x_dtype);
    __syncthreads();
    for (uint32_t h = 1; h < (1u << shift); h <<= 1) {
        for (uint32_t i = threadIdx.x; i < count / 2u; i += blockDim.x) {
            const uint32_t lo = ((i & ~(h - 1u)) << 1) | (i & (h - 1u)), hi = lo + h;      // the pairs (j, j + h) of one butterfly stage
            const float u = rot[lo], v = rot[hi];
            rot[lo] = u + v; rot[hi] = u - v;
        }
        __syncthreads();
    }
    const float scale = 1.0f / (float)(1u << shift);
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        const float v = rot[i] * scale;
        const size_t o = (size_t)b * K + c0 + i;
        if (out_split) {
            const __half hi = __float2half_rn(v);
            out_split[o] = __half_as_ushort(hi);
            out_split[(size_t)batch * K + o] = __half_as_ushort(__float2half_rn(v - __half2float(hi)));
        } else {
            out32[o] = v;
        }
    }
}

int launch_polar_rotate(const void *x, int x_dtype, uint32_t K, uint32_t block_shift, uint32_t batch, float *out32, uint16_t *out_split, void *stream)
{
    // a CTA's stretch of columns: whole blocks, 1024 columns where the block allows
    const uint32_t block = 1u << block_shift, width = std::max(block, 1024u), threads = width / 4u;
    if (threads > 1024u) return (int)cudaErrorInvalidValue;
    polar_rotate_kernel<<<dim3((K + width - 1u) / width, batch), threads, width * 4u, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_dtype, K, block_shift, batch, out32, out_split);
    g_launches++;
    return (int)cudaGetLastError();
}

template <int BT>
__global__ void __launch_bounds__(256) gemv_polar_codes_kernel(const PolarCodesArgs a)
{
    extern __shared__ float polar_lut[];
    for (uint32_t i = threadIdx.x; i < a.entries * 32u; i += blockDim.x) polar_lut[i] = __ldg(a.centroids + (i >> 5));
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row0 = (blockIdx.x * (blockDim.x >> 5) + warp) * 2u;
    if (row0 >= a.N) return;
    const uint32_t lut_lane = (uint32_t)__cvta_generic_to_shared(polar_lut) + lane * 4u, emask = (a.entries - 1u) << 7;
    const uint32_t blocks_per_row = a.K >> a.block_shift;
    const uint8_t *src[2];
    const uint16_t *nrm[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint32_t row = min(row0 + r, a.N - 1u);
        src[r] = a.codes + (size_t)row * a.K;
        nrm[r] = a.norms + (size_t)row * blocks_per_row;
    }
    float acc[2][BT];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int b = 0; b < BT; b++) acc[r][b] = 0.0f;
    uint32_t wc[2][4], wn[2][4];
    auto load_w = [&](uint32_t c, uint32_t (&w)[2][4]) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c < a.K) v = __ldg(reinterpret_cast<const uint4 *>(src[r] + c));
            w[r][0] = v.x; w[r][1] = v.y; w[r][2] = v.z; w[r][3] = v.w;
        }
    };
    uint32_t c = lane * 16u;
    load_w(c, wc);
    for (; c < a.K; c += 512u) {
        load_w(c + 512u, wn);
        const uint32_t blk = c >> a.block_shift;                    // the lane's sixteen columns lie in one block (block >= 16)
        const float n0 = half_bits_to_float(__ldg(nrm[0] + blk)), n1 = half_bits_to_float(__ldg(nrm[1] + blk));
        float p[2][BT];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < BT; b++) p[r][b] = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float xv[BT][4];
#pragma unroll
            for (int b = 0; b < BT; b++) {
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if ((uint32_t)b < a.batch) v = __ldg(reinterpret_cast<const float4 *>(a.xrot + (size_t)b * a.K + c + 4u * q));
                xv[b][0] = v.x; xv[b][1] = v.y; xv[b][2] = v.z; xv[b][3] = v.w;
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint32_t w = wc[r][q];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t off = (i == 0 ? w << 7 : w >> (8 * i - 7)) & emask;         // 128 * code
                    float cv;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(cv) : "r"(lut_lane + off));
#pragma unroll
                    for (int b = 0; b < BT; b++) p[r][b] = fmaf(cv, xv[b][i], p[r][b]);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < BT; b++) { acc[0][b] = fmaf(n0, p[0][b], acc[0][b]); acc[1][b] = fmaf(n1, p[1][b], acc[1][b]); }
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int q = 0; q < 4; q++) wc[r][q] = wn[r][q];
    }
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int b = 0; b < BT; b++) {
            float v = acc[r][b];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            const uint32_t row = row0 + r;
            if (lane == 0 && row < a.N && (uint32_t)b < a.batch)
                store_y(a.y, (size_t)b * a.N + row, v + (a.bias ? __ldg(a.bias + row) : 0.0f), a.y_dtype);
        }
}

// The same product on the warp-level tensor cores, for blocks of 64 columns and more.  The operands of
// mma.sync.m16n8k16 are fp16, a centroid and a rotated activation are fp32: each is split into the fp16 nearest to it
// and the fp16 nearest to the remainder (c = c_hi + c_lo to about 2^-22), and the product is taken as
// c_hi x_hi + (c_hi x_lo + c_lo x_hi), three instructions per sixteen columns with fp32 accumulation; the term left
// out is 2^-22 of the result.  The centroid table holds both halves of an entry in one 32-bit word, once per lane
// (conflict-free, as above); two look-ups and two byte permutes give the pair registers {hi_a, hi_b}, {lo_a, lo_b} of
// two adjacent columns, which is the order the activations are stored in, so they need no permutation.  Lane (g, t)
// takes sixteen codes of rows g and g + 8 per 64-column span (one 16-byte load each, the next span's requested
// before this one's are consumed) and the same sixteen columns of activation row g from the caller's split copy
// (xsplit: [hi | lo][batch][K] fp16).  A CTA is a 16-row tile; its warps share the spans and meet in shared memory.
template <int NB>
__global__ void __launch_bounds__(512) gemv_polar_mma_kernel(const PolarCodesArgs a)
{
    extern __shared__ uint32_t polar_lut2[];                     // [entries][32 lanes]: lo << 16 | hi
    __shared__ float red[kMmaMaxWarps][NB][16][8];
    for (uint32_t i = threadIdx.x; i < a.entries * 32u; i += blockDim.x) {
        const float c = __ldg(a.centroids + (i >> 5));
        const __half hi = __float2half_rn(c), lo = __float2half_rn(c - __half2float(hi));
        polar_lut2[i] = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, g = lane >> 2, t = lane & 3u;
    const uint32_t row0 = blockIdx.x * 16u, nspans = a.K >> 6, blocks_per_row = a.K >> a.block_shift;
    const uint32_t lut_lane = (uint32_t)__cvta_generic_to_shared(polar_lut2) + lane * 4u, emask = (a.entries - 1u) << 7;
    const uint8_t *pw[2];
    const uint16_t *pn[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint32_t row = min(row0 + r * 8u + g, a.N - 1u);
        pw[r] = a.codes + (size_t)row * a.K + t * 16u;
        pn[r] = a.norms + (size_t)row * blocks_per_row;
    }
    // activation rows 8n + g: their hi and lo halves, or the zero block with no stride where a row does not exist
    const uint16_t *xh[NB], *xl[NB];
    uint32_t xstep[NB];
    float tot[NB][4];
#pragma unroll
    for (int n = 0; n < NB; n++) {
        const bool has = 8u * n + g < a.batch;
        xh[n] = has ? a.xsplit + (size_t)(8u * n + g) * a.K + t * 16u : reinterpret_cast<const uint16_t *>(kZeroBlock);
        xl[n] = has ? xh[n] + (size_t)a.batch * a.K : xh[n];
        xstep[n] = has ? 64u : 0u;
#pragma unroll
        for (int i = 0; i < 4; i++) tot[n][i] = 0.0f;
    }

    auto load_span = [&](uint32_t s, uint32_t (&w)[2][4], uint16_t (&nr)[2]) {
        if (s >= nspans) return;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(pw[r] + s * 64u));
            w[r][0] = v.x; w[r][1] = v.y; w[r][2] = v.z; w[r][3] = v.w;
            nr[r] = __ldg(pn[r] + ((s << 6) >> a.block_shift));
        }
    };
    auto compute_span = [&](uint32_t s, const uint32_t (&w)[2][4], const uint16_t (&nr)[2]) {
        uint32_t hi[2][8], lo[2][8];                              // [row g, row g + 8][pair]: columns 2 pair, 2 pair + 1 of the lane's sixteen
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int p = 0; p < 2; p++) {
                    const uint32_t wj = w[r][j];
                    const uint32_t oa = (p == 0 ? wj << 7 : wj >> 9) & emask, ob = (p == 0 ? wj >> 1 : wj >> 17) & emask;      // 128 * code
                    uint32_t ea, eb;
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(ea) : "r"(lut_lane + oa));
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(eb) : "r"(lut_lane + ob));
                    hi[r][2 * j + p] = __byte_perm(ea, eb, 0x5410u);
                    lo[r][2 * j + p] = __byte_perm(ea, eb, 0x7632u);
                }
        const float fa = half_bits_to_float(nr[0]), fb = half_bits_to_float(nr[1]);
#pragma unroll
        for (int n = 0; n < NB; n++) {
            uint32_t xq[2][8];                                    // [hi, lo][pair of adjacent columns]
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint4 vh = __ldg(reinterpret_cast<const uint4 *>(xh[n] + s * xstep[n]) + h), vl = __ldg(reinterpret_cast<const uint4 *>(xl[n] + s * xstep[n]) + h);
                xq[0][4 * h] = vh.x; xq[0][4 * h + 1] = vh.y; xq[0][4 * h + 2] = vh.z; xq[0][4 * h + 3] = vh.w;
                xq[1][4 * h] = vl.x; xq[1][4 * h + 1] = vl.y; xq[1][4 * h + 2] = vl.z; xq[1][4 * h + 3] = vl.w;
            }
            float c[4], d[4];
            mma_m16n8k16_first<false>(c, hi[0][0], hi[1][0], hi[0][1], hi[1][1], xq[0][0], xq[0][1]);
            mma_m16n8k16_first<false>(d, hi[0][0], hi[1][0], hi[0][1], hi[1][1], xq[1][0], xq[1][1]);
            mma_m16n8k16<false>(d, lo[0][0], lo[1][0], lo[0][1], lo[1][1], xq[0][0], xq[0][1]);
#pragma unroll
            for (int m = 1; m < 4; m++) {
                mma_m16n8k16<false>(c, hi[0][2 * m], hi[1][2 * m], hi[0][2 * m + 1], hi[1][2 * m + 1], xq[0][2 * m], xq[0][2 * m + 1]);
                mma_m16n8k16<false>(d, hi[0][2 * m], hi[1][2 * m], hi[0][2 * m + 1], hi[1][2 * m + 1], xq[1][2 * m], xq[1][2 * m + 1]);
                mma_m16n8k16<false>(d, lo[0][2 * m], lo[1][2 * m], lo[0][2 * m + 1], lo[1][2 * m + 1], xq[0][2 * m], xq[0][2 * m + 1]);
            }
            tot[n][0] = fmaf(fa, c[0] + d[0], tot[n][0]); tot[n][1] = fmaf(fa, c[1] + d[1], tot[n][1]);
            tot[n][2] = fmaf(fb, c[2] + d[2], tot[n][2]); tot[n][3] = fmaf(fb, c[3] + d[3], tot[n][3]);
        }
    };

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t wbuf[2][2][4];
    uint16_t nbuf[2][2];
    load_span(warp, wbuf[0], nbuf[0]);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t s = warp; s < nspans; s += 2u * nwarps) {
#pragma unroll
        for (int dd = 0; dd < 2; dd++) {
            const uint32_t sd = s + dd * nwarps;
            if (sd >= nspans) break;
            load_span(sd + nwarps, wbuf[dd ^ 1], nbuf[dd ^ 1]);
            compute_span(sd, wbuf[dd], nbuf[dd]);
        }
    }
#pragma unroll
    for (int n = 0; n < NB; n++) {
        red[warp][n][g][2 * t] = tot[n][0]; red[warp][n][g][2 * t + 1] = tot[n][1];
        red[warp][n][g + 8][2 * t] = tot[n][2]; red[warp][n][g + 8][2 * t + 1] = tot[n][3];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < NB * 128u; i += blockDim.x) {
        const uint32_t n = i >> 7, r = (i >> 3) & 15u, b = 8u * n + (i & 7u), row = row0 + r;
        float v = 0.0f;
        for (uint32_t w = 0; w < nwarps; w++) v += red[w][n][r][i & 7u];
        if (row < a.N && b < a.batch) store_y(a.y, (size_t)b * a.N + row, v + (a.bias ? __ldg(a.bias + row) : 0.0f), a.y_dtype);
    }
}

// K a multiple of 16 and of the block, the block a power of two >= 16, entries a power of two <= 256, codes and the
// activations 16-byte aligned, batch <= 8: checked by the caller.  With a split copy of the activations (xsplit) and
// blocks of 64 columns or more: the tensor-core form, batch <= 32.
int launch_gemv_polar_codes(const PolarCodesArgs &a, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)a.entries * 128u;                   // the table, once per lane
    if (a.xsplit) {
        const uint32_t tiles = (a.N + 15u) / 16u, nspans = a.K >> 6;
        cudaError_t e = cudaSuccess;
        if (a.batch <= 8) e = launch_packed_mma(gemv_polar_mma_kernel<1>, 0u, tiles, nspans, st, a, smem);
        else if (a.batch <= 16) e = launch_packed_mma(gemv_polar_mma_kernel<2>, 0u, tiles, nspans, st, a, smem);
        else {
            // 32 KB of meeting space beside a table of up to 32 KB: past the 48 KB a kernel gets without asking
            if (smem > 16u * 1024u) e = cudaFuncSetAttribute(gemv_polar_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess) e = launch_packed_mma(gemv_polar_mma_kernel<4>, 0u, tiles, nspans, st, a, smem);
        }
        g_launches++;
        return (int)e;
    }
    const uint32_t warps = 8, grid = (a.N + warps * 2u - 1u) / (warps * 2u);
    if (a.batch > 8) return (int)cudaErrorInvalidValue;
    if (a.batch <= 1) gemv_polar_codes_kernel<1><<<grid, warps * 32, smem, st>>>(a);
    else if (a.batch <= 2) gemv_polar_codes_kernel<2><<<grid, warps * 32, smem, st>>>(a);
    else if (a.batch <= 4) gemv_polar_codes_kernel<4><<<grid, warps * 32, smem, st>>>(a);
    else gemv_polar_codes_kernel<8><<<grid, warps * 32, smem, st>>>(a);
    g_launches++;
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Fused decode -> fp16 operand pieces -> tcgen05 MMA (accumulator in tensor memory), for up to 128 activation rows.
//
//   Y[m, n] = sum_k X[m, k] * W[n, k]        (INT4 weights, 3 per step, 96-row tiles)
//
// Work split (stream-K): the tiles, in (row block, column segment) order, are cut into one contiguous range per
// CTA, one persistent CTA per SM, so every SM decodes the same number of tiles whatever the shape.  A range covers
// parts of one or more row blocks; up to four row blocks (one TMEM accumulator each) are in flight at a time and
// the warps take the tiles of the range round-robin.  Every 16 decoded columns a warp has a 96 x 16 fp16 piece of
// W ((q - 7) * scale) in shared memory, has fetched the matching piece of X (16-byte asynchronous copies straight
// from the row-major activations), and one elected lane issues
//     tcgen05.mma.cta_group::1.kind::f16   D[128 tokens x 96 rows] (fp32, TMEM) += Xpiece * Wpiece^T
// (M = 128, N = 96, K = 16; both operands K-major without swizzle: 8 x 16-byte core matrices, 128 bytes apart
// along K, 256 bytes apart along rows).  Rows of D depend only on the same rows of X, so token rows past the
// batch are never staged: the MMA reads whatever follows in shared memory and those rows of D are never stored.
// All warps of the CTA accumulate into the same TMEM tile, which is what lets each of them be at a different K
// position: accumulator space (512 columns per SM), not tensor time, is the scarce resource.  tcgen05.commit onto
// mbarriers tells a warp when its staging buffers may be overwritten and tells the CTA when a group is complete;
// the epilogue reads TMEM with tcgen05.ld.  A row block that one CTA decoded alone is written straight to Y;
// otherwise each contributor stores its fp32 partial tile and takes a ticket, and the last one to arrive adds the
// partial tiles in CTA order and writes Y (no CTA ever waits for another).  Every wait is bounded; TMEM is always
// released.
// ---------------------------------------------------------------------------
constexpr int kGemmMaxThreads = 512;
constexpr uint32_t kGemmTokens = 128, kGemmRows = 96;
constexpr uint32_t kGemmMaxM = 512;          // activation rows one pass takes: up to four 128-row tiles share every decoded piece
constexpr uint32_t kXPieceBytes = kGemmTokens * 16 * 2, kWPieceBytes = kGemmRows * 16 * 2;
constexpr uint32_t kGemmAccs = 4, kTmemCols = 128 * kGemmAccs;   // four accumulators, 128 columns apart (96 used): all of TMEM
constexpr uint32_t kGemmMaxContrib = 160, kGemmCtlBytes = 384 + 2 * kGemmMaxContrib * 4;   // 1664: keeps the pieces 128-byte aligned
constexpr uint32_t kGemmSlotFloats = kGemmTokens * kGemmRows;

// bytes of one warp's X staging piece: up to 128 token rows rounded up to 8; more rows are staged as whole 128-row tiles
__host__ __device__ inline uint32_t gemm_x_stride(uint32_t m) { return m <= kGemmTokens ? ((m + 7u) & ~7u) * 32u : ((m + 127u) / 128u) * kXPieceBytes; }
__host__ __device__ inline uint32_t gemm_m_tiles(uint32_t m) { return (m + kGemmTokens - 1u) / kGemmTokens; }

size_t gemm_smem_bytes(uint32_t p, uint32_t warps, uint32_t m)
{
    // the last warp's MMA reads a full 128-row piece: keep that much behind the last staged piece
    return smem_table_bytes(p) + kGemmCtlBytes + (size_t)warps * (kWPieceBytes + gemm_x_stride(m)) + kXPieceBytes + ring_smem_bytes<RingSmall>(warps);
}
size_t gemm_partial_bytes(uint32_t grid, uint32_t m) { return (size_t)grid * 2 * gemm_m_tiles(m) * kGemmSlotFloats * sizeof(float); }

// K-major, no-swizzle shared-memory matrix descriptor: start address, leading (K) and stride (row-group) byte offsets
// in units of 16 bytes, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__host__ __device__ __forceinline__ uint32_t piece_offset(uint32_t row, uint32_t col) { return (row >> 3) * 256u + (col >> 3) * 128u + (row & 7u) * 16u + (col & 7u) * 2u; }

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void gemm_wait(uint32_t bar, uint32_t parity, uint32_t *status, bool &dead)
{
    if (dead) return;
    for (uint32_t i = 0; i < (1u << 22); i++)
        if (mbar_test(bar, parity)) return;
    *status = 2u;
    dead = true;
}

struct GemmArgs {
    const uint32_t *table;
    const TileDesc *tiles;
    const uint8_t  *stream;
    const uint2    *scales_t; // [K/group][nrb * 32] words {s0 | s1 << 16, s2}: see GemvArgs::scales_t
    void           *y;        // [M, N]
    const float    *bias;
    float          *partials; // [grid][2][128][96]
    uint32_t       *counters; // [nrb], zero between launches
    uint32_t       *status;
    uint32_t N, K, group, p, nseg, nrb, M;
    uint32_t head_bytes;      // see TiledWeights::head_bytes
    int y_dtype;
};

// X [M, K] fp32 or bf16 -> fp16, same layout: kind::f16 MMAs take both operands in one 16-bit format, and the weight
// pieces are fp16 ((q - 7) * scale is exact to fp16 rounding, bf16 would lose three bits of it)
__global__ void gemm_x_to_half_kernel(const void *x, int x_dtype, __half *out, size_t n)
{
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    if (i + 3 < n && x_dtype == EOQ_B200_F32) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i / 4);
        __half2 h[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
        *reinterpret_cast<uint2 *>(out + i) = *reinterpret_cast<const uint2 *>(h);
    } else {
        for (size_t k = i; k < min(i + 4, n); k++) out[k] = __float2half_rn(load_x(x, k, x_dtype));
    }
}

struct GemmWarp {             // per warp, warp-uniform
    uint32_t wp, xp;          // shared addresses of the W and X staging pieces
    uint32_t mma_bar, x_bar;
    uint32_t np;              // pieces issued so far: piece i is the i-th completion on both barriers
};

// Two tiled bulk copies bring one X piece: box = [rows of the batch rounded up to 8] x [8 columns = 16 bytes] each, so
// that shared memory holds it as K-major core matrices (8 rows x 16 bytes, contiguous); rows past the batch are
// filled with zeros by the copy.  Columns c..c+7 land at dst, c+8..c+15 behind them.
// With more than 128 token rows the same is done once per 128-row tile (rows past the batch of the last tile read as zeros).
__device__ __forceinline__ void gemm_fetch_x(const CUtensorMap *xmap, uint32_t dst, uint32_t half_bytes, uint32_t c, uint32_t bar,
                                             uint32_t m_tiles)
{
    mbar_expect_tx(bar, 2u * half_bytes * m_tiles);
    for (uint32_t j = 0; j < m_tiles; j++) {
        const uint32_t at = dst + j * 2u * half_bytes, row = j * kGemmTokens;
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                     ::"r"(at), "l"(reinterpret_cast<uint64_t>(xmap)), "r"(c), "r"(row), "r"(bar) : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                     ::"r"(at + half_bytes), "l"(reinterpret_cast<uint64_t>(xmap)), "r"(c + 8u), "r"(row), "r"(bar) : "memory");
    }
}

// Decode 16 columns of the warp's tile into its W piece.  A few steps in, once the previous MMA is known to have read
// both staging pieces, the copy of this piece's X is started so that it lands while the rest decodes.
template <bool RING>
__device__ __forceinline__ void gemm_decode_piece(uint32_t tab_addr, uint32_t &x, WordState &ws, uint32_t mask, uint32_t p,
                                                  const float (&sc)[3], const GemmWarp &gw, const CUtensorMap *xmap, uint32_t c,
                                                  uint32_t x_half_bytes, uint32_t m_tiles, uint32_t lane, uint32_t *status, bool &dead)
{
    using F = Fmt<3, 4>;
    using F0 = Int4Field<F::field_bit(0)>;
    using F1 = Int4Field<F::field_bit(1)>;
    using F2 = Int4Field<F::field_bit(2)>;
    const uint32_t mg0 = F0::magic_reg(), mg1 = F1::magic_reg(), mg2 = F2::magic_reg();
#pragma unroll
    for (int half = 0; half < 2; half++) {
        float w[3][8];
#pragma unroll
        for (int s = 0; s < 8; s++) {
            uint32_t u0, u1, u2;
            rans_step_int4<F0::kMask, F1::kMask, F2::kMask>(tab_addr, x, mask, p, F::kBiasMask, mg0, mg1, mg2, u0, u1, u2);
            w[0][s] = (__uint_as_float(u0) - (F0::kBase + 7.0f)) * sc[0];      // (base + n) - (base + 7) is exact
            w[1][s] = (__uint_as_float(u1) - (F1::kBase + 7.0f)) * sc[1];
            w[2][s] = (__uint_as_float(u2) - (F2::kBase + 7.0f)) * sc[2];
            rans_renorm<RING>(x, ws);
            if (half == 0 && s == 3) {
                // the previous MMA was issued four steps ago: it has read both staging pieces by now
                {
                    if (gw.np > 0) gemm_wait(gw.mma_bar, (gw.np - 1u) & 1u, status, dead);
                    if (lane == 0) gemm_fetch_x(xmap, gw.xp, x_half_bytes, c, gw.x_bar, m_tiles);
                    __syncwarp();
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 3; j++) {
            __half2 h[4];
#pragma unroll
            for (int q = 0; q < 4; q++) h[q] = __floats2half2_rn(w[j][2 * q], w[j][2 * q + 1]);
            const uint4 v = *reinterpret_cast<const uint4 *>(h);
            const uint32_t addr = gw.wp + piece_offset(lane * 3 + j, half * 8);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
    }
}

// 16 consecutive outputs of one token row: y[idx .. idx+15] = v + bias, as two 16-byte stores when the row allows
__device__ __forceinline__ void gemm_store16(void *y, size_t idx, const float (&v)[16], uint32_t n0, uint32_t N, int dtype)
{
    if (dtype != EOQ_B200_F32 && n0 + 16u <= N && (idx & 7u) == 0) {
        uint32_t pk[8];
#pragma unroll
        for (int q = 0; q < 8; q++) {
            if (dtype == EOQ_B200_F16) {
                const __half2 h = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
                pk[q] = *reinterpret_cast<const uint32_t *>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
                pk[q] = *reinterpret_cast<const uint32_t *>(&h);
            }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(y) + idx);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    } else {
#pragma unroll
        for (uint32_t q = 0; q < 16; q++)
            if (n0 + q < N) store_y(y, idx + q, v[q], dtype);
    }
}

// The last contributor of a shared row block adds the partial tiles (slots listed in `contrib`, CTA order) and writes Y.
__device__ __forceinline__ void gemm_sum_partials(const GemmArgs &a, uint32_t rb, const volatile uint32_t *contrib, uint32_t n)
{
    constexpr uint32_t kU = 6;                       // float4 loads in flight per thread and contributor
    const uint32_t nvec = a.M * (kGemmRows / 4);
    const size_t slot_floats = (size_t)gemm_m_tiles(a.M) * kGemmSlotFloats;
    for (uint32_t v0 = threadIdx.x; v0 < nvec; v0 += blockDim.x * kU) {
        float4 acc[kU];
#pragma unroll
        for (uint32_t u = 0; u < kU; u++) acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t k = 0; k < n; k++) {
            const float4 *src = reinterpret_cast<const float4 *>(a.partials + (size_t)contrib[k] * slot_floats);
            float4 t[kU];
#pragma unroll
            for (uint32_t u = 0; u < kU; u++) {
                const uint32_t v = v0 + u * blockDim.x;
                t[u] = v < nvec ? __ldcg(src + v) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (uint32_t u = 0; u < kU; u++) { acc[u].x += t[u].x; acc[u].y += t[u].y; acc[u].z += t[u].z; acc[u].w += t[u].w; }
        }
#pragma unroll
        for (uint32_t u = 0; u < kU; u++) {
            const uint32_t v = v0 + u * blockDim.x;
            if (v >= nvec) continue;
            const uint32_t tt = v / (kGemmRows / 4), col = rb * kGemmRows + (v % (kGemmRows / 4)) * 4u;
            const float o[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
#pragma unroll
            for (uint32_t q = 0; q < 4; q++)
                if (col + q < a.N) store_y(a.y, (size_t)tt * a.N + col + q, o[q] + (a.bias ? __ldg(a.bias + col + q) : 0.0f), a.y_dtype);
        }
    }
}

__global__ void __launch_bounds__(kGemmMaxThreads, 1) gemm_tiles_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, nwarps = blockDim.x >> 5;
    uint32_t *tab = reinterpret_cast<uint32_t *>(smem);
    uint8_t *ctl = smem + smem_table_bytes(a.p);
    uint8_t *wp_base = ctl + kGemmCtlBytes;
    uint8_t *xp_base = wp_base + nwarps * kWPieceBytes;     // 128-byte aligned, as tiled bulk copies require
    uint8_t *ring_area = xp_base + nwarps * gemm_x_stride(a.M) + kXPieceBytes;

    if ((smem_addr(xp_base) & 127u) != 0) {      // tiled bulk copies need 128-byte aligned destinations: refuse rather than fault
        if (tid == 0) *a.status = 3u;
        return;
    }
    // control block: table barrier, TMEM slot, group barrier, ticket flags, per-warp barriers, two contributor lists
    const uint32_t tab_bar = smem_addr(ctl), slot_addr = smem_addr(ctl + 16), grp_bar = smem_addr(ctl + 32);
    volatile uint32_t *flag = reinterpret_cast<volatile uint32_t *>(ctl + 48);          // [2]
    const uint32_t mma_bar0 = smem_addr(ctl + 64), x_bar0 = smem_addr(ctl + 64 + 128);
    volatile uint32_t *contrib = reinterpret_cast<volatile uint32_t *>(ctl + 384);      // [2][kGemmMaxContrib]

    // Everything that has to come from global memory is requested before anything is waited for: the decode table
    // (bulk copy onto a barrier), then each warp's first tile (descriptor, L2 prefetch, first ring chunks).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // see launch_with_pdl
    if (tid == 0) {
        mbar_init(tab_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(tab_bar, 4u << a.p);
        for (uint32_t off = 0; off < (4u << a.p); off += 16384u)
            bulk_copy_g2s(smem_addr(tab) + off, reinterpret_cast<const uint8_t *>(a.table) + off, min(16384u, (4u << a.p) - off), tab_bar);
    }
    // this CTA's range of tiles
    const uint64_t T = (uint64_t)a.nrb * a.nseg;
    const uint32_t t_lo = (uint32_t)(T * blockIdx.x / gridDim.x), t_hi = (uint32_t)(T * (blockIdx.x + 1) / gridDim.x);
    const uint32_t rb_first = t_lo / a.nseg, rb_last = (t_hi - 1u) / a.nseg;
    RingCtlT<RingSmall> ring;
    ring_setup(ring, ring_area, warp, nwarps, lane, a.status);
    // up to four 128-row token tiles share one decoded piece, each with its own accumulator: 4 / m_tiles row blocks in flight
    const uint32_t m_tiles = gemm_m_tiles(a.M), rbs_in_flight = kGemmAccs / m_tiles;
    uint32_t tile = t_lo + warp;
    const uint32_t g0_hi = min(t_hi, (rb_first + rbs_in_flight) * a.nseg);
    bool have = tile < g0_hi;
    TileDesc d;
    if (have) d = a.tiles[tile];           // requested here, needed by tile_open below

    if (tid == 0) {
        mbar_init(grp_bar, nwarps);
        for (uint32_t i = 0; i < nwarps; i++) { mbar_init(mma_bar0 + i * 8, 1); mbar_init(x_bar0 + i * 8, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the .sync.aligned tensor-memory instructions below need the whole warp at the same instruction: lanes that took
    // a lane-0-only branch or left a polling loop at different times are brought back together first
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (have) tile_open(ring, d, tile_src(a.stream, a.head_bytes, tile, d), lane);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = lds_u32(slot_addr);
    bool dead = false;       // a wait gave up: stop waiting, finish quickly, report through the status word
    gemm_wait(tab_bar, 0u, a.status, dead);
    // nothing above read an input of this call or wrote global memory; X, bias, Y and the scratch come after this
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint32_t mask = (1u << a.p) - 1u, p = a.p, tab_addr = smem_addr(tab);
    // fp32 accumulate, A = X and B = W both fp16 and K-major, N = 96, M = 128
    const uint32_t idesc = (1u << 4) | ((kGemmRows >> 3) << 17) | ((kGemmTokens >> 4) << 24);
    GemmWarp gw;
    gw.wp = smem_addr(wp_base) + warp * kWPieceBytes;
    gw.xp = smem_addr(xp_base) + warp * gemm_x_stride(a.M);
    gw.mma_bar = mma_bar0 + warp * 8;
    gw.x_bar = x_bar0 + warp * 8;
    gw.np = 0;
    const uint32_t x_half_bytes = gemm_x_stride(a.M) / (2u * m_tiles);      // one 8-column half of one token tile of an X piece
    // warps 0..7: warp w owns TMEM lanes 32*(w%4).. (tokens) and columns 48*(w/4).. (weight rows of a block) of every
    // accumulator; it clears them before a group and reads them back after it
    const uint32_t tok = (warp & 3u) * 32u + lane, col0 = (warp >> 2) * 48u;
    const uint32_t taddr_w = tmem_base + (((warp & 3u) * 32u) << 16) + col0;

    uint32_t grp = 0;
    for (uint32_t rb0 = rb_first; t_lo < t_hi && rb0 <= rb_last; rb0 += rbs_in_flight, grp++) {
        const uint32_t g_lo = max(t_lo, rb0 * a.nseg), g_hi = min(t_hi, (rb0 + rbs_in_flight) * a.nseg);
        const uint32_t nparts = (g_hi - 1u) / a.nseg - rb0 + 1u;
        if (grp > 0) {
            tile = g_lo + warp;
            have = tile < g_hi;
            if (have) {
                d = a.tiles[tile];
                tile_open(ring, d, tile_src(a.stream, a.head_bytes, tile, d), lane);
            }
        }
        __syncwarp();
        if (warp < 8) {
            for (uint32_t pa = 0; pa < nparts * m_tiles; pa++)
#pragma unroll
                for (uint32_t i = 0; i < 3; i++)
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
                                 ::"r"(taddr_w + pa * 128u + i * 16u), "r"(0u) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        while (have) {
            const TileSrc base = tile_src(a.stream, a.head_bytes, tile, d);
            const uint32_t d_tmem = tmem_base + (tile / a.nseg - rb0) * m_tiles * 128u;
            uint32_t x;
            WordState ws;
            const bool ring_mode = tile_begin(ring, ws, d, base, lane, x);
            // ask L2 for the warp's next tile while this one decodes
            const uint32_t next = tile + nwarps;
            if (next < g_hi && lane == 0) {
                const TileDesc nd = a.tiles[next];
                if (a.head_bytes) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.stream + (size_t)next * a.head_bytes), "r"(a.head_bytes) : "memory");
                if ((nd.len64 << 6) > a.head_bytes)
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.stream + ((size_t)nd.off64 << 6)), "r"((nd.len64 << 6) - a.head_bytes) : "memory");
            }
            const uint32_t row = d.row0 + lane * 3;
            // transposed copy of the scales: the three scales of a lane's rows for one group are one 8-byte word, the
            // words of the 32 lanes contiguous (zero for rows past the matrix)
            const uint2 *srow = a.scales_t + row / 3u;
            const uint32_t sc_stride = a.nrb * 32u;
            uint2 sc_next = ldg_u32x2_pinned(srow + (size_t)(d.col0 / a.group) * sc_stride);
            float sc[3] = {0.0f, 0.0f, 0.0f};
            const uint32_t cend = d.col0 + d.ncols;
            for (uint32_t c = d.col0; c < cend; c += 16) {
                if (c == d.col0 || c % a.group == 0) {
                    // scales of this group were requested a group ago; request the next group's now
                    const uint32_t g = c / a.group;
                    sc[0] = half_bits_to_float((uint16_t)sc_next.x);
                    sc[1] = half_bits_to_float((uint16_t)(sc_next.x >> 16));
                    sc[2] = half_bits_to_float((uint16_t)sc_next.y);
                    if ((g + 1) * a.group < cend) sc_next = ldg_u32x2_pinned(srow + (size_t)(g + 1) * sc_stride);
                }
                if (ring_mode) {
                    {
                        ring_sync_step(ring, ws, lane);
                    }
                    gemm_decode_piece<true>(tab_addr, x, ws, mask, p, sc, gw, &xmap, c, x_half_bytes, m_tiles, lane, a.status, dead);
                } else {
                    gemm_decode_piece<false>(tab_addr, x, ws, mask, p, sc, gw, &xmap, c, x_half_bytes, m_tiles, lane, a.status, dead);
                }
                {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    gemm_wait(gw.x_bar, gw.np & 1u, a.status, dead);
                }
                {
                    if (lane == 0) {
                        // X piece: 8-row groups 128 bytes apart, its two column halves x_half_bytes apart; one MMA per token
                        // tile, all on the same decoded W piece
                        for (uint32_t j = 0; j < m_tiles; j++)
                            umma_f16(d_tmem + j * 128u, umma_desc(gw.xp + j * 2u * x_half_bytes, x_half_bytes, 128), umma_desc(gw.wp, 128, 256), idesc, 1u);
                        umma_commit(gw.mma_bar);
                    }
                    __syncwarp();
                }
                gw.np++;
            }
            tile_end(ring, ring_mode);
            tile = next;
            have = tile < g_hi;
            if (have) {
                d = a.tiles[tile];
                tile_open(ring, d, tile_src(a.stream, a.head_bytes, tile, d), lane);
            }
        }
        // every MMA this warp issued for the group is behind this commit
        if (lane == 0) umma_commit(grp_bar);
        __syncwarp();
        gemm_wait(grp_bar, grp & 1u, a.status, dead);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // a CTA's first row block and its last are the only ones it can share with other CTAs: partial slots 0 and 1
        bool shared_any = false;
        for (uint32_t pa = 0; pa < nparts; pa++) {
            const uint32_t rb = rb0 + pa;
            const bool full = max(t_lo, rb * a.nseg) == rb * a.nseg && min(t_hi, (rb + 1) * a.nseg) == (rb + 1) * a.nseg;
            shared_any |= !full;
            if (warp < 8) {
                const size_t slot_floats = (size_t)m_tiles * kGemmSlotFloats;
                for (uint32_t j = 0; j < m_tiles; j++) {
                    const uint32_t token = j * kGemmTokens + tok;
                    float *slot = a.partials + ((size_t)blockIdx.x * 2 + (rb == rb_first ? 0u : 1u)) * slot_floats + (size_t)token * kGemmRows + col0;
#pragma unroll
                    for (uint32_t i = 0; i < 3; i++) {
                        uint32_t r[16];
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                                       "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                     : "r"(taddr_w + (pa * m_tiles + j) * 128u + i * 16u) : "memory");
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (token < a.M) {
                            if (full) {
                                const uint32_t n0 = rb * kGemmRows + col0 + i * 16u;
                                float v[16];
#pragma unroll
                                for (uint32_t q = 0; q < 16; q++) v[q] = __uint_as_float(r[q]) + (a.bias && n0 + q < a.N ? __ldg(a.bias + n0 + q) : 0.0f);
                                gemm_store16(a.y, (size_t)token * a.N + n0, v, n0, a.N, a.y_dtype);
                            } else {
#pragma unroll
                                for (uint32_t q = 0; q < 16; q += 4)
                                    __stcg(reinterpret_cast<float4 *>(slot + i * 16u + q),
                                           make_float4(__uint_as_float(r[q]), __uint_as_float(r[q + 1]), __uint_as_float(r[q + 2]), __uint_as_float(r[q + 3])));
                            }
                        }
                        __syncwarp();      // lanes past the batch skipped the stores: rejoin before the next aligned load
                    }
                }
            }
        }
        if (shared_any) {
            // tickets: the last contributor of a row block to arrive adds the partial tiles, always in CTA order
            __threadfence();
            __syncthreads();
            if (tid < 2) {
                // thread 0 looks after the CTA's first row block, thread 1 after its last
                const uint32_t rb = tid == 0 ? rb_first : rb_last;
                const bool in_group = rb >= rb0 && rb < rb0 + nparts && (tid == 0 || rb_last != rb_first);
                const bool full = max(t_lo, rb * a.nseg) == rb * a.nseg && min(t_hi, (rb + 1) * a.nseg) == (rb + 1) * a.nseg;
                uint32_t result = 0;
                if (in_group && !full) {
                    const uint32_t g = gridDim.x;
                    const uint32_t c_first = (uint32_t)((((uint64_t)rb * a.nseg + 1) * g - 1) / T);
                    const uint32_t c_last = (uint32_t)((((uint64_t)(rb + 1) * a.nseg) * g - 1) / T);
                    const uint32_t n = min(c_last - c_first + 1u, kGemmMaxContrib);
                    const uint32_t old = atomicAdd(a.counters + rb, 1u);
                    if (old == n - 1u) {
                        a.counters[rb] = 0u;
                        for (uint32_t i = 0; i < n; i++) {
                            const uint32_t c = c_first + i;
                            const uint32_t c_rb_first = (uint32_t)(T * c / g) / a.nseg;
                            contrib[tid * kGemmMaxContrib + i] = c * 2u + (c_rb_first == rb ? 0u : 1u);
                        }
                        result = n;
                    }
                }
                flag[tid] = result;
            }
            __syncthreads();
            const uint32_t n0 = flag[0], n1 = flag[1];
            if (n0 | n1) __threadfence();
            if (n0) gemm_sum_partials(a, rb_first, contrib, n0);
            if (n1) gemm_sum_partials(a, rb_last, contrib + kGemmMaxContrib, n1);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    __syncwarp();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static std::atomic<int> g_gemm_warps{0};        // 0 = as many as fit shared memory
void set_gemm_warps(int v) { g_gemm_warps.store(v < 0 ? 0 : v); }

uint32_t gemm_grid(uint32_t nrb, uint32_t nseg)
{
    const uint64_t T = (uint64_t)nrb * nseg;
    return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)device_sm_count(), T));
}

// x: [M, K] row-major, M <= 128.  fp32 and bf16 activations are first rounded to fp16 into `xhalf` ([128, K] fp16 scratch).
int launch_gemm_tc(const uint32_t *table, const TileDesc *tiles, const uint8_t *stream, const uint2 *scales_t, const void *x,
                   void *xhalf, float *partials, uint32_t *counters, void *y, const float *bias, uint32_t *status, uint32_t N,
                   uint32_t K, uint32_t group, uint32_t p, uint32_t nseg, uint32_t nrb, uint32_t head_bytes, uint32_t M, int x_dtype, int y_dtype,
                   void *stream_)
{
    static std::mutex mu;
    static size_t attr_set[16] = {0};
    if (M == 0 || M > kGemmMaxM) return (int)cudaErrorInvalidValue;
    uint32_t warps = 16;
    const int want = g_gemm_warps.load();
    if (want >= 2 && want <= 16) warps = (uint32_t)want;
    while (warps > 2 && gemm_smem_bytes(p, warps, M) > 227 * 1024) warps -= 2;
    const size_t smem = gemm_smem_bytes(p, warps, M);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    if (std::min<uint64_t>((uint64_t)nseg + 1, gemm_grid(nrb, nseg)) > kGemmMaxContrib) return (int)cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (attr_set[dev & 15] < smem) {
            e = cudaFuncSetAttribute(gemm_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            attr_set[dev & 15] = 227 * 1024;
        }
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
    GemmArgs a;
    const void *x16 = x;
    if (x_dtype != EOQ_B200_F16) {
        const size_t n = (size_t)M * K;
        gemm_x_to_half_kernel<<<(unsigned)((n / 4 + 256) / 256), 256, 0, st>>>(x, x_dtype, reinterpret_cast<__half *>(xhalf), n);
        g_launches++;
        x16 = xhalf;
    }
    // tensor map over X [M, K] fp16: boxes of (M rounded up to 8) rows x 8 columns, rows past M read as zeros
    static EncodeTiledFn encode = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!encode) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return (int)cudaErrorNotSupported;
            encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
    }
    CUtensorMap xmap;
    const cuuint64_t gdim[2] = {K, M}, gstride[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {8, M <= kGemmTokens ? gemm_x_stride(M) / 32 : kGemmTokens}, estride[2] = {1, 1};
    if (encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x16), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return (int)cudaErrorInvalidValue;
    a.table = table; a.tiles = tiles; a.stream = stream; a.scales_t = scales_t; a.y = y; a.bias = bias;
    a.partials = partials; a.counters = counters; a.status = status;
    a.N = N; a.K = K; a.group = group; a.p = p; a.nseg = nseg; a.nrb = nrb; a.M = M;
    a.head_bytes = head_bytes;
    a.y_dtype = y_dtype;
    e = launch_with_pdl(gemm_tiles_kernel, dim3(gemm_grid(nrb, nseg)), dim3(warps * 32), smem, st, a, xmap);
    g_launches++;
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}


// ---------------------------------------------------------------------------
// Device-side tile encoder: the tiled layout built on the GPU from symbols that are already there (a tensor decoded
// from the wire format, or symbols copied in), byte-identical to the host builder (rans_host.cpp: build_tiled).
//
//   tile_hist_kernel     counts the joint symbols (G codes of `bits` bits per rANS step); the host turns the counts into
//                        frequencies and the decode table (a few thousand numbers);
//   tile_encode_kernel   one warp per tile, one lane per rANS stream: walks the tile's columns right to left, pushes
//                        16-bit words into a scratch column {word | step << 16}, leaves the final states, the word
//                        counts, the tile's row count (longest lane, rounded up to even) and how far the lanes' read
//                        positions drift apart;
//   tile_scatter_kernel  after the host has laid the tiles out (head region, packed tails): writes states and word rows
//                        to their place in the stream, words in decode order (last pushed first), zeros past a lane's end.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) tile_hist_kernel(const uint8_t *__restrict__ sym, uint32_t N, uint32_t K, uint32_t Npad,
                                                          uint32_t G, uint32_t bits, unsigned long long *__restrict__ counts)
{
    extern __shared__ uint32_t hist[];
    const uint32_t alphabet = 1u << (bits * G), mask = (1u << bits) - 1u;
    for (uint32_t i = threadIdx.x; i < alphabet; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint64_t quads = (uint64_t)(Npad / G) * (K / 4);            // four columns of one row group per item
    for (uint64_t q = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t rg = (uint32_t)(q / (K / 4)), c = (uint32_t)(q % (K / 4)) * 4u;
        uint32_t v[4] = {0, 0, 0, 0};
        for (uint32_t j = 0; j < G; j++) {
            const uint32_t r = rg * G + j;
            const uint32_t w = *reinterpret_cast<const uint32_t *>(sym + (size_t)(r < N ? r : r % N) * K + c);
#pragma unroll
            for (uint32_t u = 0; u < 4; u++) v[u] |= ((w >> (8u * u)) & mask) << (bits * j);
        }
#pragma unroll
        for (uint32_t u = 0; u < 4; u++) atomicAdd(&hist[v[u]], 1u);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < alphabet; i += blockDim.x)
        if (hist[i]) atomicAdd(&counts[i], (unsigned long long)hist[i]);
}

__global__ void __launch_bounds__(128) tile_encode_kernel(const TileEncodeArgs a)
{
    const uint32_t lane = threadIdx.x & 31u, t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= a.ntiles) return;
    const TileDesc d = a.tiles[t];
    const uint32_t mask = (1u << a.bits) - 1u;
    const uint8_t *src[3] = {nullptr, nullptr, nullptr};
    for (uint32_t j = 0; j < a.G; j++) {
        const uint32_t r = d.row0 + lane * a.G + j;
        src[j] = a.sym + (size_t)(r < a.N ? r : r % a.N) * a.K + d.col0;
    }
    uint32_t *col = a.scratch + (size_t)t * a.max_ncols * 32u + lane;       // this lane's pushed words, [k][lane]
    uint32_t x = 1u << 16, cnt = 0;
    for (uint32_t c = d.ncols; c-- > 0;) {
        uint32_t v = 0;
        for (uint32_t j = 0; j < a.G; j++) v |= ((uint32_t)src[j][c] & mask) << (a.bits * j);
        const uint2 fc = __ldg(a.freq_cum + v);
        if ((unsigned long long)x >= ((unsigned long long)fc.x << (32u - a.p))) {
            col[(size_t)cnt * 32u] = (x & 0xFFFFu) | (c << 16);
            cnt++;
            x >>= 16;
        }
        x = ((x / fc.x) << a.p) + (x % fc.x) + fc.y;
    }
    a.state[(size_t)t * 32u + lane] = x;
    a.count[(size_t)t * 32u + lane] = cnt;
    const uint32_t longest = (__reduce_max_sync(0xffffffffu, cnt) + 1u) & ~1u;
    // drift: the lanes' read positions after each step, in decode order (the word pushed last is read first)
    uint32_t pos = 0, drift = 0;
    for (uint32_t c = 0; c < d.ncols; c++) {
        if (pos < cnt && (col[(size_t)(cnt - 1u - pos) * 32u] >> 16) == c) pos++;
        drift = max(drift, __reduce_max_sync(0xffffffffu, pos) - __reduce_min_sync(0xffffffffu, pos));
    }
    if (lane == 0) a.info[t] = make_uint2(longest, drift);
}

__global__ void __launch_bounds__(128) tile_scatter_kernel(const TileScatterArgs a)
{
    const uint32_t lane = threadIdx.x & 31u, t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= a.ntiles) return;
    const TileDesc d = a.tiles[t];
    const uint32_t H = a.head_bytes, rows = ((d.len64 << 6) - 128u) >> 6;
    uint8_t *head = a.stream + (size_t)t * H, *tail = a.stream + ((size_t)d.off64 << 6) - H;
    auto at = [&](uint32_t b) { return b < H ? head + b : tail + b; };          // byte b of the tile
    *reinterpret_cast<uint32_t *>(at(4u * lane)) = a.state[(size_t)t * 32u + lane];
    const uint32_t cnt = a.count[(size_t)t * 32u + lane];
    const uint32_t *col = a.scratch + (size_t)t * a.max_ncols * 32u + lane;
    for (uint32_t k = 0; k < rows; k++) {
        const uint16_t w = k < cnt ? (uint16_t)col[(size_t)(cnt - 1u - k) * 32u] : (uint16_t)0;
        *reinterpret_cast<uint16_t *>(at(128u + k * 64u + lane * 2u)) = w;
    }
}

int launch_tile_hist(const uint8_t *sym, uint32_t N, uint32_t K, uint32_t Npad, uint32_t G, uint32_t bits, unsigned long long *counts,
                     void *stream)
{
    const uint32_t grid = (uint32_t)std::max(1, device_sm_count()) * 4u;
    tile_hist_kernel<<<grid, 256, sizeof(uint32_t) << (bits * G), reinterpret_cast<cudaStream_t>(stream)>>>(sym, N, K, Npad, G, bits, counts);
    g_launches++;
    return (int)cudaGetLastError();
}

int launch_tile_encode(const TileEncodeArgs &a, void *stream)
{
    tile_encode_kernel<<<(a.ntiles + 3u) / 4u, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    g_launches++;
    return (int)cudaGetLastError();
}

int launch_tile_scatter(const TileScatterArgs &a, void *stream)
{
    tile_scatter_kernel<<<(a.ntiles + 3u) / 4u, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    g_launches++;
    return (int)cudaGetLastError();
}

}  // namespace eoq
