// sm_100a kernels of the EOQ hot path.
//
//   gemv_tiles_kernel     fused rANS decode -> unpack -> scale -> GEMV, batch 1..8
//   decode_tiles_kernel   rANS decode of the tiled layout to packed INT4 / bytes / dequantised matrix
//   decode_v1_kernel      decode of the reference wire format (one thread per independent block)
//
// All three are integer/byte streaming kernels bounded by instruction issue and
// by HBM, not by tensor throughput; nothing here is shaped into a GEMM.
#include "eoq_internal.h"

#include <algorithm>
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

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

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

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
template <int B>
struct Int4Field {
    static constexpr uint32_t kMask = 0xFu << B;
    static constexpr uint32_t kMagic = (uint32_t)(150 - B) << 23;       // exponent of 2^(23-B)
    static constexpr float kBase = (float)(1u << (23 - B));
    static constexpr bool kPreSubtract = B < 15;
    static constexpr float kCorr = kPreSubtract ? 0.0f : kBase + 7.0f;
    __device__ __forceinline__ static float value(uint32_t e)
    {
        float m = __uint_as_float((e & kMask) | kMagic);
        if (kPreSubtract) m -= kBase + 7.0f;
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

// Shared-memory carve-up of the fused kernel (bytes).
__host__ __device__ inline size_t smem_table_bytes(uint32_t p) { return (size_t)4 << p; }
size_t gemv_smem_bytes(uint32_t K, uint32_t p, uint32_t bt, uint32_t kind)
{
    size_t b = smem_table_bytes(p) + (size_t)K * bt * 4;
    b += kind == EOQ_B200_KIND_Q5_POLAR ? 32 * 32 * 4 : (size_t)(K / 16) * bt * 4;
    return b;
}

// One rANS step: table lookup, state update; returns the entry.
__device__ __forceinline__ uint32_t rans_step(const uint32_t *tab, uint32_t &x, uint32_t mask, uint32_t p, uint32_t bias_mask)
{
    const uint32_t e = tab[x & mask];
    x = (e >> 23) * (x >> p) + (e & bias_mask);
    return e;
}

// Renormalise from the lane's private word column (one 16-bit word at most,
// since p <= 16).  `w` always holds the lane's next unread word.
__device__ __forceinline__ void rans_renorm(uint32_t &x, uint32_t &w, const uint16_t *&ptr)
{
    if (x < 65536u) {
        x = (x << 16) | w;
        ptr += 32;
        w = __ldg(ptr);
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
template <int G, int BITS, int BT, int KIND>
__global__ void __launch_bounds__(kThreads, 1) gemv_tiles_kernel(const GemvArgs a)
{
    using F = Fmt<G, BITS>;
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tab = reinterpret_cast<uint32_t *>(smem);
    float *xs = reinterpret_cast<float *>(smem + smem_table_bytes(a.p));
    float *aux = xs + (size_t)a.K * BT;   // INT4: [K/16][BT] sums; polar: [32][32] centroids

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t K = a.K, M = 1u << a.p;

    for (uint32_t i = tid * 4; i < M; i += kThreads * 4)
        *reinterpret_cast<uint4 *>(tab + i) = __ldg(reinterpret_cast<const uint4 *>(a.table + i));
    for (uint32_t i = tid; i < K * BT; i += kThreads) {
        const uint32_t c = i / BT, b = i % BT;
        xs[i] = b < a.batch ? load_x(a.x, (size_t)b * K + c, a.x_dtype) : 0.0f;
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
                const float s = h == 32 ? 1.0f / 64.0f : 1.0f;
                xs[c * BT + b] = (u + v) * s;
                xs[(c + h) * BT + b] = (u - v) * s;
            }
            __syncthreads();
        }
    } else {
        for (uint32_t i = tid; i < K / 16 * BT; i += kThreads) {
            const uint32_t u = i / BT, b = i % BT;
            float s = 0.0f;
#pragma unroll
            for (int k = 0; k < 16; k++) s += xs[(u * 16 + k) * BT + b];
            aux[i] = s;
        }
        __syncthreads();
    }

    const uint32_t mask = M - 1u, p = a.p;
    const uint32_t sgroups = K / a.group;
    for (uint32_t t = blockIdx.x + gridDim.x * warp; t < a.ntiles; t += gridDim.x * kWarps) {
        const TileDesc d = a.tiles[t];
        const uint8_t *base = a.stream + ((size_t)d.off64 << 6);
        uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(base) + lane);
        const uint16_t *ptr = reinterpret_cast<const uint16_t *>(base + 128) + lane;
        uint32_t w = __ldg(ptr);
        const uint32_t row = d.row0 + lane * G;

        float y[G][BT];
#pragma unroll
        for (int j = 0; j < G; j++)
#pragma unroll
            for (int b = 0; b < BT; b++) y[j][b] = 0.0f;

        uint32_t c = d.col0;
        const uint32_t cend = c + d.ncols;
        while (c < cend) {
            const uint32_t g = c / a.group;
            const uint32_t rstart = c, rend = min(cend, (g + 1) * a.group);
            float sc[G];
#pragma unroll
            for (int j = 0; j < G; j++)
                sc[j] = row + j < a.N ? half_bits_to_float(__ldg(a.scales + (size_t)(row + j) * sgroups + g)) : 0.0f;
            float acc[G][BT];
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) acc[j][b] = 0.0f;

#pragma unroll 2
            for (; c < rend; c += 4) {
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
                    const uint32_t e = rans_step(tab, x, mask, p, F::kBiasMask);
                    if (KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                        {
                            const float m = Int4Field<F::field_bit(0)>::value(e);
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[0][b] = fmaf(m, xv[s][b], acc[0][b]);
                        }
                        if (G > 1) {
                            const float m = Int4Field<F::field_bit(G > 1 ? 1 : 0)>::value(e);
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[G > 1 ? 1 : 0][b] = fmaf(m, xv[s][b], acc[G > 1 ? 1 : 0][b]);
                        }
                        if (G > 2) {
                            const float m = Int4Field<F::field_bit(G > 2 ? 2 : 0)>::value(e);
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[G > 2 ? 2 : 0][b] = fmaf(m, xv[s][b], acc[G > 2 ? 2 : 0][b]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < G; j++) {
                            const uint32_t code = (e >> F::field_bit(j)) & F::kFieldMask;
                            const float m = aux[code * 32 + lane];
#pragma unroll
                            for (int b = 0; b < BT; b++) acc[j][b] = fmaf(m, xv[s][b], acc[j][b]);
                        }
                    }
                    rans_renorm(x, w, ptr);
                }
            }

            if (KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                float rs[BT];
#pragma unroll
                for (int b = 0; b < BT; b++) rs[b] = 0.0f;
                for (uint32_t u = rstart / 16; u < rend / 16; u++)
#pragma unroll
                    for (int b = 0; b < BT; b++) rs[b] += aux[u * BT + b];
                const float corr[3] = {Int4Field<F::field_bit(0)>::kCorr,
                                       Int4Field<F::field_bit(G > 1 ? 1 : 0)>::kCorr,
                                       Int4Field<F::field_bit(G > 2 ? 2 : 0)>::kCorr};
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

        if (a.nseg > 1) {
            float *mine = a.partials + ((size_t)d.seg * a.Npad + row) * BT;
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) __stcg(mine + j * BT + b, y[j][b]);
            __threadfence();
            __syncwarp();
            uint32_t ticket = 0;
            if (lane == 0) ticket = atomicAdd(a.counters + d.rb, 1u);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket != a.nseg - 1) continue;
            __threadfence();
#pragma unroll
            for (int j = 0; j < G; j++)
#pragma unroll
                for (int b = 0; b < BT; b++) y[j][b] = 0.0f;
            for (uint32_t s = 0; s < a.nseg; s++) {
                const float *src = a.partials + ((size_t)s * a.Npad + row) * BT;
#pragma unroll
                for (int j = 0; j < G; j++)
#pragma unroll
                    for (int b = 0; b < BT; b++) y[j][b] += __ldcg(src + j * BT + b);
            }
            if (lane == 0) a.counters[d.rb] = 0u;
        }
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

template <int G, int BITS, int KIND>
static int launch_gemv_bt(const GemvArgs &a, cudaStream_t st)
{
    const uint32_t bt = a.batch <= 1 ? 1 : a.batch <= 2 ? 2 : a.batch <= 4 ? 4 : 8;
    const size_t smem = gemv_smem_bytes(a.K, a.p, bt, KIND);
    void (*kern)(const GemvArgs) = nullptr;
    switch (bt) {
        case 1: kern = gemv_tiles_kernel<G, BITS, 1, KIND>; break;
        case 2: kern = gemv_tiles_kernel<G, BITS, 2, KIND>; break;
        case 4: kern = gemv_tiles_kernel<G, BITS, 4, KIND>; break;
        default: kern = gemv_tiles_kernel<G, BITS, 8, KIND>; break;
    }
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
    const int sms = device_sm_count();
    uint32_t grid = (uint32_t)(sms * per_sm);
    grid = max(1u, min(grid, a.ntiles));
    kern<<<grid, kThreads, smem, st>>>(a);
    g_launches++;
    return (int)cudaGetLastError();
}

int launch_gemv(const GemvArgs &a, uint32_t G, uint32_t bits, uint32_t kind, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4) {
        if (G == 1) return launch_gemv_bt<1, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 2) return launch_gemv_bt<2, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 3) return launch_gemv_bt<3, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    }
    if (kind == EOQ_B200_KIND_Q5_POLAR && bits == 5) {
        if (G == 1) return launch_gemv_bt<1, 5, EOQ_B200_KIND_Q5_POLAR>(a, st);
        if (G == 2) return launch_gemv_bt<2, 5, EOQ_B200_KIND_Q5_POLAR>(a, st);
    }
    return (int)cudaErrorInvalidValue;
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
    __syncthreads();

    const uint32_t mask = M - 1u, p = a.p, sgroups = K / a.group;
    for (uint32_t t = blockIdx.x + gridDim.x * warp; t < a.ntiles; t += gridDim.x * nwarps) {
        const TileDesc d = a.tiles[t];
        const uint8_t *base = a.stream + ((size_t)d.off64 << 6);
        uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(base) + lane);
        const uint16_t *ptr = reinterpret_cast<const uint16_t *>(base + 128) + lane;
        uint32_t w = __ldg(ptr);
        const uint32_t row = d.row0 + lane * G;
        for (uint32_t c = d.col0; c < d.col0 + d.ncols; c += 8) {
            uint32_t sym[G][8];
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const uint32_t e = rans_step(tab, x, mask, p, F::kBiasMask);
#pragma unroll
                for (int j = 0; j < G; j++) sym[j][s] = (e >> F::field_bit(j)) & F::kFieldMask;
                rans_renorm(x, w, ptr);
            }
#pragma unroll
            for (int j = 0; j < G; j++) {
                const uint32_t r = row + j;
                if (r >= a.N) continue;
                if (a.out_sym) {
                    if (a.packed) {
                        uint32_t v = 0;
#pragma unroll
                        for (int s = 0; s < 8; s++) v |= sym[j][s] << (4 * s);
                        *reinterpret_cast<uint32_t *>(a.out_sym + (size_t)r * (K / 2) + c / 2) = v;
                    } else {
                        uint2 v = make_uint2(0, 0);
#pragma unroll
                        for (int s = 0; s < 4; s++) { v.x |= sym[j][s] << (8 * s); v.y |= sym[j][s + 4] << (8 * s); }
                        *reinterpret_cast<uint2 *>(a.out_sym + (size_t)r * K + c) = v;
                    }
                }
                if (a.out_deq && KIND == EOQ_B200_KIND_INT4_ABSMAX) {
                    // group is a multiple of 16 and c of 8, so the eight columns share one scale
                    const float sc = half_bits_to_float(__ldg(a.scales + (size_t)r * sgroups + c / a.group));
                    float v[8];
#pragma unroll
                    for (int s = 0; s < 8; s++) v[s] = (float)((int)sym[j][s] - 7) * sc;
                    const size_t o = (size_t)r * K + c;
                    if (a.out_dtype == EOQ_B200_F32) {
                        float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.out_deq) + o);
                        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
                    } else if (a.out_dtype == EOQ_B200_F16) {
                        __half2 h[4];
#pragma unroll
                        for (int s = 0; s < 4; s++) h[s] = __floats2half2_rn(v[2 * s], v[2 * s + 1]);
                        *reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(a.out_deq) + o) = *reinterpret_cast<uint4 *>(h);
                    } else {
                        __nv_bfloat162 h[4];
#pragma unroll
                        for (int s = 0; s < 4; s++) h[s] = __floats2bfloat162_rn(v[2 * s], v[2 * s + 1]);
                        *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(a.out_deq) + o) = *reinterpret_cast<uint4 *>(h);
                    }
                }
            }
        }
    }
}

template <int G, int BITS, int KIND>
static int launch_decode_tiles_t(const DecodeArgs &a, cudaStream_t st)
{
    const size_t smem = smem_table_bytes(a.p);
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
    if (kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4) {
        if (G == 1) return launch_decode_tiles_t<1, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 2) return launch_decode_tiles_t<2, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
        if (G == 3) return launch_decode_tiles_t<3, 4, EOQ_B200_KIND_INT4_ABSMAX>(a, st);
    }
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

int launch_decode_v1(const uint8_t *d_stream, const uint32_t *d_offsets, const uint32_t *d_sizes,
                     const V1Table *d_table, void *d_out, int out_elem_bytes, uint32_t nblocks,
                     uint32_t block_size, uint32_t total, uint32_t p, void *stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (nblocks == 0) return 0;
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
        store_y(out, i, (float)code * half_bits_to_float(__ldg(scales + flat / group)), out_dtype);
    }
}

int launch_dequant_packed(const uint8_t *packed, const uint16_t *scales, uint32_t K, uint32_t row_bytes, uint32_t bits,
                          uint32_t group, uint32_t row_lo, uint32_t row_hi, void *out, int out_dtype, void *stream)
{
    const uint64_t count = (uint64_t)(row_hi - row_lo) * K;
    if (count == 0) return 0;
    const uint32_t grid = (uint32_t)std::min<uint64_t>((count + 255) / 256, (uint64_t)device_sm_count() * 16);
    dequant_packed_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(packed, scales, K, row_bytes, bits, group,
                                                                                     row_lo, count, out, out_dtype);
    g_launches++;
    return (int)cudaGetLastError();
}

}  // namespace eoq
