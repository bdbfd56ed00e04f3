/*
 * eoq_b200.h -- C ABI of libeoq_b200.so, the sm_100a implementation of EOQ's
 * inference hot path: blocked rANS decode of entropy-coded quantised weights,
 * fused with per-group dequantisation and the GEMV that consumes them.
 *
 * Plain C: pointers and sizes only.  Every compute entry point runs on the
 * GPU; there is no CPU fallback.  On a machine without a CUDA device the
 * compute entry points return EOQ_ERR_CUDA (or -1 for the eoq_cuda_* family),
 * after argument validation, which never touches the device.
 *
 * Part 1 mirrors the reference's C interface one-for-one (same names, argument
 * meaning and error behaviour); each declaration cites the reference
 * declaration it replaces.  Part 2 is the fused path, which the reference
 * plans (PLANO_NIVEL2.md:19, core/eoq_linear.py:49-51) but does not have.
 */
#ifndef EOQ_B200_H
#define EOQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================================================== *
 * Part 1 -- drop-in for llamacpp_integration/eoq_rans_v2.h,
 *           eoq_parallel_decode.h and eoq_cuda_decompress.cu
 * ===================================================================== */

/* eoq_rans_v2.h:36-45.  EOQ_ERR_CUDA and EOQ_ERR_UNSUPPORTED are additions. */
typedef enum {
    EOQ_OK                   =  0,
    EOQ_ERR_NULL_PTR         = -1,
    EOQ_ERR_BUFFER_TOO_SMALL = -2,
    EOQ_ERR_CORRUPT_STREAM   = -3,
    EOQ_ERR_INVALID_HEADER   = -4,
    EOQ_ERR_ALLOC            = -5,
    EOQ_ERR_THREAD           = -6,   /* also: task skipped after a cancel request */
    EOQ_ERR_OVERFLOW         = -7,
    EOQ_ERR_CUDA             = -8,   /* no device, or a CUDA call failed */
    EOQ_ERR_UNSUPPORTED      = -9    /* legal input this build does not handle */
} eoq_error_t;

/* eoq_rans_v2.h:48 */
const char *eoq_error_string(eoq_error_t err);

/* eoq_rans_v2.h:54-62 (same field order and widths). */
typedef struct {
    uint32_t original_type;
    uint32_t num_blocks;
    uint32_t freq_table_size;    /* alphabet, 1..4096 (symbols are written as bytes) */
    uint32_t precision_bits;     /* 1..16 */
    uint32_t rans_block_size;    /* symbols per independent rANS block */
    uint32_t compressed_size;    /* bytes of payload, metadata included */
    uint32_t uncompressed_size;  /* symbols == output bytes */
} eoq_tensor_header_t;

/* eoq_rans_v2.h:77-81 */
typedef int (*eoq_progress_fn)(size_t bytes_decoded, size_t bytes_total, void *user_data);

/* eoq_rans_v2.h:87-91.  n_threads is accepted and ignored: every rANS block of
 * the tensor is decoded by its own GPU thread in one launch. */
typedef struct {
    uint32_t        n_threads;
    eoq_progress_fn progress_cb;
    void           *progress_ud;
} eoq_decode_opts_t;

/* eoq_rans_v2.h:94 */
#define EOQ_DECODE_OPTS_DEFAULT { 0, NULL, NULL }

/* eoq_rans_v2.h:116-123.  Host buffers in, host buffer out.  Payload layout
 * [u16 freq x A][u32 block_offsets x B][blocks] (eoq_rans_v2.c:606-619).
 * Checks, in the reference's order: NULL -> zero length (OK) -> header ->
 * out_cap -> comp_size -> metadata size -> offsets monotone and in range
 * (eoq_rans_v2.c:586-599, :542-545) -> 1+state_len <= block bytes (:392). */
eoq_error_t eoq_decode_tensor_v2(const eoq_tensor_header_t *header, const uint8_t *compressed,
                                 size_t comp_size, void *output, size_t out_cap,
                                 const eoq_decode_opts_t *opts);

/* eoq_rans_v2.h:129-133 */
int eoq_decode_tensor(const eoq_tensor_header_t *header, const uint8_t *compressed, void *output);

/* eoq_rans_v2.h:139 */
eoq_error_t eoq_validate_header(const eoq_tensor_header_t *header);

/* eoq_rans_v2.h:155-160 */
struct eoq_sym_info {
    uint16_t symbol;
    uint16_t freq;
    uint16_t cum_freq;
    uint16_t _pad;
};

/* eoq_rans_v2.h:166-174.  Same fields; `stream` and `sym_info` are owned by
 * the decoder object (device-side state is kept behind `sym_info`). */
typedef struct {
    uint32_t             state;
    const uint8_t       *stream;
    size_t               stream_pos;
    size_t               stream_end;
    uint32_t             precision_bits;
    uint32_t             precision_mask;
    struct eoq_sym_info *sym_info;
} eoq_decoder_t;

/* eoq_rans_v2.h:187-208: single-block decoder for advanced use. */
eoq_error_t eoq_decoder_init(eoq_decoder_t *dec, const uint16_t *freq_table, uint32_t alphabet_size,
                             uint32_t precision_bits, const uint8_t *block_data, size_t block_size);
eoq_error_t eoq_decoder_decode(eoq_decoder_t *dec, uint8_t *out, uint32_t count);
void        eoq_decoder_free(eoq_decoder_t *dec);

/* eoq_parallel_decode.h:35-46 */
typedef struct {
    const eoq_tensor_header_t *header;
    const uint8_t             *compressed_data;
    size_t                     compressed_size;
    void                      *output;
    size_t                     output_capacity;
    eoq_error_t                result;
    int                        task_index;
} eoq_decode_task_t;

/* eoq_parallel_decode.h:64-68: nonzero return requests cancellation; calls are
 * serialised and tensors_done increases by one per call. */
typedef int (*eoq_parallel_progress_fn)(int tensors_done, int tensors_total, void *user_data);

/* eoq_parallel_decode.h:74-78.  num_threads bounds the number of CUDA streams
 * (and pinned staging slots) tensors are pipelined over; 0 = automatic. */
typedef struct {
    int                      num_threads;
    eoq_parallel_progress_fn progress_cb;
    void                    *progress_ud;
} eoq_parallel_opts_t;

/* eoq_parallel_decode.h:80 */
#define EOQ_PARALLEL_OPTS_DEFAULT { 0, NULL, NULL }

/* eoq_parallel_decode.h:100-104.  Returns the first non-OK task result
 * (eoq_parallel_decode.c:290-300); num_tasks <= 0 is OK; NULL tasks with
 * num_tasks > 0 is EOQ_ERR_NULL_PTR (:155-156); tasks not started after a
 * cancel request get EOQ_ERR_THREAD (:72-82, :197-205). */
eoq_error_t eoq_parallel_decode(eoq_decode_task_t *tasks, int num_tasks, const eoq_parallel_opts_t *opts);

/* eoq_parallel_decode.h:106-111: default options. */
static inline eoq_error_t eoq_parallel_decode_auto(eoq_decode_task_t *tasks, int num_tasks)
{
    return eoq_parallel_decode(tasks, num_tasks, NULL);
}

/* eoq_parallel_decode.h:121 */
int eoq_detect_num_threads(void);

/* eoq_cuda_decompress.cu:405-410.  `stream` is a cudaStream_t passed as void*. */
int eoq_cuda_decode_tensor(const eoq_tensor_header_t *header, const uint8_t *compressed,
                           uint8_t *output, void *stream);

/* eoq_cuda_decompress.cu:213-221: device table entry {symbol, freq, cum}. */
typedef struct {
    uint16_t symbol;
    uint16_t freq;
    uint16_t cum_freq;
    uint16_t _pad;
} eoq_sym_info_packed;

/* eoq_cuda_decompress.cu:529-540.  All pointers are device pointers; asynchronous. */
int eoq_cuda_decode_tensor_device(const uint8_t *d_compressed_stream, const uint32_t *d_block_offsets,
                                  const uint32_t *d_block_sizes, const eoq_sym_info_packed *d_sym_info,
                                  uint8_t *d_output, uint32_t num_rans_blocks, uint32_t rans_block_size,
                                  uint32_t total_symbols, uint32_t precision_bits, void *cuda_stream);

/* eoq_cuda_decompress.cu:864-1021: batch context, at most 1024 tensors.  As in the
 * reference the caller owns the struct (stack or heap) and starts with
 * eoq_cuda_batch_init; here it is small and its per-tensor staging lives behind `impl`,
 * allocated by the first prepare_tensor and released by sync_and_free, after which the
 * struct may be reused or simply dropped.  `stream` is a cudaStream_t kept as void*. */
#define EOQ_CUDA_MAX_BATCH_TENSORS 1024                           /* :862 */
typedef struct eoq_cuda_batch_ctx {
    void    *impl;
    void    *stream;
    uint32_t n_tensors;
    uint32_t reserved;
} eoq_cuda_batch_ctx_t;
void eoq_cuda_batch_init(eoq_cuda_batch_ctx_t *ctx, void *stream);                       /* :882-887 */
int  eoq_cuda_batch_prepare_tensor(eoq_cuda_batch_ctx_t *ctx, const eoq_tensor_header_t *header,
                                   const uint8_t *compressed_host, uint8_t *d_output);   /* :900-975 */
int  eoq_cuda_batch_launch(eoq_cuda_batch_ctx_t *ctx);           /* :985-1003 */
int  eoq_cuda_batch_sync_and_free(eoq_cuda_batch_ctx_t *ctx);    /* :1008-1021 */
/* Heap-allocated variants for bindings that cannot hold a C struct by value. */
eoq_cuda_batch_ctx_t *eoq_cuda_batch_create(void *stream);
void eoq_cuda_batch_destroy(eoq_cuda_batch_ctx_t *ctx);

/* ===================================================================== *
 * Part 2 -- the fused path and the Python-facing codec entry points
 * ===================================================================== */

/* Blocked decode behind core/rans_blocked.py:124-165 (BlockedRANSDecoder) and
 * core/rans_bitpacked.py:126-154.  `freq` is the NORMALISED table (sum 2^p, all
 * >= 1; the caller normalises as core/rans.py:85-153 does).  `data`/`offsets`
 * are host pointers.  out_elem_bytes is 1 or 2.  If out_on_device is nonzero
 * `out` is a device pointer and the call is asynchronous on `stream`. */
eoq_error_t eoq_b200_decode_blocked(const uint32_t *freq, uint32_t alphabet, uint32_t precision_bits,
                                    const uint8_t *data, size_t data_len, const uint32_t *offsets,
                                    uint32_t num_blocks, uint32_t block_size, uint32_t num_symbols,
                                    void *out, int out_elem_bytes, int out_on_device, void *stream);

/* Host encoder behind core/rans_blocked.py:72-114 (wire-compatible with
 * core/rans.py:210-276).  Writes blocks back to back into `out` and their
 * offsets into `offsets`; *out_len in = capacity, out = bytes used. */
eoq_error_t eoq_b200_encode_blocked(const uint32_t *freq, uint32_t alphabet, uint32_t precision_bits,
                                    const uint32_t *symbols, uint32_t num_symbols, uint32_t block_size,
                                    uint8_t *out, size_t *out_len, uint32_t *offsets);

/* A weight matrix resident in HBM as entropy-coded tiles. */
typedef struct eoq_b200_weight eoq_b200_weight_t;

#define EOQ_B200_KIND_INT4_ABSMAX 0   /* w = (sym - 7) * scale[flat/group], core/quantized_linear.py:189-217 */
#define EOQ_B200_KIND_Q5_POLAR    1   /* w_block = norm/sqrt(d) * (centroid[sym] @ H), core/polar_quant.py:216-264 */
/* The other symmetric absmax widths a mixed-bit model uses (core/weight_packing.py:35-51, bits_fn of
 * core/rans_bitpacked.py:161-251): symbol = code + qmax, qmax = 2^(bits-1) - 1, w = (sym - qmax) * scale. */
#define EOQ_B200_KIND_INT2_ABSMAX 2   /* symbols 0..2,   three weights per rANS step */
#define EOQ_B200_KIND_INT3_ABSMAX 3   /* symbols 0..6,   three weights per rANS step */
#define EOQ_B200_KIND_INT8_ABSMAX 4   /* symbols 0..254, one weight per rANS step */

#define EOQ_B200_F16  0
#define EOQ_B200_BF16 1
#define EOQ_B200_F32  2
#define EOQ_B200_I8   3   /* eoq_b200_dequant_packed only: the signed codes, unscaled */

typedef struct {
    uint32_t kind;             /* EOQ_B200_KIND_* */
    uint32_t rows, cols;       /* N (out_features), K (in_features) */
    uint32_t group;            /* quantisation group: 128 (INT4) or 64 (polar) */
    uint32_t symbols_per_step; /* 0 = choose; weights coded jointly per rANS step */
    uint32_t precision_bits;   /* 0 = choose */
    uint32_t target_tiles;     /* 0 = choose from the device's SM count */
    const float *centroids;    /* polar only: 32 floats (host) */
} eoq_b200_weight_opts_t;

typedef struct {
    uint32_t rows, cols, padded_rows, group, kind;
    uint32_t symbols_per_step, precision_bits, alphabet;
    uint32_t num_tiles, num_col_segments;
    uint64_t stream_bytes;     /* entropy-coded tiles incl. initial states and padding */
    uint64_t table_bytes, scale_bytes, desc_bytes;
    uint64_t scratch_bytes;    /* per-call partial sums + counters (batch 8) */
    double   bits_per_weight;  /* stream_bytes*8 / (rows*cols) */
} eoq_b200_weight_info_t;

/* The tiled layout on the host, before upload: lets a loader build it once,
 * keep it (the arrays may be written to a cache file) and inspect it without a
 * device.  Tile t: rows [row0, row0 + 32*G), columns [col0, col0 + ncols);
 * its bytes are 32 x u32 initial states, then rows of 32 x u16 renormalisation
 * words (lane l reads column l, top to bottom).  The first head_bytes of tile
 * t lie at stream + t*head_bytes (a fixed stride, so a kernel can fetch them
 * from the tile index alone), the remaining 64*len64 - head_bytes at
 * stream + 64*off64. */
typedef struct eoq_b200_tiles eoq_b200_tiles_t;
typedef struct { uint32_t row0, col0, ncols, seg, off64, len64; } eoq_b200_tile_desc_t;   /* len64: tile bytes (head + tail) / 64 */
typedef struct {
    uint32_t rows, cols, padded_rows, group, kind, bits;
    uint32_t symbols_per_step, precision_bits;
    uint32_t num_tiles, num_col_segments;
    const uint32_t *table;               /* 1 << precision_bits entries: freq<<23 | sym<<(23-G*bits) | slot-cum */
    const eoq_b200_tile_desc_t *tiles;
    const uint8_t *stream;
    uint64_t stream_bytes;
    uint32_t max_lane_drift;             /* largest gap, in word rows, between two lanes' read positions in any tile */
    uint32_t head_bytes;                 /* 0, 1024 or 2048: bytes of every tile kept at the fixed stride */
} eoq_b200_tiles_view_t;
eoq_error_t eoq_b200_tiles_build(const uint8_t *symbols, const eoq_b200_weight_opts_t *opts, eoq_b200_tiles_t **out);
eoq_error_t eoq_b200_tiles_view(const eoq_b200_tiles_t *t, eoq_b200_tiles_view_t *view);
void        eoq_b200_tiles_free(eoq_b200_tiles_t *t);

/* Build from decoded symbols (host, one byte per weight, row-major N x K;
 * INT4: code+7 in 0..14, polar: centroid index 0..31) and fp16 scales (host;
 * flat N*K/group, as QuantizedLinear.scales / PolarQuantResult.norms). */
eoq_error_t eoq_b200_weight_from_symbols(const uint8_t *symbols, const uint16_t *scales_fp16,
                                         const eoq_b200_weight_opts_t *opts, eoq_b200_weight_t **out);

/* The same from symbols that are already in the current device's memory (one byte
 * per weight, row-major N x K): counted, encoded into tiles and laid out on the
 * device, byte-identical to what eoq_b200_tiles_build makes on the host.  Scales
 * on the host.  eoq_b200_weight_from_symbols and eoq_b200_weight_from_rans take
 * this route themselves after copying / decoding their input to the device. */
eoq_error_t eoq_b200_weight_from_device_symbols(const uint8_t *d_symbols, const uint16_t *scales_fp16,
                                                const eoq_b200_weight_opts_t *opts, eoq_b200_weight_t **out);

/* Upload tiles built by eoq_b200_tiles_build to the current device (may be called
 * repeatedly, e.g. once per GPU that holds a replica).  centroids: polar only. */
eoq_error_t eoq_b200_weight_from_tiles(const eoq_b200_tiles_t *tiles, const uint16_t *scales_fp16,
                                       const float *centroids, eoq_b200_weight_t **out);

/* Build from the reference's serialised `RANS` container
 * (core/rans_blocked.py:176-214), i.e. what .eoq files and
 * CompressedTensorData.rans_bytes hold: the wire-format blocks are decoded on
 * the GPU and re-tiled once, at load time. */
eoq_error_t eoq_b200_weight_from_rans(const uint8_t *rans_container, size_t size,
                                      const uint16_t *scales_fp16, const eoq_b200_weight_opts_t *opts,
                                      eoq_b200_weight_t **out);

void        eoq_b200_weight_destroy(eoq_b200_weight_t *w);
eoq_error_t eoq_b200_weight_info(const eoq_b200_weight_t *w, eoq_b200_weight_info_t *info);

/* y[b, :] = W x[b, :] (+ bias), the fused replacement for
 * QuantizedLinear.forward (core/quantized_linear.py:222-228) at batch 1..8:
 * decode -> unpack -> scale -> dot product in one kernel; decoded symbols are
 * never written to memory.  x is [batch, K], y is [batch, N], row-major, device
 * pointers of the given element types; bias is fp32 [N] or NULL; accumulation
 * is fp32.  Asynchronous on `stream`.  One launch serves up to 2 or 4 rows of x
 * (INT4, depending on the tile size) or up to 8 (Q5 polar); larger batches are
 * consecutive launches over row slices on the same stream.  Scratch is part of
 * the weight and allocated when it is created, with one exception: an INT4
 * weight whose tiles do not fit the two-tiles-per-warp kernel (or that is run
 * with "gemv_pairs" = 0) allocates the other kernel's scratch in its first call,
 * which should therefore not be made inside stream capture. */
eoq_error_t eoq_b200_gemv(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch,
                          void *y, int y_dtype, const float *bias, void *stream);

/* Y = X W^T (+ bias) for many activation rows (prefill), the fused replacement for
 * dequantize-then-matmul (core/quantized_linear.py:222-228, core/quantized_matmul.py:91-176)
 * when m is too large for the GEMV kernel: the compressed tiles are decoded once per 128
 * activation rows and the decoded fp16 pieces go from shared memory straight into tensor-core
 * MMAs (tcgen05, fp32 accumulator in tensor memory); the dequantised matrix never exists in
 * HBM.  x is [m, K], y is [m, N], row-major device pointers, both 16-byte aligned; fp16
 * activations enter the tensor cores as they are, fp32 and bf16 ones are rounded to fp16 first
 * (the tensor cores take both operands in one 16-bit format, and the weights are
 * (q - 7) * scale in fp16), so |x| must stay below 65504.  INT4 weights in the
 * default layout (3 weights per step) only; others return EOQ_ERR_UNSUPPORTED.  Asynchronous
 * on `stream`. */
eoq_error_t eoq_b200_gemm(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t m,
                          void *y, int y_dtype, const float *bias, void *stream);

/* Row-sharded GEMV with the all-gather of the output slices fused into the kernel (no
 * counterpart in the reference, whose multi-GPU plan stops at "shard by rows").  One process
 * per GPU; rank r holds the weight rows [row_offset, row_offset + N) of an n_total-row layer.
 * Every rank creates a gather object (one device allocation of `slots` output buffers plus
 * flags), passes the 64-byte handle it gets to all other ranks by any means (the Python side
 * uses torch.distributed), and connects.  eoq_b200_gemv_gather is ONE kernel: it computes this
 * rank's rows, writes them into its own full-size output, sends them as 8-byte words straight
 * into slot `slot` of every peer's receive buffer (plain stores over NVLink; an aligned 8-byte
 * store arrives whole, so the epoch inside the word is the flag and no fence is needed; with
 * 16-bit outputs one word carries the three rows of a lane plus a 16-bit epoch), and then waits
 * for the words of the other ranks and unpacks them.  The wait is bounded (about a second, or
 * eoq_b200_gather_set_timeout_ms); when it runs out the kernel returns all the same and
 * eoq_b200_gather_status reports EOQ_ERR_CUDA once.  After the call, work queued on `stream`
 * may read the full [batch, n_total] result at eoq_b200_gather_buffer(g, slot).
 * Rules: shards are equal and in rank order (row_offset = rank * N, n_total = world * N); all
 * ranks make the same sequence of calls; consecutive calls use different slots (a fast rank
 * may send the next gather while a slow one still unpacks the previous one);
 * batch * n_total * sizeof(y) <= slot_bytes; world <= 8; the weight, the gather object and the
 * current device must be the same GPU (else EOQ_ERR_UNSUPPORTED, nothing is launched).
 * eoq_b200_gather_wait is the second half on its own, for receive buffers that something else
 * fills: it waits for `rows_per_rank` rows from every other rank in words of `rows_per_word`
 * rows (1..3; fp32 outputs always use one word per value) and unpacks them into the slot. */
#define EOQ_B200_IPC_HANDLE_BYTES 64
typedef struct eoq_b200_gather eoq_b200_gather_t;
eoq_error_t eoq_b200_gather_create(uint32_t world, uint32_t rank, uint32_t slots, size_t slot_bytes,
                                   eoq_b200_gather_t **out, void *ipc_handle_out);
eoq_error_t eoq_b200_gather_connect(eoq_b200_gather_t *g, const void *all_handles /* world x 64 B, by rank */);
void        eoq_b200_gather_destroy(eoq_b200_gather_t *g);
void       *eoq_b200_gather_buffer(eoq_b200_gather_t *g, uint32_t slot);
eoq_error_t eoq_b200_gather_status(eoq_b200_gather_t *g, void *stream);
eoq_error_t eoq_b200_gather_set_timeout_ms(eoq_b200_gather_t *g, uint32_t milliseconds /* 1..60000 */);
eoq_error_t eoq_b200_gather_wait(eoq_b200_gather_t *g, uint32_t slot, uint32_t rows_per_rank, uint32_t batch,
                                 int y_dtype, uint32_t rows_per_word, void *stream);
eoq_error_t eoq_b200_gemv_gather(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch, int y_dtype,
                                 const float *bias, eoq_b200_gather_t *g, uint32_t slot, uint32_t row_offset,
                                 uint32_t n_total, void *stream);

/* Same with host buffers: copies x in, runs, copies y out, synchronises. */
eoq_error_t eoq_b200_gemv_host(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch,
                               void *y, int y_dtype, const float *bias_host, void *stream);

/* The same without the final synchronisation: copies and kernel are queued on `stream` and the
 * call returns; x, y and bias_host must stay valid (and should be pinned) until the stream has
 * been synchronised, e.g. by eoq_b200_weight_status, which also reports a failed launch.
 * Several weights can be queued this way before one synchronisation; a weight must not be
 * queued again before its previous call has completed (it owns one staging buffer).  A pinned
 * y is written by the kernel itself (pinned memory is device-addressable), so no copy back is
 * queued; a pageable y is filled by a copy from the weight's device buffer. */
eoq_error_t eoq_b200_gemv_host_async(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch,
                               void *y, int y_dtype, const float *bias_host, void *stream);

/* The same product for callers that must not allocate device memory (no counterpart in the
 * reference).  A serving process that has given all of HBM to its own arena, a latency-critical
 * thread that may not take the allocator's lock, or a framework that forbids allocation while it
 * replays recorded work cannot let a library call cudaMalloc behind its back.  This entry point
 * calls no allocator at all -- neither cudaMalloc/cudaFree nor any allocating library routine:
 * the scratch the kernel needs across tiles (partial row sums per column segment and arrival
 * counters per row block) is a fixed array of EOQ_B200_GEMV_STATIC_SCRATCH_BYTES in device
 * global memory that belongs to the library image, so every GPU that loads the library
 * carries it until the process exits.  x, y and bias are still the caller's buffers.
 *
 *  - A weight whose scratch need exceeds the array (it grows with rows x column segments x
 *    batch) is refused with EOQ_ERR_BUFFER_TOO_SMALL and a message on stderr; use
 *    eoq_b200_gemv for it.
 *  - The first call on each device looks up the array's device address (one
 *    cudaGetSymbolAddress with that device current).  Make that first call outside any
 *    stream capture.
 *  - All calls on a device share the one array, and it keeps the previous call's contents.
 *    The counters are cleared on `stream` before each launch; the partial sums are always
 *    written before they are read.  Two calls that overlap on the GPU (different streams,
 *    or different weights at the same time) race on the array: serialise them.
 *  - Results are identical to eoq_b200_gemv. */
#define EOQ_B200_GEMV_STATIC_SCRATCH_BYTES (8u << 20)
eoq_error_t eoq_b200_gemv_static_scratch(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch,
                                         void *y, int y_dtype, const float *bias, void *stream);

/* Decode the tiles back to the reference's in-memory forms (device pointers,
 * asynchronous): packed INT4 as QuantizedLinear.packed_weight
 * (core/quantized_linear.py:76-91: uint8 [N, K/2], low nibble = even column),
 * or one symbol per byte [N, K], and/or the dequantised matrix [N, K] in
 * out_dtype (core/fast_dequant.py:47-87).  Either output may be NULL. */
eoq_error_t eoq_b200_weight_decode(eoq_b200_weight_t *w, uint8_t *d_symbols_or_packed, int packed,
                                   void *d_dequant, int out_dtype, void *stream);

/* Dequantise QuantizedLinear's in-memory form on the GPU, any shape and any
 * bit width the reference stores (2 and 4 packed, others one int8 per code):
 * rows [row_lo, row_hi) of d_packed [rows, row_bytes] with scales indexed over
 * the flattened matrix -> dense [row_hi-row_lo, cols] in out_dtype; with
 * out_dtype EOQ_B200_I8 the signed codes are written instead (int8, scales may
 * be NULL: unpack_4bit_fast / unpack_2bit_fast, core/fast_dequant.py:9-44).  Behind
 * core/fast_dequant.py:47-87, core/quantized_matmul.py:123-225 and
 * QuantizedLinear._dequantize_weight (core/quantized_linear.py:189-217).
 * Device pointers; asynchronous. */
eoq_error_t eoq_b200_dequant_packed(const uint8_t *d_packed, const uint16_t *d_scales_fp16, uint32_t rows, uint32_t cols,
                                    uint32_t bits, uint32_t group, uint32_t row_lo, uint32_t row_hi, void *d_out,
                                    int out_dtype, void *stream);

/* y = x @ W.T (+ bias) straight from QuantizedLinear's in-memory form, for up
 * to 8 (or 32, see below) activation rows: what QuantizedLinear.forward computes by dequantising
 * the whole matrix and calling a GEMM (core/quantized_linear.py:219-228), as
 * one pass over the packed codes (2 and 4 bits packed low bits first with the
 * code + qmax, any other width one signed code per byte) and the fp16 scales,
 * fp32 accumulation.  Needs cols a multiple of the group and of the codes in
 * sixteen bytes (32 at 4 bits, 64 at 2 bits, 16 otherwise), the group a multiple
 * of 8 and d_packed 16-byte aligned (EOQ_ERR_UNSUPPORTED otherwise: use
 * eoq_b200_dequant_packed and a GEMM).  x [batch, cols] and y [batch, rows] in
 * EOQ_B200_F16 / BF16 / F32; device pointers; asynchronous.  With cols a
 * multiple of 128 and the group a multiple of 128 the product runs on the tensor
 * cores and takes up to 32 rows: 16-bit activations (16-byte aligned) as they
 * are, fp32 activations as two fp16 halves each (the nearest fp16 and the nearest
 * to the remainder; the codes are exact, so the products carry about 2^-22),
 * which one extra small launch writes into d_scratch (batch * cols * 4 bytes,
 * 16-byte aligned, the caller's; NULL: fp32 activations take the general form).
 * More rows than the form in use takes: EOQ_ERR_UNSUPPORTED. */
eoq_error_t eoq_b200_gemv_packed(const uint8_t *d_packed, const uint16_t *d_scales_fp16, uint32_t rows, uint32_t cols,
                                 uint32_t bits, uint32_t group, const void *x, int x_dtype, uint32_t batch, void *d_scratch,
                                 void *y, int y_dtype, const float *bias, void *stream);

/* y = x @ W.T (+ bias) straight from PolarLinear's in-memory form (kernels/polar_engine.py:144-360: one centroid index
 * per byte, one fp16 norm per block of each row, 2^bits fp32 centroids), for up to 8 activation rows on the CUDA cores
 * and 32 on the tensor cores.  Two launches:
 * the activations are rotated once (every block of `block` columns times the block's normalised Hadamard matrix,
 * divided by sqrt(block): the matrix is symmetric, so the rotation the reference applies to every dequantised weight
 * block, kernels/polar_engine.py:257-264, moves to x) into d_scratch (batch * cols * 4 bytes, 16-byte aligned, the
 * caller's), then one pass over the codes.  tensor_cores = 0: CUDA cores, fp32 throughout, block a power of two >= 16;
 * 1: tensor cores (centroids and rotated activations as two fp16 halves each, fp32 accumulation: within about 1e-6 of
 * the fp32 form), block >= 64; -1: the quicker of the two for this batch.  The block must divide cols and be at most
 * 4096; d_codes 16-byte aligned (EOQ_ERR_UNSUPPORTED otherwise).  x in EOQ_B200_F16 / BF16 / F32.  Device pointers;
 * asynchronous. */
eoq_error_t eoq_b200_gemv_polar_codes(const uint8_t *d_codes, const uint16_t *d_norms_fp16, const float *d_centroids,
                                      uint32_t rows, uint32_t cols, uint32_t bits, uint32_t block, const void *x, int x_dtype,
                                      uint32_t batch, void *d_scratch, void *y, int y_dtype, const float *bias,
                                      int tensor_cores, void *stream);

/* Synchronises `stream` and reports whether any kernel that used this weight gave up on a
 * bounded wait for its staged data (EOQ_ERR_CUDA; outputs of that launch are then invalid).
 * The kernels never spin without a limit, so a fault in the copy engine ends in this error
 * rather than in a hang. */
eoq_error_t eoq_b200_weight_status(eoq_b200_weight_t *w, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* EOQ_B200_H */
