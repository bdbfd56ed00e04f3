// C ABI of libeoq_b200.so (declarations and reference citations: include/eoq_b200.h).
// Host-side validation mirrors the reference's checks and error codes; all
// decoding runs on the GPU.
#include "eoq_internal.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_runtime.h>
#include <memory>
#include <mutex>
#include <unistd.h>

using namespace eoq;

namespace {

#define CU_TRY(call)                                                                          \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "eoq_b200: %s failed: %s\n", #call, cudaGetErrorString(e__)); \
            return EOQ_ERR_CUDA;                                                              \
        }                                                                                     \
    } while (0)

bool have_device()
{
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}

// Owns a set of device allocations; frees them when it goes out of scope.
struct DeviceBuf {
    void *p = nullptr;
    DeviceBuf() = default;
    DeviceBuf(const DeviceBuf &) = delete;
    DeviceBuf &operator=(const DeviceBuf &) = delete;
    ~DeviceBuf() { if (p) cudaFree(p); }
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 1); }
    template <typename T> T *as() const { return reinterpret_cast<T *>(p); }
};

// Pieces of a validated tensor payload `[u16 freq x A][u32 offsets x B][blocks]`.
struct Payload {
    uint32_t alphabet = 0, p = 0, block = 0, total = 0, nblocks = 0;
    const uint16_t *freq = nullptr;
    const uint8_t *offsets_raw = nullptr;   // may be unaligned
    const uint8_t *stream = nullptr;
    uint32_t stream_bytes = 0;
    std::vector<uint32_t> offsets, sizes;
};

// Checks of eoq_decode_tensor_v2 (eoq_rans_v2.c:586-619), then the per-block
// checks its workers make while decoding (:542-545 offsets, :392 state length),
// done here on the host so nothing corrupt is ever launched.
eoq_error_t parse_payload(const eoq_tensor_header_t *h, const uint8_t *comp, size_t comp_size, size_t out_cap, Payload &pl)
{
    eoq_error_t rc = eoq_validate_header(h);
    if (rc != EOQ_OK) return rc;
    if (out_cap < h->uncompressed_size) return EOQ_ERR_BUFFER_TOO_SMALL;
    if (comp_size < h->compressed_size) return EOQ_ERR_CORRUPT_STREAM;
    pl.alphabet = h->freq_table_size; pl.p = h->precision_bits; pl.block = h->rans_block_size;
    pl.total = h->uncompressed_size;
    pl.nblocks = (uint32_t)(((uint64_t)pl.total + pl.block - 1) / pl.block);
    const uint64_t meta = (uint64_t)pl.alphabet * 2 + (uint64_t)pl.nblocks * 4;
    if (meta > h->compressed_size) return EOQ_ERR_CORRUPT_STREAM;
    pl.freq = reinterpret_cast<const uint16_t *>(comp);
    pl.offsets_raw = comp + (size_t)pl.alphabet * 2;
    pl.stream = comp + meta;
    pl.stream_bytes = h->compressed_size - (uint32_t)meta;
    pl.offsets.resize(pl.nblocks);
    pl.sizes.resize(pl.nblocks);
    std::memcpy(pl.offsets.data(), pl.offsets_raw, (size_t)pl.nblocks * 4);
    for (uint32_t b = 0; b < pl.nblocks; b++) {
        const uint32_t lo = pl.offsets[b];
        const uint32_t hi = b + 1 < pl.nblocks ? pl.offsets[b + 1] : pl.stream_bytes;
        if (hi < lo || hi > pl.stream_bytes) return EOQ_ERR_CORRUPT_STREAM;
        pl.sizes[b] = hi - lo;
        if (pl.sizes[b] && 1u + pl.stream[lo] > pl.sizes[b]) return EOQ_ERR_CORRUPT_STREAM;
    }
    return EOQ_OK;
}

void make_v1_table(const std::vector<uint32_t> &freq, const std::vector<uint32_t> &cdf, uint32_t p, std::vector<V1Table> &t)
{
    t.assign((size_t)1 << p, V1Table{1, 0});
    for (uint32_t s = 0; s + 1 < cdf.size(); s++)
        for (uint32_t k = cdf[s]; k < cdf[s + 1]; k++) t[k] = V1Table{freq[s], (s << 16) | (k - cdf[s])};
}

eoq_error_t table_from_u16(const uint16_t *raw16, uint32_t alphabet, uint32_t p, std::vector<V1Table> &t)
{
    std::vector<uint32_t> raw(alphabet), freq, cdf;
    for (uint32_t s = 0; s < alphabet; s++) { uint16_t v; std::memcpy(&v, raw16 + s, 2); raw[s] = v; }
    eoq_error_t rc = normalize_reference(raw.data(), alphabet, p, freq, cdf);
    if (rc != EOQ_OK) return rc;
    make_v1_table(freq, cdf, p, t);
    return EOQ_OK;
}

// One device allocation that serves a whole decode call (streams, block tables, frequencies, task descriptors,
// outputs): the decode entry points make no allocation per tensor.  Allocations are kept in a small process-wide cache
// between calls (grow-only, at most four, freed at exit), so a loader that decodes tensor after tensor allocates once.
class DeviceArena {
  public:
    DeviceArena() = default;
    DeviceArena(const DeviceArena &) = delete;
    DeviceArena &operator=(const DeviceArena &) = delete;
    ~DeviceArena() { release(); }
    cudaError_t acquire(size_t bytes)
    {
        release();
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        {
            std::lock_guard<std::mutex> lock(cache().mu);
            auto &v = cache().free_list;
            int best = -1;
            for (int i = 0; i < (int)v.size(); i++)
                if (v[i].dev == dev && v[i].cap >= bytes && (best < 0 || v[i].cap < v[best].cap)) best = i;
            if (best < 0)                         // none large enough: recycle the largest of this device rather than keep both
                for (int i = 0; i < (int)v.size(); i++)
                    if (v[i].dev == dev && (best < 0 || v[i].cap > v[best].cap)) best = i;
            if (best >= 0) { cur_ = v[best]; v.erase(v.begin() + best); }
        }
        if (cur_.p && cur_.cap < bytes) { cudaFree(cur_.p); cur_ = Block(); }
        if (!cur_.p) {
            const size_t cap = std::max<size_t>((bytes + (1u << 20)) & ~(size_t)((1u << 20) - 1), 4u << 20);
            e = cudaMalloc(&cur_.p, cap);
            if (e != cudaSuccess) { cur_ = Block(); return e; }
            cur_.cap = cap; cur_.dev = dev;
        }
        return cudaSuccess;
    }
    void release()
    {
        if (!cur_.p) return;
        std::lock_guard<std::mutex> lock(cache().mu);
        if (cache().free_list.size() < 4) cache().free_list.push_back(cur_);
        else cudaFree(cur_.p);
        cur_ = Block();
    }
    uint8_t *base() const { return static_cast<uint8_t *>(cur_.p); }

  private:
    struct Block { void *p = nullptr; size_t cap = 0; int dev = 0; };
    struct Cache { std::mutex mu; std::vector<Block> free_list; };
    static Cache &cache() { static Cache *c = new Cache(); return *c; }      // never destroyed: no CUDA call after main
    Block cur_;
};

// One tensor of a decode call.
struct V1Job {
    Payload pl;                         // validated host views of the payload
    std::vector<uint32_t> freq, cdf;    // normalised table
    uint32_t out_elem_bytes = 1;
    void *host_out = nullptr;           // where the symbols go on the host, or
    void *dev_out = nullptr;            // the caller's device buffer
    std::vector<uint8_t> own_payload;   // batch context: the caller's host bytes, kept until launch
    // placement inside the arena
    size_t at_stream = 0, at_offsets = 0, at_sizes = 0, at_freq = 0, at_table = 0, at_out = 0;
    bool lanes = false;
};

eoq_error_t job_from_payload(const eoq_tensor_header_t *h, const uint8_t *comp, size_t comp_size, size_t out_cap, V1Job &j)
{
    eoq_error_t rc = parse_payload(h, comp, comp_size, out_cap, j.pl);
    if (rc != EOQ_OK) return rc;
    std::vector<uint32_t> raw(j.pl.alphabet);
    for (uint32_t s = 0; s < j.pl.alphabet; s++) { uint16_t v; std::memcpy(&v, j.pl.freq + s, 2); raw[s] = v; }
    return normalize_reference(raw.data(), j.pl.alphabet, j.pl.p, j.freq, j.cdf);
}

// Decode `n` validated jobs: one arena, one upload of all metadata, the streams copied in, ONE launch of the lane kernel
// over every job it serves (others run the one-thread-per-block kernel), results copied to the host buffers that ask
// for it (with copy_out false they stay in the arena, at at_out, for the caller to fetch).  Asynchronous on `st`; the arena must stay acquired until the stream has been synchronised.
eoq_error_t decode_jobs(V1Job **jobs, size_t n, cudaStream_t st, DeviceArena &arena, bool copy_out = true)
{
    if (n == 0) return EOQ_OK;
    if (!have_device()) return EOQ_ERR_CUDA;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    // layout: [metadata blob: per job offsets, sizes, freq (or slot table); task descriptors; CTA map][streams][outputs]
    std::vector<V1Task> tasks;
    std::vector<size_t> task_job;
    size_t meta = 0;
    for (size_t i = 0; i < n; i++) {
        V1Job &j = *jobs[i];
        j.at_offsets = meta; meta = up(meta + (size_t)j.pl.nblocks * 4);
        j.at_sizes = meta;   meta = up(meta + (size_t)j.pl.nblocks * 4);
        j.at_freq = meta;    meta = up(meta + (size_t)j.pl.alphabet * 4);
        V1Task t = {};
        t.nblocks = j.pl.nblocks; t.block_size = j.pl.block; t.total = j.pl.total; t.p = j.pl.p; t.alphabet = j.pl.alphabet;
        t.out_elem_bytes = j.out_elem_bytes;
        t.stream = reinterpret_cast<const uint8_t *>((uintptr_t)0);       // alignment is that of the arena slice: always 256
        j.lanes = v1_lanes_enabled() && v1_task_prepare(t);
        if (j.lanes) { tasks.push_back(t); task_job.push_back(i); }
        else { j.at_table = meta; meta = up(meta + ((size_t)8 << j.pl.p)); }
    }
    uint32_t warps_per_cta = 1, grid = 0;
    size_t smem = 0;
    if (!tasks.empty()) grid = v1_plan_ctas(tasks.data(), (uint32_t)tasks.size(), warps_per_cta, smem);
    const size_t at_tasks = meta; meta = up(meta + tasks.size() * sizeof(V1Task));
    const size_t at_cta = meta;   meta = up(meta + (size_t)grid * 4);
    size_t total = meta;
    for (size_t i = 0; i < n; i++) {
        V1Job &j = *jobs[i];
        j.at_stream = total; total = up(total + j.pl.stream_bytes + 16);
        if (!j.dev_out) { j.at_out = total; total = up(total + (size_t)j.pl.total * j.out_elem_bytes + 32); }
    }
    if (arena.acquire(total) != cudaSuccess) return EOQ_ERR_ALLOC;
    uint8_t *d = arena.base();
    std::vector<uint8_t> blob(meta, 0);
    for (size_t i = 0; i < n; i++) {
        V1Job &j = *jobs[i];
        std::memcpy(blob.data() + j.at_offsets, j.pl.offsets.data(), (size_t)j.pl.nblocks * 4);
        std::memcpy(blob.data() + j.at_sizes, j.pl.sizes.data(), (size_t)j.pl.nblocks * 4);
        std::memcpy(blob.data() + j.at_freq, j.freq.data(), (size_t)j.pl.alphabet * 4);
        if (!j.lanes) {
            std::vector<V1Table> table;
            make_v1_table(j.freq, j.cdf, j.pl.p, table);
            std::memcpy(blob.data() + j.at_table, table.data(), table.size() * sizeof(V1Table));
        }
    }
    std::vector<uint32_t> cta_task(grid);
    for (size_t k = 0; k < tasks.size(); k++) {
        V1Job &j = *jobs[task_job[k]];
        V1Task &t = tasks[k];
        t.stream = d + j.at_stream; t.offsets = reinterpret_cast<const uint32_t *>(d + j.at_offsets);
        t.sizes = reinterpret_cast<const uint32_t *>(d + j.at_sizes); t.freq = reinterpret_cast<const uint32_t *>(d + j.at_freq);
        t.table = nullptr; t.out = j.dev_out ? j.dev_out : d + j.at_out;
        const uint32_t last = k + 1 < tasks.size() ? tasks[k + 1].first_cta : grid;
        for (uint32_t c = t.first_cta; c < last; c++) cta_task[c] = (uint32_t)k;
    }
    if (!tasks.empty()) {
        std::memcpy(blob.data() + at_tasks, tasks.data(), tasks.size() * sizeof(V1Task));
        std::memcpy(blob.data() + at_cta, cta_task.data(), (size_t)grid * 4);
    }
    // pageable sources are consumed before cudaMemcpyAsync returns
    CU_TRY(cudaMemcpyAsync(d, blob.data(), meta, cudaMemcpyHostToDevice, st));
    for (size_t i = 0; i < n; i++) {
        V1Job &j = *jobs[i];
        if (j.pl.stream_bytes) CU_TRY(cudaMemcpyAsync(d + j.at_stream, j.pl.stream, j.pl.stream_bytes, cudaMemcpyHostToDevice, st));
    }
    if (!tasks.empty()) {
        int e = launch_decode_v1_lanes(reinterpret_cast<const V1Task *>(d + at_tasks), reinterpret_cast<const uint32_t *>(d + at_cta), grid,
                                       warps_per_cta, smem, st);
        if (e != 0) { std::fprintf(stderr, "eoq_b200: decode launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    }
    for (size_t i = 0; i < n; i++) {
        V1Job &j = *jobs[i];
        void *out = j.dev_out ? j.dev_out : d + j.at_out;
        if (!j.lanes) {
            int e = launch_decode_v1(d + j.at_stream, reinterpret_cast<const uint32_t *>(d + j.at_offsets),
                                     reinterpret_cast<const uint32_t *>(d + j.at_sizes), reinterpret_cast<const V1Table *>(d + j.at_table), out,
                                     (int)j.out_elem_bytes, j.pl.nblocks, j.pl.block, j.pl.total, j.pl.p, j.pl.alphabet, st);
            if (e != 0) { std::fprintf(stderr, "eoq_b200: decode launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
        }
        if (j.host_out && copy_out) CU_TRY(cudaMemcpyAsync(j.host_out, out, (size_t)j.pl.total * j.out_elem_bytes, cudaMemcpyDeviceToHost, st));
    }
    return EOQ_OK;
}

eoq_error_t decode_host_to_host(const eoq_tensor_header_t *h, const uint8_t *comp, size_t comp_size, void *output,
                                size_t out_cap, cudaStream_t st)
{
    V1Job job;
    eoq_error_t rc = job_from_payload(h, comp, comp_size, out_cap, job);
    if (rc != EOQ_OK) return rc;
    job.host_out = output;
    V1Job *one = &job;
    DeviceArena arena;
    rc = decode_jobs(&one, 1, st, arena);
    if (rc != EOQ_OK) return rc;
    CU_TRY(cudaStreamSynchronize(st));
    return EOQ_OK;
}

}  // namespace

// =========================================================================
// Part 1: the reference's C interface
// =========================================================================

extern "C" const char *eoq_error_string(eoq_error_t err)
{
    switch (err) {
        case EOQ_OK: return "success";
        case EOQ_ERR_NULL_PTR: return "null pointer argument";
        case EOQ_ERR_BUFFER_TOO_SMALL: return "output buffer too small";
        case EOQ_ERR_CORRUPT_STREAM: return "corrupt compressed stream";
        case EOQ_ERR_INVALID_HEADER: return "invalid tensor header";
        case EOQ_ERR_ALLOC: return "memory allocation failed";
        case EOQ_ERR_THREAD: return "threading error";
        case EOQ_ERR_OVERFLOW: return "integer overflow";
        case EOQ_ERR_CUDA: return "CUDA device unavailable or CUDA call failed";
        case EOQ_ERR_UNSUPPORTED: return "input not supported by this build";
    }
    return "unknown error";
}

extern "C" eoq_error_t eoq_validate_header(const eoq_tensor_header_t *h)
{
    if (!h) return EOQ_ERR_NULL_PTR;
    if (h->freq_table_size == 0 || h->freq_table_size > 4096) return EOQ_ERR_INVALID_HEADER;
    if (h->precision_bits == 0 || h->precision_bits > 16) return EOQ_ERR_INVALID_HEADER;
    if (h->rans_block_size == 0) return EOQ_ERR_INVALID_HEADER;
    if ((uint64_t)h->compressed_size < (uint64_t)h->freq_table_size * 2 + 4) return EOQ_ERR_INVALID_HEADER;
    return EOQ_OK;
}

extern "C" int eoq_detect_num_threads(void)
{
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    if (n > 0) return (int)n;
    n = sysconf(_SC_NPROCESSORS_CONF);
    return n > 0 ? (int)n : 4;
}

extern "C" eoq_error_t eoq_decode_tensor_v2(const eoq_tensor_header_t *header, const uint8_t *compressed, size_t comp_size,
                                            void *output, size_t out_cap, const eoq_decode_opts_t *opts)
{
    if (!header || !compressed || !output) return EOQ_ERR_NULL_PTR;
    if (header->uncompressed_size == 0) return EOQ_OK;
    eoq_error_t rc = decode_host_to_host(header, compressed, comp_size, output, out_cap, nullptr);
    // the whole tensor is one launch, so progress is reported once, complete (eoq_rans_v2.c:757-762)
    if (rc == EOQ_OK && opts && opts->progress_cb)
        opts->progress_cb(header->uncompressed_size, header->uncompressed_size, opts->progress_ud);
    return rc;
}

extern "C" int eoq_decode_tensor(const eoq_tensor_header_t *header, const uint8_t *compressed, void *output)
{
    if (!header) return (int)EOQ_ERR_NULL_PTR;
    return (int)eoq_decode_tensor_v2(header, compressed, header->compressed_size, output, header->uncompressed_size, nullptr);
}

// Tensors are decoded in groups: the tasks of a group are validated on the host, uploaded together and decoded by ONE
// kernel launch (every rANS block of every tensor of the group is a lane of that launch).  A group is as many tasks as
// fit 256 tasks and 256 MB of symbols, whatever opts->num_threads says: the launch is only efficient when it is wide.
// Results are then delivered in task order, opts->num_threads tasks at a time (the number of tasks the reference would
// have in flight; 64 when it is 0): their symbols are copied to the callers' buffers, then the progress callback runs
// on the calling thread for each, so calls are serialised and count up by one.  After a cancel request the tasks being
// delivered complete; the rest get EOQ_ERR_THREAD and their buffers are not written, decoded on the device or not.
extern "C" eoq_error_t eoq_parallel_decode(eoq_decode_task_t *tasks, int num_tasks, const eoq_parallel_opts_t *opts)
{
    if (!tasks && num_tasks > 0) return EOQ_ERR_NULL_PTR;
    if (num_tasks <= 0) return EOQ_OK;
    int deliver = opts ? opts->num_threads : 0;
    deliver = deliver <= 0 ? 64 : std::min(deliver, 256);
    constexpr int kGroupTasks = 256;
    constexpr uint64_t kGroupSymbols = 256ull << 20;
    eoq_parallel_progress_fn cb = opts ? opts->progress_cb : nullptr;
    void *ud = opts ? opts->progress_ud : nullptr;
    cudaStream_t st = nullptr;
    const bool device_ok = have_device() && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;

    int done = 0;
    bool cancelled = false;
    DeviceArena arena;
    for (int g0 = 0; g0 < num_tasks;) {
        int g1 = g0;
        uint64_t symbols = 0;
        while (g1 < num_tasks && g1 - g0 < kGroupTasks) {
            const uint64_t add = tasks[g1].header ? tasks[g1].header->uncompressed_size : 0;
            if (g1 > g0 && symbols + add > kGroupSymbols) break;
            symbols += add;
            g1++;
        }
        if (cancelled) {
            for (int i = g0; i < g1; i++) tasks[i].result = EOQ_ERR_THREAD;          // eoq_parallel_decode.c:72-82
            g0 = g1;
            continue;
        }
        std::vector<std::unique_ptr<V1Job>> jobs;
        std::vector<V1Job *> live;
        std::vector<V1Job *> job_of(g1 - g0, nullptr);
        for (int i = g0; i < g1; i++) {
            eoq_decode_task_t &t = tasks[i];
            t.task_index = i;
            if (!t.header || !t.compressed_data || !t.output) { t.result = EOQ_ERR_NULL_PTR; continue; }
            if (t.header->uncompressed_size == 0) { t.result = EOQ_OK; continue; }
            std::unique_ptr<V1Job> j(new V1Job());
            t.result = job_from_payload(t.header, t.compressed_data, t.compressed_size, t.output_capacity, *j);
            if (t.result == EOQ_OK && !device_ok) t.result = EOQ_ERR_CUDA;
            if (t.result != EOQ_OK) continue;
            j->host_out = t.output;
            live.push_back(j.get());
            job_of[i - g0] = j.get();
            jobs.push_back(std::move(j));
        }
        eoq_error_t rc = live.empty() ? EOQ_OK : decode_jobs(live.data(), live.size(), st, arena, /*copy_out=*/false);
        for (int d0 = g0; d0 < g1; d0 += deliver) {
            const int d1 = std::min(g1, d0 + deliver);
            if (cancelled) {
                for (int i = d0; i < d1; i++) tasks[i].result = EOQ_ERR_THREAD;
                continue;
            }
            eoq_error_t drc = rc;
            bool any = false;
            for (int i = d0; i < d1 && drc == EOQ_OK; i++) {
                const V1Job *j = job_of[i - g0];
                if (!j) continue;
                any = true;
                if (cudaMemcpyAsync(j->host_out, arena.base() + j->at_out, (size_t)j->pl.total * j->out_elem_bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess)
                    drc = EOQ_ERR_CUDA;
            }
            if (drc == EOQ_OK && any && cudaStreamSynchronize(st) != cudaSuccess) drc = EOQ_ERR_CUDA;
            for (int i = d0; i < d1; i++) {
                if (job_of[i - g0] && drc != EOQ_OK) tasks[i].result = drc;
                done++;
                if (cb && !cancelled && cb(done, num_tasks, ud)) cancelled = true;
            }
        }
        if (!live.empty()) cudaStreamSynchronize(st);            // the arena is reused by the next group
        g0 = g1;
    }
    arena.release();
    if (st) cudaStreamDestroy(st);

    for (int i = 0; i < num_tasks; i++)
        if (tasks[i].result != EOQ_OK) return tasks[i].result;        // eoq_parallel_decode.c:290-300
    return EOQ_OK;
}

// -- incremental single-block decoder --------------------------------------
namespace {
struct DecoderDev {
    DeviceBuf table, block, state_pos, out;
    size_t out_cap = 0;
    uint32_t stream_off = 0;
};
}

extern "C" eoq_error_t eoq_decoder_init(eoq_decoder_t *dec, const uint16_t *freq_table, uint32_t alphabet_size,
                                        uint32_t precision_bits, const uint8_t *block_data, size_t block_size)
{
    if (!dec || !freq_table || !block_data) return EOQ_ERR_NULL_PTR;
    if (alphabet_size == 0 || alphabet_size > 4096) return EOQ_ERR_INVALID_HEADER;
    if (precision_bits == 0 || precision_bits > 16) return EOQ_ERR_INVALID_HEADER;
    dec->precision_bits = precision_bits;
    dec->precision_mask = (1u << precision_bits) - 1;
    dec->sym_info = nullptr;
    dec->state = 0; dec->stream = block_data; dec->stream_pos = 0; dec->stream_end = 0;
    std::vector<V1Table> table;
    eoq_error_t rc = table_from_u16(freq_table, alphabet_size, precision_bits, table);
    if (rc != EOQ_OK) return rc;
    uint32_t state = 0, off = 0;
    if (block_size > 0) {
        const uint32_t sl = block_data[0];
        if ((size_t)1 + sl > block_size) return EOQ_ERR_CORRUPT_STREAM;
        for (uint32_t i = 0; i < sl; i++) state = (state << 8) | block_data[1 + i];
        off = 1 + sl;
        dec->stream = block_data + off;
        dec->stream_end = block_size - off;
    }
    dec->state = state;
    if (!have_device()) return EOQ_ERR_CUDA;
    std::unique_ptr<DecoderDev> d(new DecoderDev());
    d->stream_off = off;
    if (d->table.alloc(table.size() * sizeof(V1Table)) != cudaSuccess || d->block.alloc(block_size) != cudaSuccess ||
        d->state_pos.alloc(8) != cudaSuccess)
        return EOQ_ERR_ALLOC;
    const uint32_t sp[2] = {state, 0};
    CU_TRY(cudaMemcpy(d->table.p, table.data(), table.size() * sizeof(V1Table), cudaMemcpyHostToDevice));
    if (block_size) CU_TRY(cudaMemcpy(d->block.p, block_data, block_size, cudaMemcpyHostToDevice));
    CU_TRY(cudaMemcpy(d->state_pos.p, sp, 8, cudaMemcpyHostToDevice));
    dec->sym_info = reinterpret_cast<struct eoq_sym_info *>(d.release());
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_decoder_decode(eoq_decoder_t *dec, uint8_t *out, uint32_t count)
{
    if (!dec || !out) return EOQ_ERR_NULL_PTR;
    if (!dec->sym_info) return EOQ_ERR_NULL_PTR;
    if (count == 0) return EOQ_OK;
    DecoderDev *d = reinterpret_cast<DecoderDev *>(dec->sym_info);
    if (d->out_cap < count) {
        if (d->out.p) { cudaFree(d->out.p); d->out.p = nullptr; }
        if (d->out.alloc(count) != cudaSuccess) return EOQ_ERR_ALLOC;
        d->out_cap = count;
    }
    int e = launch_decode_v1_resume(d->block.as<uint8_t>() + d->stream_off, (uint32_t)dec->stream_end, d->table.as<V1Table>(),
                                    d->state_pos.as<uint32_t>(), d->out.as<uint8_t>(), count, dec->precision_bits, nullptr);
    if (e != 0) return EOQ_ERR_CUDA;
    uint32_t sp[2];
    CU_TRY(cudaMemcpy(out, d->out.p, count, cudaMemcpyDeviceToHost));
    CU_TRY(cudaMemcpy(sp, d->state_pos.p, 8, cudaMemcpyDeviceToHost));
    dec->state = sp[0];
    dec->stream_pos = sp[1];
    return EOQ_OK;
}

extern "C" void eoq_decoder_free(eoq_decoder_t *dec)
{
    if (dec && dec->sym_info) {
        delete reinterpret_cast<DecoderDev *>(dec->sym_info);
        dec->sym_info = nullptr;
    }
}

// -- eoq_cuda_* family -------------------------------------------------------

extern "C" int eoq_cuda_decode_tensor(const eoq_tensor_header_t *header, const uint8_t *compressed, uint8_t *output, void *stream)
{
    if (!header || !compressed || !output) return -1;
    if (header->uncompressed_size == 0) return 0;
    return decode_host_to_host(header, compressed, header->compressed_size, output, header->uncompressed_size,
                               reinterpret_cast<cudaStream_t>(stream)) == EOQ_OK ? 0 : -1;
}

extern "C" int eoq_cuda_decode_tensor_device(const uint8_t *d_compressed_stream, const uint32_t *d_block_offsets,
                                             const uint32_t *d_block_sizes, const eoq_sym_info_packed *d_sym_info,
                                             uint8_t *d_output, uint32_t num_rans_blocks, uint32_t rans_block_size,
                                             uint32_t total_symbols, uint32_t precision_bits, void *cuda_stream)
{
    if (total_symbols == 0) return 0;
    if (!d_compressed_stream || !d_block_offsets || !d_block_sizes || !d_sym_info || !d_output) return -1;
    if (precision_bits == 0 || precision_bits > 16 || rans_block_size == 0) return -1;
    if (!have_device()) return -1;
    int e = launch_decode_v1_syminfo(d_compressed_stream, d_block_offsets, d_block_sizes, d_sym_info, d_output,
                                     num_rans_blocks, rans_block_size, total_symbols, precision_bits, cuda_stream);
    if (e != 0) { std::fprintf(stderr, "eoq_cuda_decode_tensor_device: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return -1; }
    return 0;
}

namespace {
struct BatchImpl {
    std::vector<std::unique_ptr<V1Job>> tensors;
    DeviceArena arena;
    bool launched = false;
};
BatchImpl *batch_impl(eoq_cuda_batch_ctx_t *ctx, bool make)
{
    if (!ctx->impl && make) ctx->impl = new (std::nothrow) BatchImpl();
    return static_cast<BatchImpl *>(ctx->impl);
}
}  // namespace

extern "C" void eoq_cuda_batch_init(eoq_cuda_batch_ctx_t *ctx, void *stream)
{
    if (!ctx) return;
    std::memset(ctx, 0, sizeof(*ctx));
    ctx->stream = stream;
}

extern "C" eoq_cuda_batch_ctx_t *eoq_cuda_batch_create(void *stream)
{
    eoq_cuda_batch_ctx_t *c = new (std::nothrow) eoq_cuda_batch_ctx_t();
    if (c) eoq_cuda_batch_init(c, stream);
    return c;
}

extern "C" int eoq_cuda_batch_prepare_tensor(eoq_cuda_batch_ctx_t *ctx, const eoq_tensor_header_t *header,
                                             const uint8_t *compressed_host, uint8_t *d_output)
{
    if (!ctx || !header || !compressed_host || !d_output) return -1;
    if (ctx->n_tensors >= EOQ_CUDA_MAX_BATCH_TENSORS) {                  // eoq_cuda_decompress.cu:906-910
        std::fprintf(stderr, "eoq_cuda_batch_prepare_tensor: batch full (%d tensors)\n", EOQ_CUDA_MAX_BATCH_TENSORS);
        return -1;
    }
    if (header->uncompressed_size == 0) return 0;
    BatchImpl *impl = batch_impl(ctx, true);
    if (!impl) return -1;
    // the caller may release its host buffer after this call (the reference uploads here): keep a copy until launch
    std::unique_ptr<V1Job> j(new V1Job());
    j->own_payload.assign(compressed_host, compressed_host + header->compressed_size);
    if (job_from_payload(header, j->own_payload.data(), header->compressed_size, header->uncompressed_size, *j) != EOQ_OK) return -1;
    j->dev_out = d_output;
    impl->tensors.push_back(std::move(j));
    ctx->n_tensors = (uint32_t)impl->tensors.size();
    return 0;
}

// One kernel launch decodes every prepared tensor (eoq_cuda_decompress.cu:985-1003 launches one kernel per tensor).
extern "C" int eoq_cuda_batch_launch(eoq_cuda_batch_ctx_t *ctx)
{
    if (!ctx) return -1;
    BatchImpl *impl = batch_impl(ctx, false);
    if (!impl || impl->tensors.empty() || impl->launched) return 0;
    std::vector<V1Job *> live;
    for (auto &t : impl->tensors) live.push_back(t.get());
    if (decode_jobs(live.data(), live.size(), reinterpret_cast<cudaStream_t>(ctx->stream), impl->arena) != EOQ_OK) return -1;
    impl->launched = true;
    return 0;
}

extern "C" int eoq_cuda_batch_sync_and_free(eoq_cuda_batch_ctx_t *ctx)
{
    if (!ctx) return -1;
    int rc = 0;
    BatchImpl *impl = batch_impl(ctx, false);
    if (impl && impl->launched && cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(ctx->stream)) != cudaSuccess) rc = -1;
    delete impl;                   // releases the staging arena; outputs belong to the caller
    ctx->impl = nullptr;
    ctx->n_tensors = 0;
    return rc;
}

extern "C" void eoq_cuda_batch_destroy(eoq_cuda_batch_ctx_t *ctx)
{
    if (!ctx) return;
    delete batch_impl(ctx, false);
    delete ctx;
}

// =========================================================================
// Part 2: Python-facing codec entry points and the fused path
// =========================================================================

extern "C" eoq_error_t eoq_b200_decode_blocked(const uint32_t *freq, uint32_t alphabet, uint32_t precision_bits,
                                               const uint8_t *data, size_t data_len, const uint32_t *offsets,
                                               uint32_t num_blocks, uint32_t block_size, uint32_t num_symbols,
                                               void *out, int out_elem_bytes, int out_on_device, void *stream)
{
    if (num_symbols == 0) return EOQ_OK;
    if (!freq || !data || !offsets || !out) return EOQ_ERR_NULL_PTR;
    if (alphabet == 0 || block_size == 0) return EOQ_ERR_INVALID_HEADER;
    if (precision_bits < 1 || precision_bits > 16) return EOQ_ERR_UNSUPPORTED;   // 32-bit device state
    if (out_elem_bytes != 1 && out_elem_bytes != 2) return EOQ_ERR_UNSUPPORTED;
    if (alphabet > (out_elem_bytes == 1 ? 256u : 65536u)) return EOQ_ERR_UNSUPPORTED;
    if (data_len > 0xFFFFFFFFull) return EOQ_ERR_OVERFLOW;
    if (num_blocks != (uint32_t)(((uint64_t)num_symbols + block_size - 1) / block_size)) return EOQ_ERR_INVALID_HEADER;
    uint64_t sum = 0;
    std::vector<uint32_t> f(freq, freq + alphabet), cdf(alphabet + 1, 0);
    for (uint32_t s = 0; s < alphabet; s++) { sum += f[s]; cdf[s + 1] = cdf[s] + f[s]; }
    if (sum != (1ull << precision_bits)) return EOQ_ERR_INVALID_HEADER;
    std::vector<uint32_t> sizes(num_blocks);
    for (uint32_t b = 0; b < num_blocks; b++) {
        const uint64_t lo = offsets[b], hi = b + 1 < num_blocks ? offsets[b + 1] : data_len;
        if (hi < lo || hi > data_len) return EOQ_ERR_CORRUPT_STREAM;
        sizes[b] = (uint32_t)(hi - lo);
        if (sizes[b] && 1u + data[lo] > sizes[b]) return EOQ_ERR_CORRUPT_STREAM;
        if (sizes[b] && data[lo] > 4) return EOQ_ERR_UNSUPPORTED;                  // state wider than 32 bits
    }
    if (!have_device()) return EOQ_ERR_CUDA;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    V1Job job;
    job.pl.alphabet = alphabet; job.pl.p = precision_bits; job.pl.block = block_size; job.pl.total = num_symbols;
    job.pl.nblocks = num_blocks; job.pl.stream = data; job.pl.stream_bytes = (uint32_t)data_len;
    job.pl.offsets.assign(offsets, offsets + num_blocks);
    job.pl.sizes = std::move(sizes);
    job.freq = std::move(f);
    job.cdf = std::move(cdf);
    job.out_elem_bytes = (uint32_t)out_elem_bytes;
    if (out_on_device) job.dev_out = out; else job.host_out = out;
    V1Job *one = &job;
    DeviceArena arena;
    eoq_error_t rc = decode_jobs(&one, 1, st, arena);
    if (rc != EOQ_OK) return rc;
    CU_TRY(cudaStreamSynchronize(st));   // the staging arena goes back to the cache on return
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_encode_blocked(const uint32_t *freq, uint32_t alphabet, uint32_t precision_bits,
                                               const uint32_t *symbols, uint32_t num_symbols, uint32_t block_size,
                                               uint8_t *out, size_t *out_len, uint32_t *offsets)
{
    if (!out_len) return EOQ_ERR_NULL_PTR;
    if (num_symbols == 0) { *out_len = 0; return EOQ_OK; }
    if (!freq || !symbols || !out || !offsets) return EOQ_ERR_NULL_PTR;
    if (alphabet == 0 || block_size == 0 || precision_bits < 1 || precision_bits > 20) return EOQ_ERR_INVALID_HEADER;
    std::vector<uint32_t> cdf(alphabet + 1, 0);
    uint64_t sum = 0;
    for (uint32_t s = 0; s < alphabet; s++) { if (!freq[s]) return EOQ_ERR_INVALID_HEADER; sum += freq[s]; cdf[s + 1] = cdf[s] + freq[s]; }
    if (sum != (1ull << precision_bits)) return EOQ_ERR_INVALID_HEADER;
    for (uint32_t i = 0; i < num_symbols; i++) if (symbols[i] >= alphabet) return EOQ_ERR_CORRUPT_STREAM;
    const uint32_t nb = (uint32_t)(((uint64_t)num_symbols + block_size - 1) / block_size);
    // blocks are independent streams: ranges of blocks are encoded on the host's cores (one range, on the calling thread,
    // for small inputs), then laid out back to back in block order
    const size_t nranges = num_symbols < (1u << 18) ? 1 : std::min<size_t>(nb, 256);
    std::vector<std::vector<uint8_t>> bytes(nranges);
    std::vector<uint32_t> sizes(nb);
    auto encode_range = [&](size_t r) {
        const uint32_t lo = (uint32_t)((uint64_t)nb * r / nranges), hi = (uint32_t)((uint64_t)nb * (r + 1) / nranges);
        std::vector<uint8_t> blk;
        for (uint32_t b = lo; b < hi; b++) {
            const uint32_t first = b * block_size, n = std::min(block_size, num_symbols - first);
            encode_block_v1(freq, cdf.data(), precision_bits, symbols + first, n, blk);
            sizes[b] = (uint32_t)blk.size();
            bytes[r].insert(bytes[r].end(), blk.begin(), blk.end());
        }
    };
    if (nranges == 1) encode_range(0); else parallel_for(nranges, encode_range);
    size_t at = 0;
    for (size_t r = 0; r < nranges; r++) {
        const uint32_t lo = (uint32_t)((uint64_t)nb * r / nranges), hi = (uint32_t)((uint64_t)nb * (r + 1) / nranges);
        if (at + bytes[r].size() > *out_len) return EOQ_ERR_BUFFER_TOO_SMALL;
        size_t off = at;
        for (uint32_t b = lo; b < hi; b++) {
            if (off > 0xFFFFFFFFull) return EOQ_ERR_OVERFLOW;
            offsets[b] = (uint32_t)off;
            off += sizes[b];
        }
        if (!bytes[r].empty()) std::memcpy(out + at, bytes[r].data(), bytes[r].size());
        at += bytes[r].size();
    }
    *out_len = at;
    return EOQ_OK;
}

// -- resident weights ---------------------------------------------------------

struct eoq_b200_weight {
    int device = 0;
    uint32_t N = 0, K = 0, Npad = 0, G = 0, bits = 0, p = 0, group = 0, kind = 0, alphabet = 0;
    uint32_t ntiles = 0, nseg = 0, nrb = 0;
    uint32_t stage_bytes = 0, max_ncols = 0;          // geometry of the pair kernel's staging buffers (see GemvArgs)
    uint32_t head_bytes = 0;                          // TiledWeights::head_bytes
    DeviceBuf scales_t;                               // transposed copy of the scales for the pair kernel (INT4 x 3 only)
    DeviceBuf pair_partials;                          // partial rows of the pair kernel, every word 0xFFFFFFFF between launches
    size_t pair_partial_bytes = 0;
    DeviceBuf table, tiles, stream, scales, centroids, partials, counters, status, xbuf, ybuf, biasbuf;
    DeviceBuf gemm_x, gemm_partials, gemm_counters;   // scratch of the tensor-core path, allocated by its first call
    uint32_t gemm_rows = 0;                           // activation rows per pass that scratch was sized for
    // The status word the kernels set when a bounded wait expires lives in pinned host memory that the device writes
    // directly (pinned allocations are device-addressable): a healthy launch never touches it, and reading it after a
    // stream synchronise needs no copy.
    uint32_t *status_host = nullptr, *status_dev = nullptr;
    uint32_t *status_word()
    {
        return status_dev;
    }
    ~eoq_b200_weight() { if (status_host) cudaFreeHost(status_host); }
    size_t stream_bytes = 0, scale_bytes = 0, partial_bytes = 0;
    std::mutex mu;   // one call at a time may use the scratch of a weight
    std::mutex scratch_mu;   // guards the late allocation of `partials`
};

namespace {

uint32_t public_kind(uint32_t family, uint32_t bits)
{
    if (family != EOQ_B200_KIND_INT4_ABSMAX) return family;
    return bits == 2 ? EOQ_B200_KIND_INT2_ABSMAX : bits == 3 ? EOQ_B200_KIND_INT3_ABSMAX : bits == 8 ? EOQ_B200_KIND_INT8_ABSMAX : EOQ_B200_KIND_INT4_ABSMAX;
}

eoq_error_t resolve_opts(const eoq_b200_weight_opts_t *o, uint32_t &bits, uint32_t &G, uint32_t &p, uint32_t &target, uint8_t &pad)
{
    if (!o) return EOQ_ERR_NULL_PTR;
    if (o->kind == EOQ_B200_KIND_INT4_ABSMAX) { bits = 4; G = o->symbols_per_step ? o->symbols_per_step : 3; pad = 7; }
    else if (o->kind == EOQ_B200_KIND_Q5_POLAR) { bits = 5; G = o->symbols_per_step ? o->symbols_per_step : 2; pad = 16; if (!o->centroids) return EOQ_ERR_NULL_PTR; }
    else if (o->kind == EOQ_B200_KIND_INT2_ABSMAX || o->kind == EOQ_B200_KIND_INT3_ABSMAX || o->kind == EOQ_B200_KIND_INT8_ABSMAX) {
        // the other widths the reference's packers know (core/weight_packing.py:35-51): one layout each
        bits = o->kind == EOQ_B200_KIND_INT2_ABSMAX ? 2 : o->kind == EOQ_B200_KIND_INT3_ABSMAX ? 3 : 8;
        const uint32_t g = bits == 8 ? 1 : 3;
        if (o->symbols_per_step && o->symbols_per_step != g) return EOQ_ERR_UNSUPPORTED;
        G = g; pad = (uint8_t)((1u << (bits - 1)) - 1u);
    }
    else return EOQ_ERR_UNSUPPORTED;
    if (G < 1 || G > (bits <= 4 ? 3u : bits == 8 ? 1u : 2u)) return EOQ_ERR_UNSUPPORTED;
    // INT4 x 3: 13 bits, a 32 KB table; 8-bit codes: 255 symbols want the finest table shared memory holds (at 12 bits the
    // rare symbols would all be rounded up to a frequency of 1 and the stream would be larger than the codes)
    p = o->precision_bits ? o->precision_bits : bits * G == 8 ? 14u : std::min(16u, std::max(12u, bits * G + 1));
    if (p > 14 || p < bits * G) return EOQ_ERR_UNSUPPORTED;        // table must fit shared memory beside x
    target = o->target_tiles;
    return EOQ_OK;
}

// `built` (optional): the stream already on the device, `built_bytes` long (tw.stream is then empty); it is taken over.
eoq_error_t upload_weight(const TiledWeights &tw, const uint16_t *scales, const float *centroids, eoq_b200_weight_t **out,
                          DeviceBuf *built = nullptr, size_t built_bytes = 0)
{
    std::unique_ptr<eoq_b200_weight> w(new eoq_b200_weight());
    CU_TRY(cudaGetDevice(&w->device));
    w->N = tw.N; w->K = tw.K; w->Npad = tw.Npad; w->G = tw.G; w->bits = tw.bits; w->p = tw.p; w->group = tw.group;
    w->kind = tw.kind; w->alphabet = tw.alphabet; w->ntiles = (uint32_t)tw.tiles.size(); w->nseg = tw.nseg; w->nrb = tw.nrb;
    w->head_bytes = tw.head_bytes;
    for (const TileDesc &d : tw.tiles) {
        w->stage_bytes = std::max(w->stage_bytes, ((d.len64 << 6) + 64u + 127u) & ~127u);
        w->max_ncols = std::max(w->max_ncols, d.ncols);
    }
    w->stream_bytes = built ? built_bytes : tw.stream.size();
    w->scale_bytes = (size_t)tw.N * (tw.K / tw.group) * 2;
    w->partial_bytes = tw.nseg > 1 ? (size_t)tw.nseg * tw.Npad * 8 * sizeof(float) : 0;
    // INT4 x 3 weights run through the pair kernel, which meets in a few partial rows; the ring kernel's scratch (one
    // row per column segment) is allocated by the first call that needs it (see ring_scratch)
    const bool pairs_layout = tw.kind == EOQ_B200_KIND_INT4_ABSMAX && tw.bits == 4 && tw.G == 3;
    // The pair kernel reuses a warp's two tile buffers after its column loop: the warp's sums (2 tiles x 3 rows x 4
    // activation rows x 32 lanes of fp32 = 3 KB) go into the first, its share of a cooperative meeting into the second.
    // Tiles shorter than that (32-column tiles, low-entropy weights) get buffers of that size all the same.
    if (pairs_layout) w->stage_bytes = std::max(w->stage_bytes, 3072u);
    if (w->table.alloc(tw.table.size() * 4) != cudaSuccess || w->tiles.alloc(tw.tiles.size() * sizeof(TileDesc)) != cudaSuccess ||
        (!built && w->stream.alloc(tw.stream.size()) != cudaSuccess) || w->scales.alloc(w->scale_bytes) != cudaSuccess ||
        (!pairs_layout && w->partials.alloc(w->partial_bytes) != cudaSuccess) || w->counters.alloc((size_t)tw.nrb * 4) != cudaSuccess ||
        w->status.alloc(4) != cudaSuccess ||
        w->xbuf.alloc((size_t)8 * tw.K * 4) != cudaSuccess || w->ybuf.alloc((size_t)8 * tw.N * 4) != cudaSuccess ||
        w->biasbuf.alloc((size_t)tw.N * 4) != cudaSuccess)
        return EOQ_ERR_ALLOC;
    if (centroids) {
        if (w->centroids.alloc(32 * 4) != cudaSuccess) return EOQ_ERR_ALLOC;
        CU_TRY(cudaMemcpy(w->centroids.p, centroids, 32 * 4, cudaMemcpyHostToDevice));
    }
    CU_TRY(cudaMemcpy(w->table.p, tw.table.data(), tw.table.size() * 4, cudaMemcpyHostToDevice));
    CU_TRY(cudaMemcpy(w->tiles.p, tw.tiles.data(), tw.tiles.size() * sizeof(TileDesc), cudaMemcpyHostToDevice));
    if (built) { w->stream.p = built->p; built->p = nullptr; }
    else CU_TRY(cudaMemcpy(w->stream.p, tw.stream.data(), tw.stream.size(), cudaMemcpyHostToDevice));
    CU_TRY(cudaMemcpy(w->scales.p, scales, w->scale_bytes, cudaMemcpyHostToDevice));
    if (pairs_layout) {
        w->pair_partial_bytes = (size_t)pair_partial_slots(tw.nrb, tw.nseg) * tw.Npad * 4 * sizeof(float);
        if (w->pair_partials.alloc(w->pair_partial_bytes) != cudaSuccess) return EOQ_ERR_ALLOC;
        CU_TRY(cudaMemset(w->pair_partials.p, 0xFF, w->pair_partial_bytes));
        // [group][row triple] -> {s0 | s1 << 16, s2}, zero for rows past N: what a lane of the pair kernel needs for one
        // run of columns, in one coalesced 8-byte load
        const uint32_t sg = tw.K / tw.group, triples = tw.Npad / 3;
        std::vector<uint32_t> t((size_t)sg * triples * 2, 0u);
        for (uint32_t g = 0; g < sg; g++)
            for (uint32_t i = 0; i < triples; i++) {
                uint32_t v[3];
                for (uint32_t j = 0; j < 3; j++) v[j] = 3 * i + j < tw.N ? scales[(size_t)(3 * i + j) * sg + g] : 0u;
                t[((size_t)g * triples + i) * 2] = v[0] | (v[1] << 16);
                t[((size_t)g * triples + i) * 2 + 1] = v[2];
            }
        if (w->scales_t.alloc(t.size() * 4) != cudaSuccess) return EOQ_ERR_ALLOC;
        CU_TRY(cudaMemcpy(w->scales_t.p, t.data(), t.size() * 4, cudaMemcpyHostToDevice));
    }
    CU_TRY(cudaMemset(w->counters.p, 0, (size_t)tw.nrb * 4));
    CU_TRY(cudaMemset(w->status.p, 0, 4));
    CU_TRY(cudaMallocHost(reinterpret_cast<void **>(&w->status_host), 64));
    std::memset(w->status_host, 0, 64);
    CU_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&w->status_dev), w->status_host, 0));
    *out = w.release();
    return EOQ_OK;
}

}  // namespace

struct eoq_b200_tiles { TiledWeights tw; };
extern "C" eoq_error_t eoq_b200_tiles_build(const uint8_t *symbols, const eoq_b200_weight_opts_t *opts, eoq_b200_tiles_t **out);
extern "C" void eoq_b200_tiles_free(eoq_b200_tiles_t *t);

// How many tiles a weight is cut into when the caller does not say.
static uint32_t default_target_tiles(const eoq_b200_weight_opts_t *opts, uint32_t bits, uint32_t G)
{
    const int sms = have_device() ? device_sm_count() : 0;
    const uint32_t warps = (uint32_t)(sms > 0 ? sms : 148) * 16;      // one wave of 16-warp CTAs
    uint32_t target = warps;
    if (opts->kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4 && G == 3) {
        // The pair kernel gives every warp two vertically adjacent tiles and stages them whole in shared memory,
        // which holds tiles of up to 7 x 16 columns: take the fewest waves of pairs whose column segments are
        // that narrow, and as many segments as fill those waves.
        const uint32_t nrb = (opts->rows + 32 * G - 1) / (32 * G), nrbp = (nrb + 1) / 2;
        const uint32_t units = opts->cols / 16, need = (units + 6) / 7;
        uint32_t nseg = 1;
        for (uint32_t waves = 1; waves <= 64; waves++) {
            nseg = std::max(1u, waves * warps / nrbp);
            if (nseg >= need) break;
        }
        target = nseg * nrb;
    }
    // by default no tile is narrower than 64 columns (an explicit target_tiles may go down to 32) ...
    const uint32_t nrb = (opts->rows + 32 * G - 1) / (32 * G);
    target = std::min<uint32_t>(target, std::max(1u, opts->cols / 64) * nrb);
    // ... except small matrices in the pair layout (row shards of a layer, narrow projections): while tile pairs of 32
    // columns still fit one wave they are taken, twice as many warps share the columns and a launch is 6-16 % shorter
    // (1376 x 4096: 9.8 -> 9.2 us, 512 x 4096: 11.0 -> 9.2 us) for 4-5 % more bytes
    if (opts->kind == EOQ_B200_KIND_INT4_ABSMAX && bits == 4 && G == 3 && opts->cols % 32u == 0 && opts->cols >= 64u &&
        (uint64_t)((nrb + 1) / 2) * (opts->cols / 32u) <= warps)
        target = (opts->cols / 32u) * nrb;
    return target;
}

// The tiled layout built on the device from symbols that are already there (one per byte, row-major [rows, cols], in
// memory this library allocated: 256-byte aligned): joint-symbol counts by a kernel, frequencies and table on the host
// (a few thousand numbers), every tile encoded by one warp, the stream laid out on the host from the tiles' sizes and
// filled by a scatter kernel.  Byte-identical to build_tiled.  EOQ_ERR_UNSUPPORTED (nothing launched) when a tile has
// 65536 columns or more or the scratch would pass 4 GB: the caller then encodes on the host.
static eoq_error_t build_tiled_device(const uint8_t *d_sym, const eoq_b200_weight_opts_t *opts, TiledWeights &tw, DeviceBuf &stream,
                                      size_t &stream_bytes, cudaStream_t st)
{
    uint32_t bits, G, p, target; uint8_t pad;
    eoq_error_t rc = resolve_opts(opts, bits, G, p, target, pad);
    if (rc != EOQ_OK) return rc;
    if (opts->rows == 0 || opts->cols == 0 || opts->group == 0) return EOQ_ERR_INVALID_HEADER;
    if (target == 0) target = default_target_tiles(opts, bits, G);
    const uint32_t family = opts->kind == EOQ_B200_KIND_Q5_POLAR ? EOQ_B200_KIND_Q5_POLAR : EOQ_B200_KIND_INT4_ABSMAX;
    rc = tiled_geometry(opts->rows, opts->cols, bits, G, p, opts->group, family, target, tw);
    if (rc != EOQ_OK) return rc;
    const size_t ntiles = tw.tiles.size();
    uint32_t max_ncols = 0;
    for (const TileDesc &d : tw.tiles) max_ncols = std::max(max_ncols, d.ncols);
    const size_t scratch_bytes = ntiles * (size_t)max_ncols * 128u;
    if (max_ncols >= 65536u || scratch_bytes > (4ull << 30)) return EOQ_ERR_UNSUPPORTED;

    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t at_counts = 0, at_fc = up(at_counts + (size_t)tw.alphabet * 8), at_tiles = up(at_fc + (size_t)tw.alphabet * 8),
                 at_state = up(at_tiles + ntiles * sizeof(TileDesc)), at_count = up(at_state + ntiles * 128), at_info = up(at_count + ntiles * 128),
                 at_scratch = up(at_info + ntiles * 8), total_tmp = at_scratch + scratch_bytes;
    DeviceArena tmp;
    if (tmp.acquire(total_tmp) != cudaSuccess) return EOQ_ERR_ALLOC;
    uint8_t *d = tmp.base();

    CU_TRY(cudaMemsetAsync(d + at_counts, 0, (size_t)tw.alphabet * 8, st));
    if (launch_tile_hist(d_sym, tw.N, tw.K, tw.Npad, G, bits, reinterpret_cast<unsigned long long *>(d + at_counts), st) != 0) return EOQ_ERR_CUDA;
    std::vector<uint64_t> count(tw.alphabet);
    CU_TRY(cudaMemcpyAsync(count.data(), d + at_counts, (size_t)tw.alphabet * 8, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    std::vector<uint32_t> freq, cum;
    rc = tiled_table(count, tw, freq, cum);
    if (rc != EOQ_OK) return rc;
    std::vector<uint32_t> fc((size_t)tw.alphabet * 2);
    for (uint32_t s = 0; s < tw.alphabet; s++) { fc[2 * s] = freq[s] ? freq[s] : 1u; fc[2 * s + 1] = cum[s]; }   // absent symbols never occur
    CU_TRY(cudaMemcpyAsync(d + at_fc, fc.data(), fc.size() * 4, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaMemcpyAsync(d + at_tiles, tw.tiles.data(), ntiles * sizeof(TileDesc), cudaMemcpyHostToDevice, st));
    TileEncodeArgs ea = {};
    ea.sym = d_sym; ea.tiles = reinterpret_cast<const TileDesc *>(d + at_tiles); ea.freq_cum = reinterpret_cast<const uint2 *>(d + at_fc);
    ea.scratch = reinterpret_cast<uint32_t *>(d + at_scratch); ea.state = reinterpret_cast<uint32_t *>(d + at_state);
    ea.count = reinterpret_cast<uint32_t *>(d + at_count); ea.info = reinterpret_cast<uint2 *>(d + at_info);
    ea.N = tw.N; ea.K = tw.K; ea.G = G; ea.bits = bits; ea.p = p; ea.ntiles = (uint32_t)ntiles; ea.max_ncols = max_ncols;
    if (launch_tile_encode(ea, st) != 0) return EOQ_ERR_CUDA;
    std::vector<uint32_t> info(ntiles * 2);
    CU_TRY(cudaMemcpyAsync(info.data(), d + at_info, ntiles * 8, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    for (size_t t = 0; t < ntiles; t++) {
        const uint32_t rows = info[2 * t], drift = info[2 * t + 1];
        tw.tiles[t].len64 = (128u + rows * 64u) >> 6;
        if (drift > kMaxRingDrift) tw.tiles[t].seg |= kTileDirectFlag;
        tw.max_drift = std::max(tw.max_drift, drift);
    }
    rc = tiled_layout(tw, stream_bytes);
    if (rc != EOQ_OK) return rc;
    if (stream.alloc(stream_bytes) != cudaSuccess) return EOQ_ERR_ALLOC;
    CU_TRY(cudaMemsetAsync(stream.p, 0, stream_bytes, st));
    CU_TRY(cudaMemcpyAsync(d + at_tiles, tw.tiles.data(), ntiles * sizeof(TileDesc), cudaMemcpyHostToDevice, st));
    TileScatterArgs sa = {};
    sa.tiles = reinterpret_cast<const TileDesc *>(d + at_tiles); sa.scratch = ea.scratch; sa.state = ea.state; sa.count = ea.count;
    sa.stream = stream.as<uint8_t>(); sa.head_bytes = tw.head_bytes; sa.ntiles = (uint32_t)ntiles; sa.max_ncols = max_ncols;
    if (launch_tile_scatter(sa, st) != 0) return EOQ_ERR_CUDA;
    CU_TRY(cudaStreamSynchronize(st));
    return EOQ_OK;
}

// A weight from symbols in device memory (this library's own allocation).  Falls back to the host encoder, through a
// copy of the symbols, where the device encoder declines.
static eoq_error_t weight_from_device_symbols(const uint8_t *d_sym, const uint16_t *scales_fp16, const eoq_b200_weight_opts_t *opts,
                                              eoq_b200_weight_t **out)
{
    TiledWeights tw;
    DeviceBuf stream;
    size_t stream_bytes = 0;
    eoq_error_t rc = build_tiled_device(d_sym, opts, tw, stream, stream_bytes, nullptr);
    if (rc == EOQ_ERR_UNSUPPORTED && tw.N != 0) {
        std::vector<uint8_t> host((size_t)opts->rows * opts->cols);
        CU_TRY(cudaMemcpy(host.data(), d_sym, host.size(), cudaMemcpyDeviceToHost));
        eoq_b200_tiles_t *t = nullptr;
        rc = eoq_b200_tiles_build(host.data(), opts, &t);
        if (rc != EOQ_OK) return rc;
        rc = upload_weight(t->tw, scales_fp16, opts->kind == EOQ_B200_KIND_Q5_POLAR ? opts->centroids : nullptr, out);
        eoq_b200_tiles_free(t);
        return rc;
    }
    if (rc != EOQ_OK) return rc;
    return upload_weight(tw, scales_fp16, opts->kind == EOQ_B200_KIND_Q5_POLAR ? opts->centroids : nullptr, out, &stream, stream_bytes);
}


extern "C" eoq_error_t eoq_b200_tiles_build(const uint8_t *symbols, const eoq_b200_weight_opts_t *opts, eoq_b200_tiles_t **out)
{
    if (!symbols || !opts || !out) return EOQ_ERR_NULL_PTR;
    *out = nullptr;
    uint32_t bits, G, p, target; uint8_t pad;
    eoq_error_t rc = resolve_opts(opts, bits, G, p, target, pad);
    if (rc != EOQ_OK) return rc;
    if (opts->rows == 0 || opts->cols == 0 || opts->group == 0) return EOQ_ERR_INVALID_HEADER;
    if (target == 0) target = default_target_tiles(opts, bits, G);
    std::unique_ptr<eoq_b200_tiles> t(new eoq_b200_tiles());
    // inside the library the integer widths are one family (the kernels are templated on the field width)
    const uint32_t family = opts->kind == EOQ_B200_KIND_Q5_POLAR ? EOQ_B200_KIND_Q5_POLAR : EOQ_B200_KIND_INT4_ABSMAX;
    rc = build_tiled(symbols, opts->rows, opts->cols, bits, G, p, opts->group, family, target, pad, t->tw);
    if (rc != EOQ_OK) return rc;
    *out = t.release();
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_tiles_view(const eoq_b200_tiles_t *t, eoq_b200_tiles_view_t *v)
{
    if (!t || !v) return EOQ_ERR_NULL_PTR;
    const TiledWeights &tw = t->tw;
    v->rows = tw.N; v->cols = tw.K; v->padded_rows = tw.Npad; v->group = tw.group; v->kind = public_kind(tw.kind, tw.bits); v->bits = tw.bits;
    v->symbols_per_step = tw.G; v->precision_bits = tw.p;
    v->num_tiles = (uint32_t)tw.tiles.size(); v->num_col_segments = tw.nseg;
    v->table = tw.table.data();
    static_assert(sizeof(eoq_b200_tile_desc_t) == sizeof(TileDesc), "tile descriptor layout");
    v->tiles = reinterpret_cast<const eoq_b200_tile_desc_t *>(tw.tiles.data());
    v->stream = tw.stream.data();
    v->stream_bytes = tw.stream.size();
    v->max_lane_drift = tw.max_drift;
    v->head_bytes = tw.head_bytes;
    return EOQ_OK;
}

extern "C" void eoq_b200_tiles_free(eoq_b200_tiles_t *t) { delete t; }

extern "C" eoq_error_t eoq_b200_weight_from_tiles(const eoq_b200_tiles_t *t, const uint16_t *scales_fp16, const float *centroids,
                                                  eoq_b200_weight_t **out)
{
    if (!t || !scales_fp16 || !out) return EOQ_ERR_NULL_PTR;
    *out = nullptr;
    if (t->tw.kind == EOQ_B200_KIND_Q5_POLAR && !centroids) return EOQ_ERR_NULL_PTR;
    if (!have_device()) return EOQ_ERR_CUDA;
    return upload_weight(t->tw, scales_fp16, t->tw.kind == EOQ_B200_KIND_Q5_POLAR ? centroids : nullptr, out);
}

extern "C" eoq_error_t eoq_b200_weight_from_symbols(const uint8_t *symbols, const uint16_t *scales_fp16,
                                                    const eoq_b200_weight_opts_t *opts, eoq_b200_weight_t **out)
{
    if (!symbols || !scales_fp16 || !opts || !out) return EOQ_ERR_NULL_PTR;
    *out = nullptr;
    if (!have_device()) {
        uint32_t bits, G, p, target; uint8_t pad;
        eoq_error_t rc = resolve_opts(opts, bits, G, p, target, pad);
        return rc != EOQ_OK ? rc : EOQ_ERR_CUDA;
    }
    // the symbols go to the device and the tiles are encoded there (the host encoder, which the device encoder matches
    // byte for byte, stays behind eoq_b200_tiles_build for callers without a device at hand)
    if (opts->rows == 0 || opts->cols == 0) return EOQ_ERR_INVALID_HEADER;
    const size_t n = (size_t)opts->rows * opts->cols;
    DeviceArena sym;
    if (sym.acquire(n) != cudaSuccess) return EOQ_ERR_ALLOC;
    CU_TRY(cudaMemcpy(sym.base(), symbols, n, cudaMemcpyHostToDevice));
    return weight_from_device_symbols(sym.base(), scales_fp16, opts, out);
}

extern "C" eoq_error_t eoq_b200_weight_from_device_symbols(const uint8_t *d_symbols, const uint16_t *scales_fp16,
                                                           const eoq_b200_weight_opts_t *opts, eoq_b200_weight_t **out)
{
    if (!d_symbols || !scales_fp16 || !opts || !out) return EOQ_ERR_NULL_PTR;
    *out = nullptr;
    if (!have_device()) return EOQ_ERR_CUDA;
    if (opts->rows == 0 || opts->cols == 0) return EOQ_ERR_INVALID_HEADER;
    if ((reinterpret_cast<uintptr_t>(d_symbols) & 3u) == 0) return weight_from_device_symbols(d_symbols, scales_fp16, opts, out);
    // the counting kernel reads four symbols at a time: an odd base address goes through an aligned copy
    const size_t n = (size_t)opts->rows * opts->cols;
    DeviceArena sym;
    if (sym.acquire(n) != cudaSuccess) return EOQ_ERR_ALLOC;
    CU_TRY(cudaMemcpy(sym.base(), d_symbols, n, cudaMemcpyDeviceToDevice));
    return weight_from_device_symbols(sym.base(), scales_fp16, opts, out);
}

extern "C" eoq_error_t eoq_b200_weight_from_rans(const uint8_t *c, size_t size, const uint16_t *scales_fp16,
                                                 const eoq_b200_weight_opts_t *opts, eoq_b200_weight_t **out)
{
    if (!c || !scales_fp16 || !opts || !out) return EOQ_ERR_NULL_PTR;
    *out = nullptr;
    // `RANS` container: magic, then 7 x u32 (version, num_symbols, block_size, num_blocks, alphabet,
    // precision_bits, data_size), u32 freq[alphabet], u32 offsets[num_blocks], data  (core/rans_blocked.py:176-214)
    if (size < 32 || std::memcmp(c, "RANS", 4) != 0) return EOQ_ERR_INVALID_HEADER;
    uint32_t h[7];
    std::memcpy(h, c + 4, 28);
    if (h[0] != 1) return EOQ_ERR_INVALID_HEADER;
    const uint32_t n = h[1], bs = h[2], nb = h[3], a = h[4], p = h[5], dsz = h[6];
    if ((uint64_t)32 + (uint64_t)a * 4 + (uint64_t)nb * 4 + dsz > size) return EOQ_ERR_CORRUPT_STREAM;
    if ((uint64_t)opts->rows * opts->cols != n) return EOQ_ERR_INVALID_HEADER;
    if (a == 0 || a > 256) return EOQ_ERR_UNSUPPORTED;
    std::vector<uint32_t> raw(a), freq, cdf, offs(nb);
    std::memcpy(raw.data(), c + 32, (size_t)a * 4);
    std::memcpy(offs.data(), c + 32 + (size_t)a * 4, (size_t)nb * 4);
    eoq_error_t rc = normalize_reference(raw.data(), a, p, freq, cdf);
    if (rc != EOQ_OK) return rc;
    if (!have_device()) return EOQ_ERR_CUDA;
    // decoded into device memory and encoded into tiles there: the symbols never visit the host
    DeviceArena sym;
    if (sym.acquire(n) != cudaSuccess) return EOQ_ERR_ALLOC;
    rc = eoq_b200_decode_blocked(freq.data(), a, p, c + 32 + (size_t)a * 4 + (size_t)nb * 4, dsz, offs.data(), nb, bs, n,
                                 sym.base(), 1, 1, nullptr);
    if (rc != EOQ_OK) return rc;
    return weight_from_device_symbols(sym.base(), scales_fp16, opts, out);
}

extern "C" void eoq_b200_weight_destroy(eoq_b200_weight_t *w) { delete w; }

extern "C" eoq_error_t eoq_b200_weight_info(const eoq_b200_weight_t *w, eoq_b200_weight_info_t *info)
{
    if (!w || !info) return EOQ_ERR_NULL_PTR;
    info->rows = w->N; info->cols = w->K; info->padded_rows = w->Npad; info->group = w->group; info->kind = public_kind(w->kind, w->bits);
    info->symbols_per_step = w->G; info->precision_bits = w->p; info->alphabet = w->alphabet;
    info->num_tiles = w->ntiles; info->num_col_segments = w->nseg;
    info->stream_bytes = w->stream_bytes;
    info->table_bytes = (uint64_t)4 << w->p;
    info->scale_bytes = w->scale_bytes;
    info->desc_bytes = (uint64_t)w->ntiles * sizeof(TileDesc);
    info->scratch_bytes = (w->partials.p ? w->partial_bytes : 0) + w->pair_partial_bytes + (uint64_t)w->nrb * 4;
    info->bits_per_weight = (double)w->stream_bytes * 8.0 / ((double)w->N * w->K);
    return EOQ_OK;
}

// The arguments every fused GEMV launch shares (inputs, outputs and scratch are the caller's to add).
static void weight_gemv_args(eoq_b200_weight_t *w, GemvArgs &a)
{
    a.table = w->table.as<uint32_t>(); a.tiles = w->tiles.as<TileDesc>(); a.stream = w->stream.as<uint8_t>();
    a.scales = w->scales.as<uint16_t>(); a.centroids = w->centroids.as<float>();
    a.status = w->status_word();
    a.N = w->N; a.K = w->K; a.Npad = w->Npad; a.group = w->group; a.p = w->p; a.ntiles = w->ntiles; a.nseg = w->nseg;
    a.nrb = w->nrb; a.stage_bytes = w->stage_bytes; a.max_ncols = w->max_ncols; a.head_bytes = w->head_bytes;
    a.scales_t = w->scales_t.as<uint2>();
}

// A weight lives on the device it was uploaded to; launching its kernels with another device current would hand
// that device pointers it cannot reach.  Refused on the host, before anything is launched.
static eoq_error_t check_device(const eoq_b200_weight_t *w, const char *where)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return EOQ_ERR_CUDA;
    if (dev != w->device) {
        std::fprintf(stderr, "%s: the weight lives on device %d but device %d is current\n", where, w->device, dev);
        return EOQ_ERR_UNSUPPORTED;
    }
    return EOQ_OK;
}

// Scratch of the one-tile-per-warp GEMV kernel: one partial row per column segment.  Weights laid out for the pair
// kernel get it on the first call that falls back to the other kernel (an allocation: not inside stream capture).
static eoq_error_t ring_scratch(eoq_b200_weight_t *w)
{
    std::lock_guard<std::mutex> lock(w->scratch_mu);
    if (w->partials.p || w->partial_bytes == 0) return EOQ_OK;
    return w->partials.alloc(w->partial_bytes) == cudaSuccess ? EOQ_OK : EOQ_ERR_ALLOC;
}

extern "C" eoq_error_t eoq_b200_gemv(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch, void *y, int y_dtype,
                                     const float *bias, void *stream)
{
    if (!w || !x || !y) return EOQ_ERR_NULL_PTR;
    if (batch == 0) return EOQ_OK;
    if (batch > 8) return EOQ_ERR_UNSUPPORTED;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    eoq_error_t drc = check_device(w, "eoq_b200_gemv");
    if (drc != EOQ_OK) return drc;
    GemvArgs a = {};
    weight_gemv_args(w, a);
    a.x = x; a.y = y; a.bias = bias; a.counters = w->counters.as<uint32_t>(); a.batch = batch;
    a.pair_partials = w->pair_partials.as<float>();
    a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    if (!gemv_takes_pairs(a, w->G, w->bits, w->kind)) {
        const uint32_t bt = batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 4 ? 4 : 8;
        if (gemv_smem_bytes(w->K, w->p, bt, w->kind) > 227 * 1024) {
            // x for this many rows does not fit shared memory beside the table: run the rows in two halves
            if (bt == 1) return EOQ_ERR_UNSUPPORTED;
            static const size_t esz[3] = {2, 2, 4};
            const uint32_t half = bt / 2, first = std::min(batch, half);
            eoq_error_t rc = eoq_b200_gemv(w, x, x_dtype, first, y, y_dtype, bias, stream);
            if (rc != EOQ_OK || batch <= half) return rc;
            return eoq_b200_gemv(w, static_cast<const uint8_t *>(x) + (size_t)first * w->K * esz[x_dtype], x_dtype, batch - first,
                                 static_cast<uint8_t *>(y) + (size_t)first * w->N * esz[y_dtype], y_dtype, bias, stream);
        }
        eoq_error_t rc = ring_scratch(w);
        if (rc != EOQ_OK) return rc;
        a.partials = w->partials.as<float>();
    }
    int e = launch_gemv(a, w->G, w->bits, w->kind, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_gemv: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gemm(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t m, void *y, int y_dtype,
                                     const float *bias, void *stream)
{
    if (!w || !x || !y) return EOQ_ERR_NULL_PTR;
    if (m == 0) return EOQ_OK;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    // the tensor-core path is built for the default INT4 layout: 3 weights per step, 96-row tiles
    if (w->kind != EOQ_B200_KIND_INT4_ABSMAX || w->G != 3 || w->bits != 4 || w->Npad != w->nrb * 96u || (w->K & 15u)) return EOQ_ERR_UNSUPPORTED;
    if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) != 0) return EOQ_ERR_UNSUPPORTED;
    eoq_error_t drc = check_device(w, "eoq_b200_gemm");
    if (drc != EOQ_OK) return drc;
    static const size_t esz[3] = {2, 2, 4};
    const uint32_t per_pass = std::min(m, kGemmRowsPerPass);
    {
        std::lock_guard<std::mutex> lock(w->mu);
        if (!w->gemm_x.p || w->gemm_rows < per_pass) {
            // fp16 copy of one pass of fp32 or bf16 activation rows, one fp32 partial tile pair per CTA and 128-row token tile, one
            // arrival counter per row block.  Sized by the rows of a pass; a later call with more rows allocates again (outside
            // stream capture), after everything queued on the old scratch has finished.
            if (w->gemm_x.p) {
                CU_TRY(cudaDeviceSynchronize());
                cudaFree(w->gemm_x.p); w->gemm_x.p = nullptr;
                cudaFree(w->gemm_partials.p); w->gemm_partials.p = nullptr;
                cudaFree(w->gemm_counters.p); w->gemm_counters.p = nullptr;
            }
            const uint32_t rows = per_pass <= 128 ? 128 : kGemmRowsPerPass;
            CU_TRY(w->gemm_x.alloc((size_t)rows * w->K * 2));
            CU_TRY(w->gemm_partials.alloc(gemm_partial_bytes(gemm_grid(w->nrb, w->nseg), rows)));
            CU_TRY(w->gemm_counters.alloc((size_t)w->nrb * 4));
            CU_TRY(cudaMemset(w->gemm_counters.p, 0, (size_t)w->nrb * 4));
            w->gemm_rows = rows;
        }
    }
    for (uint32_t m0 = 0; m0 < m; m0 += kGemmRowsPerPass) {     // up to 512 activation rows share one pass over the compressed weight
        const uint32_t mb = std::min(kGemmRowsPerPass, m - m0);
        int e = launch_gemm_tc(w->table.as<uint32_t>(), w->tiles.as<TileDesc>(), w->stream.as<uint8_t>(), w->scales_t.as<uint2>(),
                               static_cast<const uint8_t *>(x) + (size_t)m0 * w->K * esz[x_dtype], w->gemm_x.p,
                               w->gemm_partials.as<float>(), w->gemm_counters.as<uint32_t>(),
                               static_cast<uint8_t *>(y) + (size_t)m0 * w->N * esz[y_dtype], bias, w->status_word(),
                               w->N, w->K, w->group, w->p, w->nseg, w->nrb, w->head_bytes, mb, x_dtype, y_dtype, stream);
        if (e != 0) { std::fprintf(stderr, "eoq_b200_gemm: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    }
    return EOQ_OK;
}

// =========================================================================
// Row-sharded GEMV with the all-gather fused into the kernel (peer stores over NVLink)
// =========================================================================
//
// Each rank owns one device allocation, opened by every other rank through CUDA IPC:
//   [slots x slot_bytes of output][slots x receive buffer of 8-byte words][slots epochs][slots done-counters]
// A gather sends into one slot of every peer's receive buffer; consecutive gathers must use different slots (a
// fast rank may already be sending the next gather while a slow one still unpacks the previous one).
struct eoq_b200_gather {
    uint32_t world = 0, rank = 0, slots = 0;
    size_t slot_bytes = 0, slot_elems = 0, total = 0;
    int device = 0;
    uint8_t *base[kMaxPeers] = {};      // base[rank] is the local allocation
    bool opened[kMaxPeers] = {};
    DeviceBuf status;
    long long limit_ticks = 1ll << 31;  // how long a kernel waits for the peers' words (about a second at 2 GHz)
    size_t ll_off(uint32_t slot) const { return (size_t)slots * slot_bytes + (size_t)slot * slot_elems * 8; }
    size_t epoch_off(uint32_t slot) const { return ll_off(slots) + (size_t)slot * 4; }
    size_t done_off(uint32_t slot) const { return epoch_off(slots) + (size_t)slot * 4; }
};

extern "C" eoq_error_t eoq_b200_gather_create(uint32_t world, uint32_t rank, uint32_t slots, size_t slot_bytes,
                                              eoq_b200_gather_t **out, void *ipc_handle_out)
{
    if (!out || !ipc_handle_out) return EOQ_ERR_NULL_PTR;
    if (world < 2 || world > kMaxPeers || rank >= world || slots < 2 || slots > 16 || slot_bytes == 0) return EOQ_ERR_UNSUPPORTED;
    static_assert(sizeof(cudaIpcMemHandle_t) == EOQ_B200_IPC_HANDLE_BYTES, "handle size");
    std::unique_ptr<eoq_b200_gather> g(new eoq_b200_gather());
    g->world = world; g->rank = rank; g->slots = slots;
    g->slot_bytes = (slot_bytes + 255) & ~(size_t)255;
    g->slot_elems = g->slot_bytes / 2;                      // the narrowest output element is 2 bytes
    g->total = g->done_off(slots);
    CU_TRY(cudaGetDevice(&g->device));
    void *p = nullptr;
    CU_TRY(cudaMalloc(&p, g->total));
    g->base[rank] = static_cast<uint8_t *>(p);
    g->opened[rank] = false;
    CU_TRY(cudaMemset(p, 0, g->total));
    CU_TRY(g->status.alloc(4));
    CU_TRY(cudaMemset(g->status.p, 0, 4));
    CU_TRY(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(ipc_handle_out), p));
    CU_TRY(cudaDeviceSynchronize());
    *out = g.release();
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gather_connect(eoq_b200_gather_t *g, const void *all_handles)
{
    if (!g || !all_handles) return EOQ_ERR_NULL_PTR;
    const cudaIpcMemHandle_t *h = reinterpret_cast<const cudaIpcMemHandle_t *>(all_handles);
    for (uint32_t p = 0; p < g->world; p++) {
        if (p == g->rank || g->base[p]) continue;
        void *ptr = nullptr;
        CU_TRY(cudaIpcOpenMemHandle(&ptr, h[p], cudaIpcMemLazyEnablePeerAccess));
        g->base[p] = static_cast<uint8_t *>(ptr);
        g->opened[p] = true;
    }
    return EOQ_OK;
}

extern "C" void eoq_b200_gather_destroy(eoq_b200_gather_t *g)
{
    if (!g) return;
    for (uint32_t p = 0; p < g->world; p++)
        if (g->opened[p] && g->base[p]) cudaIpcCloseMemHandle(g->base[p]);
    if (g->base[g->rank]) cudaFree(g->base[g->rank]);
    delete g;
}

extern "C" void *eoq_b200_gather_buffer(eoq_b200_gather_t *g, uint32_t slot)
{
    return g && slot < g->slots ? g->base[g->rank] + (size_t)slot * g->slot_bytes : nullptr;
}

extern "C" eoq_error_t eoq_b200_gather_status(eoq_b200_gather_t *g, void *stream)
{
    if (!g) return EOQ_ERR_NULL_PTR;
    uint32_t st = 0;
    CU_TRY(cudaMemcpyAsync(&st, g->status.p, 4, cudaMemcpyDeviceToHost, reinterpret_cast<cudaStream_t>(stream)));
    CU_TRY(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
    if (st) CU_TRY(cudaMemsetAsync(g->status.p, 0, 4, reinterpret_cast<cudaStream_t>(stream)));   // reported once; the object stays usable
    return st ? EOQ_ERR_CUDA : EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gemv_gather(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch, int y_dtype,
                                            const float *bias, eoq_b200_gather_t *g, uint32_t slot, uint32_t row_offset,
                                            uint32_t n_total, void *stream)
{
    if (!w || !x || !g) return EOQ_ERR_NULL_PTR;
    if (batch == 0) return EOQ_OK;
    if (batch > 8 || x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2 || slot >= g->slots) return EOQ_ERR_UNSUPPORTED;
    static const size_t esz[3] = {2, 2, 4};
    if ((size_t)row_offset + w->N > n_total || (size_t)batch * n_total * esz[y_dtype] > g->slot_bytes) return EOQ_ERR_BUFFER_TOO_SMALL;
    if (row_offset != g->rank * w->N || (size_t)w->N * g->world != n_total) return EOQ_ERR_UNSUPPORTED;   // equal, rank-ordered shards
    for (uint32_t p = 0; p < g->world; p++)
        if (!g->base[p]) return EOQ_ERR_UNSUPPORTED;                    // eoq_b200_gather_connect has not run
    eoq_error_t drc = check_device(w, "eoq_b200_gemv_gather");
    if (drc != EOQ_OK) return drc;
    if (g->device != w->device) return EOQ_ERR_UNSUPPORTED;
    GemvArgs a = {};
    weight_gemv_args(w, a);
    a.x = x; a.bias = bias; a.counters = w->counters.as<uint32_t>(); a.batch = batch;
    a.pair_partials = w->pair_partials.as<float>();
    a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    a.world = g->world; a.rank = g->rank; a.row_offset = row_offset; a.n_total = n_total;
    for (uint32_t p = 0; p < g->world; p++) a.peer_ll[p] = reinterpret_cast<uint64_t *>(g->base[p] + g->ll_off(slot));
    a.y = g->base[g->rank] + (size_t)slot * g->slot_bytes;
    a.gather_epoch = reinterpret_cast<uint32_t *>(g->base[g->rank] + g->epoch_off(slot));
    a.gather_done = reinterpret_cast<uint32_t *>(g->base[g->rank] + g->done_off(slot));
    a.gather_status = g->status.as<uint32_t>();
    a.gather_g = w->G;
    a.gather_limit = g->limit_ticks;
    // words one sender occupies per activation row (see GemvArgs): must fit the slot's receive buffer
    const size_t wpr = y_dtype == EOQ_B200_F32 ? w->N : w->Npad / w->G;
    if ((size_t)batch * g->world * wpr > g->slot_elems) return EOQ_ERR_BUFFER_TOO_SMALL;
    if (!gemv_takes_pairs(a, w->G, w->bits, w->kind)) {
        const uint32_t bt = batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 4 ? 4 : 8;
        if (gemv_smem_bytes(w->K, w->p, bt, w->kind) > 227 * 1024) return EOQ_ERR_UNSUPPORTED;
        eoq_error_t rc = ring_scratch(w);
        if (rc != EOQ_OK) return rc;
        a.partials = w->partials.as<float>();
    }
    // one launch: the kernel sends this rank's rows, then waits for the others' and unpacks them
    int e = launch_gemv(a, w->G, w->bits, w->kind, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_gemv_gather: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gather_set_timeout_ms(eoq_b200_gather_t *g, uint32_t milliseconds)
{
    if (!g) return EOQ_ERR_NULL_PTR;
    if (milliseconds == 0 || milliseconds > 60000) return EOQ_ERR_UNSUPPORTED;
    int khz = 0, dev = g->device;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev) != cudaSuccess || khz <= 0) khz = 2000000;
    g->limit_ticks = (long long)milliseconds * khz;
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gather_wait(eoq_b200_gather_t *g, uint32_t slot, uint32_t rows_per_rank, uint32_t batch,
                                            int y_dtype, uint32_t rows_per_word, void *stream)
{
    if (!g) return EOQ_ERR_NULL_PTR;
    if (slot >= g->slots || batch == 0 || batch > 8 || y_dtype < 0 || y_dtype > 2 || rows_per_rank == 0 ||
        rows_per_word < 1 || rows_per_word > 3)
        return EOQ_ERR_UNSUPPORTED;
    static const size_t esz[3] = {2, 2, 4};
    const size_t n_total = (size_t)rows_per_rank * g->world;
    if ((size_t)batch * n_total * esz[y_dtype] > g->slot_bytes) return EOQ_ERR_BUFFER_TOO_SMALL;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return EOQ_ERR_CUDA;
    if (dev != g->device) return EOQ_ERR_UNSUPPORTED;
    GemvArgs a = {};
    a.N = rows_per_rank;
    a.Npad = (rows_per_rank + 32u * rows_per_word - 1u) / (32u * rows_per_word) * (32u * rows_per_word);
    a.batch = batch; a.y_dtype = y_dtype;
    a.world = g->world; a.rank = g->rank; a.row_offset = g->rank * rows_per_rank; a.n_total = (uint32_t)n_total;
    a.peer_ll[g->rank] = reinterpret_cast<uint64_t *>(g->base[g->rank] + g->ll_off(slot));
    a.y = g->base[g->rank] + (size_t)slot * g->slot_bytes;
    a.gather_epoch = reinterpret_cast<uint32_t *>(g->base[g->rank] + g->epoch_off(slot));
    a.gather_done = reinterpret_cast<uint32_t *>(g->base[g->rank] + g->done_off(slot));
    a.gather_status = g->status.as<uint32_t>();
    a.gather_g = rows_per_word;
    a.gather_limit = g->limit_ticks;
    const size_t wpr = y_dtype == EOQ_B200_F32 ? a.N : a.Npad / rows_per_word;
    if ((size_t)batch * g->world * wpr > g->slot_elems) return EOQ_ERR_BUFFER_TOO_SMALL;
    int e = launch_gather_wait(a, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_gather_wait: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gemv_host_async(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch, void *y, int y_dtype,
                                                const float *bias_host, void *stream)
{
    if (!w || !x || !y) return EOQ_ERR_NULL_PTR;
    if (batch == 0) return EOQ_OK;
    if (batch > 8 || x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    static const size_t esz[3] = {2, 2, 4};
    eoq_error_t drc = check_device(w, "eoq_b200_gemv_host");
    if (drc != EOQ_OK) return drc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> lock(w->mu);
    CU_TRY(cudaMemcpyAsync(w->xbuf.p, x, (size_t)batch * w->K * esz[x_dtype], cudaMemcpyHostToDevice, st));
    if (bias_host) CU_TRY(cudaMemcpyAsync(w->biasbuf.p, bias_host, (size_t)w->N * 4, cudaMemcpyHostToDevice, st));
    // A pinned (page-locked) y is device-addressable: the kernel then stores its results straight into it and the
    // copy back is not needed.  Pageable memory goes through the weight's device buffer and a copy.
    void *y_direct = nullptr;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, y) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer) y_direct = attr.devicePointer;
    else (void)cudaGetLastError();
    eoq_error_t rc = eoq_b200_gemv(w, w->xbuf.p, x_dtype, batch, y_direct ? y_direct : w->ybuf.p, y_dtype,
                                   bias_host ? w->biasbuf.as<float>() : nullptr, stream);
    if (rc != EOQ_OK) return rc;
    if (!y_direct) CU_TRY(cudaMemcpyAsync(y, w->ybuf.p, (size_t)batch * w->N * esz[y_dtype], cudaMemcpyDeviceToHost, st));
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gemv_host(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch, void *y, int y_dtype,
                                          const float *bias_host, void *stream)
{
    eoq_error_t rc = eoq_b200_gemv_host_async(w, x, x_dtype, batch, y, y_dtype, bias_host, stream);
    if (rc != EOQ_OK || batch == 0) return rc;
    return eoq_b200_weight_status(w, stream);       // reads the status word and synchronises the stream
}

extern "C" eoq_error_t eoq_b200_weight_decode(eoq_b200_weight_t *w, uint8_t *d_sym, int packed, void *d_dequant, int out_dtype, void *stream)
{
    if (!w) return EOQ_ERR_NULL_PTR;
    if (!d_sym && !d_dequant) return EOQ_OK;
    if (packed && w->bits != 4) return EOQ_ERR_UNSUPPORTED;
    if (d_dequant && w->kind != EOQ_B200_KIND_INT4_ABSMAX) return EOQ_ERR_UNSUPPORTED;      // any integer width dequantises; polar does not
    if (out_dtype < 0 || out_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    eoq_error_t drc = check_device(w, "eoq_b200_weight_decode");
    if (drc != EOQ_OK) return drc;
    DecodeArgs a;
    a.head_bytes = w->head_bytes;
    a.table = w->table.as<uint32_t>(); a.tiles = w->tiles.as<TileDesc>(); a.stream = w->stream.as<uint8_t>();
    a.scales = w->scales.as<uint16_t>(); a.centroids = w->centroids.as<float>();
    a.status = w->status_word();
    a.out_sym = d_sym; a.out_deq = d_dequant; a.N = w->N; a.K = w->K; a.group = w->group; a.p = w->p; a.ntiles = w->ntiles;
    a.packed = packed; a.out_dtype = out_dtype;
    a.scales_t = w->scales_t.as<uint2>(); a.nseg = w->nseg; a.nrb = w->nrb; a.Npad = w->Npad; a.stage_bytes = w->stage_bytes;
    int e = launch_decode_tiles(a, w->G, w->bits, w->kind, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_weight_decode: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_dequant_packed(const uint8_t *d_packed, const uint16_t *d_scales_fp16, uint32_t rows, uint32_t cols,
                                               uint32_t bits, uint32_t group, uint32_t row_lo, uint32_t row_hi, void *d_out,
                                               int out_dtype, void *stream)
{
    if (!d_packed || !d_out || (!d_scales_fp16 && out_dtype != EOQ_B200_I8)) return EOQ_ERR_NULL_PTR;   // codes alone need no scales
    if (bits < 2 || bits > 8 || group == 0 || cols == 0) return EOQ_ERR_INVALID_HEADER;
    if (row_lo > row_hi || row_hi > rows) return EOQ_ERR_INVALID_HEADER;
    if (out_dtype < 0 || out_dtype > EOQ_B200_I8) return EOQ_ERR_UNSUPPORTED;
    if (!have_device()) return EOQ_ERR_CUDA;
    // row stride of QuantizedLinear.packed_weight (core/quantized_linear.py:49-66)
    const uint32_t row_bytes = bits == 4 ? (cols + 1) / 2 : bits == 2 ? (cols + 3) / 4 : cols;
    int e = launch_dequant_packed(d_packed, d_scales_fp16, cols, row_bytes, bits, group, row_lo, row_hi, d_out, out_dtype, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_dequant_packed: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gemv_packed(const uint8_t *d_packed, const uint16_t *d_scales_fp16, uint32_t rows, uint32_t cols,
                                            uint32_t bits, uint32_t group, const void *x, int x_dtype, uint32_t batch, void *d_scratch,
                                            void *y, int y_dtype, const float *bias, void *stream)
{
    if (!d_packed || !d_scales_fp16 || !x || !y) return EOQ_ERR_NULL_PTR;
    if (batch == 0 || rows == 0) return EOQ_OK;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    if (bits < 2 || bits > 8 || group == 0 || cols == 0) return EOQ_ERR_INVALID_HEADER;
    // a lane takes sixteen aligned bytes of a row, in pieces of eight columns of one scale group: other shapes go through
    // the dequantise kernel
    const uint32_t per16 = bits == 4 ? 32u : bits == 2 ? 64u : 16u;
    if (cols % per16 || group % 8u || cols % group || (reinterpret_cast<uintptr_t>(d_packed) & 15u)) return EOQ_ERR_UNSUPPORTED;
    PackedGemvArgs a = {};
    a.packed = d_packed; a.scales = d_scales_fp16; a.x = x; a.y = y; a.bias = bias;
    a.N = rows; a.K = cols; a.group = group; a.batch = batch; a.bits = bits; a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    // row stride of QuantizedLinear.packed_weight (core/quantized_linear.py:49-66)
    a.row_bytes = bits == 4 ? cols / 2 : bits == 2 ? cols / 4 : cols;
    // fp32 activations reach the tensor cores as two fp16 halves, written into the caller's scratch by one small launch
    const bool split = x_dtype == EOQ_B200_F32 && d_scratch && (reinterpret_cast<uintptr_t>(d_scratch) & 15u) == 0 &&
                       cols % 128u == 0 && group % 128u == 0;
    if (split) a.xsplit = static_cast<const uint16_t *>(d_scratch);
    if (batch > gemv_packed_rows(a)) return EOQ_ERR_UNSUPPORTED;
    if (!have_device()) return EOQ_ERR_CUDA;
    if (split) {
        int e = launch_polar_rotate(x, x_dtype, cols, 0, batch, nullptr, static_cast<uint16_t *>(d_scratch), stream);      // block of 1: no rotation, only the split
        if (e != 0) { std::fprintf(stderr, "eoq_b200_gemv_packed: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    }
    int e = launch_gemv_packed(a, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_gemv_packed: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_gemv_polar_codes(const uint8_t *d_codes, const uint16_t *d_norms_fp16, const float *d_centroids,
                                                 uint32_t rows, uint32_t cols, uint32_t bits, uint32_t block, const void *x, int x_dtype,
                                                 uint32_t batch, void *d_scratch, void *y, int y_dtype, const float *bias,
                                                 int tensor_cores, void *stream)
{
    if (!d_codes || !d_norms_fp16 || !d_centroids || !x || !y || !d_scratch) return EOQ_ERR_NULL_PTR;
    if (batch == 0 || rows == 0) return EOQ_OK;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    if (bits < 1 || bits > 8 || block == 0 || cols == 0) return EOQ_ERR_INVALID_HEADER;
    // one row alone is quickest on the CUDA cores, several on the tensor cores (a quad of lanes takes 64 columns of one block)
    const bool split = tensor_cores < 0 ? batch >= 2 && block >= 64u : tensor_cores != 0;
    if (batch > (split ? 32u : 8u)) return EOQ_ERR_UNSUPPORTED;
    // a lane takes sixteen codes of one block with one aligned load
    if ((block & (block - 1u)) || block < (split ? 64u : 16u) || block > 4096u || cols % block ||
        ((reinterpret_cast<uintptr_t>(d_codes) | reinterpret_cast<uintptr_t>(d_scratch)) & 15u))
        return EOQ_ERR_UNSUPPORTED;
    if (!have_device()) return EOQ_ERR_CUDA;
    PolarCodesArgs a = {};
    a.codes = d_codes; a.norms = d_norms_fp16; a.centroids = d_centroids; a.y = y; a.bias = bias;
    if (split) a.xsplit = static_cast<const uint16_t *>(d_scratch);
    else a.xrot = static_cast<const float *>(d_scratch);
    a.N = rows; a.K = cols; a.batch = batch; a.entries = 1u << bits; a.y_dtype = y_dtype;
    for (a.block_shift = 4; (1u << a.block_shift) < block; a.block_shift++) {}
    int e = launch_polar_rotate(x, x_dtype, cols, a.block_shift, batch, split ? nullptr : static_cast<float *>(d_scratch),
                                split ? static_cast<uint16_t *>(d_scratch) : nullptr, stream);
    if (e == 0) e = launch_gemv_polar_codes(a, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_gemv_polar_codes: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}

extern "C" eoq_error_t eoq_b200_weight_status(eoq_b200_weight_t *w, void *stream)
{
    if (!w) return EOQ_ERR_NULL_PTR;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> lock(w->mu);
    if (!w->status_host) return EOQ_ERR_ALLOC;
    CU_TRY(cudaStreamSynchronize(st));
    return *static_cast<volatile uint32_t *>(w->status_host) ? EOQ_ERR_CUDA : EOQ_OK;
}


// Test hook (not in the public header): copy a resident weight's tile stream (what = 0), tile descriptors (1) or decode
// table (2) to the host; returns the bytes that part has, copies min(bytes, capacity).
extern "C" uint64_t eoq_b200_weight_read(eoq_b200_weight_t *w, int what, void *host, uint64_t capacity)
{
    if (!w) return 0;
    const void *src = what == 0 ? w->stream.p : what == 1 ? w->tiles.p : what == 2 ? w->table.p : nullptr;
    const uint64_t bytes = what == 0 ? w->stream_bytes : what == 1 ? (uint64_t)w->ntiles * sizeof(TileDesc) : what == 2 ? ((uint64_t)4 << w->p) : 0;
    if (src && host && cudaMemcpy(host, src, (size_t)std::min(bytes, capacity), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    return bytes;
}

extern "C" int eoq_b200_tune(const char *key, int value)
{
    if (!key) return -1;
    if (std::strcmp(key, "gemv_ctas_per_sm") == 0) { set_gemv_ctas_per_sm(value); return 0; }
    if (std::strcmp(key, "gemm_warps") == 0) { set_gemm_warps(value); return 0; }
    if (std::strcmp(key, "pdl") == 0) { set_pdl(value); return 0; }
    if (std::strcmp(key, "gemv_pairs") == 0) { set_gemv_pairs(value); return 0; }
    if (std::strcmp(key, "v1_lanes") == 0) { set_v1_lanes(value); return 0; }
    if (std::strcmp(key, "packed_warps") == 0) { set_packed_warps(value); return 0; }
    if (std::strcmp(key, "dequant_vec") == 0) { set_dequant_vec(value); return 0; }
    return -1;
}

extern "C" uint64_t eoq_b200_launch_count(void) { return launch_counter(); }

// =========================================================================
// Fused GEMV for callers that must not allocate
// =========================================================================
//
// Some callers cannot let a library reach the device allocator: a serving loop that has
// handed all of HBM to its own arena, a real-time thread where an allocator lock is a
// latency hazard, or code running under a framework that forbids allocation while it
// replays recorded work.  For them the cross-tile scratch of the fused kernel (the partial
// row sums of the column segments and the per-row-block arrival counters) lives in one
// fixed array in device global memory that is part of the loaded library.  Every GPU that
// loads the library holds the array until the process exits.
//
// In host code `g_gemv_scratch` is only a handle for the symbol, never a device address: its
// address is looked up once per device with cudaGetSymbolAddress (with that device
// current) and the resulting pointer is what the kernel receives.
constexpr size_t kGemvStaticScratchBytes = EOQ_B200_GEMV_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_gemv_scratch[kGemvStaticScratchBytes];

namespace {
struct StaticScratchMap {
    std::mutex mu;
    void *dev_ptr[64] = {nullptr};
} g_static_scratch;

// First use on a device resolves the symbol; later calls are a table lookup.
eoq_error_t static_scratch_for_current_device(unsigned char **out)
{
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return EOQ_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_scratch.mu);
    if (!g_static_scratch.dev_ptr[dev]) {
        void *p = nullptr;
        CU_TRY(cudaGetSymbolAddress(&p, g_gemv_scratch));
        g_static_scratch.dev_ptr[dev] = p;
    }
    *out = static_cast<unsigned char *>(g_static_scratch.dev_ptr[dev]);
    return EOQ_OK;
}
}  // namespace

extern "C" eoq_error_t eoq_b200_gemv_static_scratch(eoq_b200_weight_t *w, const void *x, int x_dtype, uint32_t batch,
                                                    void *y, int y_dtype, const float *bias, void *stream)
{
    if (!w || !x || !y) return EOQ_ERR_NULL_PTR;
    if (batch == 0) return EOQ_OK;
    if (batch > 8) return EOQ_ERR_UNSUPPORTED;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return EOQ_ERR_UNSUPPORTED;
    eoq_error_t drc = check_device(w, "eoq_b200_gemv_static_scratch");
    if (drc != EOQ_OK) return drc;
    GemvArgs a = {};
    weight_gemv_args(w, a);
    a.x = x; a.y = y; a.bias = bias; a.batch = batch;
    a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    // The scratch request is sized for the kernel that will run.  Two tiles per warp (the default INT4 layout): a few
    // partial rows per pair of row blocks, at most four activation rows per launch.  One tile per warp: one partial row
    // per column segment.  Layout of the array: [arrival counters, one u32 per row block, padded to 256 B][partial sums].
    const bool pairs = gemv_takes_pairs(a, w->G, w->bits, w->kind);
    const uint32_t bt = batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 4 ? 4 : 8;
    if (!pairs && gemv_smem_bytes(w->K, w->p, bt, w->kind) > 227 * 1024) {
        // same rule as eoq_b200_gemv: rows that do not fit shared memory together run in two halves
        if (bt == 1) return EOQ_ERR_UNSUPPORTED;
        static const size_t esz[3] = {2, 2, 4};
        const uint32_t half = bt / 2, first = std::min(batch, half);
        eoq_error_t rc = eoq_b200_gemv_static_scratch(w, x, x_dtype, first, y, y_dtype, bias, stream);
        if (rc != EOQ_OK || batch <= half) return rc;
        return eoq_b200_gemv_static_scratch(w, static_cast<const uint8_t *>(x) + (size_t)first * w->K * esz[x_dtype], x_dtype,
                                            batch - first, static_cast<uint8_t *>(y) + (size_t)first * w->N * esz[y_dtype],
                                            y_dtype, bias, stream);
    }
    const size_t counter_bytes = (((size_t)w->nrb * 4) + 255) & ~(size_t)255;
    const size_t partial_bytes = pairs ? (size_t)pair_partial_slots(w->nrb, w->nseg) * w->Npad * std::min(bt, 4u) * sizeof(float)
                               : w->nseg > 1 ? (size_t)w->nseg * w->Npad * bt * sizeof(float) : 0;
    if (counter_bytes + partial_bytes > kGemvStaticScratchBytes) {
        std::fprintf(stderr,
                     "eoq_b200_gemv_static_scratch: this weight needs %zu bytes of scratch for %u rows of x, the built-in array holds %zu; "
                     "use eoq_b200_gemv\n",
                     counter_bytes + partial_bytes, batch, kGemvStaticScratchBytes);
        return EOQ_ERR_BUFFER_TOO_SMALL;
    }
    unsigned char *scratch = nullptr;
    eoq_error_t rc = static_scratch_for_current_device(&scratch);
    if (rc != EOQ_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // the array keeps whatever the last call left; the counters are the only part that must start at zero
    CU_TRY(cudaMemsetAsync(scratch, 0, counter_bytes, st));
    // pair_partials stays null: the array cannot keep the "empty slot" pattern between calls, so the runs of a pair of row
    // blocks meet through store, fence and ticket in `partials`
    a.partials = reinterpret_cast<float *>(scratch + counter_bytes);
    a.counters = reinterpret_cast<uint32_t *>(scratch);
    int e = launch_gemv(a, w->G, w->bits, w->kind, stream);
    if (e != 0) { std::fprintf(stderr, "eoq_b200_gemv_static_scratch: launch failed: %s\n", cudaGetErrorString((cudaError_t)e)); return EOQ_ERR_CUDA; }
    return EOQ_OK;
}
