/*
 * A C99 caller of libeoq_b200.so, written the way a caller of the reference's C interface is
 * (llamacpp_integration/test_parallel_decode.c: zero / one / many tasks, error propagation,
 * progress and cancellation), to show that such a caller compiles against include/eoq_b200.h
 * unchanged and gets the reference's results and error codes.
 *
 *   abi_check                 argument validation only (needs no GPU)
 *   abi_check <tensors.bin>   the same, then decodes the tensors of the file on the GPU
 *
 * tensors.bin (written by the test that runs this program): u32 count, then per tensor
 * 7 x u32 header, u32 payload bytes, payload, expected symbols (uncompressed_size bytes).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "eoq_b200.h"

static int failures = 0;
#define CHECK(cond)                                                             \
    do {                                                                        \
        if (!(cond)) { printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); failures++; } \
    } while (0)

typedef struct {
    eoq_tensor_header_t header;
    uint8_t *payload;
    uint32_t payload_bytes;
    uint8_t *expected;
    uint8_t *output;
} tensor_t;

static int calls_seen, last_done, cancel_after;
static int on_progress(int done, int total, void *ud)
{
    (void)ud;
    calls_seen++;
    if (done != last_done + 1 || done > total) failures++;      /* serialised, counting up by one */
    last_done = done;
    return cancel_after > 0 && done >= cancel_after;
}

static size_t bytes_seen;
static int on_bytes(size_t done, size_t total, void *ud)
{
    (void)ud;
    bytes_seen = done;
    return done > total;
}

static void validation_only(void)
{
    eoq_parallel_opts_t popts = EOQ_PARALLEL_OPTS_DEFAULT;
    eoq_decode_opts_t dopts = EOQ_DECODE_OPTS_DEFAULT;
    eoq_decode_task_t task;
    eoq_tensor_header_t h;
    eoq_cuda_batch_ctx_t batch;
    uint8_t byte = 0;

    CHECK(popts.num_threads == 0 && popts.progress_cb == NULL && dopts.n_threads == 0 && dopts.progress_cb == NULL);
    CHECK(eoq_parallel_decode(NULL, 0, NULL) == EOQ_OK);                      /* eoq_parallel_decode.c:155-156 */
    CHECK(eoq_parallel_decode(NULL, -3, &popts) == EOQ_OK);
    CHECK(eoq_parallel_decode(NULL, 2, &popts) == EOQ_ERR_NULL_PTR);
    CHECK(eoq_parallel_decode_auto(NULL, 1) == EOQ_ERR_NULL_PTR);
    CHECK(eoq_detect_num_threads() >= 1);

    memset(&h, 0, sizeof h);
    CHECK(eoq_validate_header(NULL) == EOQ_ERR_NULL_PTR);
    CHECK(eoq_validate_header(&h) == EOQ_ERR_INVALID_HEADER);
    h.freq_table_size = 15; h.precision_bits = 12; h.rans_block_size = 256; h.compressed_size = 34;
    CHECK(eoq_validate_header(&h) == EOQ_OK);
    h.precision_bits = 17;
    CHECK(eoq_validate_header(&h) == EOQ_ERR_INVALID_HEADER);

    /* a task without buffers fails on its own and the call reports it */
    memset(&task, 0, sizeof task);
    CHECK(eoq_parallel_decode(&task, 1, NULL) == EOQ_ERR_NULL_PTR && task.result == EOQ_ERR_NULL_PTR);
    CHECK(eoq_decode_tensor_v2(NULL, &byte, 1, &byte, 1, &dopts) == EOQ_ERR_NULL_PTR);
    h.precision_bits = 12; h.uncompressed_size = 0;
    CHECK(eoq_decode_tensor_v2(&h, &byte, 1, &byte, 1, NULL) == EOQ_OK);     /* empty tensor: OK before validation */
    CHECK(strcmp(eoq_error_string(EOQ_ERR_CORRUPT_STREAM), "corrupt compressed stream") == 0);

    /* the batch context is the caller's, as in eoq_cuda_decompress.cu:864-887 */
    eoq_cuda_batch_init(&batch, NULL);
    CHECK(batch.n_tensors == 0);
    CHECK(eoq_cuda_batch_prepare_tensor(&batch, &h, &byte, NULL) == -1);
    CHECK(eoq_cuda_batch_launch(&batch) == 0);
    CHECK(eoq_cuda_batch_sync_and_free(&batch) == 0);
}

static tensor_t *load(const char *path, int *count)
{
    FILE *f = fopen(path, "rb");
    uint32_t n = 0, i;
    tensor_t *t;
    if (!f || fread(&n, 4, 1, f) != 1) { printf("cannot read %s\n", path); exit(2); }
    t = (tensor_t *)calloc(n, sizeof *t);
    for (i = 0; i < n; i++) {
        if (fread(&t[i].header, sizeof t[i].header, 1, f) != 1 || fread(&t[i].payload_bytes, 4, 1, f) != 1) exit(2);
        t[i].payload = (uint8_t *)malloc(t[i].payload_bytes + 1);
        t[i].expected = (uint8_t *)malloc(t[i].header.uncompressed_size + 1);
        t[i].output = (uint8_t *)malloc(t[i].header.uncompressed_size + 1);
        if (fread(t[i].payload, 1, t[i].payload_bytes, f) != t[i].payload_bytes) exit(2);
        if (fread(t[i].expected, 1, t[i].header.uncompressed_size, f) != t[i].header.uncompressed_size) exit(2);
    }
    fclose(f);
    *count = (int)n;
    return t;
}

static void fill(eoq_decode_task_t *tasks, tensor_t *t, int n)
{
    int i;
    memset(tasks, 0, sizeof *tasks * (size_t)n);
    for (i = 0; i < n; i++) {
        memset(t[i].output, 0xEE, t[i].header.uncompressed_size);
        tasks[i].header = &t[i].header;
        tasks[i].compressed_data = t[i].payload;
        tasks[i].compressed_size = t[i].payload_bytes;
        tasks[i].output = t[i].output;
        tasks[i].output_capacity = t[i].header.uncompressed_size;
        tasks[i].result = EOQ_ERR_THREAD;
    }
}

static int same(const tensor_t *t) { return memcmp(t->output, t->expected, t->header.uncompressed_size) == 0; }

static void decode_cases(const char *path)
{
    int n = 0, i;
    tensor_t *t = load(path, &n);
    eoq_decode_task_t *tasks = (eoq_decode_task_t *)calloc((size_t)n, sizeof *tasks);
    eoq_parallel_opts_t opts = EOQ_PARALLEL_OPTS_DEFAULT;
    eoq_decode_opts_t dopts = EOQ_DECODE_OPTS_DEFAULT;
    uint32_t keep;
    CHECK(n >= 4);

    /* many tasks, defaults */
    fill(tasks, t, n);
    CHECK(eoq_parallel_decode_auto(tasks, n) == EOQ_OK);
    for (i = 0; i < n; i++) CHECK(tasks[i].result == EOQ_OK && tasks[i].task_index == i && same(&t[i]));

    /* one task, two threads asked for, progress reported once */
    fill(tasks, t, 1);
    opts.num_threads = 2; opts.progress_cb = on_progress; calls_seen = last_done = cancel_after = 0;
    CHECK(eoq_parallel_decode(tasks, 1, &opts) == EOQ_OK && calls_seen == 1 && same(&t[0]));

    /* progress counts every tensor */
    fill(tasks, t, n);
    opts.num_threads = 3; calls_seen = last_done = cancel_after = 0;
    CHECK(eoq_parallel_decode(tasks, n, &opts) == EOQ_OK && calls_seen == n && last_done == n);

    /* error propagation: the first failing task's code comes back, the others still decode */
    fill(tasks, t, n);
    keep = t[1].header.precision_bits;
    t[1].header.precision_bits = 0;
    tasks[2].output_capacity = 1;
    opts.progress_cb = NULL;
    CHECK(eoq_parallel_decode(tasks, n, &opts) == EOQ_ERR_INVALID_HEADER);
    CHECK(tasks[0].result == EOQ_OK && same(&t[0]));
    CHECK(tasks[1].result == EOQ_ERR_INVALID_HEADER && tasks[2].result == EOQ_ERR_BUFFER_TOO_SMALL);
    CHECK(tasks[3].result == EOQ_OK && same(&t[3]));
    CHECK(t[2].output[1] == 0xEE);                                  /* nothing written past the stated capacity */
    t[1].header.precision_bits = keep;

    /* cancellation: tasks not started afterwards are marked EOQ_ERR_THREAD */
    fill(tasks, t, n);
    opts.num_threads = 1; opts.progress_cb = on_progress; calls_seen = last_done = 0; cancel_after = 2;
    CHECK(eoq_parallel_decode(tasks, n, &opts) == EOQ_ERR_THREAD);
    CHECK(tasks[0].result == EOQ_OK && tasks[1].result == EOQ_OK && tasks[n - 1].result == EOQ_ERR_THREAD);
    CHECK(calls_seen == 2);

    /* single-tensor entry points */
    memset(t[0].output, 0, t[0].header.uncompressed_size);
    dopts.progress_cb = on_bytes; bytes_seen = 0;
    CHECK(eoq_decode_tensor_v2(&t[0].header, t[0].payload, t[0].payload_bytes, t[0].output, t[0].header.uncompressed_size, &dopts) == EOQ_OK);
    CHECK(same(&t[0]) && bytes_seen == t[0].header.uncompressed_size);
    CHECK(eoq_decode_tensor_v2(&t[0].header, t[0].payload, t[0].payload_bytes - 1, t[0].output, t[0].header.uncompressed_size, NULL) == EOQ_ERR_CORRUPT_STREAM);
    memset(t[3].output, 0, t[3].header.uncompressed_size);
    CHECK(eoq_decode_tensor(&t[3].header, t[3].payload, t[3].output) == 0 && same(&t[3]));
    memset(t[2].output, 0, t[2].header.uncompressed_size);
    CHECK(eoq_cuda_decode_tensor(&t[2].header, t[2].payload, t[2].output, NULL) == 0 && same(&t[2]));
    free(tasks);
}

int main(int argc, char **argv)
{
    validation_only();
    if (argc > 1) decode_cases(argv[1]);
    printf("%s (%d failure%s)\n", failures ? "FAILED" : "ok", failures, failures == 1 ? "" : "s");
    return failures ? 1 : 0;
}
