// lev_matvec_static_scratch: the stream-schedule matvec for callers that must
// not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits at call time:
// inside a real-time decode loop whose memory was sized and pinned up front, in
// a process whose allocator owns the whole device and hands out nothing after
// start-up, or on a thread that may not take the driver's allocation lock.  The
// ordinary lev_matvec grows context-owned work buffers on demand; this entry
// point never does.  Shapes the one-launch kernel serves need no work buffer at
// all (it builds its activation tables in shared memory); for the others the
// split activation tables live in one file-scope device array of fixed size
// that every GPU loading the library carries until the process exits.
//
// Rules that follow from that design:
//   - requests whose work buffers would not fit LEV_STATIC_SCRATCH_BYTES are
//     refused with LEV_EXCEEDS_WORKLOAD and a message naming both sizes;
//   - the array is shared by every call and every context on the device and
//     keeps whatever the previous call left in it; every byte a call reads is
//     written by that call first;
//   - two calls that overlap on the GPU (different streams or contexts) race on
//     the array: callers serialise them;
//   - the first call on a device looks the array's device address up (the
//     array's name is only a host-side handle, not a pointer a kernel could
//     use) and opts the kernel in to its shared-memory size; make that first
//     call before starting any stream capture, and from one thread at a time
//     (two first calls at once would both do the look-up; they store the same
//     address, but the table is not synchronised).
#include "lev_internal.h"
#include "lev_stream.h"

#define LEV_STATIC_SCRATCH_BYTES (4u << 20)

static __device__ __align__(256) unsigned char lev_static_scratch[LEV_STATIC_SCRATCH_BYTES];

// device address of lev_static_scratch per device ordinal, resolved on first use
static unsigned char* g_scratch_addr[64];

static int scratch_address(lev_ctx* ctx, unsigned char** out) {
    if (ctx->device < 0 || ctx->device >= 64) return lev_fail(ctx, LEV_BAD_ARGUMENT, "device ordinal %d", ctx->device);
    if (!g_scratch_addr[ctx->device]) {
        LEV_CUDA(ctx, cudaSetDevice(ctx->device));
        void* p = nullptr;
        LEV_CUDA(ctx, cudaGetSymbolAddress(&p, lev_static_scratch));
        if (!p) return lev_fail(ctx, LEV_KERNEL_FAILED, "static scratch has no device address");
        g_scratch_addr[ctx->device] = (unsigned char*)p;
    }
    *out = g_scratch_addr[ctx->device];
    return LEV_OK;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

extern "C" size_t lev_static_scratch_bytes(void) { return LEV_STATIC_SCRATCH_BYTES; }

extern "C" int lev_matvec_static_scratch(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x,
                                         int64_t x_count, int n_cols, float* y, int64_t y_capacity) {
    if (!ctx || !w || !x || !y) return LEV_BAD_ARGUMENT;
    if (row0 < 0 || rows <= 0 || row0 > w->rows || rows > w->rows - row0 || rows > LEV_MAX_DIM)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "rows [%lld, +%lld) beyond the tensor's %lld rows", (long long)row0,
                        (long long)rows, (long long)w->rows);
    if (n_cols < 1 || n_cols > LEV_MAX_COLUMNS)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d outside 1...%d", n_cols, LEV_MAX_COLUMNS);
    if (x_count != (int64_t)n_cols * w->cols)
        return lev_fail(ctx, LEV_WRONG_INPUT_COUNT, "input count %lld, expected %lld", (long long)x_count,
                        (long long)((int64_t)n_cols * w->cols));
    if (y_capacity < (int64_t)n_cols * rows)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "output capacity %lld below %lld", (long long)y_capacity,
                        (long long)((int64_t)n_cols * rows));
    {   // aliasing x and y is rejected like in lev_matvec
        const char *xa = (const char*)x, *ya = (const char*)y;
        const size_t xb = (size_t)x_count * sizeof(float), yb = (size_t)n_cols * (size_t)rows * sizeof(float);
        if (xa < ya + yb && ya < xa + xb) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and y overlap");
    }
    if (!lev_stream_supported(w, row0, rows, n_cols))
        return lev_fail(ctx, LEV_UNSUPPORTED, "the stream schedule does not serve this tensor or row window");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    {   // evidence of this call (the kernels fill in grid and block)
        lev_evidence* e = &ctx->ev;
        snprintf(e->device_name, sizeof e->device_name, "%.127s", ctx->prop.name);
        snprintf(e->kernel_name, sizeof e->kernel_name, "lev_matvec_static_scratch");
        e->out_dim = rows;
        e->in_dim = w->cols;
        e->n_cols = n_cols;
        e->weight_bytes = (size_t)rows * (size_t)w->blocks_per_row * (size_t)lev_block_bytes(w->type);
        e->gpu_us = 0.f;
        e->status = LEV_OK;
    }
    // the one-launch kernel builds its tables in shared memory and needs no work buffers at all
    if (lev_dense_supported(ctx, w, row0, rows, x, n_cols)) return lev_dense_run(ctx, w, row0, rows, x, n_cols, y);

    const int terms = lev_stream_terms(n_cols);
    lev_stream_job J = {};
    J.row0 = row0;
    J.rows = rows;
    J.out_ld = rows;
    J.max_jobs = 1;
    const size_t tb = align256(lev_stream_table_bytes(w, n_cols, terms, 1, nullptr));
    if (tb > LEV_STATIC_SCRATCH_BYTES)
        return lev_fail(ctx, LEV_EXCEEDS_WORKLOAD,
                        "this call needs %zu bytes of work buffers, the static scratch holds %u; use lev_matvec", tb,
                        (unsigned)LEV_STATIC_SCRATCH_BYTES);
    unsigned char* base = nullptr;
    LEV_TRY(scratch_address(ctx, &base));
    void* tables = base;
    lev_stream_source src = {};
    src.x = x;
    src.ld = w->cols;
    LEV_TRY(lev_stream_prepare(ctx, w, src, n_cols, terms, 1, tables));
    return lev_stream_run(ctx, w, J, tables, n_cols, terms, y);
}
