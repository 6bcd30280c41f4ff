// Context, error reporting, resident weights and the host-pointer entry
// points of libleviathan_cuda.so.  Validation order follows the reference:
// geometry, byte counts, input counts, then finiteness, all before any
// device work (Sources/LeviathanCore/Q4.swift:168-191).
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>

#include <new>

#include "lev_internal.h"
#include "lev_stream.h"

extern "C" int lev_cuda_destroy(lev_ctx* ctx);
extern "C" int lev_cuda_abi_version(void) { return LEV_CUDA_ABI_VERSION; }

extern "C" const char* lev_status_name(int s) {
    switch (s) {
        case LEV_OK: return "ok";
        case LEV_BAD_DIMENSIONS: return "badDimensions";
        case LEV_WRONG_INPUT_COUNT: return "wrongInputCount";
        case LEV_NONFINITE_INPUT: return "nonFiniteInput";
        case LEV_NONFINITE_SCALE: return "nonFiniteScale";
        case LEV_NONFINITE_OUTPUT: return "nonFiniteOutput";
        case LEV_EXCEEDS_WORKLOAD: return "exceedsModelWorkload";
        case LEV_INTEGER_OVERFLOW: return "integerOverflow";
        case LEV_DEVICE_UNAVAILABLE: return "deviceUnavailable";
        case LEV_KERNEL_FAILED: return "kernelFailed";
        case LEV_TIMEOUT: return "timeout";
        case LEV_NCCL_ERROR: return "ncclError";
        case LEV_BAD_ARGUMENT: return "badArgument";
        case LEV_OUT_OF_MEMORY: return "outOfMemory";
        case LEV_BAD_OP_SPEC: return "badOpSpec";
        case LEV_UNSUPPORTED: return "unsupported";
        case LEV_GGUF_BAD_MAGIC: return "badMagic";
        case LEV_GGUF_UNSUPPORTED_VERSION: return "unsupportedVersion";
        case LEV_GGUF_TRUNCATED: return "truncated";
        case LEV_GGUF_UNKNOWN_VALUE_TYPE: return "unknownValueType";
        case LEV_GGUF_BAD_TENSOR: return "badTensor";
        case LEV_GGUF_DATA_BEYOND_EOF: return "dataBeyondEndOfFile";
        case LEV_GGUF_MISSING: return "missing";
        case LEV_GGUF_UNSUPPORTED_TENSOR_TYPE: return "unsupportedTensorType";
    }
    return "unknown";
}

int lev_fail(lev_ctx* ctx, int status, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        int n = snprintf(ctx->err, sizeof ctx->err, "%s: ", lev_status_name(status));
        if (n > 0 && n < (int)sizeof ctx->err) vsnprintf(ctx->err + n, sizeof ctx->err - n, fmt, ap);
        va_end(ap);
    }
    return status;
}

int lev_cuda_check(lev_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return LEV_OK;
    int st = (e == cudaErrorMemoryAllocation) ? LEV_OUT_OF_MEMORY : LEV_KERNEL_FAILED;
    return lev_fail(ctx, st, "%s: %s", what, cudaGetErrorString(e));
}

int lev_scratch(lev_ctx* ctx, int slot, size_t bytes, void** out) {
    if (bytes == 0) bytes = 256;
    if (ctx->scratch_bytes[slot] < bytes) {
        // a growing buffer may still be in use by work queued on the stream
        LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch[slot]) cudaFree(ctx->scratch[slot]);
        ctx->scratch[slot] = nullptr;
        ctx->scratch_bytes[slot] = 0;
        size_t want = bytes + bytes / 4;
        LEV_CUDA(ctx, cudaMalloc(&ctx->scratch[slot], want));
        ctx->scratch_bytes[slot] = want;
    }
    *out = ctx->scratch[slot];
    return LEV_OK;
}

int lev_read_status(lev_ctx* ctx, int* bits) {
    LEV_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    LEV_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
    LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *bits = *ctx->h_status;
    return LEV_OK;
}

extern "C" int lev_cuda_init(int device, lev_ctx** out_ctx) {
    if (!out_ctx) return LEV_BAD_ARGUMENT;
    *out_ctx = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) return LEV_DEVICE_UNAVAILABLE;
    if (device < 0 || device >= count) return LEV_DEVICE_UNAVAILABLE;
    lev_ctx* ctx = new (std::nothrow) lev_ctx();
    if (!ctx) return LEV_OUT_OF_MEMORY;
    memset(ctx, 0, sizeof *ctx);
    ctx->device = device;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&ctx->prop, device) != cudaSuccess) {
        delete ctx;
        return LEV_DEVICE_UNAVAILABLE;
    }
    // the kernels are built for sm_100a only; refuse anything else loudly
    if (ctx->prop.major != 10) {
        delete ctx;
        return LEV_DEVICE_UNAVAILABLE;
    }
    if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
        // the status word, then the zero-initialised counters of kernels that elect a last thread block
        cudaMalloc((void**)&ctx->d_status, (LEV_COUNTER_OFFSET + LEV_COUNTERS) * sizeof(int)) != cudaSuccess ||
        cudaMallocHost((void**)&ctx->h_status, sizeof(int)) != cudaSuccess ||
        cudaEventCreate(&ctx->ev0) != cudaSuccess || cudaEventCreate(&ctx->ev1) != cudaSuccess) {
        delete ctx;
        return LEV_DEVICE_UNAVAILABLE;
    }
    ctx->stream = ctx->own_stream;
    {   // tuning of the persistent matvec kernel, read once per context
        const char* v = getenv("LEV_CHAIN");
        ctx->chain_off = v && *v == '0';
        v = getenv("LEV_CHAIN_WARPS");
        ctx->chain_warps = v ? atoi(v) : 0;
        v = getenv("LEV_CHAIN_DEPTH");
        ctx->chain_depth = v ? atoi(v) : 0;
    }
    cudaMemsetAsync(ctx->d_status, 0, (LEV_COUNTER_OFFSET + LEV_COUNTERS) * sizeof(int), ctx->stream);
    if (lev_chain_init(ctx) != LEV_OK) {
        lev_cuda_destroy(ctx);
        return LEV_OUT_OF_MEMORY;
    }
    cudaStreamSynchronize(ctx->stream);
    *out_ctx = ctx;
    return LEV_OK;
}

extern "C" int lev_dist_destroy(lev_ctx* ctx);

extern "C" int lev_cuda_destroy(lev_ctx* ctx) {
    if (!ctx) return LEV_BAD_ARGUMENT;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->dist) lev_dist_destroy(ctx);
    for (int i = 0; i < LEV_SCR_SLOTS; i++)
        if (ctx->scratch[i]) cudaFree(ctx->scratch[i]);
    cudaFree(ctx->d_status);
    if (ctx->chain_sync) cudaFree(ctx->chain_sync);
    cudaFreeHost(ctx->h_status);
    cudaEventDestroy(ctx->ev0);
    cudaEventDestroy(ctx->ev1);
    cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return LEV_OK;
}

extern "C" const char* lev_last_error(const lev_ctx* ctx) { return ctx ? ctx->err : "null context"; }

extern "C" int lev_cuda_hardware_profile(lev_ctx* ctx, lev_hw_profile* out) {
    if (!ctx || !out) return LEV_BAD_ARGUMENT;
    memset(out, 0, sizeof *out);
    snprintf(out->device_name, sizeof out->device_name, "%.127s", ctx->prop.name);
    out->sm_count = ctx->prop.multiProcessorCount;
    out->max_threads_per_block = ctx->prop.maxThreadsPerBlock;
    out->warp_width = ctx->prop.warpSize;
    out->cc_major = ctx->prop.major;
    out->cc_minor = ctx->prop.minor;
    out->total_memory = ctx->prop.totalGlobalMem;
    out->shared_memory_per_block_optin = ctx->prop.sharedMemPerBlockOptin;
    out->l2_bytes = (size_t)ctx->prop.l2CacheSize;
    size_t free_b = 0, total_b = 0;
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    LEV_CUDA(ctx, cudaMemGetInfo(&free_b, &total_b));
    out->free_memory = free_b;
    return LEV_OK;
}

extern "C" int lev_cuda_set_stream(lev_ctx* ctx, void* s) {
    if (!ctx) return LEV_BAD_ARGUMENT;
    ctx->stream = s ? (cudaStream_t)s : ctx->own_stream;
    return LEV_OK;
}

extern "C" int lev_cuda_synchronize(lev_ctx* ctx) {
    if (!ctx) return LEV_BAD_ARGUMENT;
    // the wait also collects what kernels recorded instead of faulting: a bounded wait that ran out,
    // a cache index outside its layout
    int bits = 0;
    LEV_TRY(lev_read_status(ctx, &bits));
    if (bits & LEV_DEV_TIMEOUT) {
        // a kernel that gave up may have left arrival counters and flags of the persistent matvec kernel set
        lev_chain_reset(ctx);
        return lev_fail(ctx, LEV_TIMEOUT, "a kernel's bounded wait ran out");
    }
    if (bits & LEV_DEV_BAD_INDEX) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "a slot, position, block-table entry or token id lay outside its table");
    return LEV_OK;
}

extern "C" int64_t lev_cuda_launch_count(const lev_ctx* ctx) { return ctx ? ctx->launches : -1; }

extern "C" int lev_cuda_last_evidence(const lev_ctx* ctx, lev_evidence* out) {
    if (!ctx || !out) return LEV_BAD_ARGUMENT;
    *out = ctx->ev;
    return LEV_OK;
}

// ---------------------------------------------------------------------------
// resident weights
// ---------------------------------------------------------------------------

static int check_geometry(lev_ctx* ctx, int type, int64_t rows, int64_t cols, size_t n_bytes,
                          int64_t* bpr_out) {
    if (!lev_type_ok(type)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "ggml type %d is not on the path", type);
    int bv = lev_block_values(type), bb = lev_block_bytes(type);
    if (cols <= 0 || rows <= 0 || cols % bv != 0 || cols > LEV_MAX_DIM)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "inDim %lld, outDim %lld", (long long)cols, (long long)rows);
    int64_t bpr = cols / bv;
    // rows may exceed the per-matvec row limit for stacked expert tensors;
    // the product is what must not overflow
    unsigned __int128 need = (unsigned __int128)(uint64_t)rows * (uint64_t)bpr * (uint64_t)bb;
    if (need > (unsigned __int128)LEV_MAX_WEIGHT_BYTES)
        return lev_fail(ctx, LEV_EXCEEDS_WORKLOAD, "weights need more than %llu bytes",
                        (unsigned long long)LEV_MAX_WEIGHT_BYTES);
    if ((size_t)need != n_bytes)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "weights are %zu bytes, geometry needs %zu", n_bytes, (size_t)need);
    *bpr_out = bpr;
    return LEV_OK;
}

int lev_weights_create(lev_ctx* ctx, const void* bytes, size_t n_bytes, int type, int64_t rows,
                       int64_t cols, int on_device, bool repack, lev_weights** out) {
    int64_t bpr = 0;
    LEV_TRY(check_geometry(ctx, type, rows, cols, n_bytes, &bpr));
    if (!bytes) return lev_fail(ctx, LEV_BAD_ARGUMENT, "null weight bytes");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    lev_weights* w = new (std::nothrow) lev_weights();
    if (!w) return lev_fail(ctx, LEV_OUT_OF_MEMORY, "host allocation");
    memset(w, 0, sizeof *w);
    w->type = type;
    w->rows = rows;
    w->cols = cols;
    w->blocks_per_row = bpr;
    w->gguf_bytes = n_bytes;
    w->owns_raw = 1;
    // 256 spare bytes: vector loads of the last block may run past the end
    int st = lev_cuda_check(ctx, cudaMalloc((void**)&w->raw, n_bytes + 256), "cudaMalloc(weights)");
    if (st) {
        delete w;
        return st;
    }
    cudaMemsetAsync(w->raw + n_bytes, 0, 256, ctx->stream);
    st = lev_cuda_check(ctx,
                        cudaMemcpyAsync(w->raw, bytes, n_bytes,
                                        on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream),
                        "cudaMemcpy(weights)");
    if (!st) st = lev_launch_scale_check(ctx, w);
    int bits = 0;
    if (!st) st = lev_read_status(ctx, &bits);
    if (!st && (bits & LEV_DEV_NONFINITE_SCALE)) st = lev_fail(ctx, LEV_NONFINITE_SCALE, "a block scale is Inf or NaN");
    if (!st && repack) st = lev_repack_weights(ctx, w);
    if (st) {
        cudaFree(w->raw);
        if (w->packed) cudaFree(w->packed);
        delete w;
        return st;
    }
    *out = w;
    return LEV_OK;
}

extern "C" int lev_weights_upload(lev_ctx* ctx, const void* bytes, size_t n_bytes, int ggml_type,
                                  int64_t rows, int64_t cols, int bytes_on_device, lev_weights** out) {
    if (!ctx || !out) return LEV_BAD_ARGUMENT;
    *out = nullptr;
    if (rows > LEV_MAX_DIM) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "inDim %lld, outDim %lld", (long long)cols, (long long)rows);
    return lev_weights_create(ctx, bytes, n_bytes, ggml_type, rows, cols, bytes_on_device, true, out);
}

extern "C" int lev_weights_free(lev_ctx* ctx, lev_weights* w) {
    if (!ctx || !w) return LEV_BAD_ARGUMENT;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (w->raw && w->owns_raw) cudaFree(w->raw);
    if (w->packed) cudaFree(w->packed);
    delete w;
    return LEV_OK;
}

// Frees the GGUF-order copy of a tensor the stream schedule serves; the repacked copy (the same bytes in
// tile order) stays.  A resident tensor then occupies its GGUF size once.
extern "C" int lev_weights_release_gguf(lev_ctx* ctx, lev_weights* w) {
    if (!ctx || !w) return LEV_BAD_ARGUMENT;
    if (!w->packed) return lev_fail(ctx, LEV_UNSUPPORTED, "the tensor has no repacked copy: the GGUF-order bytes are the only ones");
    if (!w->raw) return LEV_OK;
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (w->owns_raw) cudaFree(w->raw);
    w->raw = nullptr;
    return LEV_OK;
}

extern "C" int lev_weights_info(const lev_weights* w, int* type, int64_t* rows, int64_t* cols, size_t* bytes) {
    if (!w) return LEV_BAD_ARGUMENT;
    if (type) *type = w->type;
    if (rows) *rows = w->rows;
    if (cols) *cols = w->cols;
    if (bytes) *bytes = w->gguf_bytes;
    return LEV_OK;
}

static int check_rows(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows) {
    if (row0 < 0 || rows <= 0 || row0 > w->rows || rows > w->rows - row0)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "rows [%lld, +%lld) beyond the tensor's %lld rows",
                        (long long)row0, (long long)rows, (long long)w->rows);
    if (rows > LEV_MAX_DIM) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "outDim %lld", (long long)rows);
    return LEV_OK;
}

extern "C" int lev_dequantize(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, float* out,
                              unsigned flags) {
    if (!ctx || !w || !out) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_rows(ctx, w, row0, rows));
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    float* dst = out;
    size_t n = (size_t)rows * (size_t)w->cols;
    if (flags & LEV_FLAG_HOST_IO) {
        void* p;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_Y, n * sizeof(float), &p));
        dst = (float*)p;
    }
    LEV_TRY(lev_launch_dequantize(ctx, w, row0, rows, dst));
    if (flags & LEV_FLAG_HOST_IO) {
        LEV_CUDA(ctx, cudaMemcpyAsync(out, dst, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
        LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return LEV_OK;
}

// ---------------------------------------------------------------------------
// decode matvec
// ---------------------------------------------------------------------------

static void note_evidence(lev_ctx* ctx, const char* kernel, const lev_weights* w, int64_t rows, int n_cols,
                          int grid, int block) {
    lev_evidence* e = &ctx->ev;
    snprintf(e->device_name, sizeof e->device_name, "%.127s", ctx->prop.name);
    snprintf(e->kernel_name, sizeof e->kernel_name, "%.63s", kernel);
    e->out_dim = rows;
    e->in_dim = w->cols;
    e->n_cols = n_cols;
    e->grid = grid;
    e->block = block;
    e->weight_bytes = (size_t)rows * (size_t)w->blocks_per_row * (size_t)lev_block_bytes(w->type);
    e->gpu_us = 0.f;
    e->status = LEV_OK;
}

extern "C" int lev_matvec(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x,
                          int64_t x_count, int n_cols, float* y, int64_t y_capacity, int schedule,
                          unsigned flags) {
    if (!ctx || !w || !x || !y) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_rows(ctx, w, row0, rows));
    if (n_cols < 1 || n_cols > LEV_MAX_COLUMNS)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d outside 1...%d", n_cols, LEV_MAX_COLUMNS);
    if (x_count != (int64_t)n_cols * w->cols)
        return lev_fail(ctx, LEV_WRONG_INPUT_COUNT, "input count %lld, expected %lld", (long long)x_count,
                        (long long)((int64_t)n_cols * w->cols));
    if (y_capacity < (int64_t)n_cols * rows)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "output capacity %lld below %lld", (long long)y_capacity,
                        (long long)((int64_t)n_cols * rows));
    if (schedule != LEV_SCHEDULE_AUTO && schedule != LEV_SCHEDULE_PLAIN && schedule != LEV_SCHEDULE_STREAM)
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "unknown schedule %d", schedule);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));

    const float* dx = x;
    float* dy = y;
    bool y_direct = false;
    size_t xb = (size_t)x_count * sizeof(float), yb = (size_t)n_cols * (size_t)rows * sizeof(float);
    if (flags & LEV_FLAG_HOST_IO) {
        if (flags & LEV_FLAG_CHECK_FINITE) {  // the reference checks on the host before any device work
            for (int64_t i = 0; i < x_count; i++)
                if (!isfinite(x[i])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        }
        void *px, *py;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_X, xb, &px));
        LEV_CUDA(ctx, cudaMemcpyAsync(px, x, xb, cudaMemcpyHostToDevice, ctx->stream));
        dx = (const float*)px;
        // page-locked, device-mapped output buffers are written by the kernel itself (posted writes
        // over the host link): one copy and its launch less per call
        cudaPointerAttributes pa;
        if (cudaPointerGetAttributes(&pa, y) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer &&
            !(flags & LEV_FLAG_CHECK_FINITE)) {
            dy = (float*)pa.devicePointer;
            y_direct = true;
        } else {
            (void)cudaGetLastError();  // an unregistered host pointer is not an error here
            LEV_TRY(lev_scratch(ctx, LEV_SCR_Y, yb, &py));
            dy = (float*)py;
        }
    } else {
        // aliasing x and y is rejected like scratch aliasing in the reference
        // (Sources/LeviathanCore/Gemma4.swift:2096-2100)
        const char* xa = (const char*)x;
        const char* ya = (const char*)y;
        if (xa < ya + yb && ya < xa + xb) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and y overlap");
        if (flags & LEV_FLAG_CHECK_FINITE) LEV_TRY(lev_launch_finite_check(ctx, dx, x_count, LEV_DEV_NONFINITE_INPUT));
    }

    bool stream_ok = lev_stream_supported(w, row0, rows, n_cols);
    if (schedule == LEV_SCHEDULE_STREAM && !stream_ok)
        return lev_fail(ctx, LEV_UNSUPPORTED, "the stream schedule does not serve this geometry");
    bool use_stream = schedule == LEV_SCHEDULE_STREAM || (schedule == LEV_SCHEDULE_AUTO && stream_ok);
    note_evidence(ctx, use_stream ? "lev_matvec_stream" : "lev_matvec_plain", w, rows, n_cols, 0, 0);
    if (use_stream)
        LEV_TRY(lev_launch_matvec_stream(ctx, w, row0, rows, dx, n_cols, dy));
    else
        LEV_TRY(lev_launch_matvec_plain(ctx, w, row0, rows, dx, n_cols, dy));

    if (flags & LEV_FLAG_CHECK_FINITE) LEV_TRY(lev_launch_finite_check(ctx, dy, (int64_t)n_cols * rows, LEV_DEV_NONFINITE_OUTPUT));
    if ((flags & LEV_FLAG_HOST_IO) && !y_direct)
        LEV_CUDA(ctx, cudaMemcpyAsync(y, dy, yb, cudaMemcpyDeviceToHost, ctx->stream));
    if (flags & (LEV_FLAG_CHECK_FINITE | LEV_FLAG_HOST_IO)) {
        int bits = 0;
        if (flags & LEV_FLAG_CHECK_FINITE) {
            LEV_TRY(lev_read_status(ctx, &bits));
        } else {
            LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        }
        if (bits & LEV_DEV_NONFINITE_INPUT) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        if (bits & LEV_DEV_NONFINITE_OUTPUT) return lev_fail(ctx, LEV_NONFINITE_OUTPUT, "output vector");
    }
    return LEV_OK;
}

// Several resident tensors against the same activations.  One launch when the tensors share
// format and inDim and the one-launch kernel serves them; otherwise one matvec per tensor.
extern "C" int lev_matvec_multi(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x, int64_t x_count,
                                int n_cols, float* const* y, const int64_t* y_capacity, unsigned flags) {
    if (!ctx || !w || !x || !y || !y_capacity) return LEV_BAD_ARGUMENT;
    if (n_ops < 1 || n_ops > 4) return lev_fail(ctx, LEV_BAD_ARGUMENT, "%d tensors (1...4)", n_ops);
    if (n_cols < 1 || n_cols > LEV_MAX_COLUMNS)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d outside 1...%d", n_cols, LEV_MAX_COLUMNS);
    for (int i = 0; i < n_ops; i++) {
        if (!w[i] || !y[i]) return LEV_BAD_ARGUMENT;
        if (x_count != (int64_t)n_cols * w[i]->cols)
            return lev_fail(ctx, LEV_WRONG_INPUT_COUNT, "input count %lld, tensor %d expects %lld", (long long)x_count, i,
                            (long long)((int64_t)n_cols * w[i]->cols));
        if (y_capacity[i] < (int64_t)n_cols * w[i]->rows)
            return lev_fail(ctx, LEV_BAD_DIMENSIONS, "output %d capacity %lld below %lld", i, (long long)y_capacity[i],
                            (long long)((int64_t)n_cols * w[i]->rows));
    }
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool host = flags & LEV_FLAG_HOST_IO;
    const float* dx = x;
    float* dy[4] = {nullptr, nullptr, nullptr, nullptr};
    const size_t xb = (size_t)x_count * sizeof(float);
    if (host) {
        if (flags & LEV_FLAG_CHECK_FINITE)
            for (int64_t i = 0; i < x_count; i++)
                if (!isfinite(x[i])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        void* px;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_X, xb, &px));
        LEV_CUDA(ctx, cudaMemcpyAsync(px, x, xb, cudaMemcpyHostToDevice, ctx->stream));
        dx = (const float*)px;
        size_t total = 0;
        for (int i = 0; i < n_ops; i++) total += ((size_t)n_cols * w[i]->rows * sizeof(float) + 255) & ~(size_t)255;
        void* py;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_Y, total, &py));
        size_t off = 0;
        for (int i = 0; i < n_ops; i++) {
            dy[i] = (float*)((char*)py + off);
            off += ((size_t)n_cols * w[i]->rows * sizeof(float) + 255) & ~(size_t)255;
        }
    } else {
        for (int i = 0; i < n_ops; i++) dy[i] = y[i];
        if (flags & LEV_FLAG_CHECK_FINITE) LEV_TRY(lev_launch_finite_check(ctx, dx, x_count, LEV_DEV_NONFINITE_INPUT));
    }
    lev_chain_item chain_items[4];
    for (int i = 0; i < n_ops; i++) chain_items[i] = {w[i], 0, w[i]->rows, dx, dy[i], 0, nullptr};
    if (n_cols == 1 && n_ops >= 2 && lev_chain_preferred(ctx, n_ops, chain_items)) {
        note_evidence(ctx, "lev_matvec_chain", w[0], w[0]->rows, n_cols, 0, 0);
        LEV_TRY(lev_chain_run(ctx, n_ops, chain_items));
    } else if (n_ops >= 2 && lev_dense_multi_supported(ctx, n_ops, w, dx, n_cols)) {
        note_evidence(ctx, "lev_matvec_stream_multi", w[0], w[0]->rows, n_cols, 0, 0);
        LEV_TRY(lev_dense_multi_run(ctx, n_ops, w, dx, n_cols, dy));
    } else {
        for (int i = 0; i < n_ops; i++)
            LEV_TRY(lev_matvec(ctx, w[i], 0, w[i]->rows, dx, x_count, n_cols, dy[i], (int64_t)n_cols * w[i]->rows, LEV_SCHEDULE_AUTO, 0));
    }
    if (flags & LEV_FLAG_CHECK_FINITE)
        for (int i = 0; i < n_ops; i++)
            LEV_TRY(lev_launch_finite_check(ctx, dy[i], (int64_t)n_cols * w[i]->rows, LEV_DEV_NONFINITE_OUTPUT));
    if (host)
        for (int i = 0; i < n_ops; i++)
            LEV_CUDA(ctx, cudaMemcpyAsync(y[i], dy[i], (size_t)n_cols * w[i]->rows * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    if (flags & (LEV_FLAG_CHECK_FINITE | LEV_FLAG_HOST_IO)) {
        int bits = 0;
        if (flags & LEV_FLAG_CHECK_FINITE) {
            LEV_TRY(lev_read_status(ctx, &bits));
        } else {
            LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        }
        if (bits & LEV_DEV_NONFINITE_INPUT) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        if (bits & LEV_DEV_NONFINITE_OUTPUT) return lev_fail(ctx, LEV_NONFINITE_OUTPUT, "output vector");
    }
    return LEV_OK;
}

// One-shot: upload, run with CUDA-event timing, read back, free.
static int matvec_host(lev_ctx* ctx, int type, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                       int64_t in_dim, const float* x, int64_t x_count, float* y, lev_evidence* evidence) {
    if (!ctx || !y) return LEV_BAD_ARGUMENT;
    int bv = lev_block_values(type);
    if (in_dim <= 0 || out_dim <= 0 || in_dim % bv != 0 || in_dim > LEV_MAX_DIM || out_dim > LEV_MAX_DIM)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "inDim %lld, outDim %lld", (long long)in_dim, (long long)out_dim);
    size_t need = (size_t)out_dim * (size_t)(in_dim / bv) * (size_t)lev_block_bytes(type);
    if (n_bytes != need) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "weights are %zu bytes, geometry needs %zu", n_bytes, need);
    if (x_count != in_dim) return lev_fail(ctx, LEV_WRONG_INPUT_COUNT, "input count %lld, expected %lld", (long long)x_count, (long long)in_dim);
    if (!blocks || !x) return LEV_BAD_ARGUMENT;
    for (int64_t i = 0; i < x_count; i++)
        if (!isfinite(x[i])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
    lev_weights* w = nullptr;
    LEV_TRY(lev_weights_create(ctx, blocks, n_bytes, type, out_dim, in_dim, 0, true, &w));
    void *px = nullptr, *py = nullptr;
    int st = lev_scratch(ctx, LEV_SCR_X, (size_t)in_dim * 4, &px);
    if (!st) st = lev_scratch(ctx, LEV_SCR_Y, (size_t)out_dim * 4, &py);
    if (!st) st = lev_cuda_check(ctx, cudaMemcpyAsync(px, x, (size_t)in_dim * 4, cudaMemcpyHostToDevice, ctx->stream), "copy x");
    if (!st) st = lev_cuda_check(ctx, cudaEventRecord(ctx->ev0, ctx->stream), "event");
    if (!st) st = lev_matvec(ctx, w, 0, out_dim, (const float*)px, in_dim, 1, (float*)py, out_dim, LEV_SCHEDULE_AUTO, 0);
    if (!st) st = lev_cuda_check(ctx, cudaEventRecord(ctx->ev1, ctx->stream), "event");
    if (!st) st = lev_launch_finite_check(ctx, (const float*)py, out_dim, LEV_DEV_NONFINITE_OUTPUT);
    if (!st) st = lev_cuda_check(ctx, cudaMemcpyAsync(y, py, (size_t)out_dim * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy y");
    int bits = 0;
    if (!st) st = lev_read_status(ctx, &bits);
    if (!st && (bits & LEV_DEV_NONFINITE_OUTPUT)) st = lev_fail(ctx, LEV_NONFINITE_OUTPUT, "output vector");
    if (!st) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1);
        ctx->ev.gpu_us = ms * 1000.f;
    }
    ctx->ev.status = st;
    if (evidence) *evidence = ctx->ev;
    lev_weights_free(ctx, w);
    return st;
}

extern "C" int lev_q4_0_matvec_host(lev_ctx* ctx, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                                    int64_t in_dim, const float* x, int64_t x_count, float* y, lev_evidence* ev) {
    return matvec_host(ctx, LEV_GGML_Q4_0, blocks, n_bytes, out_dim, in_dim, x, x_count, y, ev);
}
extern "C" int lev_q4_k_matvec_host(lev_ctx* ctx, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                                    int64_t in_dim, const float* x, int64_t x_count, float* y, lev_evidence* ev) {
    return matvec_host(ctx, LEV_GGML_Q4_K, blocks, n_bytes, out_dim, in_dim, x, x_count, y, ev);
}
extern "C" int lev_q6_k_matvec_host(lev_ctx* ctx, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                                    int64_t in_dim, const float* x, int64_t x_count, float* y, lev_evidence* ev) {
    return matvec_host(ctx, LEV_GGML_Q6_K, blocks, n_bytes, out_dim, in_dim, x, x_count, y, ev);
}
