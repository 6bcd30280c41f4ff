// Multi-GPU entry points: one process per GPU, NCCL over NVLink.
//
// Dense projections split output rows across ranks and all-gather y.  The MoE
// layer shards experts (lev_moe_weights_upload local_first/local_count) and
// keeps tokens data-parallel: the ranks' token rows are all-gathered, every
// rank routes all tokens (the router is replicated, so no routing metadata or
// counts ever cross the link and no host synchronisation is needed), runs the
// expert FFN for the pairs whose experts it holds, folds them into a weighted
// partial sum per token in rank order, and a reduce-scatter adds the ranks'
// partials and hands each rank its own tokens.  The across-rank addition
// order is NCCL's, so outputs agree with the single-GPU layer to f32
// rounding, not bit for bit; indices and weights are identical.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so that the library
// loads on hosts without it; only lev_dist_* need it.  No TMA multicast and
// no peer-memory operands are used anywhere.
#include <dlfcn.h>
#include <stdlib.h>

#include <new>

#include "lev_internal.h"

namespace {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[LEV_NCCL_ID_BYTES]; } nccl_unique_id;
enum { NCCL_INT32 = 2, NCCL_FLOAT32 = 7, NCCL_SUM = 0 };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(nccl_unique_id*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, nccl_unique_id, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;

bool load_nccl() {
    if (g_nccl.handle) return true;
    const char* names[] = {getenv("LEV_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return false;
#define LEV_SYM(field, name)                                   \
    *(void**)(&g_nccl.field) = dlsym(h, name);                 \
    if (!g_nccl.field) {                                       \
        dlclose(h);                                            \
        return false;                                          \
    }
    LEV_SYM(GetUniqueId, "ncclGetUniqueId")
    LEV_SYM(CommInitRank, "ncclCommInitRank")
    LEV_SYM(CommDestroy, "ncclCommDestroy")
    LEV_SYM(AllGather, "ncclAllGather")
    LEV_SYM(ReduceScatter, "ncclReduceScatter")
    LEV_SYM(GroupStart, "ncclGroupStart")
    LEV_SYM(GroupEnd, "ncclGroupEnd")
    LEV_SYM(GetErrorString, "ncclGetErrorString")
#undef LEV_SYM
    g_nccl.handle = h;
    return true;
}

// [world][tokens][rows_local] -> [tokens][world * rows_local]
__global__ void k_interleave_rows(const float* __restrict__ in, int world, int64_t tokens, int64_t rows_local,
                                  float* __restrict__ out) {
    int64_t total = (int64_t)world * tokens * rows_local;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i % rows_local, t = (i / rows_local) % tokens, w = i / (rows_local * tokens);
        out[t * (world * rows_local) + w * rows_local + r] = in[i];
    }
}

}  // namespace

struct lev_dist_state {
    ncclComm_t comm;
    int rank, world;
};

#define LEV_NCCL(ctx, call)                                                                          \
    do {                                                                                             \
        int _r = (call);                                                                             \
        if (_r != 0) return lev_fail((ctx), LEV_NCCL_ERROR, "%s: %s", #call, g_nccl.GetErrorString(_r)); \
    } while (0)

extern "C" int lev_dist_unique_id(void* id128) {
    if (!id128) return LEV_BAD_ARGUMENT;
    if (!load_nccl()) return LEV_NCCL_ERROR;
    nccl_unique_id id;
    if (g_nccl.GetUniqueId(&id) != 0) return LEV_NCCL_ERROR;
    memcpy(id128, &id, LEV_NCCL_ID_BYTES);
    return LEV_OK;
}

extern "C" int lev_dist_init(lev_ctx* ctx, int rank, int world, const void* id128) {
    if (!ctx || !id128) return LEV_BAD_ARGUMENT;
    if (world < 1 || rank < 0 || rank >= world) return lev_fail(ctx, LEV_BAD_ARGUMENT, "rank %d of %d", rank, world);
    if (ctx->dist) return lev_fail(ctx, LEV_BAD_ARGUMENT, "the context already has a communicator");
    if (!load_nccl()) return lev_fail(ctx, LEV_NCCL_ERROR, "libnccl.so.2 could not be loaded (set LEV_NCCL_LIB)");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    nccl_unique_id id;
    memcpy(&id, id128, LEV_NCCL_ID_BYTES);
    lev_dist_state* d = new (std::nothrow) lev_dist_state();
    if (!d) return lev_fail(ctx, LEV_OUT_OF_MEMORY, "host allocation");
    int r = g_nccl.CommInitRank(&d->comm, world, id, rank);
    if (r != 0) {
        delete d;
        return lev_fail(ctx, LEV_NCCL_ERROR, "ncclCommInitRank: %s", g_nccl.GetErrorString(r));
    }
    d->rank = rank;
    d->world = world;
    ctx->dist = d;
    return LEV_OK;
}

extern "C" int lev_dist_destroy(lev_ctx* ctx) {
    if (!ctx) return LEV_BAD_ARGUMENT;
    if (ctx->dist) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        g_nccl.CommDestroy(ctx->dist->comm);
        delete ctx->dist;
        ctx->dist = nullptr;
    }
    return LEV_OK;
}

extern "C" int lev_matvec_rowsplit_allgather(lev_ctx* ctx, const lev_weights* w, const float* x, int64_t x_count,
                                             int n_cols, float* y_full, int64_t y_capacity, unsigned flags) {
    if (!ctx || !w || !x || !y_full) return LEV_BAD_ARGUMENT;
    if (!ctx->dist) return lev_fail(ctx, LEV_BAD_ARGUMENT, "lev_dist_init has not been called");
    if (flags & LEV_FLAG_HOST_IO) return lev_fail(ctx, LEV_UNSUPPORTED, "multi-GPU entry points take device pointers");
    // a finite check that fails on one rank only would make that rank leave before the collective its
    // peers have already queued; every rank must issue the same sequence
    if (flags & LEV_FLAG_CHECK_FINITE)
        return lev_fail(ctx, LEV_UNSUPPORTED, "multi-GPU entry points do not take LEV_FLAG_CHECK_FINITE: check the inputs before the call");
    const int world = ctx->dist->world;
    const int64_t rl = w->rows, rt = rl * world;
    if (n_cols < 1 || n_cols > LEV_MAX_COLUMNS) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", n_cols);
    if (y_capacity < (int64_t)n_cols * rt)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "output capacity %lld below %lld", (long long)y_capacity, (long long)(n_cols * rt));
    void* s;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_DIST, (size_t)n_cols * rl * sizeof(float) + 256, &s));
    float* yl = (float*)s;
    LEV_TRY(lev_matvec(ctx, w, 0, rl, x, x_count, n_cols, yl, (int64_t)n_cols * rl, LEV_SCHEDULE_AUTO, flags));
    // every rank owns the same number of rows; column c of rank r lands at y_full[c][r * rl ...]
    LEV_NCCL(ctx, g_nccl.GroupStart());
    for (int c = 0; c < n_cols; c++)
        LEV_NCCL(ctx, g_nccl.AllGather(yl + (int64_t)c * rl, y_full + (int64_t)c * rt, (size_t)rl, NCCL_FLOAT32,
                                      ctx->dist->comm, ctx->stream));
    LEV_NCCL(ctx, g_nccl.GroupEnd());
    return LEV_OK;
}

extern "C" int lev_gemm_prefill_rowsplit_allgather(lev_ctx* ctx, const lev_weights* w, const void* x_bf16, int64_t tokens,
                                                   float* y_full, unsigned flags) {
    if (!ctx || !w || !x_bf16 || !y_full) return LEV_BAD_ARGUMENT;
    if (!ctx->dist) return lev_fail(ctx, LEV_BAD_ARGUMENT, "lev_dist_init has not been called");
    if (flags & LEV_FLAG_HOST_IO) return lev_fail(ctx, LEV_UNSUPPORTED, "multi-GPU entry points take device pointers");
    // a finite check that fails on one rank only would make that rank leave before the collective its
    // peers have already queued; every rank must issue the same sequence
    if (flags & LEV_FLAG_CHECK_FINITE)
        return lev_fail(ctx, LEV_UNSUPPORTED, "multi-GPU entry points do not take LEV_FLAG_CHECK_FINITE: check the inputs before the call");
    const int world = ctx->dist->world;
    const int64_t rl = w->rows;
    size_t part = (size_t)tokens * rl * sizeof(float);
    void* s;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_DIST, part * (world + 1) + 512, &s));
    float* yl = (float*)s;
    float* gathered = (float*)((char*)s + ((part + 255) & ~(size_t)255));
    LEV_TRY(lev_gemm_prefill(ctx, w, x_bf16, tokens, yl, flags));
    LEV_NCCL(ctx, g_nccl.AllGather(yl, gathered, (size_t)tokens * rl, NCCL_FLOAT32, ctx->dist->comm, ctx->stream));
    int64_t total = (int64_t)world * tokens * rl;
    int grid = (int)((total + 255) / 256 < (int64_t)ctx->prop.multiProcessorCount * 8 ? (total + 255) / 256
                                                                                        : ctx->prop.multiProcessorCount * 8);
    k_interleave_rows<<<grid < 1 ? 1 : grid, 256, 0, ctx->stream>>>(gathered, world, tokens, rl, y_full);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_interleave_rows");
}

extern "C" int lev_moe_layer_ep(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                                float* out, int32_t* idx_out, float* w_out, unsigned flags) {
    if (!ctx || !w || !x || !out) return LEV_BAD_ARGUMENT;
    if (!ctx->dist) return lev_fail(ctx, LEV_BAD_ARGUMENT, "lev_dist_init has not been called");
    if (flags & LEV_FLAG_HOST_IO) return lev_fail(ctx, LEV_UNSUPPORTED, "multi-GPU entry points take device pointers");
    // a finite check that fails on one rank only would make that rank leave before the collective its
    // peers have already queued; every rank must issue the same sequence
    if (flags & LEV_FLAG_CHECK_FINITE)
        return lev_fail(ctx, LEV_UNSUPPORTED, "multi-GPU entry points do not take LEV_FLAG_CHECK_FINITE: check the inputs before the call");
    if (tokens <= 0 || tokens > (1 << 20)) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "tokens %lld", (long long)tokens);
    if (top_k <= 0 || top_k > LEV_MAX_TOP_K || top_k > w->experts)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "topK %d with %d experts", top_k, w->experts);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const int world = ctx->dist->world, rank = ctx->dist->rank;
    const int64_t tall = tokens * world, pairs = tall * top_k;
    const size_t xb = ((size_t)tall * w->hidden * 4 + 255) & ~(size_t)255;
    const size_t ib = ((size_t)pairs * 4 + 255) & ~(size_t)255;
    const size_t sb = ((size_t)tall * w->experts * 4 + 255) & ~(size_t)255;
    const size_t yb = ((size_t)pairs * w->hidden * 4 + 255) & ~(size_t)255;
    void* s;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_DIST, 2 * xb + 2 * ib + sb + 256, &s));
    char* p = (char*)s;
    float* xall = (float*)p;
    p += xb;
    float* partial = (float*)p;
    p += xb;
    int32_t* idx = (int32_t*)p;
    p += ib;
    float* wts = (float*)p;
    p += ib;
    float* scores = (float*)p;
    void* d;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_MOE_D, yb + 256, &d));
    float* ypairs = (float*)d;

    // every rank routes its own tokens (the router is replicated); tokens and routing are then
    // gathered so that each rank can run the pairs of its resident experts
    int32_t* idx_l = idx + (size_t)rank * tokens * top_k;
    float* wts_l = wts + (size_t)rank * tokens * top_k;
    LEV_TRY(lev_moe_route_dev(ctx, w, x, tokens, top_k, idx_l, wts_l, scores));
    LEV_NCCL(ctx, g_nccl.GroupStart());
    LEV_NCCL(ctx, g_nccl.AllGather(x, xall, (size_t)tokens * w->hidden, NCCL_FLOAT32, ctx->dist->comm, ctx->stream));
    LEV_NCCL(ctx, g_nccl.AllGather(idx_l, idx, (size_t)tokens * top_k, NCCL_INT32, ctx->dist->comm, ctx->stream));
    LEV_NCCL(ctx, g_nccl.AllGather(wts_l, wts, (size_t)tokens * top_k, NCCL_FLOAT32, ctx->dist->comm, ctx->stream));
    LEV_NCCL(ctx, g_nccl.GroupEnd());
    LEV_TRY(lev_moe_experts_dev(ctx, w, xall, tall, top_k, idx, ypairs, nullptr));
    // slots of experts that live elsewhere are skipped: no zero fill of the pair outputs is needed
    LEV_TRY(lev_moe_combine_resident_dev(ctx, ypairs, wts, tall, top_k, w->hidden, partial, idx, w->local_first, w->local_count));
    LEV_NCCL(ctx, g_nccl.ReduceScatter(partial, out, (size_t)tokens * w->hidden, NCCL_FLOAT32, NCCL_SUM, ctx->dist->comm,
                                      ctx->stream));
    size_t own = (size_t)tokens * top_k * 4;
    if (idx_out) LEV_CUDA(ctx, cudaMemcpyAsync(idx_out, idx + (size_t)rank * tokens * top_k, own, cudaMemcpyDeviceToDevice, ctx->stream));
    if (w_out) LEV_CUDA(ctx, cudaMemcpyAsync(w_out, wts + (size_t)rank * tokens * top_k, own, cudaMemcpyDeviceToDevice, ctx->stream));
    return LEV_OK;
}
