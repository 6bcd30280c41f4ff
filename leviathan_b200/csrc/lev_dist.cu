// Multi-GPU entry points: one process per GPU on one NVSwitch box.
//
// Plumbing is NCCL (bound at run time through dlopen, so the library loads on hosts without it); the
// data paths run over peer memory: every rank allocates one "heap", the ranks exchange CUDA IPC handles
// once (an NCCL all-gather of the handles) and map each other's heaps.  A collective step is then one
// launch that stores this rank's rows straight into every peer's heap (plain peer stores over NVLink,
// no TMA, no multicast), a system-scope fence by the last thread block and one flag word per peer; the
// consumer runs a one-block wait kernel whose spins are bounded (LEV_TIMEOUT).  Flags carry an epoch
// that every call advances on the device, so a captured CUDA graph replays correctly.
//
//  * Dense projections split output rows across ranks; each rank pushes its slice of y (or its columns
//    of the prefill GEMM's Y) into every rank's copy of the full output.
//  * The MoE layer shards experts (lev_moe_weights_upload local_first / local_count) and keeps tokens
//    data-parallel.  Dispatch: every rank routes its own tokens and pushes token rows, indices and
//    weights to all ranks (a token's eight experts live on about five of eight ranks, so little is sent
//    in vain).  Each rank runs the expert FFN for the pairs whose experts it holds.  Combine: the
//    unweighted output row of every pair is stored into the heap of the rank that owns the token, at
//    [token][slot]; that rank adds its tokens' slots in rank order (one axpy per slot like
//    Sources/LeviathanCore/Gemma4.swift:3878, :2171-2175).  No floating-point sum crosses a rank, so the
//    result equals the single-GPU layer bit for bit.
//  * Where the peer mapping is not available the entry points fall back to NCCL collectives
//    (all-gather / reduce-scatter); the MoE result then agrees to f32 rounding only.
#include <dlfcn.h>
#include <stdlib.h>

#include <new>

#include "lev_internal.h"

#define LEV_MAX_RANKS 16

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

// first bytes of every heap
struct HeapHeader {
    unsigned epoch[4];    // per phase: completed rounds; a push of round e + 1 flags e + 1, the wait then advances it
    unsigned arrive;      // thread blocks of a push that have finished their stores
    unsigned waited;      // thread blocks of a wait-and-copy that have seen every flag
    unsigned pad[58];
    unsigned flag[4][LEV_MAX_RANKS];  // [phase][source rank]: epoch of the last completed push from that rank
};
constexpr size_t kHeapHeaderBytes = 4096;

struct lev_dist_state {
    ncclComm_t comm;
    int rank, world;
    char* heap;                      // this rank's heap (device memory), NULL: peer paths unavailable
    size_t heap_bytes;
    char* peer[LEV_MAX_RANKS];       // every rank's heap as mapped here (peer[rank] == heap)
};

namespace {

struct PushArgs {
    const char* src[8];   // local source of each part
    size_t bytes[8];      // multiples of 16
    size_t dst_off[8];    // byte offset in the destination heap
    size_t parity_bytes;  // added to every offset in calls of odd epoch (double buffering), 0: none
    int parts;
    char* peer[LEV_MAX_RANKS];
    int world, me, phase;
    int* status;
};

// last block of a push: everything this rank stored is visible system-wide before any flag is
__device__ void publish(char* const* peer, int world, int me, int phase) {
    HeapHeader* mine = reinterpret_cast<HeapHeader*>(peer[me]);
    __shared__ unsigned last;
    // one system-scope fence per block, by the thread that reports the block done: after the block-wide
    // barrier it orders the stores of every thread of the block
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        last = atomicAdd(&mine->arrive, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!last) return;
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&mine->epoch[phase]) + 1u;
    if (threadIdx.x == 0) {
        mine->arrive = 0u;
        __threadfence_system();  // the other blocks' stores (observed through the counter) before the flags
    }
    __syncthreads();
    if (threadIdx.x < (unsigned)world) {
        HeapHeader* h = reinterpret_cast<HeapHeader*>(peer[threadIdx.x]);
        *reinterpret_cast<volatile unsigned*>(&h->flag[phase][me]) = epoch;
    }
}

// stores `parts` local byte ranges into every rank's heap (this rank's included), then flags
__global__ void __launch_bounds__(256) k_push(PushArgs A) {
    const size_t par = (reinterpret_cast<const HeapHeader*>(A.peer[A.me])->epoch[A.phase] & 1u) ? A.parity_bytes : 0;
    for (int part = 0; part < A.parts; part++) {
        const uint4* src = reinterpret_cast<const uint4*>(A.src[part]);
        const size_t n = A.bytes[part] / 16;
        for (int r = 0; r < A.world; r++) {
            uint4* dst = reinterpret_cast<uint4*>(A.peer[(A.me + r) % A.world] + A.dst_off[part] + par);
            for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
        }
    }
    publish(A.peer, A.world, A.me, A.phase);
}

// bounded wait of one thread for rank `src`'s flag of the round after `done`
__device__ __forceinline__ bool wait_flag(const HeapHeader* h, int phase, int src, unsigned done, int* status) {
    const long long t0 = clock64();
    for (unsigned i = 1;; i++) {
        const unsigned f = *reinterpret_cast<const volatile unsigned*>(&h->flag[phase][src]);
        if ((int)(f - (done + 1u)) >= 0) return true;
        if ((i & 63u) == 0 && clock64() - t0 > 2000000000LL) {
            atomicOr(status, LEV_DEV_TIMEOUT);
            return false;
        }
        __nanosleep(30);
    }
}

// one block: thread s waits (about one second of SM clocks at most) for rank s's flag of this phase, then
// the round counts as done
__global__ void k_wait_flags(HeapHeader* h, int world, int phase, int* status) {
    const unsigned done = *reinterpret_cast<volatile unsigned*>(&h->epoch[phase]);
    if (threadIdx.x < (unsigned)world) {
        wait_flag(h, phase, threadIdx.x, done, status);
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) h->epoch[phase] = done + 1u;
}

// wait and copy out in one launch: every block waits for the flags itself, copies its share of the heap
// region (the half of this round) to the caller's buffers, and the last block advances the round
struct WaitCopyArgs {
    char* heap;
    size_t off[8], bytes[8];   // heap offset and size of each part (multiples of 16)
    char* out[8];
    size_t parity_bytes;
    int parts, world, phase;
    int* status;
};
__global__ void __launch_bounds__(256) k_wait_copy(WaitCopyArgs A) {
    HeapHeader* h = reinterpret_cast<HeapHeader*>(A.heap);
    const unsigned done = *reinterpret_cast<volatile unsigned*>(&h->epoch[A.phase]);
    if (threadIdx.x < (unsigned)A.world) {
        wait_flag(h, A.phase, threadIdx.x, done, A.status);
        __threadfence_system();
    }
    __syncthreads();
    const size_t par = (done & 1u) ? A.parity_bytes : 0;
    for (int part = 0; part < A.parts; part++) {
        const uint4* src = reinterpret_cast<const uint4*>(A.heap + A.off[part] + par);
        uint4* dst = reinterpret_cast<uint4*>(A.out[part]);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < A.bytes[part] / 16; i += (size_t)gridDim.x * blockDim.x)
            dst[i] = __ldcv(src + i);
    }
    __shared__ unsigned last;
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&h->waited, 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (last && threadIdx.x == 0) {
        h->waited = 0u;
        h->epoch[A.phase] = done + 1u;
    }
}

struct ReturnArgs {
    const float* y_pairs;   // [pairs][hidden] by global pair id; rows of resident pairs are valid
    const int32_t* idx;     // [pairs] expert of each pair
    int64_t pairs;
    int top_k, hidden, first, count;
    int64_t tokens_local;   // tokens per rank
    size_t ret_off;         // byte offset of [tokens_local * top_k][hidden] in the owner's heap
    char* peer[LEV_MAX_RANKS];
    int world, me, phase;
};

// the output row of every pair computed here goes to the heap of the rank that owns the token
__global__ void __launch_bounds__(256) k_return_rows(ReturnArgs A) {
    const int vec = A.hidden / 4;
    for (int64_t p = blockIdx.x; p < A.pairs; p += gridDim.x) {
        const int e = A.idx[p];
        if (e < A.first || e >= A.first + A.count) continue;
        const int64_t token = p / A.top_k;
        const int slot = (int)(p - token * A.top_k);
        const int owner = (int)(token / A.tokens_local);
        const int64_t tl = token - (int64_t)owner * A.tokens_local;
        const float4* src = reinterpret_cast<const float4*>(A.y_pairs + p * A.hidden);
        float4* dst = reinterpret_cast<float4*>(A.peer[owner] + A.ret_off) + (tl * A.top_k + slot) * vec;
        for (int i = threadIdx.x; i < vec; i += blockDim.x) dst[i] = src[i];
    }
    publish(A.peer, A.world, A.me, A.phase);
}

// [tokens][rows_local] of this rank -> columns [me * rows_local, ...) of every rank's [tokens][rows_total]
struct PushColsArgs {
    const float* src;
    int64_t tokens, rows_local, rows_total;
    size_t dst_off, parity_bytes;
    char* peer[LEV_MAX_RANKS];
    int world, me, phase;
};
__global__ void __launch_bounds__(256) k_push_cols(PushColsArgs A) {
    const int64_t vec = A.rows_local / 4, total = A.tokens * vec;
    const size_t par = (reinterpret_cast<const HeapHeader*>(A.peer[A.me])->epoch[A.phase] & 1u) ? A.parity_bytes : 0;
    for (int r = 0; r < A.world; r++) {
        float* base = reinterpret_cast<float*>(A.peer[(A.me + r) % A.world] + A.dst_off + par);
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t t = i / vec, c = i - t * vec;
            reinterpret_cast<float4*>(base + t * A.rows_total + (int64_t)A.me * A.rows_local)[c] =
                reinterpret_cast<const float4*>(A.src + t * A.rows_local)[c];
        }
    }
    publish(A.peer, A.world, A.me, A.phase);
}

int push_grid(lev_ctx* ctx, size_t bytes) {
    const size_t blocks = (bytes / 16 + 255) / 256;
    const size_t cap = (size_t)ctx->prop.multiProcessorCount * 2;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

int peer_wait(lev_ctx* ctx, int phase) {
    k_wait_flags<<<1, 32, 0, ctx->stream>>>(reinterpret_cast<HeapHeader*>(ctx->dist->heap), ctx->dist->world, phase, ctx->d_status);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_wait_flags");
}

void fill_peers(lev_ctx* ctx, char** peer) {
    for (int r = 0; r < LEV_MAX_RANKS; r++) peer[r] = ctx->dist->peer[r];
}

}  // namespace

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
    d->heap = nullptr;
    d->heap_bytes = 0;
    for (int r = 0; r < LEV_MAX_RANKS; r++) d->peer[r] = nullptr;
    ctx->dist = d;
    // Peer heaps.  Every step below is taken by every rank whatever its own outcome, so that the ranks'
    // collectives stay matched; a rank that failed contributes a zero handle and all ranks fall back.
    if (world <= LEV_MAX_RANKS) {
        size_t mb = 96;
        if (const char* v = getenv("LEV_DIST_HEAP_MB")) mb = (size_t)atoll(v) > 0 ? (size_t)atoll(v) : mb;
        const size_t bytes = mb << 20;
        char* heap = nullptr;
        cudaIpcMemHandle_t mine;
        memset(&mine, 0, sizeof mine);
        bool ok = cudaMalloc((void**)&heap, bytes) == cudaSuccess;
        if (ok) ok = cudaMemsetAsync(heap, 0, kHeapHeaderBytes, ctx->stream) == cudaSuccess;
        if (ok) ok = cudaIpcGetMemHandle(&mine, heap) == cudaSuccess;
        if (!ok) {
            memset(&mine, 0, sizeof mine);
            (void)cudaGetLastError();
        }
        cudaIpcMemHandle_t* dev_handles = nullptr;
        cudaIpcMemHandle_t host_handles[LEV_MAX_RANKS];
        bool exch = cudaMalloc((void**)&dev_handles, sizeof(cudaIpcMemHandle_t) * (world + 1)) == cudaSuccess;
        if (exch) exch = cudaMemcpyAsync(dev_handles + world, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess;
        if (exch) exch = g_nccl.AllGather(dev_handles + world, dev_handles, sizeof mine, 0 /* ncclInt8 */, d->comm, ctx->stream) == 0;
        if (exch) exch = cudaMemcpyAsync(host_handles, dev_handles, sizeof mine * world, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess;
        if (exch) exch = cudaStreamSynchronize(ctx->stream) == cudaSuccess;
        if (dev_handles) cudaFree(dev_handles);
        bool all = exch && ok;
        cudaIpcMemHandle_t zero;
        memset(&zero, 0, sizeof zero);
        for (int r = 0; all && r < world; r++)
            if (memcmp(&host_handles[r], &zero, sizeof zero) == 0) all = false;
        for (int r = 0; all && r < world; r++) {
            if (r == rank) {
                d->peer[r] = heap;
            } else {
                void* p = nullptr;
                if (cudaIpcOpenMemHandle(&p, host_handles[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    (void)cudaGetLastError();
                    all = false;
                } else {
                    d->peer[r] = (char*)p;
                }
            }
        }
        if (all) {
            d->heap = heap;
            d->heap_bytes = bytes;
        } else {
            for (int r = 0; r < world; r++)
                if (r != rank && d->peer[r]) cudaIpcCloseMemHandle(d->peer[r]);
            for (int r = 0; r < LEV_MAX_RANKS; r++) d->peer[r] = nullptr;
            if (heap) cudaFree(heap);
        }
    }
    return LEV_OK;
}

extern "C" int lev_dist_peer_memory(const lev_ctx* ctx) { return ctx && ctx->dist && ctx->dist->heap ? 1 : 0; }

extern "C" int lev_dist_destroy(lev_ctx* ctx) {
    if (!ctx) return LEV_BAD_ARGUMENT;
    if (ctx->dist) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        for (int r = 0; r < ctx->dist->world && r < LEV_MAX_RANKS; r++)
            if (r != ctx->dist->rank && ctx->dist->peer[r]) cudaIpcCloseMemHandle(ctx->dist->peer[r]);
        if (ctx->dist->heap) cudaFree(ctx->dist->heap);
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
    const size_t full_bytes = (((size_t)n_cols * rt * sizeof(float)) + 255) & ~(size_t)255;
    if (ctx->dist->heap && rl % 4 == 0 && ((uintptr_t)y_full & 15) == 0 && kHeapHeaderBytes + 2 * full_bytes <= ctx->dist->heap_bytes) {
        // every rank stores its slice of each column into every rank's copy of y
        PushArgs P = {};
        P.parts = n_cols;
        for (int c = 0; c < n_cols; c++) {
            P.src[c] = (const char*)(yl + (int64_t)c * rl);
            P.bytes[c] = (size_t)rl * sizeof(float);
            P.dst_off[c] = kHeapHeaderBytes + ((size_t)c * rt + (size_t)ctx->dist->rank * rl) * sizeof(float);
        }
        P.parity_bytes = full_bytes;
        fill_peers(ctx, P.peer);
        P.world = world;
        P.me = ctx->dist->rank;
        P.phase = 2;
        P.status = ctx->d_status;
        k_push<<<push_grid(ctx, (size_t)n_cols * rl * sizeof(float)), 256, 0, ctx->stream>>>(P);
        ctx->launches++;
        LEV_CUDA(ctx, cudaGetLastError());
        WaitCopyArgs Wc = {};
        Wc.heap = ctx->dist->heap;
        Wc.parts = 1;
        Wc.off[0] = kHeapHeaderBytes;
        Wc.bytes[0] = (size_t)n_cols * rt * sizeof(float);
        Wc.out[0] = (char*)y_full;
        Wc.parity_bytes = full_bytes;
        Wc.world = world;
        Wc.phase = 2;
        Wc.status = ctx->d_status;
        k_wait_copy<<<push_grid(ctx, Wc.bytes[0]), 256, 0, ctx->stream>>>(Wc);
        ctx->launches++;
        return lev_cuda_check(ctx, cudaGetLastError(), "k_wait_copy");
    }
    // every rank owns the same number of rows; column c of rank r lands at y_full[c][r * rl ...]
    LEV_NCCL(ctx, g_nccl.GroupStart());
    for (int c = 0; c < n_cols; c++)
        LEV_NCCL(ctx, g_nccl.AllGather(yl + (int64_t)c * rl, y_full + (int64_t)c * rt, (size_t)rl, NCCL_FLOAT32,
                                      ctx->dist->comm, ctx->stream));
    LEV_NCCL(ctx, g_nccl.GroupEnd());
    return LEV_OK;
}

// A list of row-split products: ops[i].w holds this rank's rows of tensor i, ops[i].y receives the
// whole output (rows_local * world floats) on every rank.  One launch of the persistent kernel for the
// local slices, one push of all slices to all ranks, one wait-and-copy.
extern "C" int lev_matvec_chain_rowsplit(lev_ctx* ctx, int n_ops, const lev_chain_op* ops) {
    if (!ctx || !ops) return LEV_BAD_ARGUMENT;
    if (!ctx->dist) return lev_fail(ctx, LEV_BAD_ARGUMENT, "lev_dist_init has not been called");
    if (n_ops < 1 || n_ops > 8) return lev_fail(ctx, LEV_BAD_ARGUMENT, "%d ops (1...8)", n_ops);
    const int world = ctx->dist->world, rank = ctx->dist->rank;
    size_t local_bytes = 0, full_bytes = 0;
    for (int i = 0; i < n_ops; i++) {
        const lev_chain_op& o = ops[i];
        if (!o.w || !o.x || !o.y) return lev_fail(ctx, LEV_BAD_ARGUMENT, "op %d: null tensor, input or output", i);
        if (o.row0 != 0 || o.rows != o.w->rows || o.rows % 16 != 0 || o.depends || o.fusion.residual)
            return lev_fail(ctx, LEV_UNSUPPORTED, "op %d: a row-split list takes whole local tensors of whole 16-row tiles, independent, without residual", i);
        if (((uintptr_t)o.y & 15) != 0) return lev_fail(ctx, LEV_BAD_ARGUMENT, "op %d: output not 16-byte aligned", i);
        local_bytes += (size_t)o.rows * sizeof(float);
        full_bytes += (size_t)o.rows * world * sizeof(float);
    }
    full_bytes = (full_bytes + 255) & ~(size_t)255;
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    void* sl;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_DIST, local_bytes + 256, &sl));
    lev_chain_op local[8];
    size_t at = 0;
    for (int i = 0; i < n_ops; i++) {
        local[i] = ops[i];
        local[i].y = (float*)((char*)sl + at);
        at += (size_t)ops[i].rows * sizeof(float);
    }
    LEV_TRY(lev_matvec_chain(ctx, n_ops, local, 0));
    if (ctx->dist->heap && kHeapHeaderBytes + 2 * full_bytes <= ctx->dist->heap_bytes) {
        PushArgs P = {};
        WaitCopyArgs Wc = {};
        P.parts = Wc.parts = n_ops;
        size_t off = kHeapHeaderBytes;
        for (int i = 0; i < n_ops; i++) {
            const size_t lb = (size_t)ops[i].rows * sizeof(float);
            P.src[i] = (const char*)local[i].y;
            P.bytes[i] = lb;
            P.dst_off[i] = off + (size_t)rank * lb;
            Wc.off[i] = off;
            Wc.bytes[i] = lb * world;
            Wc.out[i] = (char*)ops[i].y;
            off += lb * world;
        }
        P.parity_bytes = Wc.parity_bytes = full_bytes;
        fill_peers(ctx, P.peer);
        P.world = Wc.world = world;
        P.me = rank;
        P.phase = Wc.phase = 2;
        P.status = Wc.status = ctx->d_status;
        Wc.heap = ctx->dist->heap;
        k_push<<<push_grid(ctx, local_bytes), 256, 0, ctx->stream>>>(P);
        ctx->launches++;
        LEV_CUDA(ctx, cudaGetLastError());
        k_wait_copy<<<push_grid(ctx, full_bytes), 256, 0, ctx->stream>>>(Wc);
        ctx->launches++;
        return lev_cuda_check(ctx, cudaGetLastError(), "k_wait_copy");
    }
    LEV_NCCL(ctx, g_nccl.GroupStart());
    for (int i = 0; i < n_ops; i++)
        LEV_NCCL(ctx, g_nccl.AllGather(local[i].y, ops[i].y, (size_t)ops[i].rows, NCCL_FLOAT32, ctx->dist->comm, ctx->stream));
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
    const size_t full_bytes = (part * world + 255) & ~(size_t)255;
    if (ctx->dist->heap && rl % 4 == 0 && ((uintptr_t)y_full & 15) == 0 && kHeapHeaderBytes + 2 * full_bytes <= ctx->dist->heap_bytes) {
        // the local product, then its columns go straight to their place in every rank's Y
        void* sl;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_DIST, part + 256, &sl));
        LEV_TRY(lev_gemm_prefill(ctx, w, x_bf16, tokens, (float*)sl, flags));
        PushColsArgs P = {};
        P.src = (const float*)sl;
        P.tokens = tokens;
        P.rows_local = rl;
        P.rows_total = rl * world;
        P.dst_off = kHeapHeaderBytes;
        P.parity_bytes = full_bytes;
        fill_peers(ctx, P.peer);
        P.world = world;
        P.me = ctx->dist->rank;
        P.phase = 3;
        k_push_cols<<<push_grid(ctx, part), 256, 0, ctx->stream>>>(P);
        ctx->launches++;
        LEV_CUDA(ctx, cudaGetLastError());
        WaitCopyArgs Wc = {};
        Wc.heap = ctx->dist->heap;
        Wc.parts = 1;
        Wc.off[0] = kHeapHeaderBytes;
        Wc.bytes[0] = part * world;
        Wc.out[0] = (char*)y_full;
        Wc.parity_bytes = full_bytes;
        Wc.world = world;
        Wc.phase = 3;
        Wc.status = ctx->d_status;
        k_wait_copy<<<push_grid(ctx, Wc.bytes[0]), 256, 0, ctx->stream>>>(Wc);
        ctx->launches++;
        return lev_cuda_check(ctx, cudaGetLastError(), "k_wait_copy");
    }
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
    // ---- peer-memory form: dispatch and combine by peer stores, the sum stays on the token's rank ----
    {
        const size_t xl_bytes = (size_t)tokens * w->hidden * 4, il_bytes = (size_t)tokens * top_k * 4;
        const size_t ret_bytes = ((size_t)tokens * top_k * w->hidden * 4 + 255) & ~(size_t)255;
        const size_t off_x = kHeapHeaderBytes, off_idx = off_x + xb, off_wts = off_idx + ib, off_ret = off_wts + ib;
        if (ctx->dist->heap && w->hidden % 4 == 0 && xl_bytes % 16 == 0 && il_bytes % 16 == 0 && ((uintptr_t)x & 15) == 0 &&
            off_ret + ret_bytes <= ctx->dist->heap_bytes) {
            char* heap = ctx->dist->heap;
            float* xall = (float*)(heap + off_x);
            int32_t* idx = (int32_t*)(heap + off_idx);
            float* yret = (float*)(heap + off_ret);
            void* sc;
            LEV_TRY(lev_scratch(ctx, LEV_SCR_DIST, 2 * il_bytes + sb + 1024, &sc));
            int32_t* idx_l = (int32_t*)sc;
            float* wts_l = (float*)((char*)sc + ((il_bytes + 255) & ~(size_t)255));
            float* scores = (float*)((char*)sc + 2 * ((il_bytes + 255) & ~(size_t)255));
            void* d;
            LEV_TRY(lev_scratch(ctx, LEV_SCR_MOE_D, yb + 256, &d));
            float* ypairs = (float*)d;
            LEV_TRY(lev_moe_route_dev(ctx, w, x, tokens, top_k, idx_l, wts_l, scores));
            PushArgs P = {};
            P.parts = 3;
            P.src[0] = (const char*)x;
            P.bytes[0] = xl_bytes;
            P.dst_off[0] = off_x + (size_t)rank * xl_bytes;
            P.src[1] = (const char*)idx_l;
            P.bytes[1] = il_bytes;
            P.dst_off[1] = off_idx + (size_t)rank * il_bytes;
            P.src[2] = (const char*)wts_l;
            P.bytes[2] = il_bytes;
            P.dst_off[2] = off_wts + (size_t)rank * il_bytes;
            fill_peers(ctx, P.peer);
            P.world = world;
            P.me = rank;
            P.phase = 0;
            P.status = ctx->d_status;
            k_push<<<push_grid(ctx, xl_bytes), 256, 0, ctx->stream>>>(P);
            ctx->launches++;
            LEV_CUDA(ctx, cudaGetLastError());
            LEV_TRY(peer_wait(ctx, 0));
            LEV_TRY(lev_moe_experts_dev(ctx, w, xall, tall, top_k, idx, ypairs, nullptr));
            ReturnArgs R = {};
            R.y_pairs = ypairs;
            R.idx = idx;
            R.pairs = pairs;
            R.top_k = top_k;
            R.hidden = w->hidden;
            R.first = w->local_first;
            R.count = w->local_count;
            R.tokens_local = tokens;
            R.ret_off = off_ret;
            fill_peers(ctx, R.peer);
            R.world = world;
            R.me = rank;
            R.phase = 1;
            const int rgrid = (int)(pairs < (int64_t)ctx->prop.multiProcessorCount * 4 ? pairs : (int64_t)ctx->prop.multiProcessorCount * 4);
            k_return_rows<<<rgrid < 1 ? 1 : rgrid, 256, 0, ctx->stream>>>(R);
            ctx->launches++;
            LEV_CUDA(ctx, cudaGetLastError());
            LEV_TRY(peer_wait(ctx, 1));
            // this rank's tokens: one axpy per slot in rank order, like the single-GPU layer
            LEV_TRY(lev_moe_combine_dev(ctx, yret, wts_l, tokens, top_k, w->hidden, out));
            if (idx_out) LEV_CUDA(ctx, cudaMemcpyAsync(idx_out, idx_l, il_bytes, cudaMemcpyDeviceToDevice, ctx->stream));
            if (w_out) LEV_CUDA(ctx, cudaMemcpyAsync(w_out, wts_l, il_bytes, cudaMemcpyDeviceToDevice, ctx->stream));
            return LEV_OK;
        }
    }
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
