// Single-query (decode) attention over a paged KV cache, grouped-query heads, online softmax.
//
// Semantics: g4_attn (Sources/LeviathanCore/Gemma4.swift:4412-4457): query position qpos attends to
// positions [lo, qpos], lo = qpos + 1 - window when a window is set, softmax of q.k (times `scale`,
// 1.0 in that model), output = sum softmax * v; query head h reads KV head h / (qHeads / kvHeads).
// The cache is the paged pool of attn_decode_paged (rust/crates/lev-forge/src/ops.rs:1038-1101,
// rust/crates/lev-model/src/kv.rs:36-85): pools [blocks][page][kvHeads][headDim], a block table
// [slots][max_blocks], per activation column its sequence slot and query position.  Pool elements
// are fp16 (half the bytes of the reference's f32 cache, the traffic that bounds this kernel) or f32.
//
// Work split: one thread block per (position range, KV head, column); each of its warps runs its own
// online softmax over every fourth position, a lane holding headDim/32 consecutive elements of the
// row (one 16-byte load per K or V row at headDim 256 in fp16); warps, then ranges, are merged
// with the usual max / rescale rule in a fixed order.
#include <cuda_fp16.h>

#include "lev_stream.h"
#include "lev_stream_math.cuh"

namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnUnroll = 4;
constexpr int kMaxSplits = 128;

struct AttnArgs {
    const void* k_pool;
    const void* v_pool;
    const int32_t* table;  // [slots][max_blocks]
    const int32_t* slot;   // [cols]
    const int32_t* pos;    // [cols] query position (attends to 0..pos)
    const float* q;        // [cols][q_heads][hd]
    float* out;            // [cols][q_heads][hd]
    float* part_ml;        // [cols][q_heads][splits][2]
    float* part_acc;       // [cols][q_heads][splits][hd]
    int* status;
    int page, kv_heads, q_heads, max_blocks, slots, splits, window;
    int64_t blocks;
    float scale;
};

template <typename T, int VEC>
struct Row;
template <>
struct Row<__half, 8> {
    uint4 raw;
    __device__ void load(const __half* p) { raw = __ldg(reinterpret_cast<const uint4*>(p)); }
    __device__ void get(float* f) const {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 v = __half22float2(h[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
};
template <>
struct Row<__half, 4> {
    uint2 raw;
    __device__ void load(const __half* p) { raw = __ldg(reinterpret_cast<const uint2*>(p)); }
    __device__ void get(float* f) const {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const float2 v = __half22float2(h[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
};
template <>
struct Row<float, 8> {
    float4 a, b;
    __device__ void load(const float* p) {
        a = __ldg(reinterpret_cast<const float4*>(p));
        b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    }
    __device__ void get(float* f) const {
        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    }
};
template <>
struct Row<float, 4> {
    float4 a;
    __device__ void load(const float* p) { a = __ldg(reinterpret_cast<const float4*>(p)); }
    __device__ void get(float* f) const { f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w; }
};

// column checks shared by the kernels: slot and position inside the table
__device__ __forceinline__ bool column_ok(const AttnArgs& A, int col, int* slot, int* pos) {
    *slot = A.slot[col];
    *pos = A.pos[col];
    return *slot >= 0 && *slot < A.slots && *pos >= 0 && *pos < A.max_blocks * A.page;
}

template <typename T, int VEC, int GROUP>
__global__ void __launch_bounds__(kAttnWarps * 32) k_attn_split(AttnArgs A) {
    constexpr int HD = VEC * 32;
    __shared__ float sm_m[kAttnWarps][GROUP], sm_l[kAttnWarps][GROUP];
    __shared__ float sm_acc[kAttnWarps][GROUP][HD];
    const int split = blockIdx.x, kvh = blockIdx.y, col = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    pdl_launch_dependents();
    int slot, qpos;
    if (!column_ok(A, col, &slot, &qpos)) {
        if (threadIdx.x == 0 && split == 0 && kvh == 0) atomicOr(A.status, LEV_DEV_BAD_INDEX);
        return;  // the merge kernel writes NaN for this column
    }
    const int lo = (A.window != 0 && qpos + 1 > A.window) ? qpos + 1 - A.window : 0;
    const int n = qpos + 1 - lo;
    const int begin = lo + (int)((int64_t)n * split / A.splits), end = lo + (int)((int64_t)n * (split + 1) / A.splits);
    const int32_t* trow = A.table + (int64_t)slot * A.max_blocks;
    const T* kp = static_cast<const T*>(A.k_pool);
    const T* vp = static_cast<const T*>(A.v_pool);

    float qv[GROUP][VEC];
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        const float* qh = A.q + ((int64_t)col * A.q_heads + kvh * GROUP + g) * HD + lane * VEC;
#pragma unroll
        for (int i = 0; i < VEC; i++) qv[g][i] = qh[i];
    }
    float m[GROUP], l[GROUP], acc[GROUP][VEC];
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; i++) acc[g][i] = 0.f;
    }
    bool bad = false;
    for (int base = begin + warp; base < end; base += kAttnWarps * kAttnUnroll) {
        Row<T, VEC> kr[kAttnUnroll], vr[kAttnUnroll];
        bool live[kAttnUnroll];
#pragma unroll
        for (int u = 0; u < kAttnUnroll; u++) {
            const int p = base + u * kAttnWarps;
            live[u] = p < end;
            if (live[u]) {
                const int64_t blk = trow[p / A.page];
                if (blk < 0 || blk >= A.blocks) {  // a table entry outside the pool: record it, skip the row
                    bad = true;
                    live[u] = false;
                } else {
                    const int64_t at = ((blk * A.page + p % A.page) * A.kv_heads + kvh) * HD + lane * VEC;
                    kr[u].load(kp + at);
                    vr[u].load(vp + at);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kAttnUnroll; u++) {
            if (!live[u]) continue;  // warp-uniform
            float kf[VEC], vf[VEC];
            kr[u].get(kf);
            vr[u].get(vf);
#pragma unroll
            for (int g = 0; g < GROUP; g++) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; i++) s = fmaf(qv[g][i], kf[i], s);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                s *= A.scale;
                const float m_new = fmaxf(m[g], s);
                const float corr = expf(m[g] - m_new), pw = expf(s - m_new);
                l[g] = fmaf(l[g], corr, pw);
#pragma unroll
                for (int i = 0; i < VEC; i++) acc[g][i] = fmaf(acc[g][i], corr, pw * vf[i]);
                m[g] = m_new;
            }
        }
    }
    if (bad && lane == 0) atomicOr(A.status, LEV_DEV_BAD_INDEX);
    // ---- merge the warps (fixed order) ----
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        if (lane == 0) {
            sm_m[warp][g] = m[g];
            sm_l[warp][g] = l[g];
        }
#pragma unroll
        for (int i = 0; i < VEC; i++) sm_acc[warp][g][lane * VEC + i] = acc[g][i];
    }
    __syncthreads();
    for (int item = threadIdx.x; item < GROUP * HD; item += kAttnWarps * 32) {
        const int g = item / HD, i = item - g * HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) mm = fmaxf(mm, sm_m[w][g]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) {
            const float wgt = sm_m[w][g] == -INFINITY ? 0.f : expf(sm_m[w][g] - mm);
            ll = fmaf(sm_l[w][g], wgt, ll);
            a = fmaf(sm_acc[w][g][i], wgt, a);
        }
        const int64_t ph = ((int64_t)col * A.q_heads + kvh * GROUP + g) * A.splits + split;
        A.part_acc[ph * HD + i] = a;
        if (i == 0) {
            A.part_ml[ph * 2] = mm;
            A.part_ml[ph * 2 + 1] = ll;
        }
    }
}

// out[col][head] = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M); one thread per element
__global__ void k_attn_merge(AttnArgs A, int hd) {
    __shared__ float wgt[kMaxSplits];
    __shared__ float inv_l;
    const int head = blockIdx.x, col = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    float* o = A.out + ((int64_t)col * A.q_heads + head) * hd;
    int slot, qpos;
    if (!column_ok(A, col, &slot, &qpos)) {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) o[i] = __int_as_float(0x7FC00000);
        return;
    }
    const int64_t ph = ((int64_t)col * A.q_heads + head) * A.splits;
    if (threadIdx.x == 0) {
        float mm = -INFINITY;
        for (int s = 0; s < A.splits; s++) mm = fmaxf(mm, A.part_ml[(ph + s) * 2]);
        float ll = 0.f;
        for (int s = 0; s < A.splits; s++) {
            const float ms = A.part_ml[(ph + s) * 2];
            const float w = ms == -INFINITY ? 0.f : expf(ms - mm);
            wgt[s] = w;
            ll = fmaf(A.part_ml[(ph + s) * 2 + 1], w, ll);
        }
        inv_l = 1.0f / ll;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < A.splits; s++) a = fmaf(A.part_acc[(ph + s) * hd + i], wgt[s], a);
        o[i] = a * inv_l;
    }
}

// K and V rows of each column to its position of the pool (cache append)
template <typename T>
__global__ void k_kv_append(AttnArgs A, void* k_pool, void* v_pool, const float* k, const float* v, int hd) {
    const int kvh = blockIdx.x, col = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    int slot, pos;
    bool ok = column_ok(A, col, &slot, &pos);
    int64_t blk = 0;
    if (ok) {
        blk = A.table[(int64_t)slot * A.max_blocks + pos / A.page];
        ok = blk >= 0 && blk < A.blocks;
    }
    if (!ok) {
        if (threadIdx.x == 0 && kvh == 0) atomicOr(A.status, LEV_DEV_BAD_INDEX);
        return;
    }
    const int64_t at = ((blk * A.page + pos % A.page) * A.kv_heads + kvh) * hd;
    const int64_t from = ((int64_t)col * A.kv_heads + kvh) * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        static_cast<T*>(k_pool)[at + i] = (T)k[from + i];
        static_cast<T*>(v_pool)[at + i] = (T)v[from + i];
    }
}

}  // namespace

namespace {

int check_layout(lev_ctx* ctx, const lev_kv_layout* L) {
    if (!L) return LEV_BAD_ARGUMENT;
    if (L->kv_type != LEV_KV_F16 && L->kv_type != LEV_KV_F32) return lev_fail(ctx, LEV_BAD_ARGUMENT, "cache element type %d", L->kv_type);
    if (L->head_dim != 128 && L->head_dim != 256) return lev_fail(ctx, LEV_UNSUPPORTED, "head dimension %d (128 or 256)", L->head_dim);
    if (L->page <= 0 || L->kv_heads <= 0 || L->kv_heads > 1024 || L->blocks <= 0 || L->max_blocks <= 0 || L->slots <= 0 ||
        (int64_t)L->max_blocks * L->page > (int64_t)1 << 30)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "cache layout: page %d, kvHeads %d, blocks %lld, max_blocks %d, slots %d", L->page, L->kv_heads,
                        (long long)L->blocks, L->max_blocks, L->slots);
    return LEV_OK;
}

AttnArgs base_args(lev_ctx* ctx, const lev_kv_layout* L, const int32_t* table, const int32_t* slot, const int32_t* pos) {
    AttnArgs A = {};
    A.table = table;
    A.slot = slot;
    A.pos = pos;
    A.status = ctx->d_status;
    A.page = L->page;
    A.kv_heads = L->kv_heads;
    A.max_blocks = L->max_blocks;
    A.slots = L->slots;
    A.blocks = L->blocks;
    return A;
}

template <typename T, int VEC>
cudaError_t launch_split_g(int group, dim3 grid, cudaStream_t stream, const AttnArgs& A) {
    const dim3 block(kAttnWarps * 32);
    switch (group) {
        case 1: return launch_pdl(k_attn_split<T, VEC, 1>, grid, block, 0, stream, A);
        case 2: return launch_pdl(k_attn_split<T, VEC, 2>, grid, block, 0, stream, A);
        case 4: return launch_pdl(k_attn_split<T, VEC, 4>, grid, block, 0, stream, A);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

extern "C" int lev_kv_append(lev_ctx* ctx, const lev_kv_layout* L, void* k_pool, void* v_pool, const int32_t* block_table,
                             const int32_t* slot, const int32_t* pos, int n_cols, const float* k, const float* v) {
    if (!ctx || !k_pool || !v_pool || !block_table || !slot || !pos || !k || !v) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_layout(ctx, L));
    if (n_cols < 1 || n_cols > 65535) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", n_cols);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    AttnArgs A = base_args(ctx, L, block_table, slot, pos);
    const dim3 grid(L->kv_heads, n_cols), block(L->head_dim < 256 ? L->head_dim : 256);
    if (L->kv_type == LEV_KV_F16)
        LEV_CUDA(ctx, launch_pdl(k_kv_append<__half>, grid, block, 0, ctx->stream, A, k_pool, v_pool, k, v, L->head_dim));
    else
        LEV_CUDA(ctx, launch_pdl(k_kv_append<float>, grid, block, 0, ctx->stream, A, k_pool, v_pool, k, v, L->head_dim));
    ctx->launches++;
    return LEV_OK;
}

extern "C" int lev_attn_decode(lev_ctx* ctx, const lev_kv_layout* L, const void* k_pool, const void* v_pool, const int32_t* block_table,
                               const int32_t* slot, const int32_t* pos, int n_cols, int q_heads, const float* q, int window, float scale,
                               float* out) {
    if (!ctx || !k_pool || !v_pool || !block_table || !slot || !pos || !q || !out) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_layout(ctx, L));
    if (n_cols < 1 || n_cols > 65535) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", n_cols);
    if (q_heads <= 0 || q_heads % L->kv_heads != 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%d query heads over %d KV heads", q_heads, L->kv_heads);
    const int group = q_heads / L->kv_heads;
    if (group != 1 && group != 2 && group != 4) return lev_fail(ctx, LEV_UNSUPPORTED, "%d query heads per KV head (1, 2 or 4)", group);
    if (window < 0 || !isfinite(scale)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "window %d, scale %g", window, (double)scale);
    if ((((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) != 0) return lev_fail(ctx, LEV_BAD_ARGUMENT, "cache pools are not 16-byte aligned");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    // position ranges per (column, KV head): enough thread blocks for four per SM, at least 32 positions each
    const int64_t cap = (int64_t)L->max_blocks * L->page, span = window > 0 && window < cap ? window : cap;
    int64_t splits = (4 * (int64_t)ctx->prop.multiProcessorCount + (int64_t)n_cols * L->kv_heads - 1) / ((int64_t)n_cols * L->kv_heads);
    if (splits > span / 32) splits = span / 32;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 1) splits = 1;
    const int hd = L->head_dim;
    void* scr;
    const size_t heads = (size_t)n_cols * q_heads * splits;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_ATTN, heads * (hd + 2) * sizeof(float), &scr));
    AttnArgs A = base_args(ctx, L, block_table, slot, pos);
    A.k_pool = k_pool;
    A.v_pool = v_pool;
    A.q = q;
    A.out = out;
    A.part_acc = (float*)scr;
    A.part_ml = (float*)scr + heads * hd;
    A.q_heads = q_heads;
    A.splits = (int)splits;
    A.window = window;
    A.scale = scale;
    const dim3 grid((unsigned)splits, L->kv_heads, n_cols);
    cudaError_t e;
    if (L->kv_type == LEV_KV_F16)
        e = hd == 256 ? launch_split_g<__half, 8>(group, grid, ctx->stream, A) : launch_split_g<__half, 4>(group, grid, ctx->stream, A);
    else
        e = hd == 256 ? launch_split_g<float, 8>(group, grid, ctx->stream, A) : launch_split_g<float, 4>(group, grid, ctx->stream, A);
    LEV_CUDA(ctx, e);
    LEV_CUDA(ctx, launch_pdl(k_attn_merge, dim3(q_heads, n_cols), dim3(hd), 0, ctx->stream, A, hd));
    ctx->launches += 2;
    return LEV_OK;
}
