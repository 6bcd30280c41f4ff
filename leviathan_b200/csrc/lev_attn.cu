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
// Work split: one thread block per (position range, KV head, column), ranges sized so that the grid is
// one wave of two blocks per SM; the rows of a range are staged in shared memory by asynchronous
// copies issued all at once (see k_attn_split).  Warps, then ranges, are merged with the usual
// max / rescale rule in a fixed order.
#include <cuda_fp16.h>

#include "lev_stream.h"
#include "lev_stream_math.cuh"

namespace {

constexpr int kAttnWarps = 8;
constexpr int kAttnUnroll = 4;
constexpr int kMaxSplits = 128;
constexpr int kMaxRoundPages = 128;      // block-table entries one round may span
constexpr size_t kRoundBytes = 111 * 1024;  // K and V rows of a round in shared memory: two blocks per SM

struct AttnArgs {
    const void* k_pool;
    const void* v_pool;
    const int32_t* table;  // [slots][max_blocks]
    const int32_t* slot;   // [cols]
    const int32_t* pos;    // [cols] query position (attends to 0..pos)
    const float* q;        // [cols][q_heads][hd], rows q_ld elements apart
    int64_t q_ld;
    float* out;            // [cols][q_heads][hd]
    float* part_ml;        // [cols][q_heads][splits][2]
    float* part_acc;       // [cols][q_heads][splits][hd]
    int* status;
    int* counters;  // [cols][kv_heads] ranges finished so far (zero between calls); NULL: merge in a second launch
    int page, kv_heads, q_heads, max_blocks, slots, splits, window;
    int round_cap;  // positions per round of the split kernel
    int direct;     // one range per (column, KV head): the split kernel writes the output itself
    int64_t blocks;
    float scale;
};

template <typename T, int VEC>
struct Row;
template <>
struct Row<__half, 8> {
    uint4 raw;
    __device__ void load_s(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
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
    __device__ void load_s(const __half* p) { raw = *reinterpret_cast<const uint2*>(p); }
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
    __device__ void load_s(const float* p) {
        a = *reinterpret_cast<const float4*>(p);
        b = *(reinterpret_cast<const float4*>(p) + 1);
    }
    __device__ void get(float* f) const {
        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    }
};
template <>
struct Row<float, 4> {
    float4 a;
    __device__ void load_s(const float* p) { a = *reinterpret_cast<const float4*>(p); }
    __device__ void get(float* f) const { f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w; }
};

// column checks shared by the kernels: slot and position inside the table
__device__ __forceinline__ bool column_ok(const AttnArgs& A, int col, int* slot, int* pos) {
    *slot = A.slot[col];
    *pos = A.pos[col];
    return *slot >= 0 && *slot < A.slots && *pos >= 0 && *pos < A.max_blocks * A.page;
}

// 16-byte asynchronous copy global -> shared, and its group fences
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Sums each of N (4, 8 or 16) per-lane values over the warp and leaves all N sums in every lane.
// Halving exchanges: at each step a lane keeps half of its values and adds the partner's copy of
// them, so N values cost N - 1 + log2(32 / N) shuffles instead of 5 N; the sums then go through N
// floats of shared memory.  The order of additions is fixed.
template <int N>
__device__ __forceinline__ void reduce_scores(float* v, int lane, float* sm) {
    static_assert(N == 4 || N == 8 || N == 16, "batch size");
    int width = N;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        if (width > 1) {
            const int half = width / 2;
            const bool upper = (lane & o) != 0;  // this lane keeps the upper half of what it holds
#pragma unroll
            for (int i = 0; i < N / 2; i++) {
                if (i < half) {
                    const float send = upper ? v[i] : v[i + half];
                    const float keep = upper ? v[i + half] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            width = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        }
    }
    // lane holds value number idx: bit k of idx (from the top) is the lane's choice at step k
    int idx = 0, w2 = N;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        if (w2 > 1) {
            w2 /= 2;
            if (lane & o) idx += w2;
        }
    }
    constexpr int kLow = 32 / N;  // lanes that hold the same value
    __syncwarp();
    if ((lane & (kLow - 1)) == 0) sm[idx] = v[0];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = sm[i];
    __syncwarp();
}

// The last thread block of a (column, KV head) to finish its range merges all ranges of the GROUP
// query heads: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M), ranges always in index order, so
// the result does not depend on which block came last.  Called by every thread of the block after it
// has written its own partials (the first barrier inside also ends the caller's use of `scratch`);
// blocks that are not last return at once.
template <int GROUP>
__device__ void finish_ranges(const AttnArgs& A, int col, int kvh, int hd, float* scratch) {
    // scratch: (kMaxSplits + 1) * GROUP floats of shared memory the caller no longer reads
    __shared__ int sm_last;
    float(*sm_w)[kMaxSplits] = reinterpret_cast<float(*)[kMaxSplits]>(scratch);
    float* sm_inv = scratch + GROUP * kMaxSplits;
    __threadfence();  // this block's partials are visible device-wide before the count
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(A.counters + (int64_t)col * A.kv_heads + kvh, 1);
        sm_last = prev == A.splits - 1;
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();  // the other blocks' partials, published before their counts
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // statistics, one warp per head (in turn): lanes stride the ranges
    for (int gsel = warp; gsel < GROUP; gsel += (int)(blockDim.x >> 5)) {
        const int64_t ph = ((int64_t)col * A.q_heads + kvh * GROUP + gsel) * A.splits;
        float mm = -INFINITY;
        for (int sp = lane; sp < A.splits; sp += 32) mm = fmaxf(mm, __ldcg(A.part_ml + (ph + sp) * 2));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        float ll = 0.f;
        for (int s0 = 0; s0 < A.splits; s0 += 32) {  // fixed order: blocks of 32 ranges, tree inside a block
            const int sp = s0 + lane;
            float w = 0.f, lv = 0.f;
            if (sp < A.splits) {
                const float ms = __ldcg(A.part_ml + (ph + sp) * 2);
                w = ms == -INFINITY ? 0.f : __expf(ms - mm);
                lv = __ldcg(A.part_ml + (ph + sp) * 2 + 1) * w;
                sm_w[gsel][sp] = w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lv += __shfl_xor_sync(0xffffffffu, lv, o);
            ll += lv;
        }
        if (lane == 0) sm_inv[gsel] = 1.0f / ll;
    }
    __syncthreads();
    // weighted sums: one thread per (head, four consecutive elements), eight rows in flight
    const int quads = hd >> 2;
    for (int item = threadIdx.x; item < GROUP * quads; item += blockDim.x) {
        const int gsel = item / quads, qd = item - gsel * quads;
        const int64_t ph = ((int64_t)col * A.q_heads + kvh * GROUP + gsel) * A.splits;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < A.splits; s0 += 8) {
            float4 tv[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                tv[j] = s0 + j < A.splits ? __ldcg(reinterpret_cast<const float4*>(A.part_acc + (ph + s0 + j) * hd) + qd) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float wj = s0 + j < A.splits ? sm_w[gsel][s0 + j] : 0.f;
                a.x = fmaf(tv[j].x, wj, a.x);
                a.y = fmaf(tv[j].y, wj, a.y);
                a.z = fmaf(tv[j].z, wj, a.z);
                a.w = fmaf(tv[j].w, wj, a.w);
            }
        }
        const float inv = sm_inv[gsel];
        float4* o = reinterpret_cast<float4*>(A.out + ((int64_t)col * A.q_heads + kvh * GROUP + gsel) * hd) + qd;
        *o = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
    }
    if (threadIdx.x == 0) A.counters[(int64_t)col * A.kv_heads + kvh] = 0;  // ready for the next call
}

constexpr int kStages = 4;  // copy groups per round: compute on a quarter starts when it has landed

// One thread block per (position range, KV head, column).  A range is walked in rounds of at most
// `round_cap` positions.  A round: the block-table entries of its pages go to shared memory; every
// thread then requests its share of the round's K and V rows with 16-byte asynchronous copies, all at
// once, in four groups; as each group lands the warps take its positions (warp w: positions w, w + 8,
// ...), four at a time: scores first, then one rescale of the running softmax state.  The rows of a
// round are read from HBM exactly once and never pass through registers on their way in, so the
// bytes in flight per SM are bounded by shared memory (two blocks of up to 111 KB), not registers.
template <typename T, int VEC, int GROUP>
__global__ void __launch_bounds__(kAttnWarps * 32, 2) k_attn_split(AttnArgs A) {
    constexpr int HD = VEC * 32;
    constexpr int kRowBytes = HD * (int)sizeof(T);
    constexpr int kChunksPerRow = kRowBytes / 16;
    extern __shared__ __align__(128) unsigned char attn_smem[];
    __shared__ float sm_m[kAttnWarps][GROUP], sm_l[kAttnWarps][GROUP];
    __shared__ int sm_tbl[kMaxRoundPages];
    __shared__ __align__(16) float sm_sc[kAttnWarps][16];
    const int split = blockIdx.x, kvh = blockIdx.y, col = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int round_cap = A.round_cap;
    T* ks = reinterpret_cast<T*>(attn_smem);                                     // [round_cap][HD]
    T* vs = reinterpret_cast<T*>(attn_smem + (size_t)round_cap * kRowBytes);     // [round_cap][HD]
    pdl_wait();
    pdl_launch_dependents();
    int slot, qpos;
    if (!column_ok(A, col, &slot, &qpos)) {
        if (threadIdx.x == 0 && split == 0 && kvh == 0) atomicOr(A.status, LEV_DEV_BAD_INDEX);
        if ((A.counters || A.direct) && split == 0)  // no merge launch follows: this block writes the column's NaN
            for (int i = threadIdx.x; i < GROUP * (int)HD; i += blockDim.x)
                A.out[((int64_t)col * A.q_heads + kvh * GROUP) * HD + i] = __int_as_float(0x7FC00000);
        return;  // (without counters the merge kernel writes NaN for this column)
    }
    const int lo = (A.window != 0 && qpos + 1 > A.window) ? qpos + 1 - A.window : 0;
    const int n = qpos + 1 - lo;
    const int begin = lo + (int)((int64_t)n * split / A.splits), end = lo + (int)((int64_t)n * (split + 1) / A.splits);
    const int32_t* trow = A.table + (int64_t)slot * A.max_blocks;
    const unsigned char* kp = static_cast<const unsigned char*>(A.k_pool);
    const unsigned char* vp = static_cast<const unsigned char*>(A.v_pool);

    float qv[GROUP][VEC];
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        const float* qh = A.q + (int64_t)col * A.q_ld + (int64_t)(kvh * GROUP + g) * HD + lane * VEC;
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
    // positions -> pages without a division when the page size is a power of two (the usual case)
    const int page_shift = (A.page & (A.page - 1)) == 0 ? __ffs(A.page) - 1 : -1;
    auto page_of = [&](int p) { return page_shift >= 0 ? p >> page_shift : p / A.page; };
    __shared__ int sm_any_bad;
    if (threadIdx.x == 0) sm_any_bad = 0;
    for (int r0 = begin; r0 < end; r0 += round_cap) {
        const int rn = end - r0 < round_cap ? end - r0 : round_cap;  // positions of this round
        const int page0 = page_of(r0), pages = page_of(r0 + rn - 1) - page0 + 1;
        __syncthreads();  // the previous round's rows and table entries are no longer read
        for (int j = threadIdx.x; j < pages; j += kAttnWarps * 32) {
            int e = trow[page0 + j];
            if (e < 0 || e >= A.blocks) {  // an entry outside the pool is recorded and not followed
                bad = true;
                e = -1;
                sm_any_bad = 1;
            }
            sm_tbl[j] = e;
        }
        __syncthreads();
        // ---- request every row of the round, a quarter of the positions per copy group ----
        const int per_stage = (rn + kStages - 1) / kStages;
#pragma unroll
        for (int st = 0; st < kStages; st++) {
            const int j0 = st * per_stage, j1 = j0 + per_stage < rn ? j0 + per_stage : rn;
            // a warp requests whole positions: the address is formed once, lanes take 16-byte pieces
            for (int j = j0 + warp; j < j1; j += kAttnWarps) {
                const int p = r0 + j, pg = page_of(p), e = sm_tbl[pg - page0];
                if (e < 0) continue;
                const int64_t at = LEV_KV_ROW(e, p - pg * A.page, kvh, A.page, A.kv_heads) * (int64_t)kRowBytes;
                const unsigned kd = smem_u32(ks) + (unsigned)j * kRowBytes, vd = smem_u32(vs) + (unsigned)j * kRowBytes;
#pragma unroll
                for (int c = lane; c < 2 * kChunksPerRow; c += 32) {
                    const bool is_v = c >= kChunksPerRow;
                    const int cc = is_v ? c - kChunksPerRow : c;
                    cp_async16((is_v ? vd : kd) + cc * 16, (is_v ? vp : kp) + at + cc * 16);
                }
            }
            cp_async_commit();
        }
        // ---- take the groups as they land ----
        const bool any_bad = sm_any_bad != 0;  // written before the barrier that published the table
#pragma unroll
        for (int st = 0; st < kStages; st++) {
            if (st == 0) cp_async_wait<kStages - 1>();
            if (st == 1) cp_async_wait<kStages - 2>();
            if (st == 2) cp_async_wait<kStages - 3>();
            if (st == 3) cp_async_wait<0>();
            __syncthreads();  // every thread's copies of this group are visible
            const int j0 = st * per_stage, j1 = j0 + per_stage < rn ? j0 + per_stage : rn;
            for (int jb = j0 + warp; jb < j1; jb += kAttnWarps * kAttnUnroll) {
                bool live[kAttnUnroll];
                float sc[kAttnUnroll][GROUP];
#pragma unroll
                for (int u = 0; u < kAttnUnroll; u++) {
                    const int j = jb + u * kAttnWarps;
                    live[u] = j < j1;
                    if (any_bad && live[u]) live[u] = sm_tbl[page_of(r0 + j) - page0] >= 0;
                    float kf[VEC];
                    if (live[u]) {
                        Row<T, VEC> kr;
                        kr.load_s(ks + (size_t)j * HD + lane * VEC);
                        kr.get(kf);
                    }
#pragma unroll
                    for (int g = 0; g < GROUP; g++) {
                        float d = 0.f;
                        if (live[u]) {
#pragma unroll
                            for (int i = 0; i < VEC; i++) d = fmaf(qv[g][i], kf[i], d);
                        }
                        sc[u][g] = d;
                    }
                }
                reduce_scores<kAttnUnroll * GROUP>(&sc[0][0], lane, &sm_sc[warp][0]);
#pragma unroll
                for (int g = 0; g < GROUP; g++) {
                    float m_new = m[g];
#pragma unroll
                    for (int u = 0; u < kAttnUnroll; u++) {
                        sc[u][g] = live[u] ? sc[u][g] * A.scale : -INFINITY;
                        m_new = fmaxf(m_new, sc[u][g]);
                    }
                    if (m_new == -INFINITY) continue;  // nothing live so far
                    const float corr = __expf(m[g] - m_new);  // 0 the first time (m = -inf)
                    l[g] *= corr;
#pragma unroll
                    for (int i = 0; i < VEC; i++) acc[g][i] *= corr;
#pragma unroll
                    for (int u = 0; u < kAttnUnroll; u++) sc[u][g] = __expf(sc[u][g] - m_new);  // dead rows: exp(-inf) = 0
                    m[g] = m_new;
                }
#pragma unroll
                for (int u = 0; u < kAttnUnroll; u++) {
                    if (!live[u]) continue;  // warp-uniform
                    float vf[VEC];
                    Row<T, VEC> vr;
                    vr.load_s(vs + (size_t)(jb + u * kAttnWarps) * HD + lane * VEC);
                    vr.get(vf);
#pragma unroll
                    for (int g = 0; g < GROUP; g++) {
                        l[g] += sc[u][g];
#pragma unroll
                        for (int i = 0; i < VEC; i++) acc[g][i] = fmaf(sc[u][g], vf[i], acc[g][i]);
                    }
                }
            }
        }
    }
    if (bad) atomicOr(A.status, LEV_DEV_BAD_INDEX);
    // ---- merge the warps (fixed order); the row buffer is free now and holds their sums ----
    __syncthreads();
    float* sm_acc = reinterpret_cast<float*>(attn_smem);  // [kAttnWarps][GROUP][HD]
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        if (lane == 0) {
            sm_m[warp][g] = m[g];
            sm_l[warp][g] = l[g];
        }
#pragma unroll
        for (int i = 0; i < VEC; i++) sm_acc[((size_t)warp * GROUP + g) * HD + lane * VEC + i] = acc[g][i];
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
            a = fmaf(sm_acc[((size_t)w * GROUP + g) * HD + i], wgt, a);
        }
        if (A.direct) {  // the only range of this head: no partials, no merge
            A.out[((int64_t)col * A.q_heads + kvh * GROUP + g) * HD + i] = a / ll;
            continue;
        }
        const int64_t ph = ((int64_t)col * A.q_heads + kvh * GROUP + g) * A.splits + split;
        A.part_acc[ph * HD + i] = a;
        if (i == 0) {
            A.part_ml[ph * 2] = mm;
            A.part_ml[ph * 2 + 1] = ll;
        }
    }
    if (A.counters) finish_ranges<GROUP>(A, col, kvh, HD, reinterpret_cast<float*>(attn_smem));
}

// ---------------------------------------------------------------------------
// Tensor-core form of the split kernel for fp16 caches.  The rows of the range reach shared memory by
// asynchronous copies in chunks of 32 positions, a fixed number of chunks ahead of the arithmetic, so the
// stream of a block never drains inside its range (with whole rounds requested at once and a barrier
// between rounds, 32 sequences ran at 0.61 of the copy bandwidth); the rows are consumed 16 positions at a
// time by mma.sync m16n8k16 from ldmatrix fragments:
//   scores:  S[16 positions][8 columns] = K tile [16 x headDim] . Q^T, the columns being the GROUP
//            query heads of this KV head, each as two fp16 terms (q = hi + lo * 2^-11, exact to 2^-22),
//   output:  O^T[headDim][8 columns] += V^T tile [headDim x 16] . P, P the softmax weights of the
//            batch in the same two-term form.
// The 16-byte pieces of a row sit at piece ^ (row & 7), so the eight row addresses of an ldmatrix
// fall into different banks.  Rows the copies do not fill (the tail of the last batch, rows whose
// table entry was refused) are zeroed, because 0 * garbage is not 0 in a tensor core.
// ---------------------------------------------------------------------------
constexpr int kMmaWarps = 4;
constexpr int kMmaChunk = 32;   // positions per chunk of the tensor-core kernel: two batches of 16, one copy group
// chunks in shared memory per block: two blocks share an SM (3 x 32 KB at head_dim 256, 4 x 16 KB at 128)
template <int HD>
struct MmaSlots {
    static constexpr int value = HD >= 256 ? 3 : 4;
};

__device__ __forceinline__ void ldsm_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// one of the two fp16 terms of x (x = hi + lo * 2^-11)
__device__ __forceinline__ __half split_half(float x, int term) {
    const __half hi = __float2half_rn(x);
    return term ? __float2half_rn((x - __half2float(hi)) * 2048.0f) : hi;
}
__device__ __forceinline__ unsigned pack_half2(__half a, __half b) {
    const __half2 h = __halves2half2(a, b);
    return *reinterpret_cast<const unsigned*>(&h);
}

template <int HD, int GROUP>
__global__ void __launch_bounds__(kMmaWarps * 32, 2) k_attn_split_mma(AttnArgs A) {
    constexpr int kRowBytes = HD * 2, kCpr = kRowBytes / 16, kSteps = HD / 16;
    constexpr float kLo = 4.8828125e-4f;  // 2^-11
    extern __shared__ __align__(128) unsigned char attn_smem[];
    __shared__ float sm_m[kMmaWarps][GROUP], sm_l[kMmaWarps][GROUP];
    __shared__ unsigned char sm_row_ok[MmaSlots<HD>::value][kMmaChunk];  // 1: the row was copied from the cache
    const int split = blockIdx.x, kvh = blockIdx.y, col = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    // The range is walked in chunks of kMmaChunk positions; a chunk's K rows and V rows take one slot of shared memory.
    // Copies run NS - 1 chunks ahead of the arithmetic and never drain inside a range.
    constexpr int NS = MmaSlots<HD>::value, CH = kMmaChunk;
    constexpr unsigned kSlotBytes = 2u * CH * kRowBytes;
    const unsigned smem_s = smem_u32(attn_smem);
    pdl_wait();
    pdl_launch_dependents();
    int slot, qpos;
    if (!column_ok(A, col, &slot, &qpos)) {
        if (threadIdx.x == 0 && split == 0 && kvh == 0) atomicOr(A.status, LEV_DEV_BAD_INDEX);
        if ((A.counters || A.direct) && split == 0)  // no merge launch follows: this block writes the column's NaN
            for (int i = threadIdx.x; i < GROUP * (int)HD; i += blockDim.x)
                A.out[((int64_t)col * A.q_heads + kvh * GROUP) * HD + i] = __int_as_float(0x7FC00000);
        return;  // (without counters the merge kernel writes NaN for this column)
    }
    const int lo = (A.window != 0 && qpos + 1 > A.window) ? qpos + 1 - A.window : 0;
    const int n = qpos + 1 - lo;
    const int begin = lo + (int)((int64_t)n * split / A.splits), end = lo + (int)((int64_t)n * (split + 1) / A.splits);
    const int32_t* trow = A.table + (int64_t)slot * A.max_blocks;
    const unsigned char* kp = static_cast<const unsigned char*>(A.k_pool);
    const unsigned char* vp = static_cast<const unsigned char*>(A.v_pool);

    bool bad = false;
    const int page_shift = (A.page & (A.page - 1)) == 0 ? __ffs(A.page) - 1 : -1;
    auto page_of = [&](int p) { return page_shift >= 0 ? p >> page_shift : p / A.page; };
    const int nchunks = (end - begin + CH - 1) / CH;
    // Chunk c goes into slot c % NS.  Lane l of every warp looks row l of the chunk up (table entry, byte offset in the
    // pools: one round of loads per chunk instead of one per row); the warp then requests its rows (warp, warp + 4, ...)
    // with the offsets handed round by shuffles.  Rows past the range and rows whose table entry is refused are zeroed
    // and take no part (sm_row_ok).
    static_assert(CH == 32, "one lane per row of a chunk");
    auto issue = [&](int c) {
        const int r0 = begin + c * CH;
        const int rn = end - r0 < CH ? end - r0 : CH;
        const int slot_i = c % NS;
        const unsigned ks_s = smem_s + (unsigned)slot_i * kSlotBytes, vs_s = ks_s + (unsigned)CH * kRowBytes;
        int64_t at = -1;
        if (lane < rn) {
            const int p = r0 + lane, pg = page_of(p);
            const int e = trow[pg];
            if (e < 0 || e >= A.blocks) bad = true;  // an entry outside the pool is recorded and not followed
            else at = LEV_KV_ROW(e, p - pg * A.page, kvh, A.page, A.kv_heads) * (int64_t)kRowBytes;
        }
        if (warp == 0) sm_row_ok[slot_i][lane] = at >= 0;
        const unsigned at_lo = (unsigned)at, at_hi = (unsigned)((uint64_t)at >> 32);
        const unsigned ok_rows = __ballot_sync(0xffffffffu, at >= 0);
#pragma unroll
        for (int i = 0; i < CH / kMmaWarps; i++) {
            const int j = warp + i * kMmaWarps;
            const int64_t row_at = (int64_t)(((uint64_t)__shfl_sync(0xffffffffu, at_hi, j) << 32) | __shfl_sync(0xffffffffu, at_lo, j));
            const unsigned kd = ks_s + (unsigned)j * kRowBytes, vd = vs_s + (unsigned)j * kRowBytes;
            if ((ok_rows >> j) & 1u) {
#pragma unroll
                for (int cc0 = lane; cc0 < 2 * kCpr; cc0 += 32) {
                    const bool is_v = cc0 >= kCpr;
                    const int cc = is_v ? cc0 - kCpr : cc0;
                    cp_async16((is_v ? vd : kd) + ((cc ^ (j & 7)) << 4), (is_v ? vp : kp) + row_at + cc * 16);
                }
            } else {
#pragma unroll
                for (int cc0 = lane; cc0 < 2 * kCpr; cc0 += 32) {
                    const bool is_v = cc0 >= kCpr;
                    const int cc = is_v ? cc0 - kCpr : cc0;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"((is_v ? vd : kd) + (cc << 4)), "r"(0u) : "memory");
                }
            }
        }
    };
    // one copy group per chunk, an empty one past the end: "all but the newest NS - 2" then always means chunk c
#pragma unroll
    for (int c = 0; c < NS - 1; c++) {
        if (c < nchunks) issue(c);
        cp_async_commit();
    }
    // (the first chunks are on their way while the query's fragments are formed)
    // B fragments of Q^T: column g is (head g / 2, term g % 2); this lane holds dims 2t, 2t+1, 2t+8, 2t+9 of each step
    unsigned qb[kSteps][2];
    {
        const int head = g >> 1, term = g & 1;
        const bool used = head < GROUP;
        const float* qh = A.q + (int64_t)col * A.q_ld + (int64_t)(kvh * GROUP + (used ? head : 0)) * HD;
#pragma unroll
        for (int s = 0; s < kSteps; s++) {
            const float2 a = *reinterpret_cast<const float2*>(qh + s * 16 + 2 * t);
            const float2 b = *reinterpret_cast<const float2*>(qh + s * 16 + 2 * t + 8);
            qb[s][0] = used ? pack_half2(split_half(a.x, term), split_half(a.y, term)) : 0u;
            qb[s][1] = used ? pack_half2(split_half(b.x, term), split_half(b.y, term)) : 0u;
        }
    }
    // softmax state of head t (lanes t >= GROUP carry a dummy head over zero columns)
    float m = -INFINITY, l = 0.f;
    float acc[kSteps][4];  // O^T tile mt: dims mt*16 + g (and + 8), columns 2t (hi), 2t + 1 (lo)
#pragma unroll
    for (int mt = 0; mt < kSteps; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt][i] = 0.f;
    for (int c = 0; c < nchunks; c++) {
        cp_async_wait<NS - 2>();
        __syncthreads();  // chunk c is there for every warp, and every warp is done with chunk c - 1
        if (c + NS - 1 < nchunks) issue(c + NS - 1);  // into the slot chunk c - 1 has left
        cp_async_commit();
        const int r0 = begin + c * CH;
        const int rn = end - r0 < CH ? end - r0 : CH;
        const int slot_i = c % NS;
        const unsigned ks_s = smem_s + (unsigned)slot_i * kSlotBytes, vs_s = ks_s + (unsigned)CH * kRowBytes;
        // batch b of the chunk (16 positions) belongs to warp (2 c + b) % 4: the two batches of consecutive chunks go to
        // different pairs of warps
        for (int b = 0; b < CH / 16; b++) {
            if (((2 * c + b) & (kMmaWarps - 1)) != warp) continue;
            const int j0 = b * 16;
            if (j0 >= rn) continue;
            // ---- scores of the batch ----
            float cacc[4] = {0.f, 0.f, 0.f, 0.f};
            {
                float c2[4] = {0.f, 0.f, 0.f, 0.f};  // odd steps: two shorter dependent chains
                const int mi = lane >> 3, r = lane & 7;
                const int row = j0 + (mi & 1) * 8 + r;
                const unsigned base = ks_s + (unsigned)row * kRowBytes;
#pragma unroll
                for (int st = 0; st < kSteps; st++) {
                    unsigned a0, a1, a2, a3;
                    ldsm_x4(base + (((2 * st + (mi >> 1)) ^ (row & 7)) << 4), a0, a1, a2, a3);
                    mma16816((st & 1) ? c2 : cacc, a0, a1, a2, a3, qb[st][0], qb[st][1]);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) cacc[i] += c2[i];
            }
            // this lane: positions j0 + g and j0 + g + 8 of head t
            const bool live0 = j0 + g < rn && sm_row_ok[slot_i][j0 + g] != 0;
            const bool live1 = j0 + g + 8 < rn && sm_row_ok[slot_i][j0 + g + 8] != 0;
            const float s0 = live0 ? fmaf(cacc[1], kLo, cacc[0]) * A.scale : -INFINITY;
            const float s1 = live1 ? fmaf(cacc[3], kLo, cacc[2]) * A.scale : -INFINITY;
            float bm = fmaxf(s0, s1);
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 8));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 16));
            const float m_new = fmaxf(m, bm);
            float corr = 1.f, p0 = 0.f, p1 = 0.f;
            if (m_new != -INFINITY) {
                corr = __expf(m - m_new);  // 0 the first time (m = -inf)
                p0 = __expf(s0 - m_new);   // dead rows: exp(-inf) = 0
                p1 = __expf(s1 - m_new);
            }
            m = m_new;
            l = fmaf(l, corr, p0 + p1);  // this lane's share; summed over g at the end
            // the running maxima rarely move after the first chunks: a factor of one for every head leaves the sums as they are
            if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                for (int mt = 0; mt < kSteps; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[mt][i] *= corr;
            }
            // ---- P as a B fragment: column g = (head g / 2, term g % 2), positions 2t, 2t+1, 2t+8, 2t+9 ----
            unsigned pb0, pb1;
            {
                const int head = g >> 1, term = g & 1;
                const int src_a = (2 * t) * 4 + (head & 3), src_b = (2 * t + 1) * 4 + (head & 3);
                float pa0 = __shfl_sync(0xffffffffu, p0, src_a), pb_0 = __shfl_sync(0xffffffffu, p0, src_b);
                float pa1 = __shfl_sync(0xffffffffu, p1, src_a), pb_1 = __shfl_sync(0xffffffffu, p1, src_b);
                if (head >= GROUP) pa0 = pb_0 = pa1 = pb_1 = 0.f;
                pb0 = pack_half2(split_half(pa0, term), split_half(pb_0, term));
                pb1 = pack_half2(split_half(pa1, term), split_half(pb_1, term));
            }
            // ---- O^T += V^T tile . P ----
            {
                const int mi = lane >> 3, r = lane & 7;
                const int row = j0 + (mi >> 1) * 8 + r;
                const unsigned base = vs_s + (unsigned)row * kRowBytes;
#pragma unroll
                for (int mt = 0; mt < kSteps; mt++) {
                    unsigned a0, a1, a2, a3;
                    ldsm_x4_trans(base + (((2 * mt + (mi & 1)) ^ (row & 7)) << 4), a0, a1, a2, a3);
                    mma16816(acc[mt], a0, a1, a2, a3, pb0, pb1);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (bad) atomicOr(A.status, LEV_DEV_BAD_INDEX);
    // ---- merge the warps (fixed order); the row buffer is free now and holds their sums ----
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    __syncthreads();
    float* sm_acc = reinterpret_cast<float*>(attn_smem);  // [kMmaWarps][GROUP][HD]
    if (t < GROUP) {
        if (g == 0) {
            sm_m[warp][t] = m;
            sm_l[warp][t] = l;
        }
#pragma unroll
        for (int mt = 0; mt < kSteps; mt++) {
            float* o = sm_acc + ((size_t)warp * GROUP + t) * HD + mt * 16 + g;
            o[0] = fmaf(acc[mt][1], kLo, acc[mt][0]);
            o[8] = fmaf(acc[mt][3], kLo, acc[mt][2]);
        }
    }
    __syncthreads();
    for (int item = threadIdx.x; item < GROUP * HD; item += kMmaWarps * 32) {
        const int gg = item / HD, i = item - gg * HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaWarps; w++) mm = fmaxf(mm, sm_m[w][gg]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; w++) {
            const float wgt = sm_m[w][gg] == -INFINITY ? 0.f : __expf(sm_m[w][gg] - mm);
            ll = fmaf(sm_l[w][gg], wgt, ll);
            a = fmaf(sm_acc[((size_t)w * GROUP + gg) * HD + i], wgt, a);
        }
        if (A.direct) {  // the only range of this head: no partials, no merge
            A.out[((int64_t)col * A.q_heads + kvh * GROUP + gg) * HD + i] = a / ll;
            continue;
        }
        const int64_t ph = ((int64_t)col * A.q_heads + kvh * GROUP + gg) * A.splits + split;
        A.part_acc[ph * HD + i] = a;
        if (i == 0) {
            A.part_ml[ph * 2] = mm;
            A.part_ml[ph * 2 + 1] = ll;
        }
    }
    if (A.counters) finish_ranges<GROUP>(A, col, kvh, HD, reinterpret_cast<float*>(attn_smem));
}

// out[col][head] = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M)
__global__ void k_attn_merge(AttnArgs A, int hd) {
    __shared__ float wgt[kMaxSplits];
    __shared__ float inv_l;
    const int head = blockIdx.x, col = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    float* o = A.out + ((int64_t)col * A.q_heads + head) * hd;
    const int64_t ph = ((int64_t)col * A.q_heads + head) * A.splits;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kMergeWarps = 8;
    // Requested before anything is waited for: the column's slot and position, the ranges' statistics and the first
    // eight rows this warp will add (they do not depend on the statistics), one round trip to memory instead of three.
    int slot, qpos;
    const bool col_ok = column_ok(A, col, &slot, &qpos);
    float ms = -INFINITY, ls = 0.f;
    if ((int)threadIdx.x < A.splits) {
        const float2 v = *reinterpret_cast<const float2*>(A.part_ml + (ph + threadIdx.x) * 2);
        ms = v.x;
        ls = v.y;
    }
    const int qd = blockIdx.z * 32 + lane;
    float4 first_rows[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int s2 = warp + j * kMergeWarps;
        first_rows[j] = s2 < A.splits ? *reinterpret_cast<const float4*>(A.part_acc + (ph + s2) * hd + qd * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (!col_ok) {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) o[i] = __int_as_float(0x7FC00000);
        return;
    }
    // statistics: thread s holds range s (splits <= kMaxSplits <= blockDim.x); maxima and the sum go
    // through warp shuffles and one shared array, always in the same order
    __shared__ float red[kMaxSplits / 32];
    float mm = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    if (lane == 0 && warp < kMaxSplits / 32) red[warp] = mm;
    __syncthreads();
    mm = red[0];
#pragma unroll
    for (int k = 1; k < kMaxSplits / 32; k++) mm = fmaxf(mm, red[k]);
    const float w = ms == -INFINITY ? 0.f : expf(ms - mm);
    if ((int)threadIdx.x < kMaxSplits) wgt[threadIdx.x] = w;
    float ll = ls * w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
    __syncthreads();  // everyone has read red[] as maxima
    if (lane == 0 && warp < kMaxSplits / 32) red[warp] = ll;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxSplits / 32; k++) tot += red[k];
        inv_l = 1.0f / tot;
    }
    __syncthreads();
    // weighted sum of the ranges' rows: warp w takes ranges w, w + warps, ...; a lane holds four
    // consecutive elements, so a row is read in 16-byte loads, eight rows in flight per lane
    // (blockIdx.z selects which 128 elements of the head this block sums)
    __shared__ float4 sum[kMergeWarps][32];
    const int warps = kMergeWarps;
    {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = warp; sp < A.splits; sp += warps * 8) {
            float4 t[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int s2 = sp + j * warps;
                if (sp == warp) t[j] = first_rows[j];
                else t[j] = s2 < A.splits ? *reinterpret_cast<const float4*>(A.part_acc + (ph + s2) * hd + qd * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int s2 = sp + j * warps;
                const float wj = s2 < A.splits ? wgt[s2] : 0.f;
                a.x = fmaf(t[j].x, wj, a.x);
                a.y = fmaf(t[j].y, wj, a.y);
                a.z = fmaf(t[j].z, wj, a.z);
                a.w = fmaf(t[j].w, wj, a.w);
            }
        }
        sum[warp][lane] = a;
    }
    __syncthreads();
    if (threadIdx.x < 128) {
        float a = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < kMergeWarps; w2++) a += reinterpret_cast<const float*>(&sum[w2][0])[threadIdx.x];
        o[blockIdx.z * 128 + threadIdx.x] = a * inv_l;
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
    const int64_t at = LEV_KV_ROW(blk, pos % A.page, kvh, A.page, A.kv_heads) * hd;
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

template <typename T, int VEC, int GROUP>
cudaError_t launch_split(dim3 grid, size_t smem, cudaStream_t stream, const AttnArgs& A) {
    static bool configured[16] = {};  // per device: shared-memory opt-in of this instance
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 15]) {
        cudaError_t e = cudaFuncSetAttribute(k_attn_split<T, VEC, GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRoundBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_attn_split<T, VEC, GROUP>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured[dev & 15] = true;
    }
    return launch_pdl(k_attn_split<T, VEC, GROUP>, grid, dim3(kAttnWarps * 32), smem, stream, A);
}

constexpr size_t kRoundBytesMma = 112 * 1024;  // 112 rows of K and V at headDim 256: whole 16-row batches

template <int HD, int GROUP>
cudaError_t launch_split_mma(dim3 grid, size_t smem, cudaStream_t stream, const AttnArgs& A) {
    static bool configured[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 15]) {
        cudaError_t e = cudaFuncSetAttribute(k_attn_split_mma<HD, GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRoundBytesMma);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_attn_split_mma<HD, GROUP>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured[dev & 15] = true;
    }
    return launch_pdl(k_attn_split_mma<HD, GROUP>, grid, dim3(kMmaWarps * 32), smem, stream, A);
}

template <int HD>
cudaError_t launch_split_mma_g(int group, dim3 grid, size_t smem, cudaStream_t stream, const AttnArgs& A) {
    switch (group) {
        case 1: return launch_split_mma<HD, 1>(grid, smem, stream, A);
        case 2: return launch_split_mma<HD, 2>(grid, smem, stream, A);
        case 4: return launch_split_mma<HD, 4>(grid, smem, stream, A);
    }
    return cudaErrorInvalidValue;
}

template <typename T, int VEC>
cudaError_t launch_split_g(int group, dim3 grid, size_t smem, cudaStream_t stream, const AttnArgs& A) {
    switch (group) {
        case 1: return launch_split<T, VEC, 1>(grid, smem, stream, A);
        case 2: return launch_split<T, VEC, 2>(grid, smem, stream, A);
        case 4: return launch_split<T, VEC, 4>(grid, smem, stream, A);
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
    if (!L) return LEV_BAD_ARGUMENT;
    return lev_attn_decode_ld(ctx, L, k_pool, v_pool, block_table, slot, pos, n_cols, q_heads, q, (int64_t)q_heads * L->head_dim, window, scale,
                              out);
}

// The same with the columns' query rows q_ld elements apart: q may be the leading part of each row of a fused
// [n_cols][(q_heads + 2 kv_heads) * head_dim] projection output.
extern "C" int lev_attn_decode_ld(lev_ctx* ctx, const lev_kv_layout* L, const void* k_pool, const void* v_pool, const int32_t* block_table,
                                  const int32_t* slot, const int32_t* pos, int n_cols, int q_heads, const float* q, int64_t q_ld, int window,
                                  float scale, float* out) {
    if (!ctx || !k_pool || !v_pool || !block_table || !slot || !pos || !q || !out) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_layout(ctx, L));
    if (q_ld < (int64_t)q_heads * L->head_dim || q_ld % 2 != 0 || ((uintptr_t)q & 7) != 0)
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "query rows %lld elements apart (at least %lld, even, 8-byte aligned)", (long long)q_ld,
                        (long long)q_heads * L->head_dim);
    if (n_cols < 1 || n_cols > 65535) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", n_cols);
    if (q_heads <= 0 || q_heads % L->kv_heads != 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%d query heads over %d KV heads", q_heads, L->kv_heads);
    const int group = q_heads / L->kv_heads;
    if (group != 1 && group != 2 && group != 4) return lev_fail(ctx, LEV_UNSUPPORTED, "%d query heads per KV head (1, 2 or 4)", group);
    if (window < 0 || !isfinite(scale)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "window %d, scale %g", window, (double)scale);
    if ((((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) != 0) return lev_fail(ctx, LEV_BAD_ARGUMENT, "cache pools are not 16-byte aligned");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    // position ranges per (column, KV head): one wave of two thread blocks per SM, at least 32
    // positions per range; a range is walked in rounds of what fits the shared-memory budget
    const int64_t cap = (int64_t)L->max_blocks * L->page, span = window > 0 && window < cap ? window : cap;
    const int64_t heads_kv = (int64_t)n_cols * L->kv_heads;
    int64_t splits = 2 * (int64_t)ctx->prop.multiProcessorCount / heads_kv;
    if (splits > (span + 31) / 32) splits = (span + 31) / 32;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 1) splits = 1;
    const size_t row_bytes = (size_t)L->head_dim * (L->kv_type == LEV_KV_F16 ? 2 : 4);
    int64_t round_cap = (int64_t)(kRoundBytes / (2 * row_bytes));
    if (round_cap > (span + splits - 1) / splits) round_cap = (span + splits - 1) / splits;  // the longest range
    if (round_cap > (int64_t)(kMaxRoundPages - 1) * L->page) round_cap = (int64_t)(kMaxRoundPages - 1) * L->page;
    // fp16 caches go through the tensor-core kernel: a fixed number of 32-position chunks in shared memory
    const bool use_mma = L->kv_type == LEV_KV_F16;
    size_t smem = (size_t)round_cap * 2 * row_bytes;
    if (use_mma) smem = (size_t)(L->head_dim >= 256 ? MmaSlots<256>::value : MmaSlots<128>::value) * kMmaChunk * 2 * row_bytes;
    const size_t merge_bytes = (size_t)kAttnWarps * group * L->head_dim * sizeof(float);
    if (smem < merge_bytes) smem = merge_bytes;
    const int hd = L->head_dim;
    void* scr;
    const size_t heads = (size_t)n_cols * q_heads * splits;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_ATTN, heads * (hd + 2) * sizeof(float), &scr));
    AttnArgs A = base_args(ctx, L, block_table, slot, pos);
    A.k_pool = k_pool;
    A.v_pool = v_pool;
    A.q = q;
    A.q_ld = q_ld;
    A.out = out;
    A.part_acc = (float*)scr;
    A.part_ml = (float*)scr + heads * hd;
    A.q_heads = q_heads;
    A.splits = (int)splits;
    A.round_cap = (int)round_cap;
    A.window = window;
    A.scale = scale;
    // The kernels can also let the last block of each (column, KV head) merge the ranges itself (A.counters).  No
    // call takes that form: at 4096 positions the serial tail of that block costs more than the second launch
    // (18.4 us against 16.9 us per call).
    A.direct = splits == 1;  // short windows, or enough columns to fill the GPU: no partials at all
    const bool one_launch = A.direct;
    A.counters = one_launch && !A.direct ? ctx->d_status + LEV_COUNTER_OFFSET : nullptr;
    const dim3 grid((unsigned)splits, L->kv_heads, n_cols);
    cudaError_t e;
    if (use_mma)
        e = hd == 256 ? launch_split_mma_g<256>(group, grid, smem, ctx->stream, A) : launch_split_mma_g<128>(group, grid, smem, ctx->stream, A);
    else if (L->kv_type == LEV_KV_F16)
        e = hd == 256 ? launch_split_g<__half, 8>(group, grid, smem, ctx->stream, A) : launch_split_g<__half, 4>(group, grid, smem, ctx->stream, A);
    else
        e = hd == 256 ? launch_split_g<float, 8>(group, grid, smem, ctx->stream, A) : launch_split_g<float, 4>(group, grid, smem, ctx->stream, A);
    LEV_CUDA(ctx, e);
    if (!one_launch) LEV_CUDA(ctx, launch_pdl(k_attn_merge, dim3(q_heads, n_cols, hd / 128), dim3(256), 0, ctx->stream, A, hd));
    ctx->launches += one_launch ? 1 : 2;
    return LEV_OK;
}
