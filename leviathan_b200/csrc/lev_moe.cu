// Routed mixture-of-experts composite: router decision, token->expert
// grouping, grouped expert FFN over Q4_0 weights, ordered weighted combine.
//
// Router logits.  The reference computes them with an f32 GPU kernel
// (Sources/LeviathanCore/Gemma4.swift:4160-4172) and states no CPU form, so
// the summation order is fixed here and restated term for term by the CPU
// oracle: partial p[l] (l = 0..31) accumulates elements l, l+32, l+64, ... in
// ascending order with a correctly rounded double fma; the 32 partials are
// combined by an xor butterfly (distance 16, 8, 4, 2, 1) of double adds and
// the result is rounded once to f32.
//
// Router decision (Sources/LeviathanCore/Gemma4.swift:3797-3810): m = max
// score (f32); e_i = exp(double(s_i -f32 m)); sum in ascending index order;
// p_i = e_i / sum; order by p descending, ties to the lower index; the first
// top_k; w_k = float(p_k / sum of selected p).
//
// Grouping: stable counting sort of pair ids (token*top_k + rank) by expert,
// entirely on the device, followed by a job table that cuts every expert's
// run of pairs into groups of up to `cmax` columns.  The expert FFN is then
// two grouped launches of the stream schedule (gate_up, down) driven by that
// table; no host synchronisation happens anywhere in the layer.
#include <math.h>

#include <new>

#include "lev_internal.h"
#include "lev_stream.h"
#include "lev_stream_math.cuh"

namespace {

__device__ __forceinline__ double warp_butterfly(double v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Router logits.  Summation order (the oracle states the same): lane l of a warp adds the
// products of elements l, l+32, l+64, ... in ascending order as double FMAs starting from zero,
// the 32 lane sums meet in an xor butterfly (16, 8, 4, 2, 1), one rounding to f32.
//
// Plain form: one warp per (token, 8 experts), operands straight from global memory.
__global__ void __launch_bounds__(256) k_router_logits_plain(const float* __restrict__ rw, const float* __restrict__ x,
                                                             int64_t tokens, int experts, int hidden,
                                                             float* __restrict__ scores, int* status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t tok = (int64_t)blockIdx.y * 8 + warp;
    const int e0 = blockIdx.x * 8;
    if (tok >= tokens) return;
    double acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.0;
    const float* xr = x + tok * hidden;
    for (int i = lane; i < hidden; i += 32) {
        double xv = (double)xr[i];
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (e0 + j < experts) acc[j] = fma((double)__ldg(rw + (int64_t)(e0 + j) * hidden + i), xv, acc[j]);
    }
    bool bad = false;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float s = (float)warp_butterfly(acc[j]);
        if (e0 + j < experts) {
            bad |= !isfinite(s);
            if (lane == 0) scores[tok * experts + e0 + j] = s;
        }
    }
    if (bad && lane == 0) atomicOr(status, LEV_DEV_NONFINITE_OUTPUT);
}

// Staged form: a CTA of 8 warps takes 8 experts x 8 tokens; every warp brings its expert's row
// and one token's activations into shared memory with one bulk copy each (all 16 rows are in
// flight at once: the plain form is bound by the latency of 88 dependent rounds of loads), then
// the warps share the 8 x 8 products in register tiles of 2 x 4.  Needs 16-byte aligned rows.
__global__ void __launch_bounds__(256) k_router_logits(const float* __restrict__ rw, const float* __restrict__ x,
                                                       int64_t tokens, int experts, int hidden,
                                                       float* __restrict__ scores, int* status) {
    extern __shared__ __align__(128) unsigned char rsm[];
    __shared__ __align__(8) unsigned long long bar;
    float* ws = reinterpret_cast<float*>(rsm);      // [8][hidden]
    float* xs = ws + (size_t)8 * hidden;            // [8][hidden]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.x * 8 + warp;
    const int64_t t0 = (int64_t)blockIdx.y * 8;
    const int ntok = (int)(tokens - t0 < 8 ? tokens - t0 : 8);
    const unsigned bar_s = (unsigned)__cvta_generic_to_shared(&bar);
    const unsigned row_bytes = (unsigned)hidden * 4u;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar_s), "r"(8));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();
    if (lane == 0) {
        const unsigned bytes = (e < experts ? row_bytes : 0u) + (warp < ntok ? row_bytes : 0u);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_s), "r"(bytes) : "memory");
        if (e < experts)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                             (unsigned)__cvta_generic_to_shared(ws + (size_t)warp * hidden)),
                         "l"(rw + (int64_t)e * hidden), "r"(row_bytes), "r"(bar_s)
                         : "memory");
    }
    // the router rows are constants and already on their way; the activations belong to the launch before
    pdl_launch_dependents();
    pdl_wait();
    if (lane == 0) {
        if (warp < ntok)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                             (unsigned)__cvta_generic_to_shared(xs + (size_t)warp * hidden)),
                         "l"(x + (t0 + warp) * hidden), "r"(row_bytes), "r"(bar_s)
                         : "memory");
    }
    // bounded wait for the 16 rows
    bool landed = false;
    {
        const long long t_start = clock64();
        for (unsigned i = 1; !landed; i++) {
            unsigned ok;
            asm volatile(
                "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                : "=r"(ok)
                : "r"(bar_s), "r"(0)
                : "memory");
            landed = ok != 0;
            if (!landed && (i & 63u) == 0 && clock64() - t_start > 2000000000LL) break;
        }
    }
    if (!landed) {
        if (threadIdx.x == 0) atomicOr(status, LEV_DEV_TIMEOUT);
        return;
    }
    // warp w computes experts {2a, 2a+1} x tokens {4b .. 4b+3} of the tile (a = w & 3, b = w >> 2):
    // six conversions to double and six shared-memory loads feed eight FMAs
    const int ea = 2 * (warp & 3), tb = 4 * (warp >> 2);
    const int e0 = blockIdx.x * 8 + ea;
    if (e0 >= experts || tb >= ntok) return;
    double acc[2][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.0;
    const float* w0 = ws + (size_t)ea * hidden;
    const float* x0 = xs + (size_t)tb * hidden;
    for (int i = lane; i < hidden; i += 32) {
        const double wv0 = (double)w0[i], wv1 = (double)w0[hidden + i];
#pragma unroll
        for (int b = 0; b < 4; b++) {
            if (tb + b < ntok) {
                const double xv = (double)x0[(size_t)b * hidden + i];
                acc[0][b] = fma(wv0, xv, acc[0][b]);
                acc[1][b] = fma(wv1, xv, acc[1][b]);
            }
        }
    }
    bool bad = false;
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) {
            if (tb + b < ntok && e0 + a < experts) {
                float sv = (float)warp_butterfly(acc[a][b]);
                bad |= !isfinite(sv);
                if (lane == 0) scores[(t0 + tb + b) * experts + e0 + a] = sv;
            }
        }
    if (bad && lane == 0) atomicOr(status, LEV_DEV_NONFINITE_OUTPUT);
}

// Decode form (up to four tokens): one warp, one expert.  The expert's router row is requested before the
// dependency wait (it is a constant), the tokens' rows after it; 128 experts then pull their 11 KB rows through 128
// SMs at once, where the staged form above makes 16 SMs pull 90 KB each and leaves half of its warps without work.
// Same lane order, same bits.
constexpr int kRouterWarpTokens = 4;

__global__ void __launch_bounds__(32) k_router_logits_warp(const float* __restrict__ rw, const float* __restrict__ x,
                                                           int tokens, int experts, int hidden,
                                                           float* __restrict__ scores, int* status) {
    extern __shared__ __align__(128) unsigned char rsm[];
    __shared__ __align__(8) unsigned long long bar;
    float* ws = reinterpret_cast<float*>(rsm);   // [hidden]
    float* xs = ws + hidden;                      // [tokens][hidden]
    const int lane = threadIdx.x, e = blockIdx.x;
    const unsigned bar_s = (unsigned)__cvta_generic_to_shared(&bar);
    const unsigned row_bytes = (unsigned)hidden * 4u;
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar_s), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_s), "r"(row_bytes * (unsigned)(1 + tokens)) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                         (unsigned)__cvta_generic_to_shared(ws)),
                     "l"(rw + (int64_t)e * hidden), "r"(row_bytes), "r"(bar_s)
                     : "memory");
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncwarp();
    if (lane < tokens)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                         (unsigned)__cvta_generic_to_shared(xs + (size_t)lane * hidden)),
                     "l"(x + (int64_t)lane * hidden), "r"(row_bytes), "r"(bar_s)
                     : "memory");
    bool landed = false;
    {
        const long long t_start = clock64();
        for (unsigned i = 1; !landed; i++) {
            unsigned ok;
            asm volatile(
                "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                : "=r"(ok)
                : "r"(bar_s), "r"(0)
                : "memory");
            landed = ok != 0;
            if (!landed && (i & 63u) == 0 && clock64() - t_start > 2000000000LL) break;
        }
    }
    if (!__all_sync(0xffffffffu, landed)) {
        if (lane == 0) atomicOr(status, LEV_DEV_TIMEOUT);
        return;
    }
    double acc[kRouterWarpTokens];
#pragma unroll
    for (int t = 0; t < kRouterWarpTokens; t++) acc[t] = 0.0;
    // A single token: eight columns of the lane at a time, their loads and conversions issued together, the additions
    // in ascending order (with more tokens the conversion unit is busy either way and the plain loop is as fast).
    int i = lane;
    if (tokens == 1) {
        for (; i + 7 * 32 < hidden; i += 8 * 32) {
            double wv[8], xv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                wv[u] = (double)ws[i + 32 * u];
                xv[u] = (double)xs[i + 32 * u];
            }
#pragma unroll
            for (int u = 0; u < 8; u++) acc[0] = fma(wv[u], xv[u], acc[0]);
        }
    }
    for (; i < hidden; i += 32) {
        const double wv = (double)ws[i];
#pragma unroll
        for (int t = 0; t < kRouterWarpTokens; t++)
            if (t < tokens) acc[t] = fma(wv, (double)xs[(size_t)t * hidden + i], acc[t]);
    }
    bool bad = false;
#pragma unroll
    for (int t = 0; t < kRouterWarpTokens; t++) {
        if (t < tokens) {
            const float sv = (float)warp_butterfly(acc[t]);
            bad |= !isfinite(sv);
            if (lane == 0) scores[(int64_t)t * experts + e] = sv;
        }
    }
    if (bad && lane == 0) atomicOr(status, LEV_DEV_NONFINITE_OUTPUT);
}

// Tiled form for 128 tokens or more: a CTA of 16 warps takes 16 experts x 32 tokens and walks the hidden
// dimension in chunks (two chunk buffers: the next chunk's bulk copies fly while this one is used); warp w keeps
// a 4 x 8 tile of double accumulators (experts 4 * (w & 3) ..., tokens 8 * (w >> 2) ...), so twelve conversions to
// double feed thirty-two FMAs where the 2 x 4 tile above needs six for eight.  512 tokens x 128 experts are 128
// CTAs: one wave, four warps per scheduler (the 16 x 16 tile of eight warps that preceded this form made 256 CTAs of
// one per SM, a wave and three quarters, and ran 46 us where this one runs 35 us).  A lane still adds
// its columns lane, lane + 32, ... in ascending order (chunk lengths are multiples of 32), so the bits equal the
// other forms'.
constexpr int kRouterChunk = 576;        // floats per row and chunk
constexpr int kRouterTileTokens = 32;    // 48 rows (16 experts, 32 tokens) x 2304 B x 2 buffers = 216 KB
constexpr int kRouterTileRows = 16 + kRouterTileTokens;

__global__ void __launch_bounds__(512) k_router_logits_tile(const float* __restrict__ rw, const float* __restrict__ x,
                                                            int64_t tokens, int experts, int hidden,
                                                            float* __restrict__ scores, int* status) {
    extern __shared__ __align__(128) unsigned char rsm[];
    __shared__ __align__(8) unsigned long long bars[2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e_base = blockIdx.x * 16;
    const int64_t t_base = (int64_t)blockIdx.y * kRouterTileTokens;
    const int ne = experts - e_base < 16 ? experts - e_base : 16;
    const int nt = (int)(tokens - t_base < kRouterTileTokens ? tokens - t_base : kRouterTileTokens);
    const int nchunks = (hidden + kRouterChunk - 1) / kRouterChunk;
    float* const base = reinterpret_cast<float*>(rsm);
    if (threadIdx.x == 0) {
        for (int b = 0; b < 2; b++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(&bars[b])), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    // buffer rows 0..15: the experts' chunk, rows 16..47: the tokens' chunk.  Warp 0 announces the chunk's bytes and
    // requests the expert rows (lane r: row r), warp 1 requests the token rows.
    auto request = [&](int c) {
        const int len = hidden - c * kRouterChunk < kRouterChunk ? hidden - c * kRouterChunk : kRouterChunk;
        const unsigned bar_s = (unsigned)__cvta_generic_to_shared(&bars[c & 1]);
        const float* src = nullptr;
        int row = 0;
        if (warp == 0) {
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_s), "r"((unsigned)((ne + nt) * len * 4)) : "memory");
            row = lane;
            if (lane < ne) src = rw + (int64_t)(e_base + lane) * hidden + (int64_t)c * kRouterChunk;
        } else {
            row = 16 + lane;
            if (lane < nt) src = x + (t_base + lane) * hidden + (int64_t)c * kRouterChunk;
        }
        if (src)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                             (unsigned)__cvta_generic_to_shared(base + ((size_t)(c & 1) * kRouterTileRows + row) * kRouterChunk)),
                         "l"(src), "r"((unsigned)len * 4u), "r"(bar_s)
                         : "memory");
    };
    if (warp < 2) {
        request(0);
        if (nchunks > 1) request(1);
    }
    const int ea = 4 * (warp & 3), tb = 8 * (warp >> 2);
    const bool works = ea < ne && tb < nt;
    double acc[4][8];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 8; b++) acc[a][b] = 0.0;
    for (int c = 0; c < nchunks; c++) {
        const unsigned bar_s = (unsigned)__cvta_generic_to_shared(&bars[c & 1]);
        bool landed = false;
        const long long t_start = clock64();
        for (unsigned i = 1; !landed; i++) {
            unsigned ok;
            asm volatile(
                "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                : "=r"(ok)
                : "r"(bar_s), "r"((unsigned)((c >> 1) & 1))
                : "memory");
            landed = ok != 0;
            if (!landed && (i & 63u) == 0 && clock64() - t_start > 2000000000LL) break;
        }
        if (!__syncthreads_and(landed ? 1 : 0)) {  // every thread leaves together
            if (threadIdx.x == 0) atomicOr(status, LEV_DEV_TIMEOUT);
            return;
        }
        if (works) {
            const int len = hidden - c * kRouterChunk < kRouterChunk ? hidden - c * kRouterChunk : kRouterChunk;
            const float* w0 = base + ((size_t)(c & 1) * kRouterTileRows + ea) * kRouterChunk;
            const float* x0 = base + ((size_t)(c & 1) * kRouterTileRows + 16 + tb) * kRouterChunk;
            for (int i = lane; i < len; i += 32) {
                double wv[4], xv[8];
#pragma unroll
                for (int a = 0; a < 4; a++) wv[a] = (double)w0[(size_t)a * kRouterChunk + i];
#pragma unroll
                for (int b = 0; b < 8; b++) xv[b] = (double)x0[(size_t)b * kRouterChunk + i];
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int b = 0; b < 8; b++) acc[a][b] = fma(wv[a], xv[b], acc[a][b]);
            }
        }
        __syncthreads();  // the buffer is free again
        if (warp < 2 && c + 2 < nchunks) request(c + 2);
    }
    if (!works) return;
    bool bad = false;
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const float sv = (float)warp_butterfly(acc[a][b]);
            if (ea + a < ne && tb + b < nt) {
                bad |= !isfinite(sv);
                if (lane == 0) scores[(t_base + tb + b) * experts + e_base + ea + a] = sv;
            }
        }
    if (bad && lane == 0) atomicOr(status, LEV_DEV_NONFINITE_OUTPUT);
}

// Grouping and job table, one CTA.  Experts outside [first, first+count) are
// not resident on this GPU; their pairs are left out.
struct GroupArgs {
    const int32_t* idx;  // [pairs]
    int pairs, top_k, experts, first, count, cmax;
    int32_t* counts;     // [experts]
    int32_t* offsets;    // [experts + 1]
    int32_t* perm;       // [pairs] pair ids in grouped order
    // job table (all optional)
    int* njobs;          // [1]
    int* job_slice;      // [max_jobs] local expert index
    int* job_token;      // [max_jobs][cmax] token of each column, -1 = none
    int* job_pos;        // [max_jobs][cmax] grouped position, -1 = none
    int* job_pair;       // [max_jobs][cmax] pair id, -1 = none
    int* status;
};

// one warp per token
// fuse_group (single CTA, at most 32 token-slot pairs): warp 0 also builds the grouping and the
// one-column-per-job table of k_group for these pairs, which saves a launch on the decode path
__global__ void __launch_bounds__(128) k_router_topk(const float* __restrict__ scores, int64_t tokens, int experts,
                                                     int top_k, const float* __restrict__ expert_scale,
                                                     int32_t* __restrict__ idx, float* __restrict__ weights, GroupArgs G,
                                                     int fuse_group) {
    extern __shared__ double sp[];  // [warps][experts] probabilities; selected ones are set to -1
    // With the grouping fused in, the kernels that follow read the job table before their own
    // dependency wait: they may only start when this grid has completed.
    const bool fuse = (fuse_group & 1) != 0;
    if (!fuse) pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // One block per token (fuse_group bit 1): the token's exponentials and divisions are spread over the block's four
    // warps; its sum and its selection stay with warp 0, in the same order.  Otherwise one warp per token, four tokens
    // per block: the form the fused grouping of two to four decode tokens needs, which wants them in one block.
    const bool solo = (fuse_group & 2) != 0;
    const int64_t tok = solo ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * 4 + warp;
    const bool has_token = solo || tok < tokens;
    const bool selects = solo ? warp == 0 : tok < tokens;
    const int first = solo ? (int)threadIdx.x : lane, step = solo ? (int)blockDim.x : 32;
    double* p = sp + (solo ? (size_t)0 : (size_t)warp * experts);
    __shared__ double solo_sum;
    __shared__ int sm_idx[32];
    if (has_token) {
        const float* s = scores + tok * experts;
        float m = -INFINITY;
        for (int i0 = lane; i0 < experts; i0 += 128) {  // four scores per round, requested together
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) v[j] = i0 + 32 * j < experts ? s[i0 + 32 * j] : -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) m = fmaxf(m, v[j]);
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        for (int i = first; i < experts; i += step) p[i] = exp((double)(s[i] - m));
    }
    if (solo) __syncthreads();
    else __syncwarp();
    // ascending sequential sum like the reference's reduce(0, +); the loads are issued eight at a
    // time so that only the additions are serial
    double sum = 0.0;
    if (selects) {
        if (lane == 0) {
            int i = 0;
            for (; i + 8 <= experts; i += 8) {
                double v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) v[u] = p[i + u];
#pragma unroll
                for (int u = 0; u < 8; u++) sum += v[u];
            }
            for (; i < experts; i++) sum += p[i];
            if (solo) solo_sum = sum;
        }
        sum = __shfl_sync(0xffffffffu, sum, 0);
    }
    if (solo) {
        __syncthreads();
        sum = solo_sum;
    }
    if (has_token)
        for (int i = first; i < experts; i += step) p[i] = p[i] / sum;
    if (solo) __syncthreads();
    else __syncwarp();
    if (selects) {
    double psel = 0.0, prob_sum = 0.0;  // lane k keeps the k-th selected probability (top_k <= 64: two per lane)
    double psel2 = 0.0;
    int isel = -1, isel2 = -1;
    for (int k = 0; k < top_k; k++) {
        double best = -1.0;
        int bi = 0x7fffffff;
        for (int i = lane; i < experts; i += 32) {
            double v = p[i];
            if (v > best) {  // ascending i: the first maximum is the lowest index
                best = v;
                bi = i;
            }
        }
        // The warp's maximum, ties to the lowest index: candidates are probabilities (>= 0), whose bit patterns order
        // like unsigned integers, so three warp reductions on the halves of (pattern + 1; 0 = this lane has none) and
        // on the index replace five rounds of shuffles and compares.
        {
            const unsigned long long key = bi != 0x7fffffff ? (unsigned long long)__double_as_longlong(best) + 1ull : 0ull;
            const unsigned hi = (unsigned)(key >> 32), lo = (unsigned)key;
            const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
            const unsigned ml = __reduce_max_sync(0xffffffffu, hi == mh ? lo : 0u);
            const bool wins = hi == mh && lo == ml;
            bi = (int)__reduce_min_sync(0xffffffffu, wins ? (unsigned)bi : 0x7fffffffu);
            best = (mh | ml) != 0u ? __longlong_as_double((long long)((((unsigned long long)mh << 32) | ml) - 1ull)) : -1.0;
        }
        // Non-finite scores make every probability NaN: no comparison above succeeds and bi keeps its
        // sentinel.  Record it and select a valid index (the rank) with weight zero rather than
        // follow the sentinel into shared memory.
        if (bi >= experts) {
            if (lane == 0) atomicOr(G.status, LEV_DEV_NONFINITE_OUTPUT);
            bi = k < experts ? k : 0;
            best = 0.0;
        }
        prob_sum += best;  // rank order, like topIdx.reduce
        if (lane == (k & 31)) {
            if (k < 32) {
                psel = best;
                isel = bi;
            } else {
                psel2 = best;
                isel2 = bi;
            }
        }
        if (lane == 0) p[bi] = -1.0;
        __syncwarp();
    }
    if (lane < top_k) {
        float sc = expert_scale ? expert_scale[isel] : 1.0f;
        idx[tok * top_k + lane] = isel;
        if (fuse && tok * top_k + lane < 32) sm_idx[tok * top_k + lane] = isel;  // the grouping below reads them here
        weights[tok * top_k + lane] = prob_sum > 0.0 ? __fmul_rn((float)(psel / prob_sum), sc) : 0.0f;
    }
    if (lane + 32 < top_k) {
        float sc = expert_scale ? expert_scale[isel2] : 1.0f;
        idx[tok * top_k + lane + 32] = isel2;
        weights[tok * top_k + lane + 32] = prob_sum > 0.0 ? __fmul_rn((float)(psel2 / prob_sum), sc) : 0.0f;
    }
    }
    if (!fuse) return;
    __syncthreads();  // every token's indices are written (and visible inside the CTA)
    if (warp != 0) return;
    // pair `lane`: stable position among the resident pairs ordered by (expert, pair)
    const int e = lane < G.pairs ? sm_idx[lane] : -1;
    const bool res = e >= G.first && e < G.first + G.count;
    if (lane < G.pairs && (e < 0 || e >= G.experts)) atomicOr(G.status, LEV_DEV_NONFINITE_INPUT);
    int pos = 0;
    for (int j = 0; j < G.pairs; j++) {
        const int ej = sm_idx[j];
        const bool rj = ej >= G.first && ej < G.first + G.count;
        if (rj && (ej < e || (ej == e && j < lane))) pos++;
    }
    const int total = __popc(__ballot_sync(0xffffffffu, res));
    for (int ex = lane; ex < G.experts; ex += 32) {
        int cnt = 0, before = 0;
        for (int j = 0; j < G.pairs; j++) {
            const int ej = sm_idx[j];
            const bool rj = ej >= G.first && ej < G.first + G.count;
            cnt += rj && ej == ex;
            before += rj && ej < ex;
        }
        G.counts[ex] = cnt;
        G.offsets[ex] = before;
    }
    if (lane == 0) {
        G.offsets[G.experts] = total;
        if (G.njobs) *G.njobs = total;
    }
    if (res) {
        G.perm[pos] = lane;
        if (G.job_slice) {
            G.job_slice[pos] = e - G.first;
            G.job_token[pos] = lane / G.top_k;
            G.job_pos[pos] = pos;
            G.job_pair[pos] = lane;
        }
    }
}

__global__ void __launch_bounds__(1024) k_group(GroupArgs G) {
    extern __shared__ int sh[];  // hist[experts], offs[experts + 1], jobbase[experts + 1]
    int* hist = sh;
    int* offs = sh + G.experts;
    int* jobbase = offs + G.experts + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    for (int e = tid; e < G.experts; e += blockDim.x) hist[e] = 0;
    pdl_wait();  // see k_group_fast: waits for the router, never triggers its dependents early
    __syncthreads();
    bool bad = false;
    for (int i = tid; i < G.pairs; i += blockDim.x) {
        int e = G.idx[i];
        if (e < 0 || e >= G.experts) bad = true;
        else if (e >= G.first && e < G.first + G.count) atomicAdd(&hist[e], 1);
    }
    if (bad) atomicOr(G.status, LEV_DEV_NONFINITE_INPUT);
    __syncthreads();
    if (warp == 0) {
        // exclusive scans over experts: each lane owns a contiguous run
        int per = (G.experts + 31) / 32, b = lane * per, e1 = min(b + per, G.experts);
        int s = 0, js = 0;
        for (int e = b; e < e1; e++) {
            s += hist[e];
            js += (hist[e] + G.cmax - 1) / G.cmax;
        }
        int incl = s, jincl = js;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, d), jv = __shfl_up_sync(0xffffffffu, jincl, d);
            if (lane >= d) {
                incl += v;
                jincl += jv;
            }
        }
        int run = incl - s, jrun = jincl - js;
        for (int e = b; e < e1; e++) {
            offs[e] = run;
            jobbase[e] = jrun;
            run += hist[e];
            jrun += (hist[e] + G.cmax - 1) / G.cmax;
        }
        if (lane == 31) {
            offs[G.experts] = incl;
            jobbase[G.experts] = jincl;
        }
    }
    __syncthreads();
    for (int e = tid; e < G.experts; e += blockDim.x) {
        G.counts[e] = hist[e];
        G.offsets[e] = offs[e];
    }
    if (tid == 0) {
        G.offsets[G.experts] = offs[G.experts];
        if (G.njobs) *G.njobs = jobbase[G.experts];
    }
    // stable placement: a warp walks all pairs for one expert at a time
    for (int e = G.first + warp; e < G.first + G.count; e += nwarps) {
        if (hist[e] == 0) continue;
        int base = offs[e], seen = 0;
        for (int i0 = 0; i0 < G.pairs && seen < hist[e]; i0 += 32) {
            int i = i0 + lane;
            bool hit = i < G.pairs && G.idx[i] == e;
            unsigned mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                int r = seen + __popc(mask & ((1u << lane) - 1u));
                int pos = base + r;
                G.perm[pos] = i;
                if (G.job_slice) {
                    int j = jobbase[e] + r / G.cmax, c = r % G.cmax;
                    G.job_token[j * G.cmax + c] = i / G.top_k;
                    G.job_pos[j * G.cmax + c] = pos;
                    G.job_pair[j * G.cmax + c] = i;
                }
            }
            seen += __popc(mask);
        }
        if (G.job_slice) {
            int nj = (hist[e] + G.cmax - 1) / G.cmax;
            for (int j = lane; j < nj; j += 32) G.job_slice[jobbase[e] + j] = e - G.first;
            // empty columns of the expert's last job
            int tail = nj * G.cmax - hist[e];
            if (lane < tail) {
                int j = jobbase[e] + nj - 1, c = G.cmax - 1 - lane;
                G.job_token[j * G.cmax + c] = -1;
                G.job_pos[j * G.cmax + c] = -1;
                G.job_pair[j * G.cmax + c] = -1;
            }
        }
    }
}

// Same result as k_group for pair counts whose per-chunk histograms fit shared memory: pairs are
// cut into chunks of 32 in index order; chunk histograms, a scan over chunks per expert, then
// every pair finds its stable position as offset[expert] + pairs of that expert in earlier
// chunks + earlier lanes of its own chunk.  No pass over all pairs per expert.
__global__ void __launch_bounds__(1024) k_group_fast(GroupArgs G, int nchunks) {
    extern __shared__ int sh[];  // hist[experts], offs[experts + 1], jobbase[experts + 1], ch[nchunks][experts]
    int* hist = sh;
    int* offs = sh + G.experts;
    int* jobbase = offs + G.experts + 1;
    int* ch = jobbase + G.experts + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    for (int e = tid; e < G.experts; e += blockDim.x) hist[e] = 0;
    for (int i = tid; i < nchunks * G.experts; i += blockDim.x) ch[i] = 0;
    // Launched with programmatic serialization so that the CTA is resident while the router still
    // runs.  It never triggers its own dependents early: the kernels that follow read the job
    // table before their own dependency wait and rely on this grid having completed.
    pdl_wait();
    __syncthreads();
    bool bad = false;
    for (int c = warp; c < nchunks; c += nwarps) {
        const int i = c * 32 + lane;
        if (i < G.pairs) {
            const int e = G.idx[i];
            if (e < 0 || e >= G.experts) bad = true;
            else if (e >= G.first && e < G.first + G.count) {
                atomicAdd(&ch[c * G.experts + e], 1);
                atomicAdd(&hist[e], 1);
            }
        }
    }
    if (bad) atomicOr(G.status, LEV_DEV_NONFINITE_INPUT);
    __syncthreads();
    if (warp == 0) {
        int per = (G.experts + 31) / 32, b = lane * per, e1 = min(b + per, G.experts);
        int s = 0, js = 0;
        for (int e = b; e < e1; e++) {
            s += hist[e];
            js += (hist[e] + G.cmax - 1) / G.cmax;
        }
        int incl = s, jincl = js;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, d), jv = __shfl_up_sync(0xffffffffu, jincl, d);
            if (lane >= d) {
                incl += v;
                jincl += jv;
            }
        }
        int run = incl - s, jrun = jincl - js;
        for (int e = b; e < e1; e++) {
            offs[e] = run;
            jobbase[e] = jrun;
            run += hist[e];
            jrun += (hist[e] + G.cmax - 1) / G.cmax;
        }
        if (lane == 31) {
            offs[G.experts] = incl;
            jobbase[G.experts] = jincl;
        }
    } else {
        // exclusive scan over chunks, one thread per expert
        for (int e = tid - 32; e < G.experts; e += blockDim.x - 32) {
            int run = 0;
            for (int c = 0; c < nchunks; c++) {
                const int v = ch[c * G.experts + e];
                ch[c * G.experts + e] = run;
                run += v;
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < G.experts; e += blockDim.x) {
        G.counts[e] = hist[e];
        G.offsets[e] = offs[e];
        if (G.job_slice && e >= G.first && e < G.first + G.count) {
            const int nj = (hist[e] + G.cmax - 1) / G.cmax;
            for (int j = 0; j < nj; j++) G.job_slice[jobbase[e] + j] = e - G.first;
            // empty columns of the expert's last job (wide jobs, which only the grouped GEMM uses, are
            // described by their first position and the expert's count: their tails are not filled)
            for (int r = hist[e]; r < nj * G.cmax && G.cmax <= 8; r++) {
                const int q = (jobbase[e] + nj - 1) * G.cmax + (r - (nj - 1) * G.cmax);
                G.job_token[q] = -1;
                G.job_pos[q] = -1;
                G.job_pair[q] = -1;
            }
        }
    }
    if (tid == 0) {
        G.offsets[G.experts] = offs[G.experts];
        if (G.njobs) *G.njobs = jobbase[G.experts];
    }
    for (int c = warp; c < nchunks; c += nwarps) {
        const int i = c * 32 + lane;
        int e = -1 - lane;  // lanes without a resident pair match nobody
        if (i < G.pairs) {
            const int v = G.idx[i];
            if (v >= G.first && v < G.first + G.count && v < G.experts) e = v;
        }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const int r = ch[c * G.experts + e] + __popc(same & ((1u << lane) - 1u));
            const int pos = offs[e] + r;
            G.perm[pos] = i;
            if (G.job_slice) {
                const int q = (jobbase[e] + r / G.cmax) * G.cmax + r % G.cmax;
                G.job_token[q] = i / G.top_k;
                G.job_pos[q] = pos;
                G.job_pair[q] = i;
            }
        }
    }
}

// out[t][h] = sum_k w[t][k] * y[t][k][h]: a separate multiply and add per
// slot in rank order from zero (Sources/LeviathanCore/Gemma4.swift:4459-4466)
// residual != NULL: out = residual + alpha * sum, the bits of lev_axpy applied to the plain sum (out may be residual)
__global__ void k_combine(const float* __restrict__ y, const float* __restrict__ w, int64_t tokens, int top_k,
                          int hidden, float* out, const int32_t* __restrict__ idx, int first, int count,
                          const float* residual, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    int64_t total = tokens * hidden;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t t = i / hidden;
        int h = (int)(i - t * hidden);
        float acc = 0.f;
        const float rv = residual ? residual[i] : 0.f;
        // eight slots at a time: their loads are requested together, the additions stay in slot order
        for (int k0 = 0; k0 < top_k; k0 += 8) {
            float wv[8], yv[8];
            bool use[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int k = k0 + j;
                // expert-parallel partial: slots whose expert lives on another GPU were never computed here
                use[j] = k < top_k;
                if (use[j] && idx) {
                    const int e = idx[t * top_k + k];
                    use[j] = e >= first && e < first + count;
                }
                wv[j] = use[j] ? w[t * top_k + k] : 0.f;
                yv[j] = use[j] ? y[(t * top_k + k) * hidden + h] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (use[j]) acc = __fadd_rn(acc, __fmul_rn(wv[j], yv[j]));
        }
        out[i] = residual ? fmaf(alpha, acc, rv) : acc;
    }
}

int grid_for(lev_ctx* ctx, int64_t n, int block, int per_sm) {
    int64_t g = (n + block - 1) / block, cap = (int64_t)ctx->prop.multiProcessorCount * per_sm;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

int check_tokens(lev_ctx* ctx, const lev_moe_weights* w, int64_t tokens, int top_k) {
    if (tokens <= 0 || tokens > (1 << 20)) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "tokens %lld", (long long)tokens);
    if (top_k <= 0 || top_k > LEV_MAX_TOP_K || top_k > w->experts)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "topK %d with %d experts", top_k, w->experts);
    return LEV_OK;
}

}  // namespace

// ---------------------------------------------------------------------------
// weights
// ---------------------------------------------------------------------------
extern "C" int lev_moe_weights_upload(lev_ctx* ctx, const float* router_w, const uint8_t* gu, size_t gu_bytes,
                                      const uint8_t* dn, size_t dn_bytes, int experts, int hidden, int inter,
                                      int local_first, int local_count, int on_device, lev_moe_weights** out) {
    if (!ctx || !out) return LEV_BAD_ARGUMENT;
    *out = nullptr;
    // region bounds of Sources/LeviathanCore/MoELowering.swift (dims <= 8192, multiples of 32)
    if (hidden <= 0 || inter <= 0 || hidden % 32 || inter % 32 || hidden > 8192 || inter > 8192)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "hidden %d, expertIntermediate %d", hidden, inter);
    if (experts <= 0 || experts > LEV_MAX_EXPERTS || local_first < 0 || local_count <= 0 || local_first + local_count > experts)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "experts %d, local [%d, +%d)", experts, local_first, local_count);
    size_t gu_stride = (size_t)(2 * inter) * (hidden / 32) * 18, dn_stride = (size_t)hidden * (inter / 32) * 18;
    if (gu_bytes != gu_stride * local_count || dn_bytes != dn_stride * local_count)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "packed slice sizes do not match the shape (%zu / %zu bytes, need %zu / %zu)",
                        gu_bytes, dn_bytes, gu_stride * local_count, dn_stride * local_count);
    if (!router_w || !gu || !dn) return lev_fail(ctx, LEV_BAD_ARGUMENT, "null weights");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    lev_moe_weights* w = new (std::nothrow) lev_moe_weights();
    if (!w) return lev_fail(ctx, LEV_OUT_OF_MEMORY, "host allocation");
    memset(w, 0, sizeof *w);
    w->experts = experts;
    w->hidden = hidden;
    w->inter = inter;
    w->local_first = local_first;
    w->local_count = local_count;
    size_t rb = (size_t)experts * hidden * sizeof(float);
    int st = lev_cuda_check(ctx, cudaMalloc((void**)&w->router_w, rb), "cudaMalloc(router)");
    if (!st)
        st = lev_cuda_check(ctx,
                            cudaMemcpyAsync(w->router_w, router_w, rb,
                                            on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream),
                            "copy router");
    if (!st) st = lev_weights_create(ctx, gu, gu_bytes, LEV_GGML_Q4_0, (int64_t)local_count * 2 * inter, hidden, on_device, true, &w->gate_up);
    if (!st) st = lev_weights_create(ctx, dn, dn_bytes, LEV_GGML_Q4_0, (int64_t)local_count * hidden, inter, on_device, true, &w->down);
    if (!st) st = lev_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "sync");
    if (st) {
        lev_moe_weights_free(ctx, w);
        return st;
    }
    *out = w;
    return LEV_OK;
}

// Drops the GGUF-order copies of the expert tensors.  The decode-sized forms of the layer (below 512 token-slot
// pairs) read the repacked copies only; the tensor-core form reads the GGUF bytes, so a layer released here
// runs larger batches through the multi-column stream kernels instead.
extern "C" int lev_moe_weights_release_gguf(lev_ctx* ctx, lev_moe_weights* w) {
    if (!ctx || !w || !w->gate_up || !w->down) return LEV_BAD_ARGUMENT;
    LEV_TRY(lev_weights_release_gguf(ctx, w->gate_up));
    return lev_weights_release_gguf(ctx, w->down);
}

extern "C" int lev_moe_weights_free(lev_ctx* ctx, lev_moe_weights* w) {
    if (!ctx || !w) return LEV_BAD_ARGUMENT;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (w->router_w) cudaFree(w->router_w);
    if (w->gate_up) lev_weights_free(ctx, w->gate_up);
    if (w->down) lev_weights_free(ctx, w->down);
    delete w;
    return LEV_OK;
}

// ---------------------------------------------------------------------------
// device-pointer stages
// ---------------------------------------------------------------------------
static int route_dev_impl(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, int32_t* idx,
                          float* weights, float* scores, const GroupArgs* fuse);

int lev_moe_route_dev(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, int32_t* idx,
                     float* weights, float* scores) {
    return route_dev_impl(ctx, w, x, tokens, top_k, idx, weights, scores, nullptr);
}

static int route_dev_impl(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, int32_t* idx,
                          float* weights, float* scores, const GroupArgs* fuse) {
    if ((tokens + 7) / 8 > 65535) return lev_fail(ctx, LEV_EXCEEDS_WORKLOAD, "%lld tokens in one routing call (at most 524280)", (long long)tokens);
    dim3 grid((unsigned)((w->experts + 7) / 8), (unsigned)((tokens + 7) / 8));
    const size_t stage = (size_t)16 * w->hidden * sizeof(float);
    const bool aligned = w->hidden % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w->router_w & 15) == 0;
    if (aligned && tokens >= 128) {   // below that the tiles are too few to cover the SMs and the 8 x 8 form is the faster one
        const size_t tile_smem = (size_t)2 * kRouterTileRows * kRouterChunk * sizeof(float);
        static bool configured_tile[16] = {};
        if (!configured_tile[ctx->device & 15]) {
            LEV_CUDA(ctx, cudaFuncSetAttribute(k_router_logits_tile, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem));
            configured_tile[ctx->device & 15] = true;
        }
        dim3 tgrid((unsigned)((w->experts + 15) / 16), (unsigned)((tokens + kRouterTileTokens - 1) / kRouterTileTokens));
        LEV_CUDA(ctx, launch_pdl(k_router_logits_tile, tgrid, dim3(512), tile_smem, ctx->stream, (const float*)w->router_w, x, tokens,
                                 (int)w->experts, (int)w->hidden, scores, ctx->d_status));
    } else if (aligned && tokens <= kRouterWarpTokens && (size_t)(1 + tokens) * w->hidden * sizeof(float) <= 200 * 1024) {
        const size_t warp_smem = (size_t)(1 + tokens) * w->hidden * sizeof(float);
        static bool configured_warp[16] = {};
        if (!configured_warp[ctx->device & 15]) {
            LEV_CUDA(ctx, cudaFuncSetAttribute(k_router_logits_warp, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            configured_warp[ctx->device & 15] = true;
        }
        LEV_CUDA(ctx, launch_pdl(k_router_logits_warp, dim3((unsigned)w->experts), dim3(32), warp_smem, ctx->stream, (const float*)w->router_w, x,
                                 (int)tokens, (int)w->experts, (int)w->hidden, scores, ctx->d_status));
    } else if (stage <= 200 * 1024 && aligned) {
        static bool configured[16] = {};
        if (!configured[ctx->device & 15]) {
            LEV_CUDA(ctx, cudaFuncSetAttribute(k_router_logits, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            configured[ctx->device & 15] = true;
        }
        LEV_CUDA(ctx, launch_pdl(k_router_logits, grid, dim3(256), stage, ctx->stream, (const float*)w->router_w, x, tokens,
                                 (int)w->experts, (int)w->hidden, scores, ctx->d_status));
    } else {
        k_router_logits_plain<<<grid, 256, 0, ctx->stream>>>(w->router_w, x, tokens, w->experts, w->hidden, scores, ctx->d_status);
    }
    ctx->launches++;
    LEV_CUDA(ctx, cudaGetLastError());
    size_t smem = (size_t)4 * w->experts * sizeof(double);
    GroupArgs G = {};
    if (fuse) G = *fuse;
    G.status = ctx->d_status;  // the selection loop reports non-finite scores there
    static_assert((size_t)4 * LEV_MAX_EXPERTS * sizeof(double) <= 48 * 1024, "k_router_topk runs without a shared-memory opt-in");
    // one block per token, except where the fused grouping needs two to four tokens in one block
    const bool per_token = tokens == 1 || !fuse;
    LEV_CUDA(ctx, launch_pdl(k_router_topk, dim3((unsigned)(per_token ? tokens : (tokens + 3) / 4)), dim3(128), smem, ctx->stream,
                             (const float*)scores, tokens, (int)w->experts, top_k, (const float*)nullptr, idx, weights, G,
                             (fuse ? 1 : 0) | (per_token ? 2 : 0)));
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_router_topk");
}

// grouped dequant-GEMM on the tensor cores (lev_gemm_tc.cu)
bool lev_gemm_grouped_supported(const lev_weights* w, int rows_per_expert);
int lev_gemm_grouped_job_tokens(void);
int lev_gemm_grouped_run(lev_ctx* ctx, const lev_weights* w, int rows_per_expert, const void* xg_bf16, int64_t capacity_rows,
                         int max_jobs, const int* njobs, const int* job_slice, const int* job_pos, const int* offsets,
                         int first_expert, const int* out_row, float* out, int64_t out_ld);
int lev_gather_bf16(lev_ctx* ctx, const float* x, const int* perm, const int* total_pos, int64_t max_pos, int top_k, int cols,
                    void* out_bf16);
int lev_act_grouped_bf16(lev_ctx* ctx, const float* gu, const int* total_pos, int64_t max_pos, int inter, void* out_bf16);

struct JobTable {
    int cmax, max_jobs;
    int *njobs, *job_slice, *job_token, *job_pos, *job_pair;
};

static int group_dev(lev_ctx* ctx, const int32_t* idx, int64_t tokens, int top_k, int experts, int first, int count,
                     int32_t* counts, int32_t* offsets, int32_t* perm, JobTable* jt) {
    GroupArgs G;
    G.idx = idx;
    G.pairs = (int)(tokens * top_k);
    G.top_k = top_k;
    G.experts = experts;
    G.first = first;
    G.count = count;
    G.cmax = jt ? jt->cmax : 1;
    G.counts = counts;
    G.offsets = offsets;
    G.perm = perm;
    G.njobs = jt ? jt->njobs : nullptr;
    G.job_slice = jt ? jt->job_slice : nullptr;
    G.job_token = jt ? jt->job_token : nullptr;
    G.job_pos = jt ? jt->job_pos : nullptr;
    G.job_pair = jt ? jt->job_pair : nullptr;
    G.status = ctx->d_status;
    size_t smem = (size_t)(3 * experts + 2) * sizeof(int);
    const int nchunks = (G.pairs + 31) / 32;
    const size_t fast = smem + (size_t)nchunks * experts * sizeof(int);
    if (nchunks > 0 && fast <= 160 * 1024) {
        static bool configured[16] = {};
        if (!configured[ctx->device & 15]) {
            LEV_CUDA(ctx, cudaFuncSetAttribute(k_group_fast, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
            configured[ctx->device & 15] = true;
        }
        LEV_CUDA(ctx, launch_pdl(k_group_fast, dim3(1), dim3(1024), fast, ctx->stream, G, nchunks));
    } else {
        LEV_CUDA(ctx, launch_pdl(k_group, dim3(1), dim3(1024), smem, ctx->stream, G));
    }
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_group");
}

static int lev_moe_launch_act(lev_ctx* ctx, const float* gu, const int* perm, const int* total_pos, int64_t pairs,
                              int inter, float* act);

// expert FFN for the pairs whose experts are resident; y_pairs is [pairs][hidden]
// indexed by pair id (token*top_k + rank); act_out (optional) likewise [pairs][inter]
static int experts_dev_impl(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                            const int32_t* idx, float* y_pairs, float* act_out, bool pre_grouped);

int lev_moe_experts_dev(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                       const int32_t* idx, float* y_pairs, float* act_out) {
    return experts_dev_impl(ctx, w, x, tokens, top_k, idx, y_pairs, act_out, false);
}

// decode-sized calls run one job per (token, slot) pair on the one-launch kernel
static bool moe_sliced(lev_ctx* ctx, const lev_moe_weights* w, int64_t pairs, const float* x) {
    const int64_t gu_rows = 2 * (int64_t)w->inter;
    return pairs <= 64 && lev_dense_jobs_supported(ctx, w->gate_up, gu_rows, (int)pairs, 1, x, w->hidden) &&
           lev_dense_jobs_supported(ctx, w->down, w->hidden, (int)pairs, 1, x, gu_rows);
}

// mid-sized calls: one job per expert and up to four of its tokens, still on the one-launch kernel
static bool moe_sliced4(lev_ctx* ctx, const lev_moe_weights* w, int64_t pairs, const float* x) {
    const int64_t gu_rows = 2 * (int64_t)w->inter;
    int64_t mj = (int64_t)w->local_count + pairs / 4;
    if (mj > pairs) mj = pairs;
    return lev_dense_jobs_supported(ctx, w->gate_up, gu_rows, (int)mj, 4, x, w->hidden) &&
           lev_dense_jobs_supported(ctx, w->down, w->hidden, (int)mj, 4, x, gu_rows);
}

// the grouping tables of a call inside the context's scratch (same layout for the same arguments)
static int group_tables(lev_ctx* ctx, const lev_moe_weights* w, int64_t pairs, int cmax, int max_jobs, int32_t** counts,
                        int32_t** offsets, int32_t** perm, JobTable* jt) {
    size_t ints = (size_t)w->experts * 2 + 1 + pairs + 1 + max_jobs + (size_t)3 * max_jobs * cmax + 64;
    void* gb;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_MOE_B, ints * sizeof(int), &gb));
    int* p = (int*)gb;
    *counts = p;
    p += w->experts;
    *offsets = p;
    p += w->experts + 1;
    *perm = p;
    p += pairs;
    jt->cmax = cmax;
    jt->max_jobs = max_jobs;
    jt->njobs = p;
    p += 1;
    jt->job_slice = p;
    p += max_jobs;
    jt->job_token = p;
    p += (size_t)max_jobs * cmax;
    jt->job_pos = p;
    p += (size_t)max_jobs * cmax;
    jt->job_pair = p;
    return LEV_OK;
}

static int experts_dev_impl(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                            const int32_t* idx, float* y_pairs, float* act_out, bool pre_grouped) {
    const int64_t pairs = tokens * top_k;
    const int64_t gu_rows_ = 2 * (int64_t)w->inter;
    // decode-sized calls: one job per (token, slot) pair on the one-launch kernel, whose CTAs
    // build their activation tables themselves (no preparation launches, no table memory)
    const bool sliced = moe_sliced(ctx, w, pairs, x);
    // prefill-sized calls: grouped dequant-GEMM on the tensor cores (bf16 operands, f32 accumulate;
    // the 2e-2 bar of tensor-core prefill applies to this form)
    // Mid-sized calls (one job per expert and four of its tokens) take the one-launch kernel as far as its tables
    // allow -- 84 tokens of the 128-expert top-8 shape: 180 us at 64 tokens, 222 at 84, where the grouped GEMM costs a
    // flat 300 us up to about 128 tokens -- and from 1024 pairs on the GEMM is preferred wherever it applies.
    const bool sliced4_early = !sliced && pairs < 1024 && moe_sliced4(ctx, w, pairs, x);
    const int64_t min_pairs = 512;
    const bool tensor = !sliced && !sliced4_early && pairs >= min_pairs && w->hidden % 4 == 0 && lev_gemm_grouped_supported(w->gate_up, (int)gu_rows_) &&
                        lev_gemm_grouped_supported(w->down, w->hidden);
    const bool sliced4 = sliced4_early || (!sliced && !tensor && moe_sliced4(ctx, w, pairs, x));
    const int cmax = sliced ? 1 : tensor ? lev_gemm_grouped_job_tokens() : sliced4 ? 4 : (pairs <= 2 * (int64_t)w->local_count ? 4 : 8), terms = 2;
    int64_t mj = (int64_t)w->local_count + pairs / cmax;
    if (mj > pairs) mj = pairs;
    const int max_jobs = (int)mj;

    // grouping tables
    int32_t *counts, *offsets, *perm;
    JobTable jt;
    LEV_TRY(group_tables(ctx, w, pairs, cmax, max_jobs, &counts, &offsets, &perm, &jt));
    if (!pre_grouped)
        LEV_TRY(group_dev(ctx, idx, tokens, top_k, w->experts, w->local_first, w->local_count, counts, offsets, perm, &jt));

    // gate_up: columns = tokens of each job, outputs in grouped order [pos][2*inter]
    const int64_t gu_rows = 2 * (int64_t)w->inter;
    size_t tb_gu = lev_stream_table_bytes(w->gate_up, cmax, terms, max_jobs, nullptr);
    size_t tb_dn = lev_stream_table_bytes(w->down, cmax, terms, max_jobs, nullptr);
    size_t tb = tb_gu > tb_dn ? tb_gu : tb_dn;
    size_t gu_bytes = ((size_t)pairs * gu_rows * sizeof(float) + 255) & ~(size_t)255;
    if (tensor) tb = (((size_t)pairs * w->hidden * 2 + 255) & ~(size_t)255) + (((size_t)pairs * w->inter * 2 + 255) & ~(size_t)255);
    void* cb;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_MOE_C, gu_bytes + tb + 256, &cb));
    float* gu = (float*)cb;
    void* tables = (char*)cb + gu_bytes;
    if (tensor) {
        void* xg = tables;
        void* actg = (char*)tables + (((size_t)pairs * w->hidden * 2 + 255) & ~(size_t)255);
        const int* total_pos = offsets + w->experts;
        LEV_TRY(lev_gather_bf16(ctx, x, perm, total_pos, pairs, top_k, w->hidden, xg));
        LEV_TRY(lev_gemm_grouped_run(ctx, w->gate_up, (int)gu_rows, xg, pairs, max_jobs, jt.njobs, jt.job_slice, jt.job_pos, offsets,
                                     w->local_first, nullptr, gu, gu_rows));
        LEV_TRY(lev_act_grouped_bf16(ctx, gu, total_pos, pairs, w->inter, actg));
        LEV_TRY(lev_gemm_grouped_run(ctx, w->down, w->hidden, actg, pairs, max_jobs, jt.njobs, jt.job_slice, jt.job_pos, offsets,
                                     w->local_first, perm, y_pairs, w->hidden));
        if (act_out) LEV_TRY(lev_moe_launch_act(ctx, gu, perm, offsets + w->experts, pairs, w->inter, act_out));
        return LEV_OK;
    }
    if (sliced || sliced4) {
        LEV_TRY(lev_dense_jobs_run(ctx, w->gate_up, gu_rows, max_jobs, cmax, jt.njobs, jt.job_slice, jt.job_token, jt.job_pos, x,
                                   w->hidden, 0, gu, gu_rows));
        LEV_TRY(lev_dense_jobs_run(ctx, w->down, w->hidden, max_jobs, cmax, jt.njobs, jt.job_slice, jt.job_pos, jt.job_pair, gu,
                                   gu_rows, w->inter, y_pairs, w->hidden));
        if (act_out) LEV_TRY(lev_moe_launch_act(ctx, gu, perm, offsets + w->experts, pairs, w->inter, act_out));
        return LEV_OK;
    }

    lev_stream_source src = {};
    src.x = x;
    src.ld = w->hidden;
    src.rowmap = jt.job_token;
    src.njobs_dev = jt.njobs;
    LEV_TRY(lev_stream_prepare(ctx, w->gate_up, src, cmax, terms, max_jobs, tables));
    lev_stream_job J = {};
    J.rows = gu_rows;
    J.out_ld = gu_rows;
    J.max_jobs = max_jobs;
    J.njobs_dev = jt.njobs;
    J.job_slice = jt.job_slice;
    J.outmap = jt.job_pos;
    LEV_TRY(lev_stream_run(ctx, w->gate_up, J, tables, cmax, terms, gu));

    // down: columns = gelu_tanh(gate) * up of each grouped position, outputs by pair id
    lev_stream_source src2 = {};
    src2.x = gu;
    src2.ld = gu_rows;
    src2.rowmap = jt.job_pos;
    src2.njobs_dev = jt.njobs;
    src2.gelu_inter = w->inter;
    LEV_TRY(lev_stream_prepare(ctx, w->down, src2, cmax, terms, max_jobs, tables));
    lev_stream_job J2 = {};
    J2.rows = w->hidden;
    J2.out_ld = w->hidden;
    J2.max_jobs = max_jobs;
    J2.njobs_dev = jt.njobs;
    J2.job_slice = jt.job_slice;
    J2.outmap = jt.job_pair;
    LEV_TRY(lev_stream_run(ctx, w->down, J2, tables, cmax, terms, y_pairs));
    if (act_out) {
        // activations by pair id, recomputed from the gate_up outputs (diagnostic output)
        LEV_TRY(lev_moe_launch_act(ctx, gu, perm, offsets + w->experts, pairs, w->inter, act_out));
    }
    return LEV_OK;
}

namespace {
__device__ __forceinline__ float gelu_tanh_up_f32(float g, float u) {
    float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    float e = expf(-2.0f * fabsf(inner));
    float th = copysignf((1.0f - e) / (1.0f + e), inner);
    return 0.5f * g * (1.0f + th) * u;
}
// act[pair id][i] from gu[grouped position][2*inter]; positions beyond the grouped count are skipped
__global__ void k_act(const float* __restrict__ gu, const int* __restrict__ perm, const int* __restrict__ total_pos,
                      int64_t pairs, int inter, float* __restrict__ act) {
    int64_t n = (int64_t)(*total_pos) * inter;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t pos = i / inter;
        int k = (int)(i - pos * inter);
        const float* r = gu + pos * 2 * inter;
        act[(int64_t)perm[pos] * inter + k] = gelu_tanh_up_f32(r[k], r[inter + k]);
    }
}
}  // namespace

static int lev_moe_launch_act(lev_ctx* ctx, const float* gu, const int* perm, const int* total_pos, int64_t pairs,
                              int inter, float* act) {
    k_act<<<grid_for(ctx, pairs * inter, 256, 8), 256, 0, ctx->stream>>>(gu, perm, total_pos, pairs, inter, act);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_act");
}

int lev_moe_combine_dev(lev_ctx* ctx, const float* y, const float* wts, int64_t tokens, int top_k, int hidden, float* out) {
    return lev_moe_combine_resident_dev(ctx, y, wts, tokens, top_k, hidden, out, nullptr, 0, 0);
}

// idx != NULL: only the slots routed to experts [first, first + count) enter the sum
int lev_moe_combine_resident_dev(lev_ctx* ctx, const float* y, const float* wts, int64_t tokens, int top_k, int hidden,
                                 float* out, const int32_t* idx, int first, int count) {
    return lev_moe_combine_residual_dev(ctx, y, wts, tokens, top_k, hidden, out, idx, first, count, nullptr, 1.0f);
}

int lev_moe_combine_residual_dev(lev_ctx* ctx, const float* y, const float* wts, int64_t tokens, int top_k, int hidden,
                                 float* out, const int32_t* idx, int first, int count, const float* residual, float alpha) {
    LEV_CUDA(ctx, launch_pdl(k_combine, dim3(grid_for(ctx, tokens * hidden, 256, 8)), dim3(256), (size_t)0, ctx->stream, y, wts,
                             tokens, top_k, hidden, out, idx, first, count, residual, alpha));
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_combine");
}

// ---------------------------------------------------------------------------
// host-buffer staging helpers
// ---------------------------------------------------------------------------
namespace {
struct Stage {
    lev_ctx* ctx;
    char* base = nullptr;
    size_t cap = 0, off = 0;
    int init(lev_ctx* c, size_t bytes) {
        ctx = c;
        void* p;
        int st = lev_scratch(c, LEV_SCR_X, bytes + 4096, &p);
        base = (char*)p;
        cap = bytes + 4096;
        return st;
    }
    void* take(size_t bytes) {
        void* p = base + off;
        off += (bytes + 255) & ~(size_t)255;
        return p;
    }
};
int status_to_error(lev_ctx* ctx, unsigned flags, bool sync) {
    if (flags & LEV_FLAG_CHECK_FINITE) {
        int bits = 0;
        LEV_TRY(lev_read_status(ctx, &bits));
        if (bits & LEV_DEV_TIMEOUT) return lev_fail(ctx, LEV_TIMEOUT, "a bounded device wait ran out");
        if (bits & LEV_DEV_NONFINITE_INPUT) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        if (bits & LEV_DEV_NONFINITE_OUTPUT) return lev_fail(ctx, LEV_NONFINITE_OUTPUT, "router scores or outputs");
    } else if (sync) {
        LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return LEV_OK;
}
}  // namespace

extern "C" int lev_moe_route(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                             int32_t* idx, float* weights, float* scores, unsigned flags) {
    if (!ctx || !w || !x || !idx || !weights) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_tokens(ctx, w, tokens, top_k));
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool host = flags & LEV_FLAG_HOST_IO;
    size_t xb = (size_t)tokens * w->hidden * 4, ib = (size_t)tokens * top_k * 4, sb = (size_t)tokens * w->experts * 4;
    Stage S;
    LEV_TRY(S.init(ctx, (host ? xb + 2 * ib : 0) + sb + 2048));
    const float* dx = x;
    int32_t* didx = idx;
    float* dw = weights;
    float* dscores = (scores && !host) ? scores : (float*)S.take(sb);
    if (host) {
        if (flags & LEV_FLAG_CHECK_FINITE)
            for (int64_t i = 0; i < tokens * w->hidden; i++)
                if (!isfinite(x[i])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        float* px = (float*)S.take(xb);
        LEV_CUDA(ctx, cudaMemcpyAsync(px, x, xb, cudaMemcpyHostToDevice, ctx->stream));
        dx = px;
        didx = (int32_t*)S.take(ib);
        dw = (float*)S.take(ib);
    } else if (flags & LEV_FLAG_CHECK_FINITE) {
        LEV_TRY(lev_launch_finite_check(ctx, dx, tokens * w->hidden, LEV_DEV_NONFINITE_INPUT));
    }
    LEV_TRY(lev_moe_route_dev(ctx, w, dx, tokens, top_k, didx, dw, dscores));
    if (host) {
        LEV_CUDA(ctx, cudaMemcpyAsync(idx, didx, ib, cudaMemcpyDeviceToHost, ctx->stream));
        LEV_CUDA(ctx, cudaMemcpyAsync(weights, dw, ib, cudaMemcpyDeviceToHost, ctx->stream));
        if (scores) LEV_CUDA(ctx, cudaMemcpyAsync(scores, dscores, sb, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return status_to_error(ctx, flags, host);
}

extern "C" int lev_moe_group(lev_ctx* ctx, const int32_t* idx, int64_t tokens, int top_k, int experts, int32_t* counts,
                             int32_t* offsets, int32_t* perm, unsigned flags) {
    if (!ctx || !idx || !counts || !offsets || !perm) return LEV_BAD_ARGUMENT;
    if (tokens <= 0 || top_k <= 0 || top_k > LEV_MAX_TOP_K || experts <= 0 || experts > LEV_MAX_EXPERTS ||
        tokens * top_k > (1 << 24))
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "tokens %lld, topK %d, experts %d", (long long)tokens, top_k, experts);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool host = flags & LEV_FLAG_HOST_IO;
    size_t pb = (size_t)tokens * top_k * 4, eb = (size_t)(experts + 1) * 4;
    const int32_t* didx = idx;
    int32_t *dc = counts, *dof = offsets, *dp = perm;
    Stage S;
    if (host) {
        for (int64_t i = 0; i < tokens * top_k; i++)
            if (idx[i] < 0 || idx[i] >= experts) return lev_fail(ctx, LEV_BAD_ARGUMENT, "expert index %d outside 0..%d", idx[i], experts - 1);
        LEV_TRY(S.init(ctx, 2 * pb + 2 * eb + 2048));
        int32_t* pi = (int32_t*)S.take(pb);
        LEV_CUDA(ctx, cudaMemcpyAsync(pi, idx, pb, cudaMemcpyHostToDevice, ctx->stream));
        didx = pi;
        dc = (int32_t*)S.take(eb);
        dof = (int32_t*)S.take(eb);
        dp = (int32_t*)S.take(pb);
    }
    LEV_TRY(group_dev(ctx, didx, tokens, top_k, experts, 0, experts, dc, dof, dp, nullptr));
    if (host) {
        LEV_CUDA(ctx, cudaMemcpyAsync(counts, dc, (size_t)experts * 4, cudaMemcpyDeviceToHost, ctx->stream));
        LEV_CUDA(ctx, cudaMemcpyAsync(offsets, dof, eb, cudaMemcpyDeviceToHost, ctx->stream));
        LEV_CUDA(ctx, cudaMemcpyAsync(perm, dp, pb, cudaMemcpyDeviceToHost, ctx->stream));
        LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return LEV_OK;
}

extern "C" int lev_moe_experts(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                               const int32_t* idx, float* y_slots, float* act_out, unsigned flags) {
    if (!ctx || !w || !x || !idx || !y_slots) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_tokens(ctx, w, tokens, top_k));
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool host = flags & LEV_FLAG_HOST_IO;
    const int64_t pairs = tokens * top_k;
    size_t xb = (size_t)tokens * w->hidden * 4, ib = (size_t)pairs * 4, yb = (size_t)pairs * w->hidden * 4,
           ab = (size_t)pairs * w->inter * 4;
    const float* dx = x;
    const int32_t* didx = idx;
    float *dy = y_slots, *da = act_out;
    Stage S;
    if (host) {
        for (int64_t i = 0; i < pairs; i++)
            if (idx[i] < 0 || idx[i] >= w->experts) return lev_fail(ctx, LEV_BAD_ARGUMENT, "expert index %d outside 0..%d", idx[i], w->experts - 1);
        LEV_TRY(S.init(ctx, xb + ib + yb + (act_out ? ab : 0) + 2048));
        float* px = (float*)S.take(xb);
        int32_t* pi = (int32_t*)S.take(ib);
        LEV_CUDA(ctx, cudaMemcpyAsync(px, x, xb, cudaMemcpyHostToDevice, ctx->stream));
        LEV_CUDA(ctx, cudaMemcpyAsync(pi, idx, ib, cudaMemcpyHostToDevice, ctx->stream));
        dx = px;
        didx = pi;
        dy = (float*)S.take(yb);
        if (act_out) da = (float*)S.take(ab);
    }
    if (w->local_count != w->experts) LEV_CUDA(ctx, cudaMemsetAsync(dy, 0, yb, ctx->stream));  // pairs of absent experts stay zero
    LEV_TRY(lev_moe_experts_dev(ctx, w, dx, tokens, top_k, didx, dy, da));
    if (host) {
        LEV_CUDA(ctx, cudaMemcpyAsync(y_slots, dy, yb, cudaMemcpyDeviceToHost, ctx->stream));
        if (act_out) LEV_CUDA(ctx, cudaMemcpyAsync(act_out, da, ab, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return status_to_error(ctx, flags, host);
}

extern "C" int lev_moe_combine(lev_ctx* ctx, const float* y_slots, const float* weights, int64_t tokens, int top_k,
                               int hidden, float* out, unsigned flags) {
    if (!ctx || !y_slots || !weights || !out) return LEV_BAD_ARGUMENT;
    if (tokens <= 0 || top_k <= 0 || top_k > LEV_MAX_TOP_K || hidden <= 0)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "tokens %lld, topK %d, hidden %d", (long long)tokens, top_k, hidden);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool host = flags & LEV_FLAG_HOST_IO;
    size_t yb = (size_t)tokens * top_k * hidden * 4, wb = (size_t)tokens * top_k * 4, ob = (size_t)tokens * hidden * 4;
    const float *dy = y_slots, *dw = weights;
    float* dout = out;
    Stage S;
    if (host) {
        // merge coefficients are checked finite before use (Sources/LeviathanCore/Gemma4.swift:2101-2106)
        for (int64_t i = 0; i < tokens * top_k; i++)
            if (!isfinite(weights[i])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "routed merge weights must be finite");
        LEV_TRY(S.init(ctx, yb + wb + ob + 2048));
        float* py = (float*)S.take(yb);
        float* pw = (float*)S.take(wb);
        LEV_CUDA(ctx, cudaMemcpyAsync(py, y_slots, yb, cudaMemcpyHostToDevice, ctx->stream));
        LEV_CUDA(ctx, cudaMemcpyAsync(pw, weights, wb, cudaMemcpyHostToDevice, ctx->stream));
        dy = py;
        dw = pw;
        dout = (float*)S.take(ob);
    }
    LEV_TRY(lev_moe_combine_dev(ctx, dy, dw, tokens, top_k, hidden, dout));
    if (host) {
        LEV_CUDA(ctx, cudaMemcpyAsync(out, dout, ob, cudaMemcpyDeviceToHost, ctx->stream));
        LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return LEV_OK;
}

static int moe_layer_device(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, float* out,
                            int32_t* idx_out, float* w_out, const float* residual, float alpha);

int lev_moe_layer_device(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, float* out,
                         int32_t* idx_out, float* w_out) {
    return moe_layer_device(ctx, w, x, tokens, top_k, out, idx_out, w_out, nullptr, 1.0f);
}

static int moe_layer_device(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, float* out,
                            int32_t* idx_out, float* w_out, const float* residual, float alpha) {
    const int64_t pairs = tokens * top_k;
    size_t ib = ((size_t)pairs * 4 + 255) & ~(size_t)255, sb = ((size_t)tokens * w->experts * 4 + 255) & ~(size_t)255;
    void* a;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_MOE_A, 2 * ib + sb + 256, &a));
    int32_t* idx = idx_out ? idx_out : (int32_t*)a;
    float* wts = w_out ? w_out : (float*)((char*)a + ib);
    float* scores = (float*)((char*)a + 2 * ib);
    void* d;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_MOE_D, (size_t)pairs * w->hidden * 4 + 256, &d));
    if (pairs <= 32 && tokens <= 4 && moe_sliced(ctx, w, pairs, x)) {
        // decode: the top-k kernel also groups the pairs (one job per pair)
        int32_t *counts, *offsets, *perm;
        JobTable jt;
        LEV_TRY(group_tables(ctx, w, pairs, 1, (int)pairs, &counts, &offsets, &perm, &jt));
        GroupArgs G = {};
        G.idx = idx;
        G.pairs = (int)pairs;
        G.top_k = top_k;
        G.experts = w->experts;
        G.first = w->local_first;
        G.count = w->local_count;
        G.cmax = 1;
        G.counts = counts;
        G.offsets = offsets;
        G.perm = perm;
        G.njobs = jt.njobs;
        G.job_slice = jt.job_slice;
        G.job_token = jt.job_token;
        G.job_pos = jt.job_pos;
        G.job_pair = jt.job_pair;
        G.status = ctx->d_status;
        LEV_TRY(route_dev_impl(ctx, w, x, tokens, top_k, idx, wts, scores, &G));
        LEV_TRY(experts_dev_impl(ctx, w, x, tokens, top_k, idx, (float*)d, nullptr, true));
    } else {
        LEV_TRY(lev_moe_route_dev(ctx, w, x, tokens, top_k, idx, wts, scores));
        LEV_TRY(lev_moe_experts_dev(ctx, w, x, tokens, top_k, idx, (float*)d, nullptr));
    }
    return lev_moe_combine_residual_dev(ctx, (const float*)d, wts, tokens, top_k, w->hidden, out, nullptr, 0, 0, residual, alpha);
}

// out = residual + alpha * layer(x): the layer with the residual step of the decoder loop (g4_axpy,
// Sources/LeviathanCore/Gemma4.swift:3878) folded into the combine launch.  Device pointers; out may be residual.
extern "C" int lev_moe_layer_residual(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                                      const float* residual, float alpha, float* out, unsigned flags) {
    if (!ctx || !w || !x || !out || !residual) return LEV_BAD_ARGUMENT;
    if (flags & (LEV_FLAG_HOST_IO | LEV_FLAG_CHECK_FINITE))
        return lev_fail(ctx, LEV_UNSUPPORTED, "the layer with a folded residual takes device pointers and no finite checks");
    if (!isfinite(alpha)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "alpha %g", (double)alpha);
    LEV_TRY(check_tokens(ctx, w, tokens, top_k));
    if (w->local_count != w->experts)
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "experts are sharded on this context: use lev_moe_layer_ep");
    const size_t xb = (size_t)tokens * w->hidden * sizeof(float);
    if (out != x && (const char*)out < (const char*)x + xb && (const char*)x < (const char*)out + xb)
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and out overlap");
    if (out == x) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and out overlap");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    return moe_layer_device(ctx, w, x, tokens, top_k, out, nullptr, nullptr, residual, alpha);
}

extern "C" int lev_moe_layer(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                             float* out, int32_t* idx_out, float* w_out, unsigned flags) {
    if (!ctx || !w || !x || !out) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_tokens(ctx, w, tokens, top_k));
    if (w->local_count != w->experts)
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "experts are sharded on this context: use lev_moe_layer_ep");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool host = flags & LEV_FLAG_HOST_IO;
    size_t xb = (size_t)tokens * w->hidden * 4, ib = (size_t)tokens * top_k * 4;
    const float* dx = x;
    float* dout = out;
    int32_t* didx = idx_out;
    float* dw = w_out;
    Stage S;
    if (host) {
        if (flags & LEV_FLAG_CHECK_FINITE)
            for (int64_t i = 0; i < tokens * w->hidden; i++)
                if (!isfinite(x[i])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector");
        LEV_TRY(S.init(ctx, 2 * xb + 2 * ib + 2048));
        float* px = (float*)S.take(xb);
        LEV_CUDA(ctx, cudaMemcpyAsync(px, x, xb, cudaMemcpyHostToDevice, ctx->stream));
        dx = px;
        dout = (float*)S.take(xb);
        didx = (int32_t*)S.take(ib);
        dw = (float*)S.take(ib);
    } else if (flags & LEV_FLAG_CHECK_FINITE) {
        LEV_TRY(lev_launch_finite_check(ctx, dx, tokens * w->hidden, LEV_DEV_NONFINITE_INPUT));
    }
    LEV_TRY(lev_moe_layer_device(ctx, w, dx, tokens, top_k, dout, didx, dw));
    if (flags & LEV_FLAG_CHECK_FINITE) LEV_TRY(lev_launch_finite_check(ctx, dout, tokens * w->hidden, LEV_DEV_NONFINITE_OUTPUT));
    if (host) {
        LEV_CUDA(ctx, cudaMemcpyAsync(out, dout, xb, cudaMemcpyDeviceToHost, ctx->stream));
        if (idx_out) LEV_CUDA(ctx, cudaMemcpyAsync(idx_out, didx, ib, cudaMemcpyDeviceToHost, ctx->stream));
        if (w_out) LEV_CUDA(ctx, cudaMemcpyAsync(w_out, dw, ib, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return status_to_error(ctx, flags, host);
}
