// Schedule 1 ("stream"): decode matvec over a fragment-major repack of the
// GGUF blocks, tuned for HBM streaming on sm_100a.  Serves the dense matvec
// (lev_matvec) and, in grouped form, the expert FFN of the routed MoE.
//
// Layout.  Weights are regrouped once at upload (a lossless permutation of
// the same bytes) into tiles of 16 rows.  A tile is a sequence of K-steps of
// 2304 bytes: one 256-column block for Q4_K (16 row headers, then 4 chunks of
// 64 columns), four 64-column chunks for Q4_0 (each 64 B of scales + 512 B of
// nibbles).  Inside a chunk the bytes are ordered so that lane (g = lane/4,
// t = lane%4) of a warp finds at offset 16*lane the 8 bytes of row g and the
// 8 bytes of row g+8 that it feeds into mma.sync.m16n8k16 A fragments.
//
// Arithmetic.  A nibble n masked in place inside a 16-bit lane is the bit
// pattern of the fp16 subnormal n * 2^-24 (the fp16 encoding is linear up to
// 2047), so two LOP3 per 32-bit word turn packed nibbles into A fragments
// with no integer->float conversion; nibbles sitting at bits 4..7 come out
// multiplied by 16 and the matching activations are pre-divided by 16.  The
// f32 activations are split exactly into fp16 terms (x = h0 + h1*2^-11
// + h2*2^-22; three terms while 3*columns <= 8, else two) that occupy
// separate mma columns, so the tensor-core products are exact and the only
// rounding is the f32 accumulation.  Block scales are applied to the f32
// accumulators per sub-block; the Q4_0 "-8" offset enters as the accumulator
// initial value and the Q4_K min term is accumulated on CUDA cores.
//
// Data movement.  The whole tensor (or, grouped, the list of expert slices)
// is one linear stream of K-steps cut into equal contiguous ranges, one per
// warp of a grid that is resident all at once.  Every warp owns a private
// ring of kDepth shared-memory stages filled by bulk asynchronous copies
// (cp.async.bulk global->shared completing on an mbarrier) that it issues
// itself: about kDepth*2304 bytes per warp are in flight, no registers hold
// them and warps never wait for each other.
//
// Reduction.  Tiles that lie wholly in one warp's range are written straight
// to y; for the others each warp leaves one f32 per (row, column) in a
// partials record and bumps the tile's counter; the warp that arrives last
// adds the records in warp order, so the same call always gives the same
// bits regardless of arrival order.
#include <cuda_fp16.h>
#include <stdlib.h>

#include "lev_internal.h"
#include "lev_stream.h"

namespace {

constexpr float kHiScale = 0.0625f;  // activations of k-slots fed by nibbles at bits 4..7
constexpr int kDepth = 4;            // ring stages per warp
constexpr int kStepBytes = 2304;
constexpr int kWarpsPerCta = 8;
constexpr unsigned kWaitPolls = 1u << 24;  // bound of every mbarrier wait

__device__ __forceinline__ void mma16816(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_z(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                           unsigned b1) {
    // zero accumulator input: lets the compiler use the zero register for C
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ float h2f_bits(unsigned bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
}
// float(byte k of w) without the conversion unit: 2^23 + byte, minus 2^23
__device__ __forceinline__ float byte_to_float(unsigned w, unsigned k) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u + k)) - 8388608.0f;
}

// ---------------------------------------------------------------------------
// activation preparation
// ---------------------------------------------------------------------------
// Column element of k-slot pair for lane t, mma m (0..3), register r (0: b0,
// 1: b1), half h (0, 1) inside a 64-column chunk.
//   Q4_K: bytes 8t..8t+7 of the chunk's 32 bytes; mma 0,1 take low nibbles
//         (columns = byte index), mma 2,3 high nibbles (columns 32 + byte).
//   Q4_0: the chunk is two 32-value blocks; bytes 4t..4t+3 of each block;
//         mma 0,1 = block 0 low / high nibbles, mma 2,3 = block 1.
template <int TYPE>
__device__ __forceinline__ int chunk_col(int t, int m, int r, int h) {
    if (TYPE == LEV_GGML_Q4_K) return (m >> 1) * 32 + 8 * t + 4 * (m & 1) + r + 2 * h;
    return (m >> 1) * 32 + (m & 1) * 16 + 4 * t + r + 2 * h;
}
template <int TYPE>
__device__ __forceinline__ bool chunk_hi(int m) {
    return TYPE == LEV_GGML_Q4_K ? (m >> 1) : (m & 1);
}

// term `term` of the exact fp16 split of v: v = h0 + h1*2^-11 + h2*2^-22.
// The 1/16 of the high-nibble slots is applied BEFORE the split so that every
// term is exactly representable even when it lands in the fp16 subnormals.
__device__ __forceinline__ float split_term(float v, int term) {
    float h0 = __half2float(__float2half_rn(v));
    if (term == 0) return h0;
    float r1 = (v - h0) * 2048.0f;
    float h1 = __half2float(__float2half_rn(r1));
    if (term == 1) return h1;
    return __half2float(__float2half_rn((r1 - h1) * 2048.0f));
}

// gelu_tanh(gate) * up in f32 exactly as the reference kernel states it
// (Sources/LeviathanCore/Gemma4.swift:4364-4377): tanh through exp(-2|x|)
__device__ __forceinline__ float gelu_tanh_up(float g, float u) {
    float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    float e = expf(-2.0f * fabsf(inner));
    float th = copysignf((1.0f - e) / (1.0f + e), inner);
    float gelu = 0.5f * g * (1.0f + th);
    return gelu * u;
}

struct PrepArgs {
    const float* x;        // source rows
    int64_t ld;            // elements between source rows
    int64_t cols;          // K of the matvec
    const int* rowmap;     // [job][cmax] source row of each column, -1 = none; NULL: row = column
    const int* njobs_dev;  // device count of jobs, NULL: gridDim.y jobs
    int cmax;              // activation columns per job
    int terms, glt;        // glt = cmax * terms live mma columns
    int chunks;            // padded 64-column chunks
    int gelu_inter;        // > 0: source value = gelu_tanh(x[e]) * x[gelu_inter + e]
    float* act_out;        // optional [row][cols] copy of the (gelu) source values
    unsigned* frag;        // [job][chunk][glt][4][8]
    float* aux;            // Q4_K: [job][sub-block][cmax] ; Q4_0: [job][chunk][2][glt]
    int* status;
};

__device__ __forceinline__ float prep_src(const PrepArgs& P, int row, int64_t e) {
    if (row < 0 || e >= P.cols) return 0.f;
    const float* p = P.x + (int64_t)row * P.ld;
    return P.gelu_inter > 0 ? gelu_tanh_up(p[e], p[P.gelu_inter + e]) : p[e];
}

// the 8 half2 fragment registers of (job, chunk, mma column col, lane t)
template <int TYPE>
__device__ __forceinline__ bool prep_frag(const PrepArgs& P, int job, int chunk, int col, int t, uint4* dst) {
    const int c = col / P.terms, term = col - c * P.terms;
    const int row = P.rowmap ? P.rowmap[job * P.cmax + c] : c;
    bool bad = false;
    unsigned regs[8];
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int r = 0; r < 2; r++) {
            float v[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float xv = prep_src(P, row, (int64_t)chunk * 64 + chunk_col<TYPE>(t, m, r, h));
                float s = split_term(chunk_hi<TYPE>(m) ? xv * kHiScale : xv, term);
                bad |= !isfinite(s);
                v[h] = s;
            }
            __half2 hv = __floats2half2_rn(v[0], v[1]);
            regs[m * 2 + r] = *reinterpret_cast<unsigned*>(&hv);
        }
    dst[0] = make_uint4(regs[0], regs[1], regs[2], regs[3]);
    dst[1] = make_uint4(regs[4], regs[5], regs[6], regs[7]);
    return bad;
}

// one 32-column sum by a whole warp: lane i holds element i, xor butterfly (fixed order).
// Q4_K: which = activation column c, sums the true x of sub-block sb of the chunk.
// Q4_0: which = mma column, sums what the tensor core sees of block sb: low-nibble
//       slots carry term(x), high-nibble slots term(x/16) against nibbles worth 16x.
template <int TYPE>
__device__ __forceinline__ float prep_sum32(const PrepArgs& P, int job, int chunk, int sb, int which, int lane) {
    const int c = TYPE == LEV_GGML_Q4_K ? which : which / P.terms;
    const int term = TYPE == LEV_GGML_Q4_K ? 0 : which - c * P.terms;
    const int row = P.rowmap ? P.rowmap[job * P.cmax + c] : c;
    const int64_t e = (int64_t)chunk * 64 + sb * 32 + lane;
    float xv = prep_src(P, row, e);
    if (P.act_out && term == 0 && row >= 0 && e < P.cols) P.act_out[(int64_t)row * P.cols + e] = xv;
    float s = xv;
    if (TYPE != LEV_GGML_Q4_K) s = lane < 16 ? split_term(xv, term) : 16.0f * split_term(xv * kHiScale, term);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    return TYPE == LEV_GGML_Q4_K ? s : -8.0f * 5.9604644775390625e-08f * s;
}

// the same sum by one thread (four interleaved partial sums, fixed order), for the fused path
template <int TYPE>
__device__ __forceinline__ float prep_sum32_serial(const PrepArgs& P, int chunk, int sb, int which) {
    const int c = TYPE == LEV_GGML_Q4_K ? which : which / P.terms;
    const int term = TYPE == LEV_GGML_Q4_K ? 0 : which - c * P.terms;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; i++) {
        float xv = prep_src(P, c, (int64_t)chunk * 64 + sb * 32 + i);
        float s = xv;
        if (TYPE != LEV_GGML_Q4_K) s = i < 16 ? split_term(xv, term) : 16.0f * split_term(xv * kHiScale, term);
        acc[i & 3] += s;
    }
    float s = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    return TYPE == LEV_GGML_Q4_K ? s : -8.0f * 5.9604644775390625e-08f * s;
}

// grid (chunks, jobs); one warp per 8 mma columns
template <int TYPE>
__global__ void k_prepare_x(PrepArgs P) {
    const int chunk = blockIdx.x, job = blockIdx.y;
    if (P.njobs_dev && job >= *P.njobs_dev) return;
    const int lane = threadIdx.x & 31, nt = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int col = nt * 8 + g;
    bool bad = false;
    if (col < P.glt)
        bad = prep_frag<TYPE>(P, job, chunk, col, t,
                              reinterpret_cast<uint4*>(P.frag) + ((((int64_t)job * P.chunks + chunk) * P.glt + col) * 4 + t) * 2);
    if (TYPE == LEV_GGML_Q4_K) {
        if (nt == 0)
            for (int c = 0; c < P.cmax; c++)
#pragma unroll
                for (int sb = 0; sb < 2; sb++) {
                    float s = prep_sum32<TYPE>(P, job, chunk, sb, c, lane);
                    if (lane == 0) P.aux[(((int64_t)job * P.chunks + chunk) * 2 + sb) * P.cmax + c] = s;
                }
    } else {
        for (int cc = 0; cc < 8; cc++) {
            const int col2 = nt * 8 + cc;  // uniform across the warp
            if (col2 >= P.glt) break;
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {
                float s = prep_sum32<TYPE>(P, job, chunk, blk, col2, lane);
                if (lane == 0) P.aux[(((int64_t)job * P.chunks + chunk) * 2 + blk) * P.glt + col2] = s;
            }
        }
    }
    if (bad) atomicOr(P.status, LEV_DEV_NONFINITE_INPUT);
}

// ---------------------------------------------------------------------------
// repack (device): raw GGUF blocks -> fragment-major tiles
// ---------------------------------------------------------------------------
// Q4_K: per (tile, block) 144 units of 16 B: 16 headers (row order), then per
// 64-column chunk c 32 lane units {row g bytes 32c+8t..+8, row g+8 same}.
__global__ void k_repack_q4k(const uint8_t* __restrict__ raw, int64_t rows, int64_t bpr, int64_t tiles,
                             uint4* __restrict__ out) {
    int64_t total = tiles * bpr * 144;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        int64_t tb = u / 144;
        int k = (int)(u - tb * 144);
        int64_t tile = tb / bpr, b = tb - tile * bpr;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (k < 16) {
            int64_t row = tile * 16 + k;
            if (row < rows) v = *reinterpret_cast<const uint4*>(raw + (row * bpr + b) * LEV_Q4_K_BYTES);
        } else {
            int c = (k - 16) >> 5, lane = (k - 16) & 31, g = lane >> 2, t = lane & 3;
            int64_t r0 = tile * 16 + g, r1 = r0 + 8;
            if (r0 < rows) {
                uint2 a = *reinterpret_cast<const uint2*>(raw + (r0 * bpr + b) * LEV_Q4_K_BYTES + 16 + 32 * c + 8 * t);
                v.x = a.x;
                v.y = a.y;
            }
            if (r1 < rows) {
                uint2 a = *reinterpret_cast<const uint2*>(raw + (r1 * bpr + b) * LEV_Q4_K_BYTES + 16 + 32 * c + 8 * t);
                v.z = a.x;
                v.w = a.y;
            }
        }
        out[u] = v;
    }
}

// Q4_0: per (tile, chunk of two blocks) 36 units of 16 B: 4 units of scales
// {per g: row g blk0, row g blk1, row g+8 blk0, row g+8 blk1 as fp16}, then
// 32 lane units {row g: blk0 bytes 4t..4t+3, blk1 bytes 4t..4t+3; row g+8 same}.
// Chunks beyond the row's blocks (padding to whole K-steps) are zero.
__device__ __forceinline__ unsigned q40_scale(const uint8_t* raw, int64_t rows, int64_t bpr, int64_t row, int64_t blk) {
    if (row >= rows || blk >= bpr) return 0u;
    return *reinterpret_cast<const unsigned short*>(raw + (row * bpr + blk) * LEV_Q4_0_BYTES);
}
__device__ __forceinline__ unsigned q40_word(const uint8_t* raw, int64_t rows, int64_t bpr, int64_t row, int64_t blk, int t) {
    if (row >= rows || blk >= bpr) return 0u;
    const unsigned short* p = reinterpret_cast<const unsigned short*>(raw + (row * bpr + blk) * LEV_Q4_0_BYTES + 2 + 4 * t);
    return (unsigned)p[0] | ((unsigned)p[1] << 16);
}
__global__ void k_repack_q40(const uint8_t* __restrict__ raw, int64_t rows, int64_t bpr, int64_t tiles, int64_t chunks,
                             uint4* __restrict__ out) {
    int64_t total = tiles * chunks * 36;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        int64_t tc = u / 36;
        int k = (int)(u - tc * 36);
        int64_t tile = tc / chunks, ch = tc - tile * chunks;
        int64_t b0 = 2 * ch, b1 = b0 + 1;
        uint4 v;
        if (k < 4) {
            int64_t ra = tile * 16 + 2 * k, rb = ra + 1;
            v.x = q40_scale(raw, rows, bpr, ra, b0) | (q40_scale(raw, rows, bpr, ra, b1) << 16);
            v.y = q40_scale(raw, rows, bpr, ra + 8, b0) | (q40_scale(raw, rows, bpr, ra + 8, b1) << 16);
            v.z = q40_scale(raw, rows, bpr, rb, b0) | (q40_scale(raw, rows, bpr, rb, b1) << 16);
            v.w = q40_scale(raw, rows, bpr, rb + 8, b0) | (q40_scale(raw, rows, bpr, rb + 8, b1) << 16);
        } else {
            int lane = k - 4, g = lane >> 2, t = lane & 3;
            int64_t r0 = tile * 16 + g, r1 = r0 + 8;
            v.x = q40_word(raw, rows, bpr, r0, b0, t);
            v.y = q40_word(raw, rows, bpr, r0, b1, t);
            v.z = q40_word(raw, rows, bpr, r1, b0, t);
            v.w = q40_word(raw, rows, bpr, r1, b1, t);
        }
        out[u] = v;
    }
}

// ---------------------------------------------------------------------------
// streaming kernel
// ---------------------------------------------------------------------------
struct StreamArgs {
    const uint4* wp;        // packed weights: first tile of this call (dense) or of the tensor (grouped)
    int steps_per_tile;     // K-steps per tile
    int tiles_per_job;      // tiles of one job (one expert slice; the whole call when dense)
    int max_warps;          // warps of the grid
    int total_steps;        // dense: tiles * steps_per_tile
    const int* njobs_dev;   // grouped: device count of jobs (total steps = jobs * tiles_per_job * steps_per_tile)
    const int* job_slice;   // grouped: [job] index of the expert slice, in units of tiles_per_job tiles
    const int* outmap;      // grouped: [job][cmax] output row of each column, -1 = none; NULL: column index
    int64_t rows;           // rows of one job
    int64_t out_ld;         // elements between output columns
    int chunks;             // padded 64-column chunks of the activation tables
    const uint4* frag;      // [job][chunk][glt][4] x 32 B
    const float* aux;       // Q4_K: [job][sub-block][cmax] ; Q4_0: [job][chunk][2][glt]
    int cmax, terms, glt;
    float* partials;        // [warp][2][cmax][16]
    int* tile_count;        // [job tiles], zero between launches
    int* status;            // device status word
    float* y;
    int debug;              // bit 0: skip the arithmetic (data-movement timing only)
    int fused_prep;         // XS only: build the activation tables in shared memory from prep.x
    PrepArgs prep;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
// bounded wait: false when the phase did not complete within kWaitPolls polls
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned i = 0; i < kWaitPolls; i++) {
        unsigned ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// address of K-step s of the global stream
__device__ __forceinline__ const unsigned char* step_src(const StreamArgs& A, int s) {
    int gt = s / A.steps_per_tile, k = s - gt * A.steps_per_tile;
    int64_t tile = gt;
    if (A.job_slice) {
        int job = gt / A.tiles_per_job;
        tile = (int64_t)A.job_slice[job] * A.tiles_per_job + (gt - job * A.tiles_per_job);
    }
    return reinterpret_cast<const unsigned char*>(A.wp) + (tile * A.steps_per_tile + k) * (int64_t)kStepBytes;
}

// XS: activation tables of the (single) job are staged in shared memory
template <int TYPE, int NT, bool XS>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 2) k_stream(StreamArgs A) {
    constexpr int kMaxC = 4 * NT;  // 8*NT mma columns hold at most 4*NT activation columns
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[kWarpsPerCta][kDepth];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;

    const int total = A.njobs_dev ? *A.njobs_dev * A.tiles_per_job * A.steps_per_tile : A.total_steps;
    int range = (total + A.max_warps - 1) / A.max_warps;
    if (range < 2) range = 2;
    const int gw = blockIdx.x * kWarpsPerCta + warp;
    const int s0 = gw * range;
    const int n = (s0 + range <= total ? s0 + range : total) - s0;

    unsigned char* ring = smem_raw + (size_t)warp * kDepth * kStepBytes;
    const unsigned ring_s = smem_u32(ring), bar_s = smem_u32(&bars[warp][0]);
    if (lane == 0 && n > 0) {
#pragma unroll
        for (int d = 0; d < kDepth; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
#pragma unroll
        for (int d = 0; d < kDepth; d++)
            if (d < n) bulk_load(ring_s + d * kStepBytes, step_src(A, s0 + d), kStepBytes, bar_s + 8 * d);
    }
    // dense calls stage the activation tables once per CTA while the first
    // weight bytes are on their way
    const uint4* sfrag = nullptr;
    const float* saux = nullptr;
    if (XS) {
        uint4* xs = reinterpret_cast<uint4*>(smem_raw + (size_t)kWarpsPerCta * kDepth * kStepBytes);
        const int nfrag = A.chunks * A.glt * 8;  // uint4 units
        const int naux = TYPE == LEV_GGML_Q4_K ? A.chunks * 2 * A.cmax : A.chunks * 2 * A.glt;
        float* sa = reinterpret_cast<float*>(xs + nfrag);
        if (A.fused_prep) {
            // each CTA splits the activations itself while its first weight
            // bytes are in flight: no separate preparation launch
            bool bad = false;
            for (int i = threadIdx.x; i < A.chunks * A.glt * 4; i += blockDim.x) {
                int tt = i & 3, col = (i >> 2) % A.glt, chunk = (i >> 2) / A.glt;
                bad |= prep_frag<TYPE>(A.prep, 0, chunk, col, tt, xs + (size_t)i * 2);
            }
            // 32-column sums, one thread each so that the loads of all sums are in flight together
            const int per = TYPE == LEV_GGML_Q4_K ? A.cmax : A.glt;
            for (int i = threadIdx.x; i < naux; i += blockDim.x)
                sa[i] = prep_sum32_serial<TYPE>(A.prep, i / (2 * per), (i / per) & 1, i % per);
            if (bad && blockIdx.x == 0) atomicOr(A.status, LEV_DEV_NONFINITE_INPUT);
        } else {
            for (int i = threadIdx.x; i < nfrag; i += blockDim.x) xs[i] = __ldg(A.frag + i);
            for (int i = threadIdx.x; i < naux; i += blockDim.x) sa[i] = __ldg(A.aux + i);
        }
        __syncthreads();
        sfrag = xs;
        saux = sa;
    }
    if (n <= 0) return;  // no block-wide barrier below this line
    __syncwarp();

    int gt = s0 / A.steps_per_tile;        // global tile index (job * tiles_per_job + tile)
    int k = s0 - gt * A.steps_per_tile;    // K-step inside the tile
    int seg_k0 = k;                        // where this warp's segment of the tile began
    int pend_tile[2] = {-1, -1};           // global tiles with a partials record of this warp
    const int first_gt = gt;

    float yacc[NT][4];
    float mina[kMaxC], minb[kMaxC];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxC; c++) mina[c] = minb[c] = 0.f;

    int job = gt / A.tiles_per_job;
    const uint4* jfrag = XS ? sfrag : A.frag + (int64_t)job * A.chunks * A.glt * 8;
    const float* jaux = XS ? saux
                           : A.aux + (int64_t)job * (TYPE == LEV_GGML_Q4_K ? A.chunks * 2 * A.cmax : A.chunks * 2 * A.glt);

    for (int i = 0; i < n; i++) {
        const int slot = i % kDepth;
        if (!mbar_wait(bar_s + 8 * slot, (unsigned)(i / kDepth) & 1u)) {
            if (lane == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
            return;
        }
        const uint4* st = reinterpret_cast<const uint4*>(ring + slot * kStepBytes);

        if (!(A.debug & 1))
#pragma unroll
        for (int c = 0; c < 4; c++) {
            // ---- activation fragments of this chunk ----
            const int ch = k * 4 + c;
            uint4 x0[NT], x1[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                x0[nt] = make_uint4(0, 0, 0, 0);
                x1[nt] = x0[nt];
                if (nt * 8 + g < A.glt) {
                    const uint4* p = jfrag + ((ch * A.glt + nt * 8 + g) * 4 + t) * 2;
                    x0[nt] = XS ? p[0] : __ldg(p);
                    x1[nt] = XS ? p[1] : __ldg(p + 1);
                }
            }
            if (TYPE == LEV_GGML_Q4_K) {
                const uint4 q = st[16 + c * 32 + lane];
                // 6-bit scales of sub-blocks 2c, 2c+1 of rows g (h0) and g+8 (h1)
                // (rust/crates/lev-cpu/src/lib.rs:64-74), four per word
                const uint4 h0 = st[g], h1 = st[8 + g];
                unsigned sa = c < 2 ? (h0.y & 0x3F3F3F3Fu) : ((h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u));
                unsigned sb = c < 2 ? (h1.y & 0x3F3F3F3Fu) : ((h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u));
                float dA = h2f_bits(h0.x & 0xffffu) * 16777216.0f, dB = h2f_bits(h1.x & 0xffffu) * 16777216.0f;  // d * 2^24
                float sA_lo = dA * byte_to_float(sa, 2 * (c & 1)), sA_hi = dA * byte_to_float(sa, 2 * (c & 1) + 1);
                float sB_lo = dB * byte_to_float(sb, 2 * (c & 1)), sB_hi = dB * byte_to_float(sb, 2 * (c & 1) + 1);
                unsigned w0 = q.x, w1 = q.y, w2 = q.z, w3 = q.w;
                unsigned w0s = w0 >> 8, w1s = w1 >> 8, w2s = w2 >> 8, w3s = w3 >> 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    float lo[4], hi[4];
                    mma16816_z(lo, w0 & 0x000F000Fu, w2 & 0x000F000Fu, w0s & 0x000F000Fu, w2s & 0x000F000Fu, x0[nt].x, x0[nt].y);
                    mma16816(lo, w1 & 0x000F000Fu, w3 & 0x000F000Fu, w1s & 0x000F000Fu, w3s & 0x000F000Fu, x0[nt].z, x0[nt].w);
                    mma16816_z(hi, w0 & 0x00F000F0u, w2 & 0x00F000F0u, w0s & 0x00F000F0u, w2s & 0x00F000F0u, x1[nt].x, x1[nt].y);
                    mma16816(hi, w1 & 0x00F000F0u, w3 & 0x00F000F0u, w1s & 0x00F000F0u, w3s & 0x00F000F0u, x1[nt].z, x1[nt].w);
                    yacc[nt][0] = fmaf(sA_lo, lo[0], fmaf(sA_hi, hi[0], yacc[nt][0]));
                    yacc[nt][1] = fmaf(sA_lo, lo[1], fmaf(sA_hi, hi[1], yacc[nt][1]));
                    yacc[nt][2] = fmaf(sB_lo, lo[2], fmaf(sB_hi, hi[2], yacc[nt][2]));
                    yacc[nt][3] = fmaf(sB_lo, lo[3], fmaf(sB_hi, hi[3], yacc[nt][3]));
                }
            } else {
                const uint2 sc = reinterpret_cast<const uint2*>(st + c * 36)[g];
                const uint4 q = st[c * 36 + 4 + lane];
                // d * 2^24 for (row g, blk0), (row g, blk1), (row g+8, blk0), (row g+8, blk1)
                float dA0 = h2f_bits(sc.x & 0xffffu) * 16777216.0f, dA1 = h2f_bits(sc.x >> 16) * 16777216.0f;
                float dB0 = h2f_bits(sc.y & 0xffffu) * 16777216.0f, dB1 = h2f_bits(sc.y >> 16) * 16777216.0f;
                unsigned w0 = q.x, w1 = q.y, w2 = q.z, w3 = q.w;
                unsigned w0s = w0 >> 8, w1s = w1 >> 8, w2s = w2 >> 8, w3s = w3 >> 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    // accumulators start at -8 * 2^-24 * (sum of the block's activations)
                    float k00 = 0.f, k01 = 0.f, k10 = 0.f, k11 = 0.f;
                    const int cb = nt * 8 + 2 * t;
                    const float* bp = jaux + (ch * 2) * A.glt + cb;
                    if (cb < A.glt) {
                        k00 = XS ? bp[0] : __ldg(bp);
                        k10 = XS ? bp[A.glt] : __ldg(bp + A.glt);
                    }
                    if (cb + 1 < A.glt) {
                        k01 = XS ? bp[1] : __ldg(bp + 1);
                        k11 = XS ? bp[A.glt + 1] : __ldg(bp + A.glt + 1);
                    }
                    float a0[4] = {k00, k01, k00, k01}, a1[4] = {k10, k11, k10, k11};
                    mma16816(a0, w0 & 0x000F000Fu, w2 & 0x000F000Fu, w0s & 0x000F000Fu, w2s & 0x000F000Fu, x0[nt].x, x0[nt].y);
                    mma16816(a0, w0 & 0x00F000F0u, w2 & 0x00F000F0u, w0s & 0x00F000F0u, w2s & 0x00F000F0u, x0[nt].z, x0[nt].w);
                    mma16816(a1, w1 & 0x000F000Fu, w3 & 0x000F000Fu, w1s & 0x000F000Fu, w3s & 0x000F000Fu, x1[nt].x, x1[nt].y);
                    mma16816(a1, w1 & 0x00F000F0u, w3 & 0x00F000F0u, w1s & 0x00F000F0u, w3s & 0x00F000F0u, x1[nt].z, x1[nt].w);
                    yacc[nt][0] = fmaf(dA0, a0[0], fmaf(dA1, a1[0], yacc[nt][0]));
                    yacc[nt][1] = fmaf(dA0, a0[1], fmaf(dA1, a1[1], yacc[nt][1]));
                    yacc[nt][2] = fmaf(dB0, a0[2], fmaf(dB1, a1[2], yacc[nt][2]));
                    yacc[nt][3] = fmaf(dB0, a0[3], fmaf(dB1, a1[3], yacc[nt][3]));
                }
            }
        }
        if (TYPE == LEV_GGML_Q4_K && !(A.debug & 1)) {
            // min term: this lane owns sub-blocks 2t, 2t+1 of its two rows
            const uint4 h0 = st[g], h1 = st[8 + g];
            unsigned ma = t < 2 ? (h0.z & 0x3F3F3F3Fu) : (((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u));
            unsigned mb = t < 2 ? (h1.z & 0x3F3F3F3Fu) : (((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u));
            int sh = 16 * (t & 1);
            float dminA = h2f_bits(h0.x >> 16), dminB = h2f_bits(h1.x >> 16);
            float mA0 = dminA * (float)((ma >> sh) & 0xffu), mA1 = dminA * (float)((ma >> (sh + 8)) & 0xffu);
            float mB0 = dminB * (float)((mb >> sh) & 0xffu), mB1 = dminB * (float)((mb >> (sh + 8)) & 0xffu);
            const float* sx0 = jaux + (k * 8 + 2 * t) * A.cmax;
#pragma unroll
            for (int c = 0; c < kMaxC; c++) {
                if (c < A.cmax) {
                    float x0 = XS ? sx0[c] : __ldg(sx0 + c), x1 = XS ? sx0[A.cmax + c] : __ldg(sx0 + A.cmax + c);
                    mina[c] = fmaf(mA0, x0, fmaf(mA1, x1, mina[c]));
                    minb[c] = fmaf(mB0, x0, fmaf(mB1, x1, minb[c]));
                }
            }
        }

        // every lane has consumed its shared-memory reads of this stage: refill it
        __syncwarp();
        if (lane == 0 && i + kDepth < n)
            bulk_load(ring_s + slot * kStepBytes, step_src(A, s0 + i + kDepth), kStepBytes, bar_s + 8 * slot);

        k++;
        if (k == A.steps_per_tile || i == n - 1) {
            // ---- this warp's segment of the tile ends: fold to one f32 per (row, column) ----
            const bool whole = seg_k0 == 0 && k == A.steps_per_tile;
            const int rec = gt == first_gt ? 0 : 1;
            const int tile_in_job = gt - job * A.tiles_per_job;
            float* pbuf = A.partials + ((int64_t)(gw * 2 + rec) * A.cmax) * 16;
#pragma unroll
            for (int c = 0; c < kMaxC; c++) {
                if (c < A.cmax) {
                    float va = 0.f, vb = 0.f;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
#pragma unroll
                        for (int jj = 0; jj < 2; jj++) {
                            int col = nt * 8 + 2 * t + jj;
                            int xc = col / A.terms, term = col - xc * A.terms;
                            float sc = term == 0 ? 1.0f : (term == 1 ? 4.8828125e-4f : 2.384185791015625e-7f);
                            if (xc == c) {
                                va = fmaf(yacc[nt][jj], sc, va);
                                vb = fmaf(yacc[nt][2 + jj], sc, vb);
                            }
                        }
                    if (TYPE == LEV_GGML_Q4_K) {
                        va -= mina[c];
                        vb -= minb[c];
                    }
                    va += __shfl_xor_sync(0xffffffffu, va, 1);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 1);
                    va += __shfl_xor_sync(0xffffffffu, va, 2);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 2);
                    if (t == 0) {
                        if (whole) {
                            const int oc = A.outmap ? A.outmap[job * A.cmax + c] : c;
                            int64_t r = (int64_t)tile_in_job * 16 + g;
                            if (oc >= 0) {
                                if (r < A.rows) A.y[(int64_t)oc * A.out_ld + r] = va;
                                if (r + 8 < A.rows) A.y[(int64_t)oc * A.out_ld + r + 8] = vb;
                            }
                        } else {
                            __stcg(pbuf + c * 16 + g, va);
                            __stcg(pbuf + c * 16 + g + 8, vb);
                        }
                    }
                }
            }
            if (!whole) pend_tile[rec] = gt;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
            for (int c = 0; c < kMaxC; c++) mina[c] = minb[c] = 0.f;
            gt++;
            k = 0;
            seg_k0 = 0;
            if (!XS && gt - job * A.tiles_per_job >= A.tiles_per_job) {
                job++;
                jfrag = A.frag + (int64_t)job * A.chunks * A.glt * 8;
                jaux = A.aux + (int64_t)job * (TYPE == LEV_GGML_Q4_K ? A.chunks * 2 * A.cmax : A.chunks * 2 * A.glt);
            }
        }
    }

    // ---- tiles shared with other warps: the last arriver adds the records in warp order ----
#pragma unroll
    for (int rec = 0; rec < 2; rec++) {
        const int pt = pend_tile[rec];
        if (pt < 0) continue;
        __threadfence();
        __syncwarp();
        const int w_first = (pt * A.steps_per_tile) / range;
        const int w_last = (pt * A.steps_per_tile + A.steps_per_tile - 1) / range;
        int prev = 0;
        if (lane == 0) prev = atomicAdd(A.tile_count + pt, 1);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == w_last - w_first) {
            __threadfence();
            const int pjob = pt / A.tiles_per_job, ptile = pt - pjob * A.tiles_per_job;
            for (int idx = lane; idx < A.cmax * 16; idx += 32) {
                float acc = 0.f;
                for (int w = w_first; w <= w_last; w++) {
                    int wrec = (w * range) / A.steps_per_tile == pt ? 0 : 1;
                    acc += __ldcg(A.partials + ((int64_t)(w * 2 + wrec) * A.cmax) * 16 + idx);
                }
                const int c = idx >> 4;
                const int oc = A.outmap ? A.outmap[pjob * A.cmax + c] : c;
                int64_t r = (int64_t)ptile * 16 + (idx & 15);
                if (oc >= 0 && r < A.rows) A.y[(int64_t)oc * A.out_ld + r] = acc;
            }
            if (lane == 0) A.tile_count[pt] = 0;
        }
    }
}

int grid_cap(lev_ctx* ctx, int64_t work, int block, int per_sm) {
    int64_t g = (work + block - 1) / block, cap = (int64_t)ctx->prop.multiProcessorCount * per_sm;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

template <int TYPE, int NT, bool XS>
int launch_stream(lev_ctx* ctx, int grid, size_t smem, const StreamArgs& A) {
    static size_t configured[16] = {};  // per device: largest dynamic shared memory opted in so far
    if (configured[ctx->device & 15] < smem) {
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_stream<TYPE, NT, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[ctx->device & 15] = smem;
    }
    k_stream<TYPE, NT, XS><<<grid, kWarpsPerCta * 32, smem, ctx->stream>>>(A);
    return LEV_OK;
}

int env_int(const char* name, int fallback) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : fallback;
}

}  // namespace

int lev_stream_terms(int n_cols) { return 3 * n_cols <= 8 ? 3 : 2; }

// 64-column chunks of the activation tables; Q4_0 rows are padded with zero
// blocks to whole K-steps of four chunks
int64_t lev_stream_chunks(const lev_weights* w) {
    int64_t c = (w->cols + 63) / 64;
    return w->type == LEV_GGML_Q4_0 ? (c + 3) / 4 * 4 : c;
}

int lev_repack_weights(lev_ctx* ctx, lev_weights* w) {
    if (w->type != LEV_GGML_Q4_K && w->type != LEV_GGML_Q4_0) return LEV_OK;  // other types: plain schedule
    int64_t tiles = (w->rows + 15) / 16;
    int64_t steps = lev_stream_chunks(w) / 4;
    size_t bytes = (size_t)tiles * steps * kStepBytes;
    LEV_CUDA(ctx, cudaMalloc((void**)&w->packed, bytes + 256));
    w->packed_bytes = bytes;
    w->packed_rows = tiles * 16;
    int grid = grid_cap(ctx, (int64_t)(bytes / 16), 256, 16);
    if (w->type == LEV_GGML_Q4_K)
        k_repack_q4k<<<grid, 256, 0, ctx->stream>>>(w->raw, w->rows, w->blocks_per_row, tiles, (uint4*)w->packed);
    else
        k_repack_q40<<<grid, 256, 0, ctx->stream>>>(w->raw, w->rows, w->blocks_per_row, tiles, lev_stream_chunks(w),
                                                    (uint4*)w->packed);
    ctx->launches++;
    LEV_CUDA(ctx, cudaGetLastError());
    LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return LEV_OK;
}

bool lev_stream_supported(const lev_weights* w, int64_t row0, int64_t rows, int n_cols) {
    (void)rows;
    if (!w->packed) return false;
    if (row0 % 16 != 0) return false;
    return n_cols >= 1 && n_cols <= LEV_MAX_COLUMNS;
}

size_t lev_stream_table_bytes(const lev_weights* w, int cmax, int terms, int jobs, size_t* frag_bytes) {
    int64_t chunks = lev_stream_chunks(w);
    int glt = cmax * terms;
    size_t fb = ((size_t)jobs * chunks * glt * 4 * 32 + 255) & ~(size_t)255;
    size_t ab = w->type == LEV_GGML_Q4_K ? (size_t)jobs * chunks * 2 * cmax * sizeof(float)
                                         : (size_t)jobs * chunks * 2 * glt * sizeof(float);
    ab = (ab + 255) & ~(size_t)255;
    if (frag_bytes) *frag_bytes = fb;
    return fb + ab;
}

static PrepArgs make_prep(lev_ctx* ctx, const lev_weights* w, const lev_stream_source& src, int cmax, int terms,
                          void* tables, int jobs);

int lev_stream_prepare(lev_ctx* ctx, const lev_weights* w, const lev_stream_source& src, int cmax, int terms, int jobs,
                       void* tables) {
    PrepArgs P = make_prep(ctx, w, src, cmax, terms, tables, jobs);
    int ntiles = (P.glt + 7) / 8;
    dim3 grid((unsigned)P.chunks, (unsigned)jobs);
    if (w->type == LEV_GGML_Q4_K) k_prepare_x<LEV_GGML_Q4_K><<<grid, 32 * ntiles, 0, ctx->stream>>>(P);
    else k_prepare_x<LEV_GGML_Q4_0><<<grid, 32 * ntiles, 0, ctx->stream>>>(P);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_prepare_x");
}

static PrepArgs make_prep(lev_ctx* ctx, const lev_weights* w, const lev_stream_source& src, int cmax, int terms,
                          void* tables, int jobs) {
    size_t fb;
    lev_stream_table_bytes(w, cmax, terms, jobs, &fb);
    PrepArgs P;
    P.x = src.x;
    P.ld = src.ld;
    P.cols = w->cols;
    P.rowmap = src.rowmap;
    P.njobs_dev = src.njobs_dev;
    P.cmax = cmax;
    P.terms = terms;
    P.glt = cmax * terms;
    P.chunks = (int)lev_stream_chunks(w);
    P.gelu_inter = src.gelu_inter;
    P.act_out = src.act_out;
    P.frag = (unsigned*)tables;
    P.aux = tables ? (float*)((char*)tables + fb) : nullptr;
    P.status = ctx->d_status;
    return P;
}

bool lev_stream_fuses_prepare(const lev_weights* w, int cmax, int terms) {
    size_t tb = lev_stream_table_bytes(w, cmax, terms, 1, nullptr);
    return (size_t)kWarpsPerCta * kDepth * kStepBytes + tb <= 110 * 1024;
}

// sizes of the two work buffers a call needs: per-warp partial sums and per-tile counters
void lev_stream_workspace_bytes(lev_ctx* ctx, const lev_weights* w, const lev_stream_job& J, int cmax,
                                size_t* partial_bytes, size_t* counter_bytes) {
    const int64_t steps = lev_stream_chunks(w) / 4, tiles_per_job = (J.rows + 15) / 16;
    const int64_t max_steps = (int64_t)J.max_jobs * tiles_per_job * steps;
    int ctas_per_sm = env_int("LEV_STREAM_CTAS_PER_SM", 2);
    ctas_per_sm = ctas_per_sm < 1 ? 1 : (ctas_per_sm > 2 ? 2 : ctas_per_sm);
    int grid = ctx->prop.multiProcessorCount * ctas_per_sm;
    int64_t need_warps = (max_steps + 1) / 2;
    if ((int64_t)grid * kWarpsPerCta > need_warps) grid = (int)((need_warps + kWarpsPerCta - 1) / kWarpsPerCta);
    if (grid < 1) grid = 1;
    *partial_bytes = (size_t)grid * kWarpsPerCta * 2 * cmax * 16 * sizeof(float);
    *counter_bytes = (size_t)(J.max_jobs * tiles_per_job + 2) * sizeof(int);
}

int lev_stream_run(lev_ctx* ctx, const lev_weights* w, const lev_stream_job& J, const void* tables, int cmax, int terms,
                   float* y, const lev_stream_source* fused_src) {
    size_t pb, cb;
    lev_stream_workspace_bytes(ctx, w, J, cmax, &pb, &cb);
    void *pbuf, *counters;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_PARTIALS, pb, &pbuf));
    LEV_TRY(lev_scratch_zeroed(ctx, LEV_SCR_COUNTERS, cb, &counters));
    return lev_stream_run_ws(ctx, w, J, tables, cmax, terms, y, fused_src, pbuf, counters);
}

// the launch itself, on caller-provided work buffers (counters zero on entry; left zero on exit)
int lev_stream_run_ws(lev_ctx* ctx, const lev_weights* w, const lev_stream_job& J, const void* tables, int cmax, int terms,
                      float* y, const lev_stream_source* fused_src, void* pbuf, void* counters) {
    const int glt = cmax * terms, ntiles = (glt + 7) / 8;
    const int64_t chunks = lev_stream_chunks(w), steps = chunks / 4;
    const bool grouped = J.njobs_dev != nullptr;
    const int64_t tiles_per_job = (J.rows + 15) / 16;
    const int64_t max_steps = (int64_t)J.max_jobs * tiles_per_job * steps;
    if (max_steps > 0x7fffffff / 4) return lev_fail(ctx, LEV_EXCEEDS_WORKLOAD, "stream schedule: too many K-steps");

    int ctas_per_sm = env_int("LEV_STREAM_CTAS_PER_SM", 2);
    ctas_per_sm = ctas_per_sm < 1 ? 1 : (ctas_per_sm > 2 ? 2 : ctas_per_sm);
    int grid = ctx->prop.multiProcessorCount * ctas_per_sm;
    // a call with little work uses fewer warps, each with at least two K-steps
    int64_t need_warps = (max_steps + 1) / 2;
    if ((int64_t)grid * kWarpsPerCta > need_warps) grid = (int)((need_warps + kWarpsPerCta - 1) / kWarpsPerCta);
    if (grid < 1) grid = 1;
    const int max_warps = grid * kWarpsPerCta;

    size_t fb;
    size_t tb = lev_stream_table_bytes(w, cmax, terms, 1, &fb);
    size_t ring = (size_t)kWarpsPerCta * kDepth * kStepBytes;
    // stage the tables in shared memory when the call is dense and two CTAs still fit
    bool xs = !grouped && ring + tb <= 110 * 1024;

    size_t fb_all;
    lev_stream_table_bytes(w, cmax, terms, J.max_jobs, &fb_all);
    StreamArgs A;
    A.wp = (const uint4*)w->packed + (J.row0 / 16) * steps * 144;
    A.steps_per_tile = (int)steps;
    A.tiles_per_job = (int)tiles_per_job;
    A.max_warps = max_warps;
    A.total_steps = (int)max_steps;
    A.njobs_dev = J.njobs_dev;
    A.job_slice = J.job_slice;
    A.outmap = J.outmap;
    A.rows = J.rows;
    A.out_ld = J.out_ld;
    A.chunks = (int)chunks;
    A.frag = (const uint4*)tables;
    A.aux = (const float*)((const char*)tables + fb_all);
    A.cmax = cmax;
    A.terms = terms;
    A.glt = glt;
    A.partials = (float*)pbuf;
    A.tile_count = (int*)counters;
    A.status = ctx->d_status;
    A.y = y;
    A.debug = env_int("LEV_STREAM_DEBUG", 0);
    A.fused_prep = 0;
    if (fused_src) {
        if (!xs) return lev_fail(ctx, LEV_BAD_ARGUMENT, "stream schedule: tables do not fit shared memory");
        A.fused_prep = 1;
        A.prep = make_prep(ctx, w, *fused_src, cmax, terms, nullptr, 1);
    } else {
        A.prep = PrepArgs();
    }
    size_t smem = ring + (xs ? tb : 0);
    int st;
#define LEV_PICK(T)                                                                                          \
    (ntiles == 1 ? (xs ? launch_stream<T, 1, true>(ctx, grid, smem, A) : launch_stream<T, 1, false>(ctx, grid, smem, A)) \
                 : (xs ? launch_stream<T, 2, true>(ctx, grid, smem, A) : launch_stream<T, 2, false>(ctx, grid, smem, A)))
    st = w->type == LEV_GGML_Q4_K ? LEV_PICK(LEV_GGML_Q4_K) : LEV_PICK(LEV_GGML_Q4_0);
#undef LEV_PICK
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = grid;
    ctx->ev.block = kWarpsPerCta * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_stream");
}

int lev_launch_matvec_stream(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols,
                             float* y) {
    const int terms = lev_stream_terms(n_cols);
    lev_stream_source src = {};
    src.x = x;
    src.ld = w->cols;
    lev_stream_job J = {};
    J.row0 = row0;
    J.rows = rows;
    J.out_ld = rows;
    J.max_jobs = 1;
    // building the tables inside every CTA is available but measured slower than the
    // separate preparation launch, so it is opt-in
    if (lev_stream_fuses_prepare(w, n_cols, terms) && getenv("LEV_STREAM_FUSED_PREP"))
        return lev_stream_run(ctx, w, J, nullptr, n_cols, terms, y, &src);
    void* tables;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_XPREP, lev_stream_table_bytes(w, n_cols, terms, 1, nullptr) + 256, &tables));
    LEV_TRY(lev_stream_prepare(ctx, w, src, n_cols, terms, 1, tables));
    return lev_stream_run(ctx, w, J, tables, n_cols, terms, y, nullptr);
}
