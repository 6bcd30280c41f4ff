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
// f32 activations are split into two fp16 terms (x = h0 + h1*2^-11, exact to
// 2^-22 relative) that occupy separate mma columns, so the tensor-core
// products are exact and the remaining rounding is the f32 accumulation.  Block scales are applied to the f32
// accumulators per sub-block; the Q4_0 "-8" offset enters as the accumulator
// initial value and the Q4_K min term is accumulated on CUDA cores.
//
// Data movement.  Tiles are handed to CTAs in groups whose K-steps the CTA's warps split
// evenly (a dense call sizes the groups so that the whole tensor is one resident wave; a
// grouped call, whose tile count only the device knows, lets the CTAs stride over groups).
// Every warp owns a private ring of shared-memory stages filled by bulk asynchronous copies
// (cp.async.bulk global->shared completing on an mbarrier) that it issues itself; no registers
// hold data in flight and warps never wait for each other.
//
// Reduction.  Tiles that lie wholly in one warp's range are written straight to y; for the
// others each warp leaves one f32 per (row, column) in a shared-memory record and the CTA adds
// the records in warp order after a barrier, so the same call always gives the same bits.
//
// This file serves the grouped expert FFN, dense calls with 5..8 columns and dense calls whose
// activation tables do not fit shared memory; lev_dense.cu holds the one-launch kernel for the
// rest.
#include "lev_stream.h"
#include "lev_stream_math.cuh"

namespace {


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

// One sum of a chunk's activations by a whole warp (xor butterfly, fixed order).
// Q4_K: which = activation column c; the true x of the 32-value sub-block sb (0, 1).
// Q4_0: which = mma column; what the tensor core sees of block sb (0, 1), times -8 * 2^-24:
//       low-nibble slots carry term(x), high-nibble slots term(x/16) against nibbles worth 16x.
// Q6_K: which = mma column; the same for the two 16-value sub-blocks 2*sb, 2*sb+1 (lanes
//       0..15 / 16..31), times -32 * 2^-24; the result of sub-block 2*sb + (lane >> 4).
template <int TYPE>
__device__ __forceinline__ float prep_sum32(const PrepArgs& P, int job, int chunk, int sb, int which, int lane) {
    const int c = TYPE == LEV_GGML_Q4_K ? which : which / P.terms;
    const int term = TYPE == LEV_GGML_Q4_K ? 0 : which - c * P.terms;
    const int row = P.rowmap ? P.rowmap[job * P.cmax + c] : c;
    const int64_t e = (int64_t)chunk * 64 + sb * 32 + lane;
    float xv = prep_src(P, row, e);
    if (P.act_out && term == 0 && row >= 0 && e < P.cols) P.act_out[(int64_t)row * P.cols + e] = xv;
    float s = xv;
    if (TYPE == LEV_GGML_Q4_0) s = lane < 16 ? split_term(xv, term) : 16.0f * split_term(xv * kHiScale, term);
    if (TYPE == LEV_GGML_Q6_K) s = sb == 0 ? split_term(xv, term) : 16.0f * split_term(xv * kHiScale, term);
#pragma unroll
    for (int d = (TYPE == LEV_GGML_Q6_K ? 8 : 16); d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (TYPE == LEV_GGML_Q4_K) return s;
    return (TYPE == LEV_GGML_Q6_K ? -32.0f : -8.0f) * 5.9604644775390625e-08f * s;
}

// grid (chunks, jobs); one warp per 8 mma columns

template <int TYPE>
__global__ void k_prepare_x(PrepArgs P) {
    pdl_launch_dependents();
    pdl_wait();  // x may be the previous kernel's output, and that kernel may still read the tables
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
    } else if (TYPE == LEV_GGML_Q6_K) {
        for (int cc = 0; cc < 8; cc++) {
            const int col2 = nt * 8 + cc;  // uniform across the warp
            if (col2 >= P.glt) break;
#pragma unroll
            for (int half = 0; half < 2; half++) {  // sub-blocks 2*half, 2*half+1 of the chunk
                float s = prep_sum32<TYPE>(P, job, chunk, half, col2, lane);
                if ((lane & 15) == 0)
                    P.aux[(((int64_t)job * P.chunks + chunk) * 4 + 2 * half + (lane >> 4)) * P.glt + col2] = s;
            }
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

// Q6_K: per (tile, block) 210 units of 16 B:
//   [0, 16)    the 16 int8 sub-block scales of each row (row order)
//   [16, 18)   the fp16 d of the 16 rows
//   [18, 146)  per chunk c (64 columns) 32 lane units: the low 4 bits of the levels; lane (g, t)
//              holds 8 B of row g then 8 B of row g+8.  In a row's two words W0, W1, the level of
//              element 16m + 4t + j of the chunk sits in word m&1, low (m<2) or high (m>=2)
//              nibble of byte {0, 2, 1, 3}[j]  -- the order the A-fragment masks pick them up.
//   [146, 210) per chunk 32 lane units of 8 B: the high 2 bits, one word per row; the field of
//              (m, j) sits at bit {4, 6, 2, 0, 8, 10, 12, 14}[2m + (j >> 1)] + 16 * (j & 1).
__device__ __forceinline__ unsigned q6k_level(const uint8_t* blk, int e) {  // stored 6-bit level of element e (0..255)
    int hb = e >> 7, rem = e & 127, grp = rem >> 5, l = rem & 31;
    unsigned ql = blk[64 * hb + ((grp & 1) ? 32 : 0) + l];
    unsigned lo = (grp & 2) ? (ql >> 4) : (ql & 15u);
    unsigned hi = (blk[128 + 32 * hb + l] >> (2 * grp)) & 3u;
    return lo | (hi << 4);
}
__global__ void k_repack_q6k(const uint8_t* __restrict__ raw, int64_t rows, int64_t bpr, int64_t tiles,
                             uint4* __restrict__ out) {
    int64_t total = tiles * bpr * 210;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        int64_t tb = u / 210;
        int k = (int)(u - tb * 210);
        int64_t tile = tb / bpr, b = tb - tile * bpr;
        unsigned w[4] = {0, 0, 0, 0};
        if (k < 16) {
            int64_t row = tile * 16 + k;
            if (row < rows) {
                const uint8_t* p = raw + (row * bpr + b) * LEV_Q6_K_BYTES + 192;
                for (int i = 0; i < 16; i++) w[i >> 2] |= (unsigned)p[i] << (8 * (i & 3));
            }
        } else if (k < 18) {
            for (int i = 0; i < 8; i++) {
                int64_t row = tile * 16 + (k - 16) * 8 + i;
                unsigned d = 0;
                if (row < rows) {
                    const uint8_t* p = raw + (row * bpr + b) * LEV_Q6_K_BYTES + 208;
                    d = (unsigned)p[0] | ((unsigned)p[1] << 8);
                }
                w[i >> 1] |= d << (16 * (i & 1));
            }
        } else if (k < 146) {
            int c = (k - 18) >> 5, lane = (k - 18) & 31, g = lane >> 2, t = lane & 3;
            for (int rr = 0; rr < 2; rr++) {
                int64_t row = tile * 16 + g + 8 * rr;
                if (row >= rows) continue;
                const uint8_t* blk = raw + (row * bpr + b) * LEV_Q6_K_BYTES;
                for (int m = 0; m < 4; m++)
                    for (int j = 0; j < 4; j++) {
                        unsigned lv = q6k_level(blk, 64 * c + 16 * m + 4 * t + j) & 15u;
                        const int byte = j == 0 ? 0 : (j == 1 ? 2 : (j == 2 ? 1 : 3));
                        w[2 * rr + (m & 1)] |= lv << (8 * byte + ((m & 2) ? 4 : 0));
                    }
            }
        } else {
            // two lanes per 16-byte unit
            int idx = (k - 146) * 2;
            for (int hl = 0; hl < 2; hl++) {
                int c = (idx + hl) >> 5, lane = (idx + hl) & 31, g = lane >> 2, t = lane & 3;
                for (int rr = 0; rr < 2; rr++) {
                    int64_t row = tile * 16 + g + 8 * rr;
                    if (row >= rows) continue;
                    const uint8_t* blk = raw + (row * bpr + b) * LEV_Q6_K_BYTES;
                    for (int m = 0; m < 4; m++)
                        for (int j = 0; j < 4; j++) {
                            unsigned hv = q6k_level(blk, 64 * c + 16 * m + 4 * t + j) >> 4;
                            const int pos[8] = {4, 6, 2, 0, 8, 10, 12, 14};
                            w[2 * hl + rr] |= hv << (pos[2 * m + (j >> 1)] + 16 * (j & 1));
                        }
                }
            }
        }
        out[u] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// ---------------------------------------------------------------------------
// streaming kernel
// ---------------------------------------------------------------------------
struct StreamArgs {
    const uint4* wp;        // packed weights: first tile of this call (dense) or of the tensor (grouped)
    int steps_per_tile;     // K-steps per tile
    int tiles_per_job;      // tiles of one job (one expert slice; the whole call when dense)
    int tiles_per_group;    // tiles one CTA works on at a time, their K-steps split over its warps
    int total_tiles;        // dense: tiles of the call
    const int* njobs_dev;   // grouped: device count of jobs (total steps = jobs * tiles_per_job * steps_per_tile)
    const int* job_slice;   // grouped: [job] index of the expert slice, in units of tiles_per_job tiles
    const int* outmap;      // grouped: [job][cmax] output row of each column, -1 = none; NULL: column index
    int64_t rows;           // rows of one job
    int64_t out_ld;         // elements between output columns
    int out_cols;           // output columns that exist (dense: the call's n_cols)
    int chunks;             // padded 64-column chunks of the activation tables
    const uint4* frag;      // [job][chunk][glt][4] x 32 B
    const float* aux;       // Q4_K: [job][sub-block][cmax] ; Q4_0: [job][chunk][2][glt]
    int cmax, terms, glt;
    int* status;            // device status word
    float* y;
    int depth;              // ring stages per warp
};

// W: warps per CTA; OCC: CTAs per SM the register budget is sized for
template <int TYPE, int CMAX, bool XS, int W, int OCC>
__global__ void __launch_bounds__(W * 32, OCC) k_stream(StreamArgs A) {
    using D = StreamDims<CMAX>;
    constexpr int NT = D::kNT, GLT = D::kGlt, TERMS = D::kTerms;
    constexpr int kWarpsPerCta = W;
    constexpr int kStepBytes = step_bytes(TYPE);
    constexpr int kAuxPerChunk = TYPE == LEV_GGML_Q4_K ? 2 * CMAX : (TYPE == LEV_GGML_Q6_K ? 4 * GLT : 2 * GLT);
    const int kDepth = A.depth;  // ring stages per warp (1..4)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[W][4];
    __shared__ float rec[W][2][CMAX][16];  // partial sums of tiles a warp shares with its neighbours
    __shared__ int rec_tile[W][2];         // group-local tile of each record, -1 = none
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int spt = A.steps_per_tile, tpg = A.tiles_per_group;
    const int total_tiles = A.njobs_dev ? *A.njobs_dev * A.tiles_per_job : A.total_tiles;
    const int groups = (total_tiles + tpg - 1) / tpg;

    // K-step range of this warp inside group grp: the group's steps are split evenly over the warps
    auto warp_range = [&](int grp, int& s, int& e, int& per) {
        int nt_here = total_tiles - grp * tpg < tpg ? total_tiles - grp * tpg : tpg;
        int nst = nt_here * spt;
        per = (nst + kWarpsPerCta - 1) / kWarpsPerCta;
        s = warp * per;
        e = s + per < nst ? s + per : nst;
        if (s > e) s = e;
    };

    unsigned char* ring = smem_raw + (size_t)warp * kDepth * kStepBytes;
    const unsigned ring_s = smem_u32(ring), bar_s = smem_u32(&bars[warp][0]);
    // fetch cursor (used by lane 0): walks this warp's K-steps over all of the CTA's groups
    int f_grp = blockIdx.x, f_s = 0, f_e = 0, f_gt = 0, f_k = 0;
    auto fetch_seek = [&]() {  // position on the first step of group f_grp
        int per;
        warp_range(f_grp, f_s, f_e, per);
        f_gt = f_grp * tpg + f_s / spt;
        f_k = f_s - (f_s / spt) * spt;
    };
    auto fetch_next = [&]() -> const unsigned char* {  // address of the next K-step, nullptr when done
        while (f_grp < groups && f_s >= f_e) {
            f_grp += gridDim.x;
            if (f_grp < groups) fetch_seek();
        }
        if (f_grp >= groups) return nullptr;
        int64_t tile = f_gt;
        if (A.job_slice) {
            int job = f_gt / A.tiles_per_job;
            tile = (int64_t)A.job_slice[job] * A.tiles_per_job + (f_gt - job * A.tiles_per_job);
        }
        const unsigned char* p = reinterpret_cast<const unsigned char*>(A.wp) + (tile * spt + f_k) * (int64_t)kStepBytes;
        f_s++;
        if (++f_k == spt) {
            f_k = 0;
            f_gt++;
        }
        return p;
    };
    if (lane == 0) {
        for (int d = 0; d < kDepth; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        if (f_grp < groups) fetch_seek();
        for (int d = 0; d < kDepth; d++) {
            const unsigned char* p = fetch_next();
            if (p) bulk_load(ring_s + d * kStepBytes, p, kStepBytes, bar_s + 8 * d);
        }
    }
    pdl_launch_dependents();
    pdl_wait();  // the weight requests above are already in flight; the tables come from the preceding launch
    // dense calls stage the activation tables once per CTA while the first weight bytes are on their way
    const uint4* jfrag = A.frag;
    const float* jaux = A.aux;
    if (XS) {
        uint4* xs = reinterpret_cast<uint4*>(smem_raw + (size_t)kWarpsPerCta * kDepth * kStepBytes);
        const int nfrag = A.chunks * GLT * 8;  // uint4 units
        const int naux = A.chunks * kAuxPerChunk;
        float* sa = reinterpret_cast<float*>(xs + nfrag);
        for (int i = threadIdx.x; i < nfrag; i += blockDim.x) xs[i] = __ldg(A.frag + i);
        for (int i = threadIdx.x; i < naux; i += blockDim.x) sa[i] = __ldg(A.aux + i);
        jfrag = xs;
        jaux = sa;
    }
    __syncthreads();

    // per-lane table offsets.  A chunk's fragments are [GLT columns][4 t] x 32 B, so lane (g, t) of
    // n-tile nt reads entry nt*32 + lane; lanes beyond the live columns read a valid entry whose
    // values land in accumulator columns nobody reads.
    LaneOffsets<CMAX> O;
    O.init(lane);

    float yacc[NT][4];
    float mina[CMAX], minb[CMAX];
    int slot = 0;          // ring stage of the next K-step
    unsigned phase = 0;    // its mbarrier phase parity
    bool dead = false;   // a bounded wait ran out: skip the work, keep meeting the barriers

    for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
        int s, e, per;
        warp_range(grp, s, e, per);
        if (lane < 2) rec_tile[warp][lane] = -1;
        int tl = s / spt;            // group-local tile
        int k = s - tl * spt;        // K-step inside the tile
        int seg_k0 = k;
        const int first_tl = tl;
        int job = (grp * tpg + tl) / A.tiles_per_job;
        if (!XS) {
            jfrag = A.frag + (int64_t)job * A.chunks * GLT * 8;
            jaux = A.aux + (int64_t)job * A.chunks * kAuxPerChunk;
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
        for (int c = 0; c < CMAX; c++) mina[c] = minb[c] = 0.f;

        for (int i = s; i < e && !dead; i++) {
            if (!mbar_wait(bar_s + 8 * slot, phase)) {
                if (lane == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
                dead = true;
                break;
            }
            const uint4* st = reinterpret_cast<const uint4*>(ring + slot * kStepBytes);
            const uint4* xchunk = jfrag + k * (4 * GLT * 8);
            const float* achunk = jaux + k * (4 * kAuxPerChunk);

            stream_step<TYPE, CMAX, XS>(st, xchunk, achunk, lane, O, yacc, mina, minb);

            // every lane has consumed its shared-memory reads of this stage: refill it
            __syncwarp();
            if (lane == 0) {
                const unsigned char* p = fetch_next();
                if (p) bulk_load(ring_s + slot * kStepBytes, p, kStepBytes, bar_s + 8 * slot);
            }
            if (++slot == kDepth) {
                slot = 0;
                phase ^= 1u;
            }

            k++;
            if (k == spt || i == e - 1) {
                // ---- this warp's segment of the tile ends: fold to one f32 per (row, column) ----
                const bool whole = seg_k0 == 0 && k == spt;
                const int r = tl == first_tl ? 0 : 1;
                const int gt = grp * tpg + tl;
                const int tile_in_job = gt - job * A.tiles_per_job;
#pragma unroll
                for (int c = 0; c < CMAX; c++) {
                    float va = 0.f, vb = 0.f;
#pragma unroll
                    for (int term = 0; term < TERMS; term++) {
                        constexpr float kScale[3] = {1.0f, 4.8828125e-4f, 2.384185791015625e-7f};  // 2^0, 2^-11, 2^-22
                        const int col = c * TERMS + term, nt = col / 8, jj = col & 1;
                        const bool mine = t == (col % 8) / 2;
                        va = fmaf(mine ? yacc[nt][jj] : 0.f, kScale[term], va);
                        vb = fmaf(mine ? yacc[nt][2 + jj] : 0.f, kScale[term], vb);
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
                            const int oc = A.outmap ? A.outmap[job * CMAX + c] : c;
                            const int64_t row = (int64_t)tile_in_job * 16 + g;
                            if (oc >= 0 && oc < A.out_cols) {
                                if (row < A.rows) A.y[(int64_t)oc * A.out_ld + row] = va;
                                if (row + 8 < A.rows) A.y[(int64_t)oc * A.out_ld + row + 8] = vb;
                            }
                        } else {
                            rec[warp][r][c][g] = va;
                            rec[warp][r][c][g + 8] = vb;
                        }
                    }
                }
                if (!whole && lane == 0) rec_tile[warp][r] = tl;
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
                for (int c = 0; c < CMAX; c++) mina[c] = minb[c] = 0.f;
                tl++;
                k = 0;
                seg_k0 = 0;
                if (!XS && grp * tpg + tl - job * A.tiles_per_job >= A.tiles_per_job) {
                    job++;
                    jfrag = A.frag + (int64_t)job * A.chunks * GLT * 8;
                    jaux = A.aux + (int64_t)job * A.chunks * kAuxPerChunk;
                }
            }
        }
        __syncthreads();
        // ---- tiles shared between warps: add the warps' records in warp order ----
        {
            const int nt_here = total_tiles - grp * tpg < tpg ? total_tiles - grp * tpg : tpg;
            for (int item = threadIdx.x; item < nt_here * CMAX * 16; item += blockDim.x) {
                const int tile = item / (CMAX * 16), idx = item - tile * (CMAX * 16);
                const int w_first = (tile * spt) / per, w_last = (tile * spt + spt - 1) / per;
                if (w_first == w_last) continue;  // one warp had the whole tile and wrote it
                float acc = 0.f;
                for (int w = w_first; w <= w_last; w++) acc += rec[w][rec_tile[w][0] == tile ? 0 : 1][0][idx];
                const int gt = grp * tpg + tile, pjob = gt / A.tiles_per_job, ptile = gt - pjob * A.tiles_per_job;
                const int c = idx >> 4;
                const int oc = A.outmap ? A.outmap[pjob * CMAX + c] : c;
                const int64_t row = (int64_t)ptile * 16 + (idx & 15);
                if (oc >= 0 && oc < A.out_cols && row < A.rows) A.y[(int64_t)oc * A.out_ld + row] = acc;
            }
        }
        __syncthreads();
    }
}

int grid_cap(lev_ctx* ctx, int64_t work, int block, int per_sm) {
    int64_t g = (work + block - 1) / block, cap = (int64_t)ctx->prop.multiProcessorCount * per_sm;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}


template <int TYPE, int CMAX, bool XS, int W, int OCC>
int launch_stream(lev_ctx* ctx, int grid, size_t smem, const StreamArgs& A) {
    static size_t configured[16] = {};  // per device: largest dynamic shared memory opted in so far
    if (configured[ctx->device & 15] < smem) {
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_stream<TYPE, CMAX, XS, W, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[ctx->device & 15] = smem;
    }
    LEV_CUDA(ctx, launch_pdl(k_stream<TYPE, CMAX, XS, W, OCC>, dim3(grid), dim3(W * 32), smem, ctx->stream, A));
    return LEV_OK;
}

// variant 0: eight warps, two CTAs per SM, tables read from global memory (grouped / oversized tables)
// variant 1: eight warps, two CTAs per SM, tables in shared memory
// variant 2: twenty-four warps, one CTA per SM, tables in shared memory
template <int TYPE, int CMAX>
int launch_stream_variant(lev_ctx* ctx, int grid, size_t smem, const StreamArgs& A, int variant) {
    if (variant == 0) return launch_stream<TYPE, CMAX, false, kWarpsPerCta, 2>(ctx, grid, smem, A);
    if (variant == 2 && CMAX <= 4) return launch_stream<TYPE, (CMAX <= 4 ? CMAX : 1), true, kWarpsWide, 1>(ctx, grid, smem, A);
    return launch_stream<TYPE, CMAX, true, kWarpsPerCta, 2>(ctx, grid, smem, A);
}

template <int TYPE>
int launch_stream_cmax(lev_ctx* ctx, int cmax, int grid, size_t smem, const StreamArgs& A, int variant) {
    switch (cmax) {
        case 1: return launch_stream_variant<TYPE, 1>(ctx, grid, smem, A, variant);
        case 2: return launch_stream_variant<TYPE, 2>(ctx, grid, smem, A, variant);
        case 3: return launch_stream_variant<TYPE, 3>(ctx, grid, smem, A, variant);
        case 4: return launch_stream_variant<TYPE, 4>(ctx, grid, smem, A, variant);
        case 5: return launch_stream_variant<TYPE, 5>(ctx, grid, smem, A, variant);
        case 6: return launch_stream_variant<TYPE, 6>(ctx, grid, smem, A, variant);
        case 7: return launch_stream_variant<TYPE, 7>(ctx, grid, smem, A, variant);
        case 8: return launch_stream_variant<TYPE, 8>(ctx, grid, smem, A, variant);
    }
    return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", cmax);
}


}  // namespace

int lev_stream_terms(int n_cols) {
    (void)n_cols;
    return 2;
}

// 64-column chunks of the activation tables; Q4_0 rows are padded with zero
// blocks to whole K-steps of four chunks
int64_t lev_stream_chunks(const lev_weights* w) {
    int64_t c = (w->cols + 63) / 64;
    return w->type == LEV_GGML_Q4_0 ? (c + 3) / 4 * 4 : c;
}

int lev_repack_weights(lev_ctx* ctx, lev_weights* w) {
    int64_t tiles = (w->rows + 15) / 16;
    int64_t steps = lev_stream_chunks(w) / 4;
    size_t bytes = (size_t)tiles * steps * step_bytes(w->type);
    LEV_CUDA(ctx, cudaMalloc((void**)&w->packed, bytes + 256));
    w->packed_bytes = bytes;
    w->packed_rows = tiles * 16;
    int grid = grid_cap(ctx, (int64_t)(bytes / 16), 256, 16);
    if (w->type == LEV_GGML_Q4_K)
        k_repack_q4k<<<grid, 256, 0, ctx->stream>>>(w->raw, w->rows, w->blocks_per_row, tiles, (uint4*)w->packed);
    else if (w->type == LEV_GGML_Q6_K)
        k_repack_q6k<<<grid, 256, 0, ctx->stream>>>(w->raw, w->rows, w->blocks_per_row, tiles, (uint4*)w->packed);
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
    size_t ab = w->type == LEV_GGML_Q4_K   ? (size_t)jobs * chunks * 2 * cmax * sizeof(float)
                : w->type == LEV_GGML_Q6_K ? (size_t)jobs * chunks * 4 * glt * sizeof(float)
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
    dim3 block(32 * ntiles);
    if (w->type == LEV_GGML_Q4_K) LEV_CUDA(ctx, launch_pdl(k_prepare_x<LEV_GGML_Q4_K>, grid, block, 0, ctx->stream, P));
    else if (w->type == LEV_GGML_Q6_K) LEV_CUDA(ctx, launch_pdl(k_prepare_x<LEV_GGML_Q6_K>, grid, block, 0, ctx->stream, P));
    else LEV_CUDA(ctx, launch_pdl(k_prepare_x<LEV_GGML_Q4_0>, grid, block, 0, ctx->stream, P));
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

int lev_stream_run(lev_ctx* ctx, const lev_weights* w, const lev_stream_job& J, const void* tables, int cmax, int terms,
                   float* y) {
    const int glt = cmax * terms;
    const int64_t chunks = lev_stream_chunks(w), steps = chunks / 4;
    const bool grouped = J.njobs_dev != nullptr;
    const int64_t tiles_per_job = (J.rows + 15) / 16;
    const int64_t max_steps = (int64_t)J.max_jobs * tiles_per_job * steps;
    if (max_steps > 0x7fffffff / 4) return lev_fail(ctx, LEV_EXCEEDS_WORKLOAD, "stream schedule: too many K-steps");
    if (terms != lev_stream_terms(cmax)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "stream schedule: %d terms with %d columns", terms, cmax);

    const size_t kStepBytes = step_bytes(w->type);
    size_t tb = lev_stream_table_bytes(w, cmax, terms, 1, nullptr);
    const int64_t total_tiles = (int64_t)J.max_jobs * tiles_per_job;
    const int sms = ctx->prop.multiProcessorCount;
    const size_t smem_cap = 200 * 1024;
    // Variant and ring depth.  Dense calls with small tables run one CTA of 24 warps per SM: the
    // tables are staged once per SM and the ring is as deep as shared memory allows, so that for
    // decode-sized tensors every byte is requested at kernel start.  Everything else runs two
    // CTAs of eight warps per SM with a four-stage ring.
    int variant = grouped ? 0 : 1, warps = kWarpsPerCta, occ = 2, depth = 4;
    if (!grouped && cmax <= 4 && (size_t)kWarpsWide * kStepBytes + tb <= smem_cap) {
        variant = 2;
        warps = kWarpsWide;
        occ = 1;
    }
    if (variant == 1 && (size_t)kWarpsPerCta * 4 * kStepBytes + tb > 110 * 1024) variant = 0;
    // Tiles are handed to CTAs in groups whose K-steps the warps split evenly; every reduction
    // then stays inside one CTA.  A dense call sizes the groups so that the whole tensor is one
    // resident wave; a grouped call, whose tile count only the device knows, uses the smallest
    // useful group and lets the CTAs stride over them.
    const int resident = sms * occ;
    int tpg = (int)((2 * warps + steps - 1) / steps);  // at least two K-steps per warp
    if (!grouped && (total_tiles + resident - 1) / resident > tpg) tpg = (int)((total_tiles + resident - 1) / resident);
    int64_t ngroups = (total_tiles + tpg - 1) / tpg;
    int grid = (int)(ngroups < resident ? ngroups : resident);
    if (grid < 1) grid = 1;
    if (variant == 2) {
        int64_t per_warp = ((int64_t)tpg * steps + warps - 1) / warps;
        int fit = (int)((smem_cap - tb) / ((size_t)warps * kStepBytes));
        depth = (int)(per_warp < fit ? per_warp : fit);
        depth = depth < 1 ? 1 : (depth > 4 ? 4 : depth);
    }
    size_t ring = (size_t)warps * depth * kStepBytes;
    const bool xs = variant != 0;

    size_t fb_all;
    lev_stream_table_bytes(w, cmax, terms, J.max_jobs, &fb_all);
    StreamArgs A;
    A.wp = (const uint4*)w->packed + (J.row0 / 16) * steps * (kStepBytes / 16);
    A.steps_per_tile = (int)steps;
    A.tiles_per_job = (int)tiles_per_job;
    A.tiles_per_group = tpg;
    A.total_tiles = (int)total_tiles;
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
    A.status = ctx->d_status;
    A.y = y;
    A.out_cols = J.outmap ? 0x7fffffff : cmax;
    size_t smem = ring + (xs ? tb : 0);
    A.depth = depth;
    int st = w->type == LEV_GGML_Q4_K   ? launch_stream_cmax<LEV_GGML_Q4_K>(ctx, cmax, grid, smem, A, variant)
             : w->type == LEV_GGML_Q6_K ? launch_stream_cmax<LEV_GGML_Q6_K>(ctx, cmax, grid, smem, A, variant)
                                        : launch_stream_cmax<LEV_GGML_Q4_0>(ctx, cmax, grid, smem, A, variant);
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = grid;
    ctx->ev.block = warps * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_stream");
}

int lev_launch_matvec_stream(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols,
                             float* y) {
    if (n_cols == 1) {
        const lev_chain_item it = {w, row0, rows, x, y, 0, nullptr};
        if (lev_chain_preferred(ctx, 1, &it)) return lev_chain_run(ctx, 1, &it);
    }
    if (lev_dense_supported(ctx, w, row0, rows, x, n_cols)) return lev_dense_run(ctx, w, row0, rows, x, n_cols, y);
    const int terms = lev_stream_terms(n_cols);
    lev_stream_source src = {};
    src.x = x;
    src.ld = w->cols;
    lev_stream_job J = {};
    J.row0 = row0;
    J.rows = rows;
    J.out_ld = rows;
    J.max_jobs = 1;
    void* tables;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_XPREP, lev_stream_table_bytes(w, n_cols, terms, 1, nullptr) + 256, &tables));
    LEV_TRY(lev_stream_prepare(ctx, w, src, n_cols, terms, 1, tables));
    return lev_stream_run(ctx, w, J, tables, n_cols, terms, y);
}
