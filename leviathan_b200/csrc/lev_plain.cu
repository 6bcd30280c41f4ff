// Schedule 0 ("plain"): one warp per weight row over the raw GGUF block bytes,
// plus the bit-exact block dequantizer and the finite checks.
//
// The dequantized value of every element is formed exactly as the reference
// decoders form it -- Q4_0: d*(nib-8) (Sources/LeviathanCore/Q4.swift:54-69);
// Q4_K: (d*sc)*q - dmin*m (rust/crates/lev-cpu/src/lib.rs:110-130); Q6_K:
// (d*sc)*level (Sources/LeviathanCore/Q6.swift:24-62) -- and then multiplied
// into an f32 accumulator per lane; lanes are combined by an xor butterfly.
// These kernels are the correctness anchor and the fallback for geometries
// the stream schedule does not serve; they are not tuned for bandwidth.
#include <cuda_fp16.h>

#include "lev_internal.h"

namespace {

__device__ __forceinline__ float h2f(unsigned bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// 6-bit scale / min of sub-block j from the 12 packed bytes held in s[3]
// (rust/crates/lev-cpu/src/lib.rs:64-74)
__device__ __forceinline__ unsigned sbyte(const unsigned* s, int i) { return (s[i >> 2] >> (8 * (i & 3))) & 0xffu; }
__device__ __forceinline__ void q4k_scale_min(const unsigned* s, int j, unsigned* sc, unsigned* mn) {
    if (j < 4) {
        *sc = sbyte(s, j) & 63u;
        *mn = sbyte(s, j + 4) & 63u;
    } else {
        *sc = (sbyte(s, j + 4) & 0x0Fu) | ((sbyte(s, j - 4) >> 6) << 4);
        *mn = (sbyte(s, j + 4) >> 4) | ((sbyte(s, j) >> 6) << 4);
    }
}

// ---- per-format element decoders: item -> values and their column index ----

// Q4_0: item = (block, byte pair j): 4 values
struct Q40Item {
    static constexpr int kValues = 4;
    __device__ static int64_t items_per_row(int64_t bpr) { return bpr * 8; }
    __device__ static void decode(const uint8_t* row, int64_t item, float* v, int64_t* col) {
        int64_t blk = item >> 3;
        int j = (int)(item & 7);
        const unsigned short* bp = (const unsigned short*)(row + blk * LEV_Q4_0_BYTES);
        float d = h2f(bp[0]);
        unsigned q = bp[1 + j];
        int l = 2 * j;
        v[0] = __fmul_rn(d, (float)(q & 15u) - 8.0f);
        v[1] = __fmul_rn(d, (float)((q >> 4) & 15u) - 8.0f);
        v[2] = __fmul_rn(d, (float)((q >> 8) & 15u) - 8.0f);
        v[3] = __fmul_rn(d, (float)(q >> 12) - 8.0f);
        col[0] = blk * 32 + l;
        col[1] = blk * 32 + 16 + l;
        col[2] = blk * 32 + l + 1;
        col[3] = blk * 32 + 16 + l + 1;
    }
};

// Q4_K: item = (block, 32-bit word of qs): 8 values
struct Q4KItem {
    static constexpr int kValues = 8;
    __device__ static int64_t items_per_row(int64_t bpr) { return bpr * 32; }
    __device__ static void decode(const uint8_t* row, int64_t item, float* v, int64_t* col) {
        int64_t blk = item >> 5;
        int wi = (int)(item & 31);
        const unsigned* bp = (const unsigned*)(row + blk * LEV_Q4_K_BYTES);
        unsigned hdr = bp[0];
        float d = h2f(hdr & 0xffffu), dmin = h2f(hdr >> 16);
        unsigned s[3] = {bp[1], bp[2], bp[3]};
        unsigned word = bp[4 + wi];
        int c = wi >> 3, l0 = 4 * (wi & 7);
        unsigned sc1, m1, sc2, m2;
        q4k_scale_min(s, 2 * c, &sc1, &m1);
        q4k_scale_min(s, 2 * c + 1, &sc2, &m2);
        float d1 = __fmul_rn(d, (float)sc1), mm1 = __fmul_rn(dmin, (float)m1);
        float d2 = __fmul_rn(d, (float)sc2), mm2 = __fmul_rn(dmin, (float)m2);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            unsigned byte = (word >> (8 * k)) & 0xffu;
            v[2 * k] = __fsub_rn(__fmul_rn(d1, (float)(byte & 15u)), mm1);
            v[2 * k + 1] = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), mm2);
            col[2 * k] = blk * 256 + c * 64 + l0 + k;
            col[2 * k + 1] = blk * 256 + c * 64 + 32 + l0 + k;
        }
    }
};

// Q6_K: item = (block, half c, l): 4 values
struct Q6KItem {
    static constexpr int kValues = 4;
    __device__ static int64_t items_per_row(int64_t bpr) { return bpr * 64; }
    __device__ static void decode(const uint8_t* row, int64_t item, float* v, int64_t* col) {
        int64_t blk = item >> 6;
        int c = (int)((item >> 5) & 1), l = (int)(item & 31);
        const uint8_t* bp = row + blk * LEV_Q6_K_BYTES;
        float d = h2f((unsigned)bp[208] | ((unsigned)bp[209] << 8));
        unsigned qa = bp[64 * c + l], qb = bp[64 * c + 32 + l], h = bp[128 + 32 * c + l];
        int is = l >> 4;
        const int8_t* sc = (const int8_t*)(bp + 192 + 8 * c + is);
        int lv0 = (int)((qa & 15u) | ((h & 3u) << 4)) - 32;
        int lv1 = (int)((qb & 15u) | (((h >> 2) & 3u) << 4)) - 32;
        int lv2 = (int)((qa >> 4) | (((h >> 4) & 3u) << 4)) - 32;
        int lv3 = (int)((qb >> 4) | (((h >> 6) & 3u) << 4)) - 32;
        v[0] = __fmul_rn(__fmul_rn(d, (float)sc[0]), (float)lv0);
        v[1] = __fmul_rn(__fmul_rn(d, (float)sc[2]), (float)lv1);
        v[2] = __fmul_rn(__fmul_rn(d, (float)sc[4]), (float)lv2);
        v[3] = __fmul_rn(__fmul_rn(d, (float)sc[6]), (float)lv3);
        int64_t base = blk * 256 + c * 128 + l;
        col[0] = base;
        col[1] = base + 32;
        col[2] = base + 64;
        col[3] = base + 96;
    }
};

template <class Item, int NC>
__global__ void __launch_bounds__(256) k_matvec_plain(const uint8_t* __restrict__ w, int64_t bpr, int block_bytes,
                                                       int64_t rows, int64_t cols, const float* __restrict__ x,
                                                       float* __restrict__ y) {
    int lane = threadIdx.x & 31;
    int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    int64_t items = Item::items_per_row(bpr);
    for (int64_t row = warp; row < rows; row += nwarps) {
        const uint8_t* rp = w + row * bpr * block_bytes;
        float acc[NC];
#pragma unroll
        for (int c = 0; c < NC; c++) acc[c] = 0.f;
        for (int64_t it = lane; it < items; it += 32) {
            float v[Item::kValues];
            int64_t col[Item::kValues];
            Item::decode(rp, it, v, col);
#pragma unroll
            for (int k = 0; k < Item::kValues; k++)
#pragma unroll
                for (int c = 0; c < NC; c++) acc[c] = fmaf(v[k], __ldg(x + (int64_t)c * cols + col[k]), acc[c]);
        }
#pragma unroll
        for (int c = 0; c < NC; c++) {
            float s = warp_sum(acc[c]);
            if (lane == 0) y[(int64_t)c * rows + row] = s;
        }
    }
}

template <class Item>
__global__ void k_dequantize(const uint8_t* __restrict__ w, int64_t bpr, int block_bytes, int64_t rows,
                             int64_t cols, float* __restrict__ out) {
    int64_t items = Item::items_per_row(bpr);
    int64_t total = rows * items;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t row = i / items, it = i - row * items;
        float v[Item::kValues];
        int64_t col[Item::kValues];
        Item::decode(w + row * bpr * block_bytes, it, v, col);
#pragma unroll
        for (int k = 0; k < Item::kValues; k++) out[row * cols + col[k]] = v[k];
    }
}

__global__ void k_scale_check(const uint8_t* __restrict__ w, int64_t blocks, int type, int* status) {
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += (int64_t)gridDim.x * blockDim.x) {
        bool bad;
        if (type == LEV_GGML_Q4_0) {
            const unsigned short* p = (const unsigned short*)(w + b * LEV_Q4_0_BYTES);
            bad = (p[0] & 0x7C00u) == 0x7C00u;
        } else if (type == LEV_GGML_Q4_K) {
            const unsigned short* p = (const unsigned short*)(w + b * LEV_Q4_K_BYTES);
            bad = (p[0] & 0x7C00u) == 0x7C00u || (p[1] & 0x7C00u) == 0x7C00u;
        } else {
            const unsigned short* p = (const unsigned short*)(w + b * LEV_Q6_K_BYTES + 208);
            bad = (p[0] & 0x7C00u) == 0x7C00u;
        }
        if (bad) atomicOr(status, LEV_DEV_NONFINITE_SCALE);
    }
}

__global__ void k_finite_check(const float* __restrict__ v, int64_t n, int bit, int* status) {
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        bad |= !isfinite(v[i]);
    if (bad) atomicOr(status, bit);
}

int grid_for(lev_ctx* ctx, int64_t work_items, int block, int per_sm) {
    int64_t g = (work_items + block - 1) / block;
    int64_t cap = (int64_t)ctx->prop.multiProcessorCount * per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

template <class Item>
int launch_plain_nc(lev_ctx* ctx, const lev_weights* w, const uint8_t* base, int64_t rows, const float* x,
                    int n_cols, float* y) {
    const int block = 256;
    int grid = grid_for(ctx, rows * 32, block, 8);
    int bb = lev_block_bytes(w->type);
    switch (n_cols) {
#define LEV_CASE(N)                                                                                         \
    case N:                                                                                                 \
        k_matvec_plain<Item, N><<<grid, block, 0, ctx->stream>>>(base, w->blocks_per_row, bb, rows, w->cols, x, y); \
        break;
        LEV_CASE(1) LEV_CASE(2) LEV_CASE(3) LEV_CASE(4) LEV_CASE(5) LEV_CASE(6) LEV_CASE(7) LEV_CASE(8)
#undef LEV_CASE
        default:
            return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", n_cols);
    }
    ctx->launches++;
    ctx->ev.grid = grid;
    ctx->ev.block = block;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_matvec_plain");
}

}  // namespace

int lev_launch_matvec_plain(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x,
                            int n_cols, float* y) {
    if (!w->raw) return lev_fail(ctx, LEV_UNSUPPORTED, "the GGUF-order copy of this tensor was released: only the stream schedule serves it");
    const uint8_t* base = w->raw + (size_t)row0 * (size_t)w->blocks_per_row * (size_t)lev_block_bytes(w->type);
    if (w->type == LEV_GGML_Q4_0) return launch_plain_nc<Q40Item>(ctx, w, base, rows, x, n_cols, y);
    if (w->type == LEV_GGML_Q4_K) return launch_plain_nc<Q4KItem>(ctx, w, base, rows, x, n_cols, y);
    return launch_plain_nc<Q6KItem>(ctx, w, base, rows, x, n_cols, y);
}

int lev_launch_dequantize(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, float* out) {
    if (!w->raw) return lev_fail(ctx, LEV_UNSUPPORTED, "the GGUF-order copy of this tensor was released");
    int bb = lev_block_bytes(w->type);
    const uint8_t* base = w->raw + (size_t)row0 * (size_t)w->blocks_per_row * (size_t)bb;
    const int block = 256;
    if (w->type == LEV_GGML_Q4_0) {
        int grid = grid_for(ctx, rows * w->blocks_per_row * 8, block, 16);
        k_dequantize<Q40Item><<<grid, block, 0, ctx->stream>>>(base, w->blocks_per_row, bb, rows, w->cols, out);
    } else if (w->type == LEV_GGML_Q4_K) {
        int grid = grid_for(ctx, rows * w->blocks_per_row * 32, block, 16);
        k_dequantize<Q4KItem><<<grid, block, 0, ctx->stream>>>(base, w->blocks_per_row, bb, rows, w->cols, out);
    } else {
        int grid = grid_for(ctx, rows * w->blocks_per_row * 64, block, 16);
        k_dequantize<Q6KItem><<<grid, block, 0, ctx->stream>>>(base, w->blocks_per_row, bb, rows, w->cols, out);
    }
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_dequantize");
}

int lev_launch_scale_check(lev_ctx* ctx, const lev_weights* w) {
    int64_t blocks = w->rows * w->blocks_per_row;
    int grid = grid_for(ctx, blocks, 256, 16);
    k_scale_check<<<grid, 256, 0, ctx->stream>>>(w->raw, blocks, w->type, ctx->d_status);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_scale_check");
}

int lev_launch_finite_check(lev_ctx* ctx, const float* v, int64_t n, int bit) {
    int grid = grid_for(ctx, n, 256, 8);
    k_finite_check<<<grid, 256, 0, ctx->stream>>>(v, n, bit, ctx->d_status);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_finite_check");
}
