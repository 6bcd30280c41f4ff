// The two ends of a decode step: the embedding row of a token id read out of a quantized tensor
// (g4_q6_embed_row, Sources/LeviathanCore/Gemma4.swift:4210-4245, called with scale = sqrt(hidden) at
// :3560-3578), and the softcap of the final logits (g4_softcap, Gemma4.swift:4496-4503, with the
// overflow-safe tanh of :4360-4367).  Token ids are device memory, so the id a previous step's argmax
// wrote feeds the next step without a host round trip.
//
// A decoded value is formed in the reference's order, ((d * s) * level) * scale for Q6_K, every product
// rounded to f32; the Q4_0 and Q4_K forms multiply their decoded value (Q4.swift:54-69,
// rust/crates/lev-cpu/src/lib.rs:110-130) by scale the same way.
#include <cuda_fp16.h>

#include "lev_internal.h"
#include "lev_stream_math.cuh"

namespace {

__device__ __forceinline__ float h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

__device__ __forceinline__ float q6k_value(const uint8_t* blk, unsigned j) {
    const float d = h2f((unsigned)blk[208] | ((unsigned)blk[209] << 8));
    const unsigned c = j >> 7, l0 = j & 127u, quarter = l0 >> 5, lane = l0 & 31u;
    const unsigned ql = blk[c * 64u + lane + ((quarter & 1u) ? 32u : 0u)];
    const unsigned h = blk[128u + c * 32u + lane];
    const float s = (float)(int)(int8_t)blk[192u + c * 8u + 2u * quarter + (lane >> 4)];
    const unsigned lo = quarter < 2u ? (ql & 15u) : (ql >> 4);
    const float level = (float)((int)(lo | (((h >> (2u * quarter)) & 3u) << 4)) - 32);
    return __fmul_rn(__fmul_rn(d, s), level);
}

__device__ __forceinline__ float q4_0_value(const uint8_t* blk, unsigned j) {
    const float d = h2f((unsigned)blk[0] | ((unsigned)blk[1] << 8));
    const unsigned b = blk[2u + (j & 15u)];
    return __fmul_rn(d, (float)(j < 16u ? (b & 15u) : (b >> 4)) - 8.0f);
}

__device__ __forceinline__ float q4k_value(const uint8_t* blk, unsigned j) {
    const float d = h2f((unsigned)blk[0] | ((unsigned)blk[1] << 8)), dmin = h2f((unsigned)blk[2] | ((unsigned)blk[3] << 8));
    const uint8_t* s = blk + 4;
    const unsigned sub = j >> 5, l = j & 31u;
    unsigned sc, mn;
    if (sub < 4) {
        sc = s[sub] & 63u;
        mn = s[sub + 4] & 63u;
    } else {
        sc = (s[sub + 4] & 15u) | ((s[sub - 4] >> 6) << 4);
        mn = (s[sub + 4] >> 4) | ((s[sub] >> 6) << 4);
    }
    const unsigned b = blk[16u + (sub >> 1) * 32u + l];
    const float q = (float)((sub & 1u) ? (b >> 4) : (b & 15u));
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), q), __fmul_rn(dmin, (float)mn));
}

// one thread per value of every requested row; a token id outside [0, rows) leaves zeros and raises the
// context's status word instead of reading past the tensor
template <int TYPE>
__global__ void __launch_bounds__(256) k_embed_rows(const uint8_t* __restrict__ w, int64_t rows, int cols, int bpr,
                                                      const int32_t* __restrict__ tokens, int64_t total, float scale,
                                                      float* __restrict__ y, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr unsigned kValues = TYPE == LEV_GGML_Q4_0 ? 32u : 256u;
    constexpr unsigned kBytes = TYPE == LEV_GGML_Q4_0 ? LEV_Q4_0_BYTES : (TYPE == LEV_GGML_Q4_K ? LEV_Q4_K_BYTES : LEV_Q6_K_BYTES);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / cols;
        const unsigned v = (unsigned)(i - t * cols);
        const int64_t row = tokens[t];
        if (row < 0 || row >= rows) {
            if (v == 0) atomicOr(status, LEV_DEV_BAD_INDEX);
            y[i] = 0.f;
            continue;
        }
        const uint8_t* blk = w + ((size_t)row * bpr + v / kValues) * kBytes;
        const unsigned j = v % kValues;
        const float val = TYPE == LEV_GGML_Q4_0 ? q4_0_value(blk, j) : (TYPE == LEV_GGML_Q4_K ? q4k_value(blk, j) : q6k_value(blk, j));
        y[i] = __fmul_rn(val, scale);
    }
}

__global__ void __launch_bounds__(256) k_softcap(float* __restrict__ x, int64_t n, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float a = x[i] / cap;
        const float e = expf(-2.0f * fabsf(a));
        x[i] = cap * copysignf((1.0f - e) / (1.0f + e), a);
    }
}

int grid_for(lev_ctx* ctx, int64_t n) {
    const int64_t blocks = (n + 255) / 256, cap = (int64_t)ctx->prop.multiProcessorCount * 8;
    return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace

extern "C" int lev_embed_rows(lev_ctx* ctx, const lev_weights* w, const int32_t* tokens, int64_t n_tokens, float scale, float* y) {
    if (!ctx || !w || !tokens || !y) return LEV_BAD_ARGUMENT;
    if (n_tokens <= 0 || n_tokens > (int64_t)1 << 24) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%lld tokens", (long long)n_tokens);
    if (!isfinite(scale)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "scale %g", (double)scale);
    if (!w->raw) return lev_fail(ctx, LEV_BAD_ARGUMENT, "the tensor's GGUF-order copy was released; embedding rows are read from it");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t total = n_tokens * w->cols;
    const int grid = grid_for(ctx, total);
    int* status = ctx->d_status;
#define LEV_EMBED(T)                                                                                                         \
    LEV_CUDA(ctx, launch_pdl(k_embed_rows<T>, dim3(grid), dim3(256), 0, ctx->stream, (const uint8_t*)w->raw, w->rows, (int)w->cols, \
                             (int)w->blocks_per_row, tokens, total, scale, y, status))
    if (w->type == LEV_GGML_Q4_0) {
        LEV_EMBED(LEV_GGML_Q4_0);
    } else if (w->type == LEV_GGML_Q4_K) {
        LEV_EMBED(LEV_GGML_Q4_K);
    } else {
        LEV_EMBED(LEV_GGML_Q6_K);
    }
#undef LEV_EMBED
    ctx->launches++;
    return LEV_OK;
}

extern "C" int lev_softcap(lev_ctx* ctx, float* x, int64_t n, float cap) {
    if (!ctx || !x) return LEV_BAD_ARGUMENT;
    if (n <= 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%lld elements", (long long)n);
    if (!(cap > 0.f) || !isfinite(cap)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "cap %g", (double)cap);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    LEV_CUDA(ctx, launch_pdl(k_softcap, dim3(grid_for(ctx, n)), dim3(256), 0, ctx->stream, x, n, cap));
    ctx->launches++;
    return LEV_OK;
}
