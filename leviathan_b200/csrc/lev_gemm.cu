// Prefill dequant-GEMM:  Y[t][r] = sum_k bf16(W[r][k]) * X[t][k],  f32 accumulate.
//
// Operand rounding follows the reference's cooperative-matrix kernels, which
// round the dequantized weights and the activations to the tensor-core input
// type and accumulate in f32 (rust/crates/lev-forge/src/coopmat.rs:236-425;
// oracle rust/crates/lev-cli/src/main.rs:1201-1217); the input type here is
// bf16.  Like the reference's blocked kernel, a CTA dequantizes a slab of
// weight rows into shared memory (bit-exact block decode, then one rounding to
// bf16) and multiplies it against a slab of tokens.
//
// This first version issues mma.sync.m16n8k16 (bf16) from shared-memory tiles:
// CTA tile 64 rows x 64 tokens, K-step 32, four warps of 32 x 32.  It is the
// correctness anchor for the path; the tcgen05/TMEM mainloop replaces the
// inner product without changing the operand rounding or the tile decode.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "lev_internal.h"

// tensor-memory form (lev_gemm_tc.cu)
bool lev_gemm_tc_supported(const lev_weights* w, const void* x_bf16, int64_t tokens);
int lev_gemm_tc_run(lev_ctx* ctx, const lev_weights* w, const void* x_bf16, int64_t tokens, float* y);

namespace {

constexpr int kTileM = 64, kTileN = 64, kTileK = 32, kPad = 8;  // row stride 40 bf16 = 80 B: conflict-free fragment loads

__device__ __forceinline__ float h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int j, unsigned* sc, unsigned* mn) {
    if (j < 4) {
        *sc = s[j] & 63u;
        *mn = s[j + 4] & 63u;
    } else {
        *sc = (s[j + 4] & 0x0Fu) | ((unsigned)(s[j - 4] >> 6) << 4);
        *mn = (unsigned)(s[j + 4] >> 4) | ((unsigned)(s[j] >> 6) << 4);
    }
}

// 16 consecutive dequantized values of one row starting at column k0 (a multiple of 16),
// formed exactly as the block decoders form them
__device__ __forceinline__ void dequant16(int type, const uint8_t* row, int64_t k0, float* v) {
    if (type == LEV_GGML_Q4_0) {
        const uint8_t* b = row + (k0 >> 5) * LEV_Q4_0_BYTES;
        float d = h2f((unsigned)b[0] | ((unsigned)b[1] << 8));
        int hi = (int)(k0 & 16);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            unsigned q = b[2 + i];
            v[i] = __fmul_rn(d, (float)(hi ? (q >> 4) : (q & 15u)) - 8.0f);
        }
    } else if (type == LEV_GGML_Q4_K) {
        const uint8_t* b = row + (k0 >> 8) * LEV_Q4_K_BYTES;
        int e = (int)(k0 & 255), c = e >> 6, hi = (e >> 5) & 1, l0 = e & 31;
        float d = h2f((unsigned)b[0] | ((unsigned)b[1] << 8)), dmin = h2f((unsigned)b[2] | ((unsigned)b[3] << 8));
        unsigned sc, mn;
        q4k_scale_min(b + 4, 2 * c + hi, &sc, &mn);
        float d1 = __fmul_rn(d, (float)sc), mm = __fmul_rn(dmin, (float)mn);
        const uint8_t* q = b + 16 + 32 * c + l0;
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = __fsub_rn(__fmul_rn(d1, (float)(hi ? (q[i] >> 4) : (q[i] & 15u))), mm);
    } else {
        const uint8_t* b = row + (k0 >> 8) * LEV_Q6_K_BYTES;
        int e = (int)(k0 & 255), c = e >> 7, grp = (e >> 5) & 3, l0 = e & 31;
        float d = h2f((unsigned)b[208] | ((unsigned)b[209] << 8));
        float ds = __fmul_rn(d, (float)(int8_t)b[192 + 8 * c + 2 * grp + (l0 >> 4)]);
        const uint8_t* ql = b + 64 * c + ((grp & 1) ? 32 : 0) + l0;
        const uint8_t* qh = b + 128 + 32 * c + l0;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            unsigned lo = (grp & 2) ? (ql[i] >> 4) : (ql[i] & 15u);
            unsigned hb = (qh[i] >> (2 * grp)) & 3u;
            v[i] = __fmul_rn(ds, (float)((int)(lo | (hb << 4)) - 32));
        }
    }
}

__device__ __forceinline__ void mma_bf16(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128) k_gemm_prefill(const uint8_t* __restrict__ w, int type, int64_t row_bytes, int64_t rows,
                                                      int64_t cols, const __nv_bfloat16* __restrict__ x, int64_t tokens,
                                                      float* __restrict__ y) {
    __shared__ __align__(16) __nv_bfloat16 sa[kTileM][kTileK + kPad];
    __shared__ __align__(16) __nv_bfloat16 sb[kTileN][kTileK + kPad];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int wm = (warp & 1) * 32, wn = (warp >> 1) * 32;
    const int64_t r0 = (int64_t)blockIdx.x * kTileM, n0 = (int64_t)blockIdx.y * kTileN;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[i][j][q] = 0.f;

    for (int64_t k0 = 0; k0 < cols; k0 += kTileK) {
        // weights: 64 rows x 32 columns = 128 runs of 16, one per thread
        {
            int r = tid >> 1, half = tid & 1;
            float v[16];
            if (r0 + r < rows) dequant16(type, w + (r0 + r) * row_bytes, k0 + 16 * half, v);
            else
#pragma unroll
                for (int i = 0; i < 16; i++) v[i] = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i += 2)
                *reinterpret_cast<__nv_bfloat162*>(&sa[r][16 * half + i]) = __floats2bfloat162_rn(v[i], v[i + 1]);
        }
        // activations: 64 tokens x 32 columns of bf16 = 256 x 16 B
        for (int i = tid; i < 256; i += 128) {
            int n = i >> 2, part = i & 3;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (n0 + n < tokens) val = *reinterpret_cast<const uint4*>(x + (n0 + n) * cols + k0 + 8 * part);
            *reinterpret_cast<uint4*>(&sb[n][8 * part]) = val;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; kk += 16) {
            unsigned a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                a[i][0] = *reinterpret_cast<const unsigned*>(&sa[wm + 16 * i + g][kk + 2 * t]);
                a[i][1] = *reinterpret_cast<const unsigned*>(&sa[wm + 16 * i + g + 8][kk + 2 * t]);
                a[i][2] = *reinterpret_cast<const unsigned*>(&sa[wm + 16 * i + g][kk + 2 * t + 8]);
                a[i][3] = *reinterpret_cast<const unsigned*>(&sa[wm + 16 * i + g + 8][kk + 2 * t + 8]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                b[j][0] = *reinterpret_cast<const unsigned*>(&sb[wn + 8 * j + g][kk + 2 * t]);
                b[j][1] = *reinterpret_cast<const unsigned*>(&sb[wn + 8 * j + g][kk + 2 * t + 8]);
            }
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) mma_bf16(acc[i][j], a[i][0], a[i][1], a[i][2], a[i][3], b[j][0], b[j][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                int64_t r = r0 + wm + 16 * i + g + (q >> 1) * 8;
                int64_t n = n0 + wn + 8 * j + 2 * t + (q & 1);
                if (r < rows && n < tokens) y[n * rows + r] = acc[i][j][q];
            }
}

__global__ void k_act_bf16(const float* __restrict__ x, int64_t n, __nv_bfloat16* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(x[i]);
}

}  // namespace

extern "C" int lev_act_bf16(lev_ctx* ctx, const float* x, int64_t n, void* out_bf16) {
    if (!ctx || !x || !out_bf16 || n <= 0) return LEV_BAD_ARGUMENT;
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    int64_t g = (n + 255) / 256, cap = (int64_t)ctx->prop.multiProcessorCount * 16;
    k_act_bf16<<<(unsigned)(g > cap ? cap : g), 256, 0, ctx->stream>>>(x, n, (__nv_bfloat16*)out_bf16);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_act_bf16");
}

extern "C" int lev_gemm_prefill(lev_ctx* ctx, const lev_weights* w, const void* x_bf16, int64_t tokens, float* y,
                                unsigned flags) {
    if (!ctx || !w || !x_bf16 || !y) return LEV_BAD_ARGUMENT;
    if (flags & LEV_FLAG_HOST_IO) return lev_fail(ctx, LEV_UNSUPPORTED, "lev_gemm_prefill takes device pointers");
    if (tokens <= 0 || tokens > (1 << 20)) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "tokens %lld", (long long)tokens);
    if (w->cols % 32) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "inDim %lld", (long long)w->cols);
    if (!w->raw) return lev_fail(ctx, LEV_UNSUPPORTED, "the GGUF-order copy of this tensor was released: prefill reads it");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    if (lev_gemm_tc_supported(w, x_bf16, tokens)) {
        snprintf(ctx->ev.kernel_name, sizeof ctx->ev.kernel_name, "lev_gemm_prefill_tcgen05");
        return lev_gemm_tc_run(ctx, w, x_bf16, tokens, y);
    }
    dim3 grid((unsigned)((w->rows + kTileM - 1) / kTileM), (unsigned)((tokens + kTileN - 1) / kTileN));
    int64_t row_bytes = w->blocks_per_row * lev_block_bytes(w->type);
    k_gemm_prefill<<<grid, 128, 0, ctx->stream>>>(w->raw, w->type, row_bytes, w->rows, w->cols,
                                                  (const __nv_bfloat16*)x_bf16, tokens, y);
    ctx->launches++;
    snprintf(ctx->ev.kernel_name, sizeof ctx->ev.kernel_name, "lev_gemm_prefill");
    return lev_cuda_check(ctx, cudaGetLastError(), "k_gemm_prefill");
}
