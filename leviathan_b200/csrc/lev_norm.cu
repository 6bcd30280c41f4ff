// The elementwise steps either side of a decode matvec — RMSNorm, gelu_tanh(gate) * up, axpy —
// as stand-alone kernels, and the fused entry points that fold them into the one-launch matvec
// (norm or activation while the activation tables are built, residual where the rows are stored).
//
// Semantics follow the reference's kernels: g4_rmsnorm y = x * (1 / sqrt(mean(x^2) + eps)) * w
// (Sources/LeviathanCore/Gemma4.swift:4247-4268; the tiled form :4323-4358 reassociates the sum and
// is gated against an f64 oracle, as this one is), g4_gelu_up (Gemma4.swift:4364-4377) and
// g4_axpy (Gemma4.swift:4459).
#include <cuda_fp16.h>

#include "lev_stream.h"
#include "lev_stream_math.cuh"

namespace {

constexpr int kNormThreads = 256;

// One CTA per vector.  The sum of squares is reduced in a fixed order (thread-strided f32 partials,
// warp tree, warps in order), so repeated runs give the same bits.  x == y is allowed: every
// thread finishes reading before the barrier and afterwards touches only its own elements.
__global__ void __launch_bounds__(kNormThreads) k_rmsnorm(const float* x, int n, const float* __restrict__ w, float eps,
                                                           float* y, float* inverse, const float* cached) {
    __shared__ float part[kNormThreads / 32];
    // Vectors of up to kNormRegs * 1024 elements whose rows are 16-byte aligned stay in registers between the two
    // passes, and the weight is requested together with them, not after the reduction.
    constexpr int kNormRegs = 4;
    const bool in_regs = (n & 3) == 0 && n <= kNormRegs * kNormThreads * 4 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
                         (!w || ((uintptr_t)w & 15) == 0);
    float4 wv[kNormRegs];
    pdl_wait();
    pdl_launch_dependents();
    if (in_regs && w) {
#pragma unroll
        for (int k = 0; k < kNormRegs; k++) {
            const int i = (threadIdx.x + k * kNormThreads) * 4;
            wv[k] = i < n ? __ldg(reinterpret_cast<const float4*>(w + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    const float* xv = x + (int64_t)blockIdx.x * n;
    float* yv = y + (int64_t)blockIdx.x * n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4 xr[kNormRegs];
    float inv;
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < kNormRegs; k++) {
            const int i = (threadIdx.x + k * kNormThreads) * 4;
            xr[k] = i < n ? *reinterpret_cast<const float4*>(xv + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (cached) {
        inv = cached[blockIdx.x];
    } else {
        float ss = 0.f;
        const int n4 = n & ~3;
        if (in_regs) {
            // the same elements in the same order as the loop below: thread t adds its chunks t, t + 256, ...
#pragma unroll
            for (int k = 0; k < kNormRegs; k++) {
                if ((threadIdx.x + k * kNormThreads) * 4 < n) {
                    ss = fmaf(xr[k].x, xr[k].x, ss);
                    ss = fmaf(xr[k].y, xr[k].y, ss);
                    ss = fmaf(xr[k].z, xr[k].z, ss);
                    ss = fmaf(xr[k].w, xr[k].w, ss);
                }
            }
        } else {
            for (int i = threadIdx.x * 4; i < n4; i += kNormThreads * 4) {
                const float4 v = *reinterpret_cast<const float4*>(xv + i);
                ss = fmaf(v.x, v.x, ss);
                ss = fmaf(v.y, v.y, ss);
                ss = fmaf(v.z, v.z, ss);
                ss = fmaf(v.w, v.w, ss);
            }
            if (threadIdx.x < n - n4) ss = fmaf(xv[n4 + threadIdx.x], xv[n4 + threadIdx.x], ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < kNormThreads / 32; k++) tot += part[k];
        inv = 1.0f / sqrtf(tot / (float)n + eps);
        if (inverse && threadIdx.x == 0) inverse[blockIdx.x] = inv;
    }
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < kNormRegs; k++) {
            const int i = (threadIdx.x + k * kNormThreads) * 4;
            if (i < n) {
                float4 v = make_float4(xr[k].x * inv, xr[k].y * inv, xr[k].z * inv, xr[k].w * inv);
                if (w) v = make_float4(v.x * wv[k].x, v.y * wv[k].y, v.z * wv[k].z, v.w * wv[k].w);
                *reinterpret_cast<float4*>(yv + i) = v;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < n; i += kNormThreads) {
        const float v = xv[i] * inv;
        yv[i] = w ? v * w[i] : v;
    }
}

// out[v][e] = gelu_tanh(src[v][e]) * src[v][inter + e]
__global__ void k_gelu_up(const float* __restrict__ src, int64_t inter, int64_t total, float* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i / inter, e = i - v * inter;
        out[i] = gelu_tanh_up(src[v * 2 * inter + e], src[v * 2 * inter + inter + e]);
    }
}

// y = r + alpha * x (r may be y)
__global__ void k_axpy(float alpha, const float* __restrict__ x, const float* r, int64_t n, float* y) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = fmaf(alpha, x[i], r[i]);
}

// Inputs of a host-buffer list that lie in pinned, device-mapped host memory: one small kernel reads them over
// the bus (16 bytes per thread, all requests in flight at once) into the device-side staging area.  It costs one
// launch where the copy engine costs a queued copy per input plus an engine-to-engine hand-over, and the list's
// kernel, launched programmatically dependent on it, fills its weight rings while the inputs travel.
struct PullArgs {
    const uint4* src[LEV_MAX_CHAIN_OPS];
    uint4* dst[LEV_MAX_CHAIN_OPS];
    unsigned n16[LEV_MAX_CHAIN_OPS];
};
__global__ void __launch_bounds__(256) k_pull(const __grid_constant__ PullArgs P) {
    pdl_launch_dependents();
    const int j = blockIdx.y;
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < P.n16[j]) P.dst[j][i] = __ldcv(P.src[j] + i);  // never from a cache: the host rewrites these bytes between calls
}

int elementwise_grid(lev_ctx* ctx, int64_t n) {
    const int64_t blocks = (n + 255) / 256, cap = (int64_t)ctx->prop.multiProcessorCount * 8;
    return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

int rmsnorm_dev(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n, const float* w, float eps, float* y, float* inverse,
                const float* cached) {
    LEV_CUDA(ctx, launch_pdl(k_rmsnorm, dim3((unsigned)vectors), dim3(kNormThreads), 0, ctx->stream, x, (int)n, w, eps, y, inverse, cached));
    ctx->launches++;
    return LEV_OK;
}

int check_vectors(lev_ctx* ctx, int64_t vectors, int64_t n) {
    if (vectors <= 0 || n <= 0 || n > LEV_MAX_DIM || vectors > (int64_t)1 << 24)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%lld vectors of %lld elements", (long long)vectors, (long long)n);
    return LEV_OK;
}

bool overlap(const void* a, size_t na, const void* b, size_t nb) {
    const char *pa = (const char*)a, *pb = (const char*)b;
    return pa < pb + nb && pb < pa + na;
}

}  // namespace

extern "C" int lev_rmsnorm(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n, const float* weight, float eps, float* y,
                           float* inverse_out) {
    if (!ctx || !x || !y) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_vectors(ctx, vectors, n));
    if (!(eps >= 0.f) || !isfinite(eps)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "epsilon %g", (double)eps);
    if (((uintptr_t)x & 15) != 0) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x is not 16-byte aligned");
    if (vectors > 1 && n % 4 != 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "several vectors need n %% 4 == 0 (got %lld)", (long long)n);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    return rmsnorm_dev(ctx, x, vectors, n, weight, eps, y, inverse_out, nullptr);
}

// the cached apply of the reference's statistics group (g4_rmsnorm_cached,
// Sources/LeviathanCore/RMSStatisticsKernels.swift:104-130): y = x * inverse[v] * w, no new reduction
extern "C" int lev_rmsnorm_cached(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n, const float* weight,
                                  const float* inverse, float* y) {
    if (!ctx || !x || !y || !inverse) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_vectors(ctx, vectors, n));
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    return rmsnorm_dev(ctx, x, vectors, n, weight, 0.f, y, nullptr, inverse);
}

extern "C" int lev_gelu_up(lev_ctx* ctx, const float* gate_up, int64_t vectors, int64_t inter, float* out) {
    if (!ctx || !gate_up || !out) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_vectors(ctx, vectors, inter));
    if (overlap(gate_up, (size_t)vectors * 2 * inter * 4, out, (size_t)vectors * inter * 4))
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "input and output overlap");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t total = vectors * inter;
    LEV_CUDA(ctx, launch_pdl(k_gelu_up, dim3(elementwise_grid(ctx, total)), dim3(256), 0, ctx->stream, gate_up, inter, total, out));
    ctx->launches++;
    return LEV_OK;
}

extern "C" int lev_axpy(lev_ctx* ctx, float alpha, const float* x, const float* r, int64_t n, float* y) {
    if (!ctx || !x || !r || !y) return LEV_BAD_ARGUMENT;
    if (n <= 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%lld elements", (long long)n);
    if (overlap(x, (size_t)n * 4, y, (size_t)n * 4)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and y overlap");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    LEV_CUDA(ctx, launch_pdl(k_axpy, dim3(elementwise_grid(ctx, n)), dim3(256), 0, ctx->stream, alpha, x, r, n, y));
    ctx->launches++;
    return LEV_OK;
}

namespace {

int check_fusion(lev_ctx* ctx, const lev_fusion* f) {
    if (!f) return LEV_OK;
    if (f->prologue != LEV_PROLOGUE_NONE && f->prologue != LEV_PROLOGUE_RMSNORM && f->prologue != LEV_PROLOGUE_GELU_UP)
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "unknown prologue %d", f->prologue);
    if (f->prologue == LEV_PROLOGUE_RMSNORM && (!(f->eps >= 0.f) || !isfinite(f->eps)))
        return lev_fail(ctx, LEV_BAD_ARGUMENT, "epsilon %g", (double)f->eps);
    if (f->residual && !isfinite(f->alpha)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "alpha %g", (double)f->alpha);
    return LEV_OK;
}

lev_dense_fusion to_dense(const lev_fusion* f) {
    lev_dense_fusion d = {};
    if (!f) return d;
    d.norm_on = f->prologue == LEV_PROLOGUE_RMSNORM;
    d.norm_w = f->norm_weight;
    d.eps = f->eps;
    d.gelu_up = f->prologue == LEV_PROLOGUE_GELU_UP;
    d.residual = f->residual;
    d.alpha = f->alpha;
    return d;
}

// the prologue as a launch of its own, into the context's scratch
int staged_prologue(lev_ctx* ctx, const lev_fusion* f, const float* x, int n_cols, int64_t cols, const float** dx) {
    *dx = x;
    if (!f || f->prologue == LEV_PROLOGUE_NONE) return LEV_OK;
    void* p;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_X, (size_t)n_cols * cols * sizeof(float), &p));
    if (f->prologue == LEV_PROLOGUE_RMSNORM) {
        LEV_TRY(rmsnorm_dev(ctx, x, n_cols, cols, f->norm_weight, f->eps, (float*)p, nullptr, nullptr));
    } else {
        const int64_t total = (int64_t)n_cols * cols;
        LEV_CUDA(ctx, launch_pdl(k_gelu_up, dim3(elementwise_grid(ctx, total)), dim3(256), 0, ctx->stream, x, cols, total, (float*)p));
        ctx->launches++;
    }
    *dx = (const float*)p;
    return LEV_OK;
}

}  // namespace

// y[c][r] = residual[c][r] + alpha * sum_k W[row0 + r][k] * a[c][k], a = prologue(x).  Device pointers.
extern "C" int lev_matvec_fused(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int64_t x_count,
                                int n_cols, const lev_fusion* fusion, float* y, int64_t y_capacity) {
    if (!ctx || !w || !x || !y) return LEV_BAD_ARGUMENT;
    if (row0 < 0 || rows <= 0 || row0 > w->rows || rows > w->rows - row0)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "rows [%lld, +%lld) beyond the tensor's %lld rows", (long long)row0, (long long)rows,
                        (long long)w->rows);
    if (n_cols < 1 || n_cols > LEV_MAX_COLUMNS) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d outside 1...%d", n_cols, LEV_MAX_COLUMNS);
    LEV_TRY(check_fusion(ctx, fusion));
    const bool gelu = fusion && fusion->prologue == LEV_PROLOGUE_GELU_UP;
    const int64_t per_col = gelu ? 2 * w->cols : w->cols;
    if (x_count != (int64_t)n_cols * per_col)
        return lev_fail(ctx, LEV_WRONG_INPUT_COUNT, "input count %lld, expected %lld", (long long)x_count, (long long)((int64_t)n_cols * per_col));
    if (y_capacity < (int64_t)n_cols * rows)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "output capacity %lld below %lld", (long long)y_capacity, (long long)((int64_t)n_cols * rows));
    const size_t yb = (size_t)n_cols * (size_t)rows * sizeof(float);
    if (overlap(x, (size_t)x_count * 4, y, yb)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and y overlap");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n_cols == 1) {
        const lev_dense_fusion d = to_dense(fusion);
        const lev_chain_item it = {w, row0, rows, x, y, 0, &d};
        if (lev_chain_preferred(ctx, 1, &it)) return lev_chain_run(ctx, 1, &it);
    }
    if (lev_dense_supported(ctx, w, row0, rows, x, n_cols)) {
        const lev_dense_fusion d = to_dense(fusion);
        return lev_dense_run(ctx, w, row0, rows, x, n_cols, y, fusion ? &d : nullptr);
    }
    // shapes the one-launch kernel does not serve: the same steps as separate launches
    const float* dx;
    LEV_TRY(staged_prologue(ctx, fusion, x, n_cols, w->cols, &dx));
    float* dy = y;
    if (fusion && fusion->residual) {
        void* p;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_Y, yb, &p));
        dy = (float*)p;
    }
    if (lev_stream_supported(w, row0, rows, n_cols))
        LEV_TRY(lev_launch_matvec_stream(ctx, w, row0, rows, dx, n_cols, dy));
    else
        LEV_TRY(lev_launch_matvec_plain(ctx, w, row0, rows, dx, n_cols, dy));
    if (fusion && fusion->residual) {
        const int64_t n = (int64_t)n_cols * rows;
        LEV_CUDA(ctx, launch_pdl(k_axpy, dim3(elementwise_grid(ctx, n)), dim3(256), 0, ctx->stream, fusion->alpha, (const float*)dy,
                                 fusion->residual, n, y));
        ctx->launches++;
    }
    return LEV_OK;
}

// Several tensors of one inDim against prologue(x) (the gate and up projections behind one norm).
// The residual epilogue is not offered here.
extern "C" int lev_matvec_multi_fused(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x, int64_t x_count, int n_cols,
                                      const lev_fusion* fusion, float* const* y, const int64_t* y_capacity) {
    if (!ctx || !w || !x || !y || !y_capacity) return LEV_BAD_ARGUMENT;
    if (n_ops < 1 || n_ops > 4) return lev_fail(ctx, LEV_BAD_ARGUMENT, "%d tensors (1...4)", n_ops);
    if (n_cols < 1 || n_cols > LEV_MAX_COLUMNS) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d outside 1...%d", n_cols, LEV_MAX_COLUMNS);
    LEV_TRY(check_fusion(ctx, fusion));
    if (fusion && fusion->residual) return lev_fail(ctx, LEV_BAD_ARGUMENT, "the multi-tensor call has no residual epilogue");
    const bool gelu = fusion && fusion->prologue == LEV_PROLOGUE_GELU_UP;
    for (int i = 0; i < n_ops; i++) {
        if (!w[i] || !y[i]) return LEV_BAD_ARGUMENT;
        const int64_t per_col = gelu ? 2 * w[i]->cols : w[i]->cols;
        if (x_count != (int64_t)n_cols * per_col)
            return lev_fail(ctx, LEV_WRONG_INPUT_COUNT, "input count %lld, tensor %d expects %lld", (long long)x_count, i,
                            (long long)((int64_t)n_cols * per_col));
        if (y_capacity[i] < (int64_t)n_cols * w[i]->rows)
            return lev_fail(ctx, LEV_BAD_DIMENSIONS, "output %d capacity %lld below %lld", i, (long long)y_capacity[i],
                            (long long)((int64_t)n_cols * w[i]->rows));
        if (overlap(x, (size_t)x_count * 4, y[i], (size_t)n_cols * w[i]->rows * 4)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "x and y overlap");
    }
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n_cols == 1) {
        const lev_dense_fusion d = to_dense(fusion);
        lev_chain_item it[4];
        for (int i = 0; i < n_ops; i++) it[i] = {w[i], 0, w[i]->rows, x, y[i], 0, &d};
        if (lev_chain_preferred(ctx, n_ops, it)) return lev_chain_run(ctx, n_ops, it);
    }
    if (lev_dense_multi_supported(ctx, n_ops, w, x, n_cols)) {
        const lev_dense_fusion d = to_dense(fusion);
        return lev_dense_multi_run(ctx, n_ops, w, x, n_cols, y, fusion ? &d : nullptr);
    }
    // one tensor at a time; the prologue runs once when it has to be staged
    bool all_dense = true;
    for (int i = 0; i < n_ops; i++) all_dense = all_dense && lev_dense_supported(ctx, w[i], 0, w[i]->rows, x, n_cols);
    if (all_dense) {
        const lev_dense_fusion d = to_dense(fusion);
        for (int i = 0; i < n_ops; i++) LEV_TRY(lev_dense_run(ctx, w[i], 0, w[i]->rows, x, n_cols, y[i], fusion ? &d : nullptr));
        return LEV_OK;
    }
    const float* dx;
    LEV_TRY(staged_prologue(ctx, fusion, x, n_cols, w[0]->cols, &dx));
    for (int i = 0; i < n_ops; i++) {
        if (lev_stream_supported(w[i], 0, w[i]->rows, n_cols))
            LEV_TRY(lev_launch_matvec_stream(ctx, w[i], 0, w[i]->rows, dx, n_cols, y[i]));
        else
            LEV_TRY(lev_launch_matvec_plain(ctx, w[i], 0, w[i]->rows, dx, n_cols, y[i]));
    }
    return LEV_OK;
}

// A list of one-column products, each with its own prologue / epilogue, executed as if in order.
// One launch when the persistent kernel serves the list; else one fused call per op.
static_assert(LEV_MAX_CHAIN_OPS == kLevChainMaxOps, "the header's limit is the kernel's");
static int chain_host(lev_ctx* ctx, int n_ops, const lev_chain_op* ops, unsigned flags);

extern "C" int lev_matvec_chain(lev_ctx* ctx, int n_ops, const lev_chain_op* ops, unsigned flags) {
    if (!ctx || !ops) return LEV_BAD_ARGUMENT;
    if (n_ops < 1 || n_ops > LEV_MAX_CHAIN_OPS) return lev_fail(ctx, LEV_BAD_ARGUMENT, "%d ops (1...%d)", n_ops, LEV_MAX_CHAIN_OPS);
    if (flags & LEV_FLAG_HOST_IO) return chain_host(ctx, n_ops, ops, flags);
    if (flags & LEV_FLAG_CHECK_FINITE)
        return lev_fail(ctx, LEV_UNSUPPORTED, "the finite checks of a list run with host buffers only (LEV_FLAG_HOST_IO)");
    lev_chain_item items[LEV_MAX_CHAIN_OPS];
    lev_dense_fusion fus[LEV_MAX_CHAIN_OPS];
    for (int i = 0; i < n_ops; i++) {
        const lev_chain_op& o = ops[i];
        if (!o.w || !o.x || !o.y) return lev_fail(ctx, LEV_BAD_ARGUMENT, "op %d: null tensor, input or output", i);
        if (o.row0 < 0 || o.rows <= 0 || o.row0 > o.w->rows || o.rows > o.w->rows - o.row0 || o.rows > LEV_MAX_DIM)
            return lev_fail(ctx, LEV_BAD_DIMENSIONS, "op %d: rows [%lld, +%lld) beyond the tensor's %lld rows", i, (long long)o.row0,
                            (long long)o.rows, (long long)o.w->rows);
        LEV_TRY(check_fusion(ctx, &o.fusion));
        const bool gelu = o.fusion.prologue == LEV_PROLOGUE_GELU_UP;
        const size_t xb = (size_t)(gelu ? 2 : 1) * o.w->cols * sizeof(float), yb = (size_t)o.rows * sizeof(float);
        if (overlap(o.x, xb, o.y, yb)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "op %d: x and y overlap", i);
        fus[i] = to_dense(&o.fusion);
        items[i].w = o.w;
        items[i].row0 = o.row0;
        items[i].rows = o.rows;
        items[i].x = o.x;
        items[i].y = o.y;
        items[i].fusion = &fus[i];
        // an op that reads what an earlier op writes, or writes what an earlier op reads or writes,
        // starts only when every earlier op has finished on the whole GPU
        int wait = o.depends != 0;
        for (int j = 0; j < i && !wait; j++) {
            const lev_chain_op& e = ops[j];
            const bool egelu = e.fusion.prologue == LEV_PROLOGUE_GELU_UP;
            const size_t exb = (size_t)(egelu ? 2 : 1) * e.w->cols * sizeof(float), eyb = (size_t)e.rows * sizeof(float);
            wait = overlap(o.x, xb, e.y, eyb) || overlap(o.y, yb, e.x, exb) || overlap(o.y, yb, e.y, eyb) ||
                   (o.fusion.residual && o.fusion.residual != o.y && overlap(o.fusion.residual, yb, e.y, eyb)) ||
                   (e.fusion.residual && overlap(o.y, yb, e.fusion.residual, eyb));
        }
        items[i].wait = wait;
    }
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    if (lev_chain_supported(ctx, n_ops, items)) {
        lev_evidence* ev = &ctx->ev;
        snprintf(ev->device_name, sizeof ev->device_name, "%.127s", ctx->prop.name);
        snprintf(ev->kernel_name, sizeof ev->kernel_name, "lev_matvec_chain");
        ev->out_dim = ops[0].rows;
        ev->in_dim = ops[0].w->cols;
        ev->n_cols = 1;
        ev->weight_bytes = 0;
        for (int i = 0; i < n_ops; i++)
            ev->weight_bytes += (size_t)ops[i].rows * (size_t)ops[i].w->blocks_per_row * (size_t)lev_block_bytes(ops[i].w->type);
        ev->gpu_us = 0.f;
        ev->status = LEV_OK;
        return lev_chain_run(ctx, n_ops, items);
    }
    for (int i = 0; i < n_ops; i++) {
        const lev_chain_op& o = ops[i];
        const bool gelu = o.fusion.prologue == LEV_PROLOGUE_GELU_UP;
        LEV_TRY(lev_matvec_fused(ctx, o.w, o.row0, o.rows, o.x, (gelu ? 2 : 1) * o.w->cols, 1, &o.fusion, o.y, o.rows));
    }
    return LEV_OK;
}

// Host buffers: every op's x and y are host pointers (independent ops only).  Distinct inputs are
// brought in once, the list runs as one launch, the outputs come back, one synchronisation.
static int chain_host(lev_ctx* ctx, int n_ops, const lev_chain_op* ops, unsigned flags) {
    lev_chain_op dev[LEV_MAX_CHAIN_OPS];
    const void* seen_x[LEV_MAX_CHAIN_OPS];
    size_t seen_off[LEV_MAX_CHAIN_OPS];
    int n_seen = 0;
    size_t xb_total = 0, yb_total = 0;
    for (int i = 0; i < n_ops; i++) {
        const lev_chain_op& o = ops[i];
        if (!o.w || !o.x || !o.y) return lev_fail(ctx, LEV_BAD_ARGUMENT, "op %d: null tensor, input or output", i);
        if (o.row0 < 0 || o.rows <= 0 || o.row0 > o.w->rows || o.rows > o.w->rows - o.row0 || o.rows > LEV_MAX_DIM)
            return lev_fail(ctx, LEV_BAD_DIMENSIONS, "op %d: rows [%lld, +%lld) beyond the tensor's %lld rows", i, (long long)o.row0,
                            (long long)o.rows, (long long)o.w->rows);
        LEV_TRY(check_fusion(ctx, &o.fusion));
        if (o.depends || o.fusion.residual || (o.fusion.prologue == LEV_PROLOGUE_RMSNORM && o.fusion.norm_weight))
            return lev_fail(ctx, LEV_UNSUPPORTED, "op %d: with host buffers the ops of a list are independent plain products", i);
        const size_t xb = (size_t)(o.fusion.prologue == LEV_PROLOGUE_GELU_UP ? 2 : 1) * o.w->cols * sizeof(float);
        if (flags & LEV_FLAG_CHECK_FINITE)
            for (size_t k = 0; k < xb / sizeof(float); k++)
                if (!isfinite(o.x[k])) return lev_fail(ctx, LEV_NONFINITE_INPUT, "activation vector of op %d", i);
        int at = -1;
        for (int j = 0; j < n_seen; j++)
            if (seen_x[j] == o.x) at = j;
        if (at < 0) {
            at = n_seen++;
            seen_x[at] = o.x;
            seen_off[at] = xb_total;
            xb_total += (xb + 255) & ~(size_t)255;
        }
        dev[i] = o;
        dev[i].x = (const float*)seen_off[at];  // offsets for now
        dev[i].y = (float*)yb_total;
        yb_total += ((size_t)o.rows * sizeof(float) + 255) & ~(size_t)255;
    }
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    void *px, *py;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_X, xb_total, &px));
    LEV_TRY(lev_scratch(ctx, LEV_SCR_Y, yb_total, &py));
    // An output buffer in pinned host memory is mapped into the device's address space: the kernel then stores
    // its rows there itself (a few posted writes per row tile) and no copy back is queued for that op.
    bool direct[LEV_MAX_CHAIN_OPS];
    for (int i = 0; i < n_ops; i++) {
        dev[i].x = (const float*)((char*)px + (size_t)dev[i].x);
        dev[i].y = (float*)((char*)py + (size_t)dev[i].y);
        direct[i] = false;
        cudaPointerAttributes pa;
        if (cudaPointerGetAttributes(&pa, ops[i].y) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer != nullptr &&
            ((uintptr_t)pa.devicePointer & 15) == 0) {
            dev[i].y = (float*)pa.devicePointer;
            direct[i] = true;
        } else {
            (void)cudaGetLastError();  // an ordinary host pointer is not an error here
        }
    }
    // Inputs: pinned and mapped ones are fetched by one kernel (k_pull), the others by one queued copy each.
    PullArgs pull = {};
    int n_pull = 0;
    unsigned pull_max = 0;
    for (int j = 0; j < n_seen; j++) {
        size_t xb = 0;
        for (int i = 0; i < n_ops; i++)
            if (ops[i].x == seen_x[j]) xb = (size_t)(ops[i].fusion.prologue == LEV_PROLOGUE_GELU_UP ? 2 : 1) * ops[i].w->cols * sizeof(float);
        cudaPointerAttributes pa;
        if (xb % 16 == 0 && xb <= ((size_t)1 << 22) && cudaPointerGetAttributes(&pa, seen_x[j]) == cudaSuccess &&
            pa.type == cudaMemoryTypeHost && pa.devicePointer != nullptr && ((uintptr_t)pa.devicePointer & 15) == 0) {
            pull.src[n_pull] = (const uint4*)pa.devicePointer;
            pull.dst[n_pull] = (uint4*)((char*)px + seen_off[j]);
            pull.n16[n_pull] = (unsigned)(xb / 16);
            if (pull.n16[n_pull] > pull_max) pull_max = pull.n16[n_pull];
            n_pull++;
        } else {
            (void)cudaGetLastError();
            LEV_CUDA(ctx, cudaMemcpyAsync((char*)px + seen_off[j], seen_x[j], xb, cudaMemcpyHostToDevice, ctx->stream));
        }
    }
    if (n_pull) {
        // an ordinary launch: it starts when everything queued before it (a list still reading the staging area) is over
        k_pull<<<dim3((pull_max + 255) / 256, (unsigned)n_pull), 256, 0, ctx->stream>>>(pull);
        LEV_TRY(lev_cuda_check(ctx, cudaGetLastError(), "k_pull"));
        ctx->launches++;
    }
    LEV_TRY(lev_matvec_chain(ctx, n_ops, dev, 0));
    for (int i = 0; i < n_ops; i++)
        if (!direct[i])
            LEV_CUDA(ctx, cudaMemcpyAsync(ops[i].y, dev[i].y, (size_t)ops[i].rows * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    LEV_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (flags & LEV_FLAG_CHECK_FINITE)
        for (int i = 0; i < n_ops; i++)
            for (int64_t k = 0; k < ops[i].rows; k++)
                if (!isfinite(ops[i].y[k])) return lev_fail(ctx, LEV_NONFINITE_OUTPUT, "output vector of op %d", i);
    return LEV_OK;
}

// ---------------------------------------------------------------------------
// Greedy token choice: index of the maximum of each row (lowest index on ties) and the gap to the
// second best, after argmax of rust/crates/lev-forge/src/ops.rs:478-517.  A (best, index, second)
// triple merges associatively and commutatively, so the row is cut into chunks over many thread
// blocks and the triples merged in a second small launch; the result does not depend on the cut.
// ---------------------------------------------------------------------------
namespace {

struct Top {
    float best, second;
    int idx;
};

__device__ __forceinline__ Top top_merge(const Top& a, const Top& b) {
    const bool take = b.best > a.best || (b.best == a.best && b.idx < a.idx);
    Top r;
    r.best = take ? b.best : a.best;
    r.idx = take ? b.idx : a.idx;
    r.second = fmaxf(take ? fmaxf(a.best, b.second) : fmaxf(b.best, a.second), take ? a.second : b.second);
    return r;
}

__device__ __forceinline__ Top top_block(Top t, Top* sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Top u;
        u.best = __shfl_xor_sync(0xffffffffu, t.best, o);
        u.second = __shfl_xor_sync(0xffffffffu, t.second, o);
        u.idx = __shfl_xor_sync(0xffffffffu, t.idx, o);
        t = top_merge(t, u);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (lane == 0) sm[warp] = t;
    __syncthreads();
    t = sm[0];
    for (int w = 1; w < warps; w++) t = top_merge(t, sm[w]);
    return t;
}

constexpr float kLowest = -3.0e38f;  // the reference's starting value: anything below it never wins

__global__ void __launch_bounds__(256) k_argmax_part(const float* __restrict__ x, int64_t n, int chunks, Top* part) {
    __shared__ Top sm[8];
    pdl_wait();
    pdl_launch_dependents();
    const int chunk = blockIdx.x, row = blockIdx.y;
    const int64_t per = ((n + chunks - 1) / chunks + 3) & ~(int64_t)3, i0 = chunk * per, i1 = i0 + per < n ? i0 + per : n;
    const float* xr = x + row * n;
    Top t = {kLowest, kLowest, 0};
    auto see = [&](float v, int64_t i) {
        if (v > t.best) {
            t.second = t.best;
            t.best = v;
            t.idx = (int)i;
        } else if (v > t.second) {
            t.second = v;
        }
    };
    const bool vec = (((uintptr_t)xr & 15) == 0) && (n % 4 == 0);
    if (vec) {
        for (int64_t i = i0 + threadIdx.x * 4; i + 3 < i1; i += 256 * 4) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(xr + i));
            see(v.x, i), see(v.y, i + 1), see(v.z, i + 2), see(v.w, i + 3);
        }
        for (int64_t i = i0 + ((i1 - i0) & ~(int64_t)3) + threadIdx.x; i < i1; i += 256) see(xr[i], i);
    } else {
        for (int64_t i = i0 + threadIdx.x; i < i1; i += 256) see(xr[i], i);
    }
    t = top_block(t, sm);
    if (threadIdx.x == 0) part[(int64_t)row * chunks + chunk] = t;
}

__global__ void __launch_bounds__(256) k_argmax_final(const Top* part, int chunks, int32_t* out, float* margin) {
    __shared__ Top sm[8];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    Top t = {kLowest, kLowest, 0};
    for (int c = threadIdx.x; c < chunks; c += 256) t = top_merge(t, part[(int64_t)row * chunks + c]);
    t = top_block(t, sm);
    if (threadIdx.x == 0) {
        out[row] = t.idx;
        if (margin) margin[row] = t.best - t.second;
    }
}

}  // namespace

extern "C" int lev_argmax(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n, int32_t* out_index, float* out_margin) {
    if (!ctx || !x || !out_index) return LEV_BAD_ARGUMENT;
    LEV_TRY(check_vectors(ctx, vectors, n));
    if (vectors > 65535) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%lld vectors", (long long)vectors);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    // chunks of at least 4096 values, about four thread blocks per SM over all rows
    int64_t chunks = (4 * (int64_t)ctx->prop.multiProcessorCount + vectors - 1) / vectors;
    if (chunks > (n + 4095) / 4096) chunks = (n + 4095) / 4096;
    if (chunks < 1) chunks = 1;
    void* scr;
    LEV_TRY(lev_scratch(ctx, LEV_SCR_ATTN, (size_t)vectors * chunks * sizeof(Top), &scr));
    LEV_CUDA(ctx, launch_pdl(k_argmax_part, dim3((unsigned)chunks, (unsigned)vectors), dim3(256), 0, ctx->stream, x, n, (int)chunks, (Top*)scr));
    LEV_CUDA(ctx, launch_pdl(k_argmax_final, dim3((unsigned)vectors), dim3(256), 0, ctx->stream, (const Top*)scr, (int)chunks, out_index, out_margin));
    ctx->launches += 2;
    return LEV_OK;
}

// ---------------------------------------------------------------------------
// The per-head steps between the q / k / v projections and the cache append of a local layer
// (Sources/LeviathanCore/Gemma4.swift:3662-3687) in one launch over a [q heads | k heads | v heads]
// row: q heads RMSNorm(q_weight) then rotary, k heads RMSNorm(k_weight) then rotary, v heads the
// scale-free RMSNorm.  Rotary as g4_rope (Gemma4.swift:4390-4410): pairs (i, i + headDim/2) turned by
// the angle inv_freq[i] * position, cos and sin in f32.  One thread block per (head, column), in place.
// ---------------------------------------------------------------------------
namespace {

// where the k and v heads also go when the call appends to a paged cache (k_pool NULL: nowhere)
struct KvTarget {
    void* k_pool;
    void* v_pool;
    const int32_t* table;
    const int32_t* slot;
    int* status;
    int64_t blocks;
    int page, max_blocks, slots, f16;
};

// the rows the launch works on: column c's q heads at q + c * q_stride, its k heads at k + c * kv_stride, its
// v heads at v + c * kv_stride (one [q | k | v] row per column, or three separate matrices)
struct QkvRows {
    float *q, *k, *v;
    int64_t q_stride, kv_stride;
};

__global__ void __launch_bounds__(128) k_qkv_norm_rope(QkvRows X, int q_heads, int kv_heads, int hd, const float* __restrict__ qw,
                                                        const float* __restrict__ kw, float eps, const float* __restrict__ inv_freq,
                                                        const int32_t* __restrict__ pos, KvTarget C) {
    __shared__ float row[512];
    __shared__ float part[4];
    pdl_wait();
    pdl_launch_dependents();
    const int head = blockIdx.x, col = blockIdx.y;
    const bool is_q = head < q_heads, is_k = !is_q && head < q_heads + kv_heads;
    float* xv = is_q ? X.q + col * X.q_stride + (int64_t)head * hd
                     : (is_k ? X.k + col * X.kv_stride + (int64_t)(head - q_heads) * hd
                             : X.v + col * X.kv_stride + (int64_t)(head - q_heads - kv_heads) * hd);
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
    // Every load that does not wait for the norm is requested up front -- the head's elements, its norm weights, the
    // rotary frequencies, the column's slot and position and, as soon as those two are there, its block-table entry --
    // so the kernel pays one round trip to memory plus the table's, not five in a row.  head_dim <= 512: at most four
    // elements and two rotary pairs per thread.
    const bool turn = (is_q || is_k) && inv_freq != nullptr;
    const bool appends = C.k_pool != nullptr && !is_q;
    const int half = hd >> 1;
    float xreg[4], wreg[4], freq[2];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int i = threadIdx.x + 128 * k;
        xreg[k] = i < hd ? xv[i] : 0.f;
    }
    const int ps = (turn || appends) ? pos[col] : 0;
    const int sl = appends ? C.slot[col] : -1;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int i = threadIdx.x + 128 * k;
        wreg[k] = (w && i < hd) ? w[i] : 1.0f;
    }
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int i = threadIdx.x + 128 * k;
        freq[k] = (turn && i < half) ? inv_freq[i] : 0.f;
    }
    // cache append of the finished k / v head (optional): the row of this column's position
    int64_t at = -1;
    if (appends) {
        int64_t blk = -1;
        if (sl >= 0 && sl < C.slots && ps >= 0 && ps < C.max_blocks * C.page) blk = C.table[(int64_t)sl * C.max_blocks + ps / C.page];
        if (blk >= 0 && blk < C.blocks) {
            at = LEV_KV_ROW(blk, ps % C.page, is_k ? head - q_heads : head - q_heads - kv_heads, C.page, kv_heads) * hd;
        } else if (threadIdx.x == 0) {
            atomicOr(C.status, LEV_DEV_BAD_INDEX);  // recorded, not followed
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++)
        if (threadIdx.x + 128 * k < hd) ss = fmaf(xreg[k], xreg[k], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf((part[0] + part[1] + part[2] + part[3]) / (float)hd + eps);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int i = threadIdx.x + 128 * k;
        if (i < hd) {
            const float v = xreg[k] * inv;
            row[i] = w ? v * wreg[k] : v;
        }
    }
    __syncthreads();
    const float p = turn ? (float)ps : 0.f;
    void* pool = is_k ? C.k_pool : C.v_pool;
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int i = threadIdx.x + 128 * k;
        if (i >= half) break;
        float a = row[i], b = row[i + half];
        if (turn) {
            float sn, cs;
            sincosf(freq[k] * p, &sn, &cs);
            const float ra = a * cs - b * sn, rb = a * sn + b * cs;
            a = ra;
            b = rb;
        }
        xv[i] = a;
        xv[i + half] = b;
        if (at >= 0) {
            if (C.f16) {
                static_cast<__half*>(pool)[at + i] = __float2half_rn(a);
                static_cast<__half*>(pool)[at + i + half] = __float2half_rn(b);
            } else {
                static_cast<float*>(pool)[at + i] = a;
                static_cast<float*>(pool)[at + i + half] = b;
            }
        }
    }
}

QkvRows one_row(float* qkv, int q_heads, int kv_heads, int hd) {
    const int64_t stride = (int64_t)(q_heads + 2 * kv_heads) * hd;
    return {qkv, qkv + (int64_t)q_heads * hd, qkv + (int64_t)(q_heads + kv_heads) * hd, stride, stride};
}

}  // namespace

extern "C" int lev_qkv_norm_rope(lev_ctx* ctx, float* qkv, int n_cols, int q_heads, int kv_heads, int head_dim, const float* q_weight,
                                 const float* k_weight, float eps, const float* inv_freq, const int32_t* pos) {
    if (!ctx || !qkv) return LEV_BAD_ARGUMENT;
    if (n_cols < 1 || n_cols > 65535 || q_heads < 0 || kv_heads < 0 || q_heads + 2 * kv_heads < 1 || q_heads + 2 * kv_heads > 65535)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%d columns, %d query heads, %d KV heads", n_cols, q_heads, kv_heads);
    if (head_dim < 2 || head_dim > 512 || head_dim % 2 != 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "head dimension %d (even, at most 512)", head_dim);
    if (!(eps >= 0.f) || !isfinite(eps)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "epsilon %g", (double)eps);
    if (inv_freq && !pos) return lev_fail(ctx, LEV_BAD_ARGUMENT, "rotary frequencies without positions");
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    KvTarget none = {};
    LEV_CUDA(ctx, launch_pdl(k_qkv_norm_rope, dim3(q_heads + 2 * kv_heads, n_cols), dim3(128), 0, ctx->stream,
                             one_row(qkv, q_heads, kv_heads, head_dim), q_heads, kv_heads, head_dim, q_weight, k_weight, eps, inv_freq, pos, none));
    ctx->launches++;
    return LEV_OK;
}

// The same launch also stores the finished k and v heads at pos[column] of sequence slot[column] of a paged
// cache (lev_kv_append's job; the append of Sources/LeviathanCore/Gemma4.swift:3688-3698 without a launch).
namespace {
int norm_rope_append(lev_ctx* ctx, QkvRows X, int n_cols, int q_heads, int head_dim, const float* q_weight, const float* k_weight, float eps,
                     const float* inv_freq, const int32_t* pos, const lev_kv_layout* L, void* k_pool, void* v_pool,
                     const int32_t* block_table, const int32_t* slot) {
    if (L->kv_type != LEV_KV_F16 && L->kv_type != LEV_KV_F32) return lev_fail(ctx, LEV_BAD_ARGUMENT, "cache element type %d", L->kv_type);
    if (L->head_dim != head_dim || L->kv_heads < 1 || L->page <= 0 || L->blocks <= 0 || L->max_blocks <= 0 || L->slots <= 0)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "cache layout does not match the heads (head_dim %d / %d)", L->head_dim, head_dim);
    if (n_cols < 1 || n_cols > 65535 || q_heads < 0 || q_heads + 2 * L->kv_heads > 65535)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%d columns, %d query heads, %d KV heads", n_cols, q_heads, L->kv_heads);
    if (head_dim < 2 || head_dim > 512 || head_dim % 2 != 0) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "head dimension %d (even, at most 512)", head_dim);
    if (!(eps >= 0.f) || !isfinite(eps)) return lev_fail(ctx, LEV_BAD_ARGUMENT, "epsilon %g", (double)eps);
    LEV_CUDA(ctx, cudaSetDevice(ctx->device));
    KvTarget C = {k_pool, v_pool, block_table, slot, ctx->d_status, L->blocks, L->page, L->max_blocks, L->slots, L->kv_type == LEV_KV_F16};
    LEV_CUDA(ctx, launch_pdl(k_qkv_norm_rope, dim3(q_heads + 2 * L->kv_heads, n_cols), dim3(128), 0, ctx->stream, X, q_heads, L->kv_heads,
                             head_dim, q_weight, k_weight, eps, inv_freq, pos, C));
    ctx->launches++;
    return LEV_OK;
}
}  // namespace

extern "C" int lev_qkv_norm_rope_append(lev_ctx* ctx, float* qkv, int n_cols, int q_heads, int head_dim, const float* q_weight,
                                        const float* k_weight, float eps, const float* inv_freq, const int32_t* pos,
                                        const lev_kv_layout* L, void* k_pool, void* v_pool, const int32_t* block_table, const int32_t* slot) {
    if (!ctx || !qkv || !pos || !L || !k_pool || !v_pool || !block_table || !slot) return LEV_BAD_ARGUMENT;
    return norm_rope_append(ctx, one_row(qkv, q_heads, L->kv_heads, head_dim), n_cols, q_heads, head_dim, q_weight, k_weight, eps, inv_freq, pos, L,
                            k_pool, v_pool, block_table, slot);
}

// q [n_cols][q_heads * head_dim], k and v [n_cols][kv_heads * head_dim] as three matrices: the form the projections
// of several sequences leave them in
extern "C" int lev_qkv_norm_rope_append_split(lev_ctx* ctx, float* q, float* k, float* v, int n_cols, int q_heads, int head_dim,
                                              const float* q_weight, const float* k_weight, float eps, const float* inv_freq,
                                              const int32_t* pos, const lev_kv_layout* L, void* k_pool, void* v_pool,
                                              const int32_t* block_table, const int32_t* slot) {
    if (!ctx || !q || !k || !v || !pos || !L || !k_pool || !v_pool || !block_table || !slot) return LEV_BAD_ARGUMENT;
    const QkvRows X = {q, k, v, (int64_t)q_heads * head_dim, (int64_t)L->kv_heads * head_dim};
    return norm_rope_append(ctx, X, n_cols, q_heads, head_dim, q_weight, k_weight, eps, inv_freq, pos, L, k_pool, v_pool, block_table, slot);
}
