// Dense decode matvec of the stream schedule in ONE launch: y[n][rows] = W[rows][K] * x[n][K]
// for n <= 4 activation columns, over the fragment-major repack (see lev_stream.cu for the
// layout and the arithmetic).
//
// What differs from the general stream kernel:
//  * No preparation launch.  Every CTA builds the activation tables (fp16 split terms in mma
//    B-fragment order, bias / min sums) in its own shared memory, straight from x.
//  * The split of work is fixed on the host: CTA c owns a run of consecutive 16-row tiles, its
//    warps split that run's K-steps evenly; a warp's share is one contiguous byte range, so the
//    fetch side is a pointer and a count.
//  * A CTA takes at most half of an SM (shared memory, registers, threads).  With programmatic
//    dependent launch the next matvec's CTAs become resident beside this one's, issue their
//    first weight requests and then wait for this launch to finish; the HBM latency and ramp-up
//    of launch i+1 hide behind the arithmetic of launch i.
//  * Sums: a warp adds its K-steps in order; tiles shared by several warps are added in warp
//    order from shared-memory records.  Same call, same bits.
#include "lev_stream.h"
#include "lev_stream_math.cuh"

namespace {

constexpr int kMaxDepth = 8;

struct DenseArgs {
    const uint4* wp;   // first tile of the call
    int spt;           // K-steps per tile
    int tiles_base;    // CTA c owns tiles_base (+1 when c < tiles_rem) consecutive tiles
    int tiles_rem;
    const float* x;    // [n_cols][x_ld]
    int64_t x_ld;
    int cols;          // K
    int chunks;        // padded 64-column chunks
    int n_cols;
    float* y;          // [n_cols][out_ld]
    int64_t rows, out_ld;
    int* status;
    int depth;         // ring stages per warp
    int debug;         // bit 0: skip the arithmetic
};

template <int TYPE, int CMAX, int W>
__global__ void __launch_bounds__(W * 32, W <= 16 ? 2 : 1) k_dense(DenseArgs A) {
    using D = StreamDims<CMAX>;
    constexpr int NT = D::kNT, GLT = D::kGlt, TERMS = D::kTerms;
    constexpr int kStepBytes = step_bytes(TYPE);
    constexpr int kAuxPerChunk = TYPE == LEV_GGML_Q4_K ? 2 * CMAX : (TYPE == LEV_GGML_Q6_K ? 4 * GLT : 2 * GLT);
    static_assert(W % 4 == 0 && TERMS == 2, "warps are dealt to the four schedulers in equal shares");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[W][kMaxDepth];
    __shared__ float rec[W][2][CMAX][16];  // partial sums of tiles a warp shares with its neighbours
    __shared__ int rec_tile[W][2];         // CTA-local tile of each record, -1 = none
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    // logical position of this warp in the CTA's run: warps of one scheduler (warp % 4) are
    // neighbours, so shares that differ by one step spread evenly over the schedulers
    const int lw = (warp & 3) * (W / 4) + (warp >> 2);
    const int spt = A.spt, depth = A.depth;
    const int cta = blockIdx.x;
    const int tile0 = cta * A.tiles_base + (cta < A.tiles_rem ? cta : A.tiles_rem);
    const int ntiles = A.tiles_base + (cta < A.tiles_rem ? 1 : 0);
    const int nst = ntiles * spt;
    const int s = (int)((int64_t)nst * lw / W), e = (int)((int64_t)nst * (lw + 1) / W);

    unsigned char* ring = smem_raw + (size_t)warp * depth * kStepBytes;
    const unsigned ring_s = smem_u32(ring), bar_s = smem_u32(&bars[warp][0]);
    const unsigned char* f_ptr = reinterpret_cast<const unsigned char*>(A.wp) + ((int64_t)tile0 * spt + s) * kStepBytes;
    int f_left = e - s;
    if (lane < 2) rec_tile[warp][lane] = -1;
    if (lane == 0) {
        for (int d = 0; d < depth; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (int d = 0; d < depth && f_left > 0; d++, f_left--, f_ptr += kStepBytes)
            bulk_load(ring_s + d * kStepBytes, f_ptr, kStepBytes, bar_s + 8 * d);
    }
    pdl_launch_dependents();
    pdl_wait();  // weights are immutable and already on their way; x and y belong to the launches before

    // ---- activation tables, built by every CTA for itself ----
    uint4* xs = reinterpret_cast<uint4*>(smem_raw + (size_t)W * depth * kStepBytes);
    float* sa = reinterpret_cast<float*>(xs + A.chunks * GLT * 8);
    {
        const int entries = A.chunks * GLT * 4, rounded = (entries + 31) & ~31;
        bool bad = false;
        for (int idx = threadIdx.x; idx < rounded; idx += W * 32) {
            const bool live = idx < entries;
            const int ii = live ? idx : entries - 1;
            const int chunk = ii / (GLT * 4), rem = ii - chunk * (GLT * 4), col = rem >> 2, tt = rem & 3;
            const int c = col >> 1, term = col & 1;
            const float* xr = A.x + (int64_t)(c < A.n_cols ? c : 0) * A.x_ld;
            float xv[4][2][2];
#pragma unroll
            for (int m = 0; m < 4; m++)
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int el = chunk * 64 + chunk_col<TYPE>(tt, m, r, h);
                        const float v = __ldg(xr + (el < A.cols ? el : 0));
                        xv[m][r][h] = (el < A.cols && c < A.n_cols) ? v : 0.f;
                    }
            unsigned regs[8];
            float seen[4];  // what the tensor core sees of each mma's four elements, summed
            float plain[2] = {0.f, 0.f};
#pragma unroll
            for (int m = 0; m < 4; m++) {
                seen[m] = 0.f;
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    float v[2];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float sv = split_term(chunk_hi<TYPE>(m) ? xv[m][r][h] * kHiScale : xv[m][r][h], term);
                        bad |= !isfinite(sv);
                        v[h] = sv;
                        seen[m] += chunk_hi<TYPE>(m) ? 16.0f * sv : sv;
                        plain[m >> 1] += xv[m][r][h];
                    }
                    __half2 hv = __floats2half2_rn(v[0], v[1]);
                    regs[m * 2 + r] = *reinterpret_cast<unsigned*>(&hv);
                }
            }
            if (live) {
                xs[ii * 2] = make_uint4(regs[0], regs[1], regs[2], regs[3]);
                xs[ii * 2 + 1] = make_uint4(regs[4], regs[5], regs[6], regs[7]);
            }
            // sums over the quad (the four tt of one chunk and column)
            if (TYPE == LEV_GGML_Q4_K) {
                // true activations of the chunk's two 32-value sub-blocks
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    float v = plain[hf];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (live && tt == 0 && term == 0) sa[(chunk * 2 + hf) * CMAX + c] = v;
                }
            } else if (TYPE == LEV_GGML_Q6_K) {
                // -32 * 2^-24 * (sum seen by the tensor core) of each 16-value sub-block
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    float v = seen[m];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (live && tt == 0) sa[(chunk * 4 + m) * GLT + col] = -32.0f * 5.9604644775390625e-08f * v;
                }
            } else {
                // -8 * 2^-24 * (sum seen by the tensor core) of each 32-value block
#pragma unroll
                for (int blk = 0; blk < 2; blk++) {
                    float v = seen[2 * blk] + seen[2 * blk + 1];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (live && tt == 0) sa[(chunk * 2 + blk) * GLT + col] = -8.0f * 5.9604644775390625e-08f * v;
                }
            }
        }
        if (bad) atomicOr(A.status, LEV_DEV_NONFINITE_INPUT);
    }
    __syncthreads();

    LaneOffsets<CMAX> O;
    O.init(lane);
    float yacc[NT][4];
    float mina[CMAX], minb[CMAX];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
    for (int c = 0; c < CMAX; c++) mina[c] = minb[c] = 0.f;

    int slot = 0;        // ring stage of the next K-step
    unsigned phase = 0;  // its mbarrier phase parity
    int tl = s / spt;    // CTA-local tile
    int k = s - tl * spt;
    int seg_k0 = k;
    const int first_tl = tl;
    for (int i = s; i < e; i++) {
        if (!mbar_wait(bar_s + 8 * slot, phase)) {
            if (lane == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
            break;
        }
        const uint4* st = reinterpret_cast<const uint4*>(ring + slot * kStepBytes);
        if (!(A.debug & 1))
            stream_step<TYPE, CMAX, true>(st, xs + k * (4 * GLT * 8), sa + k * (4 * kAuxPerChunk), lane, O, yacc, mina, minb);
        // every lane has consumed its shared-memory reads of this stage: refill it
        __syncwarp();
        if (lane == 0 && f_left > 0) {
            bulk_load(ring_s + slot * kStepBytes, f_ptr, kStepBytes, bar_s + 8 * slot);
            f_ptr += kStepBytes;
            f_left--;
        }
        if (++slot == depth) {
            slot = 0;
            phase ^= 1u;
        }
        k++;
        if (k == spt || i == e - 1) {
            // ---- this warp's segment of the tile ends: fold to one f32 per (row, column) ----
            const bool whole = seg_k0 == 0 && k == spt;
            const int r = tl == first_tl ? 0 : 1;
#pragma unroll
            for (int c = 0; c < CMAX; c++) {
                float va = 0.f, vb = 0.f;
#pragma unroll
                for (int term = 0; term < TERMS; term++) {
                    constexpr float kScale[2] = {1.0f, 4.8828125e-4f};  // 2^0, 2^-11
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
                        const int64_t row = (int64_t)(tile0 + tl) * 16 + g;
                        if (c < A.n_cols) {
                            if (row < A.rows) A.y[(int64_t)c * A.out_ld + row] = va;
                            if (row + 8 < A.rows) A.y[(int64_t)c * A.out_ld + row + 8] = vb;
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
        }
    }
    __syncthreads();
    // ---- tiles shared between warps: add the warps' records in the order of their ranges ----
    for (int item = threadIdx.x; item < ntiles * CMAX * 16; item += W * 32) {
        const int tile = item / (CMAX * 16), idx = item - tile * (CMAX * 16);
        float acc = 0.f;
        int found = 0;
#pragma unroll 1
        for (int l2 = 0; l2 < W; l2++) {
            const int pw = (l2 % (W / 4)) * 4 + l2 / (W / 4);  // the warp whose logical position is l2
            if (rec_tile[pw][0] == tile) {
                acc += rec[pw][0][0][idx];
                found++;
            } else if (rec_tile[pw][1] == tile) {
                acc += rec[pw][1][0][idx];
                found++;
            }
        }
        if (!found) continue;  // one warp had the whole tile and wrote it
        const int c = idx >> 4;
        const int64_t row = (int64_t)(tile0 + tile) * 16 + (idx & 15);
        if (c < A.n_cols && row < A.rows) A.y[(int64_t)c * A.out_ld + row] = acc;
    }
}

template <int TYPE, int CMAX, int W>
int launch_dense(lev_ctx* ctx, int grid, size_t smem, const DenseArgs& A) {
    static size_t configured[16] = {};  // per device: largest dynamic shared memory opted in so far
    if (configured[ctx->device & 15] < smem) {
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_dense<TYPE, CMAX, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[ctx->device & 15] = smem;
    }
    LEV_CUDA(ctx, launch_pdl(k_dense<TYPE, CMAX, W>, dim3(grid), dim3(W * 32), smem, ctx->stream, A));
    return LEV_OK;
}

template <int TYPE, int CMAX>
int launch_dense_w(lev_ctx* ctx, int warps, int grid, size_t smem, const DenseArgs& A) {
    if (warps == 8) return launch_dense<TYPE, CMAX, 8>(ctx, grid, smem, A);
    if (warps == 12) return launch_dense<TYPE, CMAX, 12>(ctx, grid, smem, A);
    if (warps == 16) return launch_dense<TYPE, CMAX, 16>(ctx, grid, smem, A);
    return launch_dense<TYPE, CMAX, 24>(ctx, grid, smem, A);
}

template <int TYPE>
int launch_dense_c(lev_ctx* ctx, int cmax, int warps, int grid, size_t smem, const DenseArgs& A) {
    switch (cmax) {
        case 1: return launch_dense_w<TYPE, 1>(ctx, warps, grid, smem, A);
        case 2: return launch_dense_w<TYPE, 2>(ctx, warps, grid, smem, A);
        case 3: return launch_dense_w<TYPE, 3>(ctx, warps, grid, smem, A);
        case 4: return launch_dense_w<TYPE, 4>(ctx, warps, grid, smem, A);
    }
    return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", cmax);
}

struct DensePlan {
    int warps, depth, grid;
    size_t smem;
};

// Shape of a launch, or false when the tables do not fit beside a useful ring.
bool dense_plan(lev_ctx* ctx, const lev_weights* w, int64_t rows, int n_cols, DensePlan* P) {
    if (n_cols < 1 || n_cols > 4 || env_int("LEV_DENSE", 1) == 0) return false;
    const size_t step = step_bytes(w->type);
    const size_t tb = lev_stream_table_bytes(w, n_cols, 2, 1, nullptr);
    const int64_t tiles = (rows + 15) / 16, spt = lev_stream_chunks(w) / 4;
    if (tiles < 1 || tiles * spt > 0x7fffffff / 64) return false;
    int warps = env_int("LEV_DENSE_WARPS", 12);
    if (warps != 8 && warps != 12 && warps != 16 && warps != 24) warps = 12;
    // half of an SM's shared memory unless one CTA takes the SM
    size_t cap = (size_t)env_int("LEV_DENSE_SMEM_KB", warps <= 16 ? 108 : 200) * 1024;
    const int sms = ctx->prop.multiProcessorCount;
    const int grid = (int)(tiles < sms ? tiles : sms);
    const int64_t per_cta = ((tiles + grid - 1) / grid) * spt;
    const int64_t per_warp = (per_cta + warps - 1) / warps;
    if (tb + (size_t)warps * step > cap) {
        // large tables: give the CTA the whole SM before giving up
        cap = 200 * 1024;
        if (tb + (size_t)warps * step > cap) return false;
    }
    int64_t depth = (int64_t)((cap - tb) / ((size_t)warps * step));
    if (depth > per_warp) depth = per_warp;
    if (depth > kMaxDepth) depth = kMaxDepth;
    const int forced = env_int("LEV_DENSE_DEPTH", 0);
    if (forced > 0 && forced < depth) depth = forced;
    if (depth < 1) depth = 1;
    P->warps = warps;
    P->depth = (int)depth;
    P->grid = grid;
    P->smem = (size_t)warps * depth * step + tb;
    return true;
}

}  // namespace

bool lev_dense_supported(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, int n_cols) {
    DensePlan P;
    return w->packed && row0 % 16 == 0 && dense_plan(ctx, w, rows, n_cols, &P);
}

// x: [n_cols][w->cols] device, y: [n_cols][rows] device.  No work buffers.
int lev_dense_run(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols, float* y) {
    DensePlan P;
    if (!w->packed || row0 % 16 != 0 || !dense_plan(ctx, w, rows, n_cols, &P))
        return lev_fail(ctx, LEV_UNSUPPORTED, "dense stream kernel: shape not served");
    const int64_t tiles = (rows + 15) / 16, chunks = lev_stream_chunks(w), spt = chunks / 4;
    const size_t step = step_bytes(w->type);
    DenseArgs A;
    A.wp = (const uint4*)w->packed + (row0 / 16) * spt * (int64_t)(step / 16);
    A.spt = (int)spt;
    A.tiles_base = (int)(tiles / P.grid);
    A.tiles_rem = (int)(tiles % P.grid);
    A.x = x;
    A.x_ld = w->cols;
    A.cols = (int)w->cols;
    A.chunks = (int)chunks;
    A.n_cols = n_cols;
    A.y = y;
    A.rows = rows;
    A.out_ld = rows;
    A.status = ctx->d_status;
    A.depth = P.depth;
    A.debug = env_int("LEV_STREAM_DEBUG", 0);
    int st = w->type == LEV_GGML_Q4_K   ? launch_dense_c<LEV_GGML_Q4_K>(ctx, n_cols, P.warps, P.grid, P.smem, A)
             : w->type == LEV_GGML_Q6_K ? launch_dense_c<LEV_GGML_Q6_K>(ctx, n_cols, P.warps, P.grid, P.smem, A)
                                        : launch_dense_c<LEV_GGML_Q4_0>(ctx, n_cols, P.warps, P.grid, P.smem, A);
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = P.grid;
    ctx->ev.block = P.warps * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_dense");
}
