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
#include "lev_chain_math.cuh"

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
    int sps;           // K-steps per stage
    // sliced form (JOBS): the call is a device-side list of jobs, each up to CMAX activation columns
    // against one slice (expert) of the tensor
    const int* njobs_dev;   // [1] jobs in the list
    const int* job_slice;   // [job] slice index, in units of tiles_per_job tiles
    const int* job_src;     // [job][CMAX] source row of each column's activations, -1 = none
    const int* job_out;     // [job][CMAX] output row of each column, -1 = none
    int tiles_per_job;
    int gelu_inter;         // > 0: activation e = gelu_tanh(src[e]) * src[gelu_inter + e]
    int table_stride;       // bytes between the tables of consecutive jobs in shared memory
    int max_tables;         // jobs whose tables the launch has room for in one CTA (<= kMaxJobTables)
    // multi form (MULTI): up to four tensors of one format and K against the same activations;
    // the call's tiles are the tensors' tiles in order
    int n_ops;
    const uint4* wp_op[4];  // first tile of each tensor's row window
    int tiles_cum[5];       // tiles before each tensor
    float* y_op[4];         // [n_cols][rows_op]
    int64_t rows_op[4];
    // fused steps either side of the product (dense and multi forms)
    int norm_on;            // activations are x * inv_rms(x) * norm_w, inv_rms computed by every CTA
    const float* norm_w;    // [cols] or NULL (no scale)
    float norm_eps;
    const float* residual;  // dense form: y = residual + alpha * (W x), same layout as y; NULL: y = W x
    float alpha;
};


constexpr int kMaxJobTables = 3;  // jobs whose tables one CTA of the sliced form can hold

template <int TYPE, int CMAX, int W, bool JOBS, bool MULTI = false>
__global__ void __launch_bounds__(W * 32, W <= 8 ? 2 : 1) k_dense(DenseArgs A) {
    static_assert(!(JOBS && MULTI), "a call is either a job list or a list of tensors");
    using D = StreamDims<CMAX>;
    constexpr int NT = D::kNT, GLT = D::kGlt, TERMS = D::kTerms;
    constexpr int kStepBytes = step_bytes(TYPE);
    constexpr int kAuxPerChunk = TYPE == LEV_GGML_Q4_K ? 2 * CMAX : (TYPE == LEV_GGML_Q6_K ? 4 * GLT : 2 * GLT);
    static_assert(W % 4 == 0 && TERMS == 2, "warps are dealt to the four schedulers in equal shares");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[W][kMaxDepth];  // stage filled (bulk copy landed)
    __shared__ float rec[W][2][CMAX][16];  // partial sums of tiles a warp shares with its neighbours
    __shared__ __align__(16) uint4 zero_block[2];  // one column: the fragments of lanes outside a chunk's column group
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    if (CMAX == 1 && threadIdx.x < 2) zero_block[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);  // read after the table barrier
    // logical position of this warp in the CTA's run: warps of one scheduler (warp % 4) are
    // neighbours, so shares that differ by one step spread evenly over the schedulers
    const int lw = (warp & 3) * (W / 4) + (warp >> 2);
    const int spt = A.spt, depth = A.depth;
    const int cta = blockIdx.x;
    int tiles_base = A.tiles_base, tiles_rem = A.tiles_rem;
    const int tpj = JOBS ? A.tiles_per_job : 1;
    if (JOBS) {  // the job count is only known on the device (written by a launch that has completed)
        const int total = *A.njobs_dev * tpj;
        tiles_base = total / (int)gridDim.x;
        tiles_rem = total - tiles_base * (int)gridDim.x;
    }
    const int tile0 = cta * tiles_base + (cta < tiles_rem ? cta : tiles_rem);
    const int ntiles = tiles_base + (cta < tiles_rem ? 1 : 0);
    if (ntiles == 0) return;
    const int job0 = JOBS ? tile0 / tpj : 0;
    const int njobs_here = JOBS ? (tile0 + ntiles - 1) / tpj - job0 + 1 : 1;
    if (JOBS && njobs_here > A.max_tables) {
        if (threadIdx.x == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
        return;
    }
    const int nst = ntiles * spt;
    const int s = (int)((int64_t)nst * lw / W), e = (int)((int64_t)nst * (lw + 1) / W);

    const int sps = A.sps;  // K-steps per ring stage (one bulk copy, one barrier wait)
    const unsigned stage_bytes = (unsigned)sps * kStepBytes;

    unsigned char* ring = smem_raw + (size_t)warp * depth * stage_bytes;
    const unsigned ring_s = smem_u32(ring), bar_s = smem_u32(&bars[warp][0]);
    // fetch side (lane 0): this warp's share is one contiguous byte range
    const unsigned char* f_ptr = reinterpret_cast<const unsigned char*>(A.wp) + ((int64_t)tile0 * spt + s) * kStepBytes;
    int f_left = e - s;  // K-steps not yet requested
    int f_q = s;         // sliced form: CTA-local index of the next K-step to request (one per stage)
    // sliced form: a tile's bytes sit in the slice its job names
    auto step_src = [&](int q) -> const unsigned char* {
        const int gt = tile0 + q / spt, k = q - (q / spt) * spt;
        const int job = gt / tpj, tij = gt - job * tpj;
        return reinterpret_cast<const unsigned char*>(A.wp) +
               (((int64_t)A.job_slice[job] * tpj + tij) * spt + k) * (int64_t)kStepBytes;
    };
    // sliced form, fetch cursor (lane 0): the K-steps of a job's tiles are contiguous, so the address is formed once
    // per job (divisions, a table load) and stepped in between
    const unsigned char* j_ptr = nullptr;
    int j_run = 0;  // K-steps left at j_ptr before the next job begins
    auto jobs_next = [&](int q) -> const unsigned char* {
        if (j_run == 0) {
            const int tq = q / spt, gt = tile0 + tq;
            j_ptr = step_src(q);
            j_run = (tpj - gt % tpj) * spt - (q - tq * spt);
        }
        const unsigned char* a = j_ptr;
        j_ptr += kStepBytes;
        j_run--;
        return a;
    };
    // multi form: the tensor a global tile belongs to
    auto op_of = [&](int gt) -> int {
        int o = 0;
        while (o + 1 < A.n_ops && gt >= A.tiles_cum[o + 1]) o++;
        return o;
    };
    // multi form, fetch cursor (lane 0): address of the next K-step; steps are contiguous inside a
    // tensor, so the cursor only jumps where the next tile belongs to another tensor
    const unsigned char* m_ptr = nullptr;
    int m_k = 0, m_gt = 0, m_op = 0;
    if (MULTI) {
        const int tq = s / spt;
        m_gt = tile0 + tq;
        m_k = s - tq * spt;
        m_op = op_of(m_gt);
        m_ptr = reinterpret_cast<const unsigned char*>(A.wp_op[m_op]) +
                ((int64_t)(m_gt - A.tiles_cum[m_op]) * spt + m_k) * (int64_t)kStepBytes;
    }
    auto multi_next = [&]() -> const unsigned char* {
        const unsigned char* a = m_ptr;
        m_ptr += kStepBytes;
        if (++m_k == spt) {
            m_k = 0;
            m_gt++;
            if (m_op + 1 < A.n_ops && m_gt == A.tiles_cum[m_op + 1]) {
                m_op++;
                m_ptr = reinterpret_cast<const unsigned char*>(A.wp_op[m_op]);
            }
        }
        return a;
    };
    // requests the next stage's K-steps into ring stage d (lane 0)
    auto issue_stage = [&](int d) {
        const int n = f_left < sps ? f_left : sps;
        const unsigned dst = ring_s + d * stage_bytes, bar = bar_s + 8 * d;
        if (MULTI) {
            // consecutive steps are contiguous except where the next tile belongs to another tensor
            mbar_expect(bar, n * kStepBytes);
            const unsigned char* a0 = multi_next();
            int run = 1, done = 0;
            for (int u = 1; u < n; u++) {
                const unsigned char* a = multi_next();
                if (a == a0 + (size_t)run * kStepBytes) {
                    run++;
                } else {
                    bulk_copy(dst + done * kStepBytes, a0, run * kStepBytes, bar);
                    done += run;
                    a0 = a;
                    run = 1;
                }
            }
            bulk_copy(dst + done * kStepBytes, a0, run * kStepBytes, bar);
        } else {
            bulk_load(dst, JOBS ? jobs_next(f_q) : f_ptr, n * kStepBytes, bar);  // sliced form: one K-step per stage
        }
        f_ptr += n * kStepBytes;
        f_q += n;
        f_left -= n;
    };
    if (lane == 0) {
        for (int d = 0; d < depth; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (int d = 0; d < depth && f_left > 0; d++) issue_stage(d);
    }
    LaneOffsets<CMAX> O;
    O.init(lane);
    int tl = s / spt;    // CTA-local tile
    int k = s - tl * spt;
    pdl_launch_dependents();
    pdl_wait();  // weights are immutable and already on their way; x and y belong to the launches before

    // ---- RMSNorm statistic of each activation column (fused prologue): every CTA reduces the
    // column itself, in a fixed order (thread-strided partials, warp tree, warps in order) ----
    float inv_rms[CMAX];
#pragma unroll
    for (int c = 0; c < CMAX; c++) inv_rms[c] = 1.0f;
    if (!JOBS && A.norm_on) {
        __shared__ float norm_part[W][CMAX];
#pragma unroll
        for (int c = 0; c < CMAX; c++) {
            float ss = 0.f;
            if (c < A.n_cols) {
                const float* xr = A.x + (int64_t)c * A.x_ld;
                for (int i = threadIdx.x * 4; i < A.cols; i += W * 128) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(xr + i));
                    ss = fmaf(v.x, v.x, ss);
                    ss = fmaf(v.y, v.y, ss);
                    ss = fmaf(v.z, v.z, ss);
                    ss = fmaf(v.w, v.w, ss);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) norm_part[warp][c] = ss;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < CMAX; c++) {
            float tot = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < W; w2++) tot += norm_part[w2][c];
            inv_rms[c] = 1.0f / sqrtf(tot / (float)A.cols + A.norm_eps);
        }
    }
    // ---- activation tables, built by every CTA for itself ----
    // One item = (chunk, activation column, lane-of-quad tt): the 16 activations that feed lane
    // tt's B fragments of the chunk's four mma, both split terms.
    unsigned char* tables0 = smem_raw + (size_t)W * depth * stage_bytes;
    {
        uint4* xs = reinterpret_cast<uint4*>(tables0);
        float* sa = reinterpret_cast<float*>(xs + A.chunks * GLT * 8);
        const int per_job = A.chunks * CMAX * 4;  // a multiple of 4: quads stay whole
        const int items = per_job * njobs_here;
        bool bad = false;
        for (int idx0 = warp * 32; idx0 < items; idx0 += W * 32) {
            const int idx = idx0 + lane;
            const bool live = idx < items;
            const int i2 = live ? idx : items - 1;
            const int jj = JOBS ? i2 / per_job : 0, ii = i2 - jj * per_job;
            const int chunk = ii / (CMAX * 4), rem = ii - chunk * (CMAX * 4), c = rem >> 2, tt = rem & 3;
            const int src_row = JOBS ? A.job_src[(job0 + jj) * CMAX + c] : c;
            const bool has = JOBS ? src_row >= 0 : c < A.n_cols;
            const float* xr = A.x + (int64_t)(has ? src_row : 0) * A.x_ld;
            if (JOBS) {
                xs = reinterpret_cast<uint4*>(tables0 + (size_t)jj * A.table_stride);
                sa = reinterpret_cast<float*>(xs + A.chunks * GLT * 8);
            }
            // the four elements of one mma are consecutive in x (component r + 2h, Q6_K: 2r + h)
            float xv[4][2][2];
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const int el = chunk * 64 + chunk_col<TYPE>(tt, m, 0, 0);
                float4 v = __ldg(reinterpret_cast<const float4*>(xr + (el < A.cols ? el : 0)));
                if (!JOBS && A.norm_on) {
                    float inv = inv_rms[0];
#pragma unroll
                    for (int cc = 1; cc < CMAX; cc++) inv = c == cc ? inv_rms[cc] : inv;
                    v = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
                    if (A.norm_w) {
                        const float4 nw = __ldg(reinterpret_cast<const float4*>(A.norm_w + (el < A.cols ? el : 0)));
                        v = make_float4(v.x * nw.x, v.y * nw.y, v.z * nw.z, v.w * nw.w);
                    }
                }
                if (A.gelu_inter > 0) {
                    const float4 u = __ldg(reinterpret_cast<const float4*>(xr + A.gelu_inter + (el < A.cols ? el : 0)));
                    v = make_float4(gelu_tanh_up(v.x, u.x), gelu_tanh_up(v.y, u.y), gelu_tanh_up(v.z, u.z), gelu_tanh_up(v.w, u.w));
                }
                const bool in = el < A.cols && has;
                const float q[4] = {in ? v.x : 0.f, in ? v.y : 0.f, in ? v.z : 0.f, in ? v.w : 0.f};
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int h = 0; h < 2; h++) xv[m][r][h] = q[chunk_col<TYPE>(tt, m, r, h) - chunk_col<TYPE>(tt, m, 0, 0)];
            }
            unsigned r0[8], r1[8];         // fragment registers of term 0 / term 1
            float seen0[4], seen1[4];      // what the tensor core sees of each mma's four elements, summed
            float plain[2] = {0.f, 0.f};   // true activations of the chunk's two halves
#pragma unroll
            for (int m = 0; m < 4; m++) {
                seen0[m] = seen1[m] = 0.f;
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const float sc = chunk_hi<TYPE>(m) ? kHiScale : 1.0f;
                    const float v0 = xv[m][r][0] * sc, v1 = xv[m][r][1] * sc;
                    // x = h0 + h1 * 2^-11, both exactly representable in fp16
                    const __half2 p0 = __floats2half2_rn(v0, v1);
                    const float2 f0 = __half22float2(p0);
                    const __half2 p1 = __floats2half2_rn((v0 - f0.x) * 2048.0f, (v1 - f0.y) * 2048.0f);
                    const float2 f1 = __half22float2(p1);
                    bad |= !isfinite(f0.x) | !isfinite(f0.y);
                    r0[m * 2 + r] = *reinterpret_cast<const unsigned*>(&p0);
                    r1[m * 2 + r] = *reinterpret_cast<const unsigned*>(&p1);
                    seen0[m] += f0.x + f0.y;
                    seen1[m] += f1.x + f1.y;
                    plain[m >> 1] += xv[m][r][0] + xv[m][r][1];
                }
            }
            if (live) {
                uint4* e0 = xs + (((chunk * GLT + 2 * c) * 4 + tt) * 2);
                e0[0] = make_uint4(r0[0], r0[1], r0[2], r0[3]);
                e0[1] = make_uint4(r0[4], r0[5], r0[6], r0[7]);
                e0[8] = make_uint4(r1[0], r1[1], r1[2], r1[3]);  // column 2c+1: four lanes x two units further
                e0[9] = make_uint4(r1[4], r1[5], r1[6], r1[7]);
            }
            // sums over the quad (the four tt of one chunk and column)
            if (TYPE == LEV_GGML_Q4_K) {
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    float v = plain[hf];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (live && tt == 0) sa[(chunk * 2 + hf) * CMAX + c] = v;
                }
            } else if (TYPE == LEV_GGML_Q6_K) {
                // -32 * 2^-24 * (sum seen by the tensor core) of each 16-value sub-block; levels of
                // mma 2, 3 sit 16x high against activations divided by 16
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    const float k = (chunk_hi<TYPE>(m) ? 16.0f : 1.0f) * -32.0f * 5.9604644775390625e-08f;
                    float v0 = seen0[m], v1 = seen1[m];
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
                    if (live && tt == 0) {
                        sa[(chunk * 4 + m) * GLT + 2 * c] = k * v0;
                        sa[(chunk * 4 + m) * GLT + 2 * c + 1] = k * v1;
                    }
                }
            } else {
                // -8 * 2^-24 * (sum seen by the tensor core) of each 32-value block (mma 2b: low
                // nibbles, mma 2b+1: high nibbles, worth 16x against activations divided by 16)
#pragma unroll
                for (int blk = 0; blk < 2; blk++) {
                    const float k = -8.0f * 5.9604644775390625e-08f;
                    float v0 = seen0[2 * blk] + 16.0f * seen0[2 * blk + 1], v1 = seen1[2 * blk] + 16.0f * seen1[2 * blk + 1];
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
                    if (live && tt == 0) {
                        sa[(chunk * 2 + blk) * GLT + 2 * c] = k * v0;
                        sa[(chunk * 2 + blk) * GLT + 2 * c + 1] = k * v1;
                    }
                }
            }
        }
        if (bad) atomicOr(A.status, LEV_DEV_NONFINITE_INPUT);
    }
    __syncthreads();

    // One column runs the column-group arithmetic of lev_chain_math.cuh (a third fewer instructions per K-step than
    // the general form below: one accumulator chain per K-step, block scales applied once): ya / yb are this lane's
    // sums of rows g and g + 8, the table layout is the same.
    float ya = 0.f, yb = 0.f;
    LaneConst LC;
    LC.q_off = 16u * lane;
    LC.hdr_off = 16u * g;
    LC.x_off = (unsigned)(((g & 1) * 4 + t) * 32);
    LC.grp = (unsigned)(g >> 1);
    LC.t = (unsigned)t;
    LC.g = (unsigned)g;
    LC.sh16 = 16u * (t & 1);
    LC.zero_s = smem_u32(zero_block);
    unsigned xs_s = 0, sa_s = 0;  // shared-memory addresses of the tables of the tile being worked on
    float yacc[NT][4];
    float mina[CMAX], minb[CMAX];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
    for (int c = 0; c < CMAX; c++) mina[c] = minb[c] = 0.f;

    int slot = 0;        // ring stage in use
    unsigned phase = 0;  // its mbarrier phase parity
    int seg_k0 = k;
    const int first_tl = tl;
    // tables, output row and tile-in-job of the tile being worked on
    const uint4* xs = reinterpret_cast<const uint4*>(tables0);
    const float* sa = reinterpret_cast<const float*>(xs + A.chunks * GLT * 8);
    int job = 0, tij = tile0 + tl;
    float* cur_y = A.y;
    int64_t cur_rows = A.rows, cur_ld = A.out_ld;
    int orow[CMAX];
#pragma unroll
    for (int c = 0; c < CMAX; c++) orow[c] = 0;
    // first: the warp's first tile; afterwards tiles are entered in order, and only a new job reloads anything
    auto enter_tile = [&](bool first) {
        if (JOBS) {
            if (first) {
                job = (tile0 + tl) / tpj;
                tij = tile0 + tl - job * tpj;
            } else if (++tij == tpj) {
                tij = 0;
                job++;
            } else {
                return;
            }
            xs = reinterpret_cast<const uint4*>(tables0 + (size_t)(job - job0) * A.table_stride);
            sa = reinterpret_cast<const float*>(xs + A.chunks * GLT * 8);
            xs_s = 0;  // (one column) the tables' shared-memory addresses are formed again
#pragma unroll
            for (int c = 0; c < CMAX; c++) orow[c] = A.job_out[job * CMAX + c];
        } else if (MULTI) {
            const int o = op_of(tile0 + tl);
            tij = tile0 + tl - A.tiles_cum[o];
            cur_y = A.y_op[o];
            cur_rows = cur_ld = A.rows_op[o];
        } else {
            tij = tile0 + tl;
        }
    };
    if (s < e) enter_tile(true);
    for (int i0 = s; i0 < e; i0 += sps) {
        if (!mbar_wait(bar_s + 8 * slot, phase)) {
            if (lane == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
            break;
        }
        const int i1 = i0 + sps < e ? i0 + sps : e;
        for (int i = i0; i < i1; i++) {
            const uint4* st = reinterpret_cast<const uint4*>(ring + slot * stage_bytes + (i - i0) * kStepBytes);
            if constexpr (CMAX == 1) {
                if (xs_s == 0) {
                    xs_s = smem_u32(xs);
                    sa_s = smem_u32(sa);
                    order_after(xs_s);
                }
                unsigned st_s = ring_s + (unsigned)slot * stage_bytes + (unsigned)(i - i0) * kStepBytes;
                order_after(st_s);  // the loads inside are plain asm: this keeps them behind the wait above
                chain_step<TYPE>(st_s, xs_s + (unsigned)k * 1024u, sa_s + (unsigned)k * (16u * kAuxPerChunk), LC, ya, yb);
            } else {
                stream_step<TYPE, CMAX, true>(st, xs + k * (4 * GLT * 8), sa + k * (4 * kAuxPerChunk), lane, O, yacc, mina, minb);
            }
            k++;
            if (k == spt || i == e - 1) {
                // ---- this warp's segment of the tile ends: fold to one f32 per (row, column) ----
                const bool whole = seg_k0 == 0 && k == spt;
                const int r = tl == first_tl ? 0 : 1;
#pragma unroll
                for (int c = 0; c < CMAX; c++) {
                    float va = 0.f, vb = 0.f;
                    if constexpr (CMAX == 1) {
                        va = ya;
                        vb = yb;
                    } else {
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
                    }
                    va += __shfl_xor_sync(0xffffffffu, va, 1);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 1);
                    va += __shfl_xor_sync(0xffffffffu, va, 2);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 2);
                    if (t == 0) {
                        if (whole) {
                            const int64_t row = (int64_t)tij * 16 + g;
                            const int oc = JOBS ? orow[c] : c;
                            if (JOBS ? orow[c] >= 0 : c < A.n_cols) {
                                const int64_t at = (int64_t)oc * cur_ld + row;
                                if (!JOBS && !MULTI && A.residual) {
                                    if (row < cur_rows) va = fmaf(A.alpha, va, A.residual[at]);
                                    if (row + 8 < cur_rows) vb = fmaf(A.alpha, vb, A.residual[at + 8]);
                                }
                                if (row < cur_rows) cur_y[at] = va;
                                if (row + 8 < cur_rows) cur_y[at + 8] = vb;
                            }
                        } else {
                            rec[warp][r][c][g] = va;
                            rec[warp][r][c][g + 8] = vb;
                        }
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int j = 0; j < 4; j++) yacc[nt][j] = 0.f;
#pragma unroll
                for (int c = 0; c < CMAX; c++) mina[c] = minb[c] = 0.f;
                ya = yb = 0.f;
                tl++;
                k = 0;
                seg_k0 = 0;
                if (i + 1 < e) enter_tile(false);
            }
        }
        // every lane has consumed its shared-memory reads of this stage: refill it
        __syncwarp();
        if (lane == 0 && f_left > 0) issue_stage(slot);
        if (++slot == depth) {
            slot = 0;
            phase ^= 1u;
        }
    }
    __syncthreads();
    // ---- tiles shared between warps: add the warps' records in the order of their ranges ----
    // logical warp l owns steps [nst*l/W, nst*(l+1)/W); the one holding step q is ((q+1)*W - 1) / nst
    for (int item = threadIdx.x; item < ntiles * CMAX * 16; item += W * 32) {
        const int tile = item / (CMAX * 16), idx = item - tile * (CMAX * 16);
        const int l_first = ((tile * spt + 1) * W - 1) / nst, l_last = ((tile * spt + spt) * W - 1) / nst;
        if (l_first == l_last) continue;  // one warp had the whole tile and wrote it
        float acc = 0.f;
        for (int l2 = l_first; l2 <= l_last; l2++) {
            const int pw = (l2 % (W / 4)) * 4 + l2 / (W / 4);  // the warp whose logical position is l2
            const int s2 = (int)((int64_t)nst * l2 / W), e2 = (int)((int64_t)nst * (l2 + 1) / W);
            if (s2 == e2) continue;  // more warps than K-steps: this one had nothing
            acc += rec[pw][tile == s2 / spt ? 0 : 1][0][idx];
        }
        const int c = idx >> 4;
        if (JOBS) {
            const int pjob = (tile0 + tile) / tpj, ptij = tile0 + tile - pjob * tpj, oc = A.job_out[pjob * CMAX + c];
            const int64_t row = (int64_t)ptij * 16 + (idx & 15);
            if (oc >= 0 && row < A.rows) A.y[(int64_t)oc * A.out_ld + row] = acc;
        } else if (MULTI) {
            const int o = op_of(tile0 + tile);
            const int64_t row = (int64_t)(tile0 + tile - A.tiles_cum[o]) * 16 + (idx & 15);
            if (c < A.n_cols && row < A.rows_op[o]) A.y_op[o][(int64_t)c * A.rows_op[o] + row] = acc;
        } else {
            const int64_t row = (int64_t)(tile0 + tile) * 16 + (idx & 15);
            if (c < A.n_cols && row < A.rows) {
                const int64_t at = (int64_t)c * A.out_ld + row;
                A.y[at] = A.residual ? fmaf(A.alpha, acc, A.residual[at]) : acc;
            }
        }
    }
}


template <int TYPE, int CMAX, int W, bool JOBS = false, bool MULTI = false>
int launch_dense(lev_ctx* ctx, int grid, size_t smem, const DenseArgs& A) {
    static size_t configured[16] = {};  // per device: largest dynamic shared memory opted in so far
    if (configured[ctx->device & 15] < smem) {
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_dense<TYPE, CMAX, W, JOBS, MULTI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // every instance asks for the same (largest) shared-memory carve-out: an SM whose split
        // would have to change between two launches cannot hold CTAs of both at once
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_dense<TYPE, CMAX, W, JOBS, MULTI>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           (int)cudaSharedmemCarveoutMaxShared));
        configured[ctx->device & 15] = smem;
    }
    LEV_CUDA(ctx, launch_pdl(k_dense<TYPE, CMAX, W, JOBS, MULTI>, dim3(grid), dim3(W * 32), smem, ctx->stream, A));
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
    int warps, depth, sps, grid;
    size_t smem;
};

// Shape of a launch, or false when the tables do not fit beside a useful ring.
bool dense_plan_tiles(lev_ctx* ctx, const lev_weights* w, int64_t tiles, int n_cols, DensePlan* P) {
    if (n_cols < 1 || n_cols > 4) return false;
    const size_t step = step_bytes(w->type);
    const size_t tb = lev_stream_table_bytes(w, n_cols, 2, 1, nullptr);
    const int64_t spt = lev_stream_chunks(w) / 4;
    if (tiles < 1 || tiles * spt > 0x7fffffff / 64) return false;
    const int warps = 8;
    // half of an SM's shared memory unless one CTA takes the SM
    size_t cap = (size_t)110 * 1024;
    const int sms = ctx->prop.multiProcessorCount;
    const int grid = (int)(tiles < sms ? tiles : sms);
    const int64_t per_cta = ((tiles + grid - 1) / grid) * spt;
    const int64_t per_warp = (per_cta + warps - 1) / warps;
    if (tb + (size_t)warps * step > cap) {
        // large tables: give the CTA the whole SM before giving up
        cap = 200 * 1024;
        if (tb + (size_t)warps * step > cap) return false;
    }
    // K-steps one warp can hold in shared memory, cut into stages of sps steps
    int64_t room = (int64_t)((cap - tb) / ((size_t)warps * step));
    if (room > per_warp) room = per_warp;
    int sps = 2;
    if (sps * 2 > room) sps = room >= 2 ? (int)(room / 2) : 1;  // at least two stages when there is room
    int64_t depth = room / sps;
    if (depth > kMaxDepth) depth = kMaxDepth;
    if (depth < 1) depth = 1;
    P->warps = warps;
    P->depth = (int)depth;
    P->sps = sps;
    P->grid = grid;
    P->smem = (size_t)warps * depth * sps * step + tb;
    return true;
}

bool dense_plan(lev_ctx* ctx, const lev_weights* w, int64_t rows, int n_cols, DensePlan* P) {
    return dense_plan_tiles(ctx, w, (rows + 15) / 16, n_cols, P);
}

template <int TYPE>
int launch_multi_c(lev_ctx* ctx, int cmax, int grid, size_t smem, const DenseArgs& A) {
    switch (cmax) {
        case 1: return launch_dense<TYPE, 1, 8, false, true>(ctx, grid, smem, A);
        case 2: return launch_dense<TYPE, 2, 8, false, true>(ctx, grid, smem, A);
        case 3: return launch_dense<TYPE, 3, 8, false, true>(ctx, grid, smem, A);
        case 4: return launch_dense<TYPE, 4, 8, false, true>(ctx, grid, smem, A);
    }
    return lev_fail(ctx, LEV_BAD_DIMENSIONS, "columns %d", cmax);
}

}  // namespace

// Several whole tensors of one format and K against the same activations in one launch.
bool lev_dense_multi_supported(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x, int n_cols) {
    if (n_ops < 2 || n_ops > 4 || ((uintptr_t)x & 15) != 0) return false;
    int64_t tiles = 0;
    for (int i = 0; i < n_ops; i++) {
        if (!w[i] || !w[i]->packed || w[i]->type != w[0]->type || w[i]->cols != w[0]->cols) return false;
        tiles += (w[i]->rows + 15) / 16;
    }
    DensePlan P;
    return dense_plan_tiles(ctx, w[0], tiles, n_cols, &P);
}

// prologue fields shared by the dense and multi forms
static void apply_fusion(DenseArgs& A, const lev_dense_fusion* f, int64_t cols) {
    if (!f) return;
    A.norm_on = f->norm_on;
    A.norm_w = f->norm_w;
    A.norm_eps = f->eps;
    if (f->gelu_up) {
        A.gelu_inter = (int)cols;
        A.x_ld = 2 * cols;
    }
    A.residual = f->residual;
    A.alpha = f->alpha;
}

int lev_dense_multi_run(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x, int n_cols, float* const* y,
                        const lev_dense_fusion* fusion) {
    if (!lev_dense_multi_supported(ctx, n_ops, w, x, n_cols) || (fusion && fusion->residual))
        return lev_fail(ctx, LEV_UNSUPPORTED, "multi-tensor dense kernel: shapes not served");
    const int64_t chunks = lev_stream_chunks(w[0]), spt = chunks / 4;
    DenseArgs A = {};
    int64_t tiles = 0;
    A.n_ops = n_ops;
    for (int i = 0; i < n_ops; i++) {
        A.wp_op[i] = (const uint4*)w[i]->packed;
        A.tiles_cum[i] = (int)tiles;
        A.y_op[i] = y[i];
        A.rows_op[i] = w[i]->rows;
        tiles += (w[i]->rows + 15) / 16;
    }
    for (int i = n_ops; i <= 4; i++) A.tiles_cum[i] = (int)tiles;
    DensePlan P;
    dense_plan_tiles(ctx, w[0], tiles, n_cols, &P);
    A.wp = A.wp_op[0];
    A.spt = (int)spt;
    A.tiles_base = (int)(tiles / P.grid);
    A.tiles_rem = (int)(tiles % P.grid);
    A.x = x;
    A.x_ld = w[0]->cols;
    A.cols = (int)w[0]->cols;
    A.chunks = (int)chunks;
    A.n_cols = n_cols;
    A.y = y[0];
    A.rows = w[0]->rows;
    A.out_ld = w[0]->rows;
    A.status = ctx->d_status;
    A.depth = P.depth;
    A.sps = P.sps;
    apply_fusion(A, fusion, w[0]->cols);
    const int t = w[0]->type;
    int st = t == LEV_GGML_Q4_K   ? launch_multi_c<LEV_GGML_Q4_K>(ctx, n_cols, P.grid, P.smem, A)
             : t == LEV_GGML_Q6_K ? launch_multi_c<LEV_GGML_Q6_K>(ctx, n_cols, P.grid, P.smem, A)
                                  : launch_multi_c<LEV_GGML_Q4_0>(ctx, n_cols, P.grid, P.smem, A);
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = P.grid;
    ctx->ev.block = 8 * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_dense (multi)");
}

bool lev_dense_supported(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols) {
    DensePlan P;
    // x is read in 16-byte vectors
    return w->packed && row0 % 16 == 0 && ((uintptr_t)x & 15) == 0 && dense_plan(ctx, w, rows, n_cols, &P);
}

// x: [n_cols][w->cols] device, y: [n_cols][rows] device.  No work buffers.
int lev_dense_run(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols, float* y,
                  const lev_dense_fusion* fusion) {
    DensePlan P;
    if (!w->packed || row0 % 16 != 0 || ((uintptr_t)x & 15) != 0 || !dense_plan(ctx, w, rows, n_cols, &P))
        return lev_fail(ctx, LEV_UNSUPPORTED, "dense stream kernel: shape not served");
    const int64_t tiles = (rows + 15) / 16, chunks = lev_stream_chunks(w), spt = chunks / 4;
    const size_t step = step_bytes(w->type);
    DenseArgs A = {};
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
    A.sps = P.sps;
    apply_fusion(A, fusion, w->cols);
    int st = w->type == LEV_GGML_Q4_K   ? launch_dense_c<LEV_GGML_Q4_K>(ctx, n_cols, P.warps, P.grid, P.smem, A)
             : w->type == LEV_GGML_Q6_K ? launch_dense_c<LEV_GGML_Q6_K>(ctx, n_cols, P.warps, P.grid, P.smem, A)
                                        : launch_dense_c<LEV_GGML_Q4_0>(ctx, n_cols, P.warps, P.grid, P.smem, A);
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = P.grid;
    ctx->ev.block = P.warps * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_dense");
}

// Sliced form: a device-side list of up to max_jobs jobs, job j = one activation column (row
// job_src[j] of x, optionally through gelu_tanh(gate) * up) against slice job_slice[j] of the
// tensor (slice = rows_per_job consecutive rows), result to row job_out[j] of y.
// shared-memory budget of the sliced form: half an SM when the tables allow it (so that consecutive
// launches co-reside), else the whole SM
static size_t jobs_cap(size_t tables, size_t step) {
    return tables + 8 * 2 * step <= 110 * 1024 ? 110 * 1024 : 200 * 1024;
}

bool lev_dense_jobs_supported(lev_ctx* ctx, const lev_weights* w, int64_t rows_per_job, int max_jobs, int cmax,
                              const float* x, int64_t x_ld) {
    if (!w->packed || rows_per_job % 16 != 0 || max_jobs < 1) return false;
    if (cmax != 1 && cmax != 4) return false;
    if (((uintptr_t)x & 15) != 0 || x_ld % 4 != 0) return false;
    // a CTA's run of tiles may touch at most kMaxJobTables jobs
    const int64_t tpj = rows_per_job / 16, sms = ctx->prop.multiProcessorCount;
    const int64_t max_tiles = (int64_t)max_jobs * tpj, grid = max_tiles < sms ? max_tiles : sms;
    const int64_t run = (max_tiles + grid - 1) / grid;
    if ((run + tpj - 1) / tpj + 1 > kMaxJobTables) return false;
    const size_t stride = (lev_stream_table_bytes(w, cmax, 2, 1, nullptr) + 255) & ~(size_t)255;
    const size_t step = step_bytes(w->type);
    return kMaxJobTables * stride + 8 * 2 * step <= jobs_cap(kMaxJobTables * stride, step);
}

int lev_dense_jobs_run(lev_ctx* ctx, const lev_weights* w, int64_t rows_per_job, int max_jobs, int cmax, const int* njobs_dev,
                       const int* job_slice, const int* job_src, const int* job_out, const float* x, int64_t x_ld,
                       int gelu_inter, float* y, int64_t out_ld) {
    if (!lev_dense_jobs_supported(ctx, w, rows_per_job, max_jobs, cmax, x, x_ld))
        return lev_fail(ctx, LEV_UNSUPPORTED, "sliced dense kernel: shape not served");
    const int64_t tpj = rows_per_job / 16, chunks = lev_stream_chunks(w), spt = chunks / 4;
    const size_t step = step_bytes(w->type);
    const size_t stride = (lev_stream_table_bytes(w, cmax, 2, 1, nullptr) + 255) & ~(size_t)255;
    const int sms = ctx->prop.multiProcessorCount;
    const int64_t max_tiles = (int64_t)max_jobs * tpj;
    // jobs a CTA's run of tiles can touch when the list's tiles are dealt to `ctas` CTAs
    auto tables_for = [&](int64_t ctas) -> int64_t {
        const int64_t g = max_tiles < ctas ? max_tiles : ctas, run = (max_tiles + g - 1) / g;
        const int64_t n = (run + tpj - 1) / tpj + 1;
        return n < kMaxJobTables ? n : kMaxJobTables;
    };
    // A list is a dependent step of its layer (nothing of the next launch can run beside it): two CTAs of eight
    // warps per SM when their tables and two ring stages per warp fit half an SM, else one CTA per SM with as many
    // warps as leave two stages each.
    int W = 8;
    int64_t slots = 2 * (int64_t)sms, n_tables = tables_for(slots);
    size_t cap = 110 * 1024;
    if (n_tables * stride + 8 * 2 * step > cap) {
        slots = sms;
        n_tables = tables_for(slots);
        cap = 200 * 1024;
        if (cmax == 4) W = n_tables * stride + 16 * 2 * step <= cap ? 16 : 12;
    }
    const int grid = (int)(max_tiles < slots ? max_tiles : slots);
    const int64_t per_warp = (((max_tiles + grid - 1) / grid) * spt + W - 1) / W;
    int64_t depth = (int64_t)((cap - n_tables * stride) / ((size_t)W * step));
    if (depth > per_warp) depth = per_warp;
    if (depth > kMaxDepth) depth = kMaxDepth;
    if (depth < 1) depth = 1;
    DenseArgs A = {};
    A.wp = (const uint4*)w->packed;
    A.spt = (int)spt;
    A.x = x;
    A.x_ld = x_ld;
    A.cols = (int)w->cols;
    A.chunks = (int)chunks;
    A.n_cols = cmax;
    A.y = y;
    A.rows = rows_per_job;
    A.out_ld = out_ld;
    A.status = ctx->d_status;
    A.depth = (int)depth;
    A.sps = 1;
    A.njobs_dev = njobs_dev;
    A.job_slice = job_slice;
    A.job_src = job_src;
    A.job_out = job_out;
    A.tiles_per_job = (int)tpj;
    A.gelu_inter = gelu_inter;
    A.table_stride = (int)stride;
    A.max_tables = (int)n_tables;
    const size_t smem = (size_t)W * depth * step + n_tables * stride;
    int st;
    if (cmax == 1)
        st = w->type == LEV_GGML_Q4_K   ? launch_dense<LEV_GGML_Q4_K, 1, 8, true>(ctx, grid, smem, A)
             : w->type == LEV_GGML_Q6_K ? launch_dense<LEV_GGML_Q6_K, 1, 8, true>(ctx, grid, smem, A)
                                        : launch_dense<LEV_GGML_Q4_0, 1, 8, true>(ctx, grid, smem, A);
    else if (W == 8)
        st = w->type == LEV_GGML_Q4_K   ? launch_dense<LEV_GGML_Q4_K, 4, 8, true>(ctx, grid, smem, A)
             : w->type == LEV_GGML_Q6_K ? launch_dense<LEV_GGML_Q6_K, 4, 8, true>(ctx, grid, smem, A)
                                        : launch_dense<LEV_GGML_Q4_0, 4, 8, true>(ctx, grid, smem, A);
    else if (W == 12)
        st = w->type == LEV_GGML_Q4_K   ? launch_dense<LEV_GGML_Q4_K, 4, 12, true>(ctx, grid, smem, A)
             : w->type == LEV_GGML_Q6_K ? launch_dense<LEV_GGML_Q6_K, 4, 12, true>(ctx, grid, smem, A)
                                        : launch_dense<LEV_GGML_Q4_0, 4, 12, true>(ctx, grid, smem, A);
    else
        st = w->type == LEV_GGML_Q4_K   ? launch_dense<LEV_GGML_Q4_K, 4, 16, true>(ctx, grid, smem, A)
             : w->type == LEV_GGML_Q6_K ? launch_dense<LEV_GGML_Q6_K, 4, 16, true>(ctx, grid, smem, A)
                                        : launch_dense<LEV_GGML_Q4_0, 4, 16, true>(ctx, grid, smem, A);
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = grid;
    ctx->ev.block = W * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_dense (sliced)");
}
