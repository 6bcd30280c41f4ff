// Persistent decode matvec: a list of y = W x products (one activation column) in ONE launch.
//
// The reference's decode loop records a sequence of matvec steps and submits them together
// (rust/crates/lev-model/src/gpu.rs:334-370 records, rust/crates/lev-vulkan/src/engine.rs:87-153
// runs the recorded steps); on the Swift side the FFN is `matvec(gate), matvec(up) -> geluUp ->
// matvec(down) -> axpy` (Sources/LeviathanCore/Gemma4.swift:3741-3753).  Here such a list runs as
// one grid of one thread block per SM:
//
//  * every op's K-steps (16 rows x 256 columns of packed weights, see lev_stream.cu) are split in
//    equal contiguous shares over the blocks and, inside a block, over its compute warps
//    (lev_chain_split.h).  A warp streams its share through its own ring of shared-memory slots
//    filled by cp.async.bulk; the fetch side runs ahead across op boundaries, so the HBM stream
//    does not pause where one tensor ends and the next begins;
//  * four helper warps build each op's activation tables (fp16 split terms in mma fragment order,
//    bias sums) one op ahead of the compute warps, apply the fused prologues (RMSNorm, gelu(gate)*up)
//    and, where an op reads what earlier ops of the launch wrote, wait on a grid-wide arrival
//    counter first; compute warps that reach an op whose tables are not ready help to build them;
//  * arithmetic: the fp16-subnormal tensor-core dot of lev_stream_math.cuh with the eight mma
//    columns used as four sub-block groups x two activation terms, so one accumulator chain spans a
//    whole K-step and block scales are applied once per K-step by the lane that owns the sub-block;
//  * tiles shared by warps or by blocks are finished by the last to arrive, adding partial sums in
//    a fixed order: same call, same bits.
//
// Every wait is bounded (about one second of SM clocks); on expiry the block records LEV_DEV_TIMEOUT,
// drains its own copies in flight and returns.
#include <type_traits>

#include "lev_chain_split.h"
#include "lev_stream.h"
#include "lev_stream_math.cuh"
#include "lev_chain_math.cuh"

namespace {

constexpr int kChainMaxOps = kLevChainMaxOps;
constexpr int kHelperWarps = 4;  // three table builders, one finisher of shared tiles

struct ChainOp {
    const unsigned char* wp;  // packed bytes of the op's first tile
    const float* x;           // activations [cols] (gelu form: [gate(cols) | up(cols)])
    float* y;                 // [rows]
    const float* norm_w;      // RMSNorm weight or NULL
    const float* residual;    // y = residual + alpha * (W x), or NULL
    int64_t rows;
    int type, spt, nsteps, cols, chunks;
    int wait;        // the activations are written by earlier ops of this launch
    int fence;       // a later op of the launch waits: results are fenced before the warp moves on
    int tab;         // op whose tables this op reads (itself when it builds its own)
    int tslot;       // table buffer (0 / 1) of the tables it builds
    int free_after;  // last op that reads the buffer's previous contents, -1: none
    int norm_on;
    float norm_eps;
    int gelu_inter;  // > 0: activation e = gelu_tanh(x[e]) * x[gelu_inter + e]
    float alpha;
};

struct ChainArgs {
    ChainOp op[kChainMaxOps];
    int n_ops;
    int ring_bytes, ring_stride;  // ring of every compute warp: usable bytes, bytes between the warps' rings
    int tab_off[2], rec_off;   // byte offsets in dynamic shared memory (the ring starts at 0)
    int* status;
    unsigned* sync;            // [2 * kChainMaxOps] grid arrival / departure counters
    uint2* gpart;              // [op][block][2][16] (sum, flag) of tiles shared by blocks; flags rest at 0
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ---------------------------------------------------------------------------
// activation tables of one op: one warp builds 32 items (item = chunk x lane-of-quad, one column)
// ---------------------------------------------------------------------------
template <int TYPE>
__device__ void build_piece(const ChainOp& P, int piece, int lane, unsigned char* tables, float inv, int* status) {
    constexpr int CMAX = 1, GLT = 2;
    uint4* xs = reinterpret_cast<uint4*>(tables);
    float* sa = reinterpret_cast<float*>(xs + P.chunks * GLT * 8);
    const int items = P.chunks * 4;
    const int idx = piece * 32 + lane;
    const bool live = idx < items;
    const int i2 = live ? idx : items - 1;
    const int chunk = i2 >> 2, tt = i2 & 3;
    const float* xr = P.x;
    float xv[4][2][2];
#pragma unroll
    for (int m = 0; m < 4; m++) {
        const int el = chunk * 64 + chunk_col<TYPE>(tt, m, 0, 0);
        const int at = el < P.cols ? el : 0;
        // plain loads: the activations may have been written by earlier ops of this launch
        float4 v = *reinterpret_cast<const float4*>(xr + at);
        if (P.norm_on) {
            v = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
            if (P.norm_w) {
                const float4 nw = __ldg(reinterpret_cast<const float4*>(P.norm_w + at));
                v = make_float4(v.x * nw.x, v.y * nw.y, v.z * nw.z, v.w * nw.w);
            }
        }
        if (P.gelu_inter > 0) {
            const float4 u = *reinterpret_cast<const float4*>(xr + P.gelu_inter + at);
            v = make_float4(gelu_tanh_up(v.x, u.x), gelu_tanh_up(v.y, u.y), gelu_tanh_up(v.z, u.z), gelu_tanh_up(v.w, u.w));
        }
        const bool in = el < P.cols;
        const float q[4] = {in ? v.x : 0.f, in ? v.y : 0.f, in ? v.z : 0.f, in ? v.w : 0.f};
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int h = 0; h < 2; h++) xv[m][r][h] = q[chunk_col<TYPE>(tt, m, r, h) - chunk_col<TYPE>(tt, m, 0, 0)];
    }
    unsigned r0[8], r1[8];
    float seen0[4], seen1[4];
    float plain[2] = {0.f, 0.f};
    bool bad = false;
#pragma unroll
    for (int m = 0; m < 4; m++) {
        seen0[m] = seen1[m] = 0.f;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float sc = chunk_hi<TYPE>(m) ? kHiScale : 1.0f;
            const float v0 = xv[m][r][0] * sc, v1 = xv[m][r][1] * sc;
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
        uint4* e0 = xs + ((chunk * GLT * 4 + tt) * 2);
        e0[0] = make_uint4(r0[0], r0[1], r0[2], r0[3]);
        e0[1] = make_uint4(r0[4], r0[5], r0[6], r0[7]);
        e0[8] = make_uint4(r1[0], r1[1], r1[2], r1[3]);
        e0[9] = make_uint4(r1[4], r1[5], r1[6], r1[7]);
    }
    if (TYPE == LEV_GGML_Q4_K) {
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            float v = plain[hf];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (live && tt == 0) sa[(chunk * 2 + hf) * CMAX] = v;
        }
    } else if (TYPE == LEV_GGML_Q6_K) {
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const float k = (chunk_hi<TYPE>(m) ? 16.0f : 1.0f) * -32.0f * 5.9604644775390625e-08f;
            float v0 = seen0[m], v1 = seen1[m];
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (live && tt == 0) {
                sa[(chunk * 4 + m) * GLT] = k * v0;
                sa[(chunk * 4 + m) * GLT + 1] = k * v1;
            }
        }
    } else {
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
            const float k = -8.0f * 5.9604644775390625e-08f;
            float v0 = seen0[2 * blk] + 16.0f * seen0[2 * blk + 1], v1 = seen1[2 * blk] + 16.0f * seen1[2 * blk + 1];
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (live && tt == 0) {
                sa[(chunk * 2 + blk) * GLT] = k * v0;
                sa[(chunk * 2 + blk) * GLT + 1] = k * v1;
            }
        }
    }
    if (bad) atomicOr(status, LEV_DEV_NONFINITE_INPUT);
}

__device__ __forceinline__ void build_piece_any(const ChainOp& P, int piece, int lane, unsigned char* tables, float inv, int* status) {
    if (P.type == LEV_GGML_Q4_K) build_piece<LEV_GGML_Q4_K>(P, piece, lane, tables, inv, status);
    else if (P.type == LEV_GGML_Q6_K) build_piece<LEV_GGML_Q6_K>(P, piece, lane, tables, inv, status);
    else build_piece<LEV_GGML_Q4_0>(P, piece, lane, tables, inv, status);
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
constexpr int kBuilderWarps = 3;
constexpr int kQueue = 16;                       // tiles waiting for the finishing warp
constexpr int kRecDepth = 4;                     // ops whose records and tickets are kept apart: a warp may run that far ahead
constexpr int kRingBars = 8;                     // bulk copies one compute warp may have in flight
// K-steps per bulk copy: the copy engine takes a fixed time per request, so small steps travel in pairs
__host__ __device__ constexpr unsigned copy_steps(int type) { return type == LEV_GGML_Q6_K ? 1u : 2u; }

struct TileEntry {
    float v[16];        // this block's sums of the tile's 16 rows
    int op;
    unsigned tile;
    volatile unsigned ready;  // sequence number + 1 once the entry is complete
    int pad;
};


template <int W>
__global__ void __launch_bounds__((W + kHelperWarps) * 32, 1) k_chain(const __grid_constant__ ChainArgs A) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bars[W][kRingBars];
    __shared__ __align__(16) uint4 zero_block[2];
    __shared__ __align__(16) TileEntry fq[kQueue];
    __shared__ unsigned fq_tail;
    __shared__ volatile unsigned fq_head;
    __shared__ volatile int prog[W];                      // op a compute warp works on; all earlier ones are done
    __shared__ volatile int tab_ready[kChainMaxOps];      // tables built
    __shared__ volatile int tab_open[kChainMaxOps];       // pieces may be claimed
    __shared__ int piece_next[kChainMaxOps], piece_done[kChainMaxOps];
    __shared__ int tick[kRecDepth][2 * W];                // arrivals at tiles shared by warps, per op (mod kRecDepth)
    __shared__ float norm_inv[2];                         // per table buffer
    __shared__ float hpart[kHelperWarps];
    __shared__ volatile int abort_flag;
    __shared__ volatile int fq_hurry;                     // a builder waits for the queue to drain

    typedef unsigned u32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, G = gridDim.x, n_ops = A.n_ops;
    const u32 R = (u32)A.ring_bytes;

    for (int i = threadIdx.x; i < kChainMaxOps; i += blockDim.x) {
        tab_ready[i] = 0;
        tab_open[i] = 0;
        piece_next[i] = 0;
        piece_done[i] = 0;
    }
    if (threadIdx.x < W) prog[threadIdx.x] = 0;
    for (int i = threadIdx.x; i < kRecDepth * 2 * W; i += blockDim.x) (&tick[0][0])[i] = 0;
    if (threadIdx.x < 2) zero_block[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x < kQueue) fq[threadIdx.x].ready = 0u;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        fq_hurry = 0;
        fq_tail = 0u;
        fq_head = 0u;
    }

    // share_lo[o][w]: first K-step of op o that belongs to compute warp w of this block ([o][W]: end of the
    // block's share), share_tile: the tile it lies in.  32-bit: the host side keeps nsteps * (grid + 1) below 2^32.
    __shared__ unsigned share_lo[kChainMaxOps][W + 1], share_tile[kChainMaxOps][W + 1];
    for (int i = threadIdx.x; i < n_ops * (W + 1); i += blockDim.x) {
        const int o = i / (W + 1), w = i - o * (W + 1);
        const u32 N = (u32)A.op[o].nsteps;
        const u32 cs = lev_split_lo<u32>(N, (u32)cta, (u32)G), ce = lev_split_lo<u32>(N, (u32)cta + 1u, (u32)G);
        const u32 lo = cs + lev_split_lo<u32>(ce - cs, (u32)w, (u32)W);
        share_lo[o][w] = lo;
        share_tile[o][w] = lo / (u32)A.op[o].spt;
    }
    __syncthreads();
    auto warp_range = [&](int o, int w, u32& s, u32& e) {
        s = share_lo[o][w];
        e = share_lo[o][w + 1];
    };
    auto timed_out = [&](long long& t0, unsigned i) -> bool {
        if ((i & 255u) != 0) return false;
        if (abort_flag) return true;
        const long long now = clock64();
        if (t0 == 0) t0 = now;
        else if (now - t0 > kWaitCycles) {
            abort_flag = 1;
            atomicOr(A.status, LEV_DEV_TIMEOUT);
            return true;
        }
        return false;
    };
    // one warp claims and builds pieces of op o's tables until none is left
    auto build_some = [&](int o) {
        const ChainOp& P = A.op[o];
        const int pieces = (P.chunks * 4 + 31) >> 5;
        unsigned char* tables = smem + A.tab_off[P.tslot];
        for (;;) {
            int p = 0;
            if (lane == 0) p = atomicAdd(&piece_next[o], 1);
            p = __shfl_sync(0xffffffffu, p, 0);
            if (p >= pieces) break;
            build_piece_any(P, p, lane, tables, norm_inv[P.tslot], A.status);
            __threadfence_block();
            __syncwarp();
            if (lane == 0 && atomicAdd(&piece_done[o], 1) == pieces - 1) {
                __threadfence_block();
                tab_ready[o] = 1;
            }
        }
    };

    // ring of a compute warp: bulk copies (one or two K-steps) packed back to back in R bytes; a copy that
    // does not fit before the end of the ring starts at 0 and the bytes skipped count as its own.  Lane 0
    // keeps the fetch side (it runs ahead across op boundaries), all lanes the compute side.
    unsigned char* ring = smem + (size_t)(warp < W ? warp : 0) * A.ring_stride;
    const unsigned ring_s = smem_u32(ring), bar_s = smem_u32(&bars[warp < W ? warp : 0][0]);
    int c_op = 0, f_op = -1;
    u32 c_k = 0, c_e = 0, c_seq = 0, c_pos = 0;
    const unsigned char* f_src = nullptr;
    u32 f_left = 0, f_bytes = 0, f_grp = 1, f_pos = 0, f_seq = 0, in_use = 0;
    auto fetch_next_op = [&]() {
        while (f_left == 0 && ++f_op < n_ops) {
            u32 s, e;
            warp_range(f_op, warp, s, e);
            const ChainOp& P = A.op[f_op];
            f_bytes = (u32)step_bytes(P.type);
            f_grp = copy_steps(P.type);
            f_src = P.wp + (int64_t)s * f_bytes;
            f_left = e - s;
        }
    };
    auto try_issue = [&]() {
        while (f_left != 0 && f_seq - c_seq < (u32)kRingBars) {
            const u32 nk = f_left < f_grp ? f_left : f_grp, bytes = nk * f_bytes;
            u32 p = f_pos, skip = 0;
            if (p + bytes > R) {
                skip = R - p;
                p = 0;
            }
            if (in_use + skip + bytes > R) break;
            bulk_load(ring_s + p, f_src, bytes, bar_s + 8 * (f_seq & (kRingBars - 1)));
            in_use += skip + bytes;
            f_pos = p + bytes;
            f_seq++;
            f_src += bytes;
            f_left -= nk;
            if (f_left == 0) fetch_next_op();
        }
    };
    if (warp < W) {
        warp_range(0, warp, c_k, c_e);
        while (c_k >= c_e && ++c_op < n_ops) warp_range(c_op, warp, c_k, c_e);
        if (lane == 0) {
            for (int d = 0; d < kRingBars; d++) mbar_init(bar_s + 8 * d, 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            fetch_next_op();
            try_issue();
        }
    }
    pdl_launch_dependents();
    pdl_wait();  // weights are immutable and already on their way; everything else belongs to earlier launches
    __syncthreads();

    // A tile shared by several blocks is finished by the last block that shares it: the others leave their
    // sums of the 16 rows as (value, flag) pairs, one 8-byte store each, and it adds them in block order to
    // its own and writes y.  No fence is involved (a GPU-scope fence stalls the weight stream of the whole
    // SM): a pair is complete when its flag reads 1, and the reader puts the flag back to 0 for the next launch.
    // Run by one whole warp; lanes < 16 hold this block's sum of row `lane` in `acc`.
    auto finish_shared_tile = [&](int o, u32 tile, float acc) -> bool {
        const ChainOp& P = A.op[o];
        const u32 N = (u32)P.nsteps, spt = (u32)P.spt, ta = tile * spt, tb = ta + spt;
        const u32 c0 = lev_split_owner<u32>(N, ta, (u32)G), c1 = lev_split_owner<u32>(N, tb - 1u, (u32)G);
        float tot = 0.f;
        bool ok = true;
        for (u32 cc = c0; cc < c1 && ok; cc++) {
            // with fewer K-steps than blocks some blocks have no share
            if (N < (u32)G && lev_split_lo<u32>(N, cc, (u32)G) == lev_split_lo<u32>(N, cc + 1u, (u32)G)) continue;
            uint2* gp = A.gpart + ((size_t)(o * G + cc) * 2 + (cc == c0 ? 1 : 0)) * 16;
            uint2 v = make_uint2(0u, 1u);
            long long t0 = 0;
            for (unsigned i = 1;; i++) {
                if (lane < 16) v = __ldcv(gp + lane);
                if (__all_sync(0xffffffffu, v.y == 1u)) break;
                if (timed_out(t0, i)) {
                    ok = false;
                    break;
                }
                __nanosleep(40);
            }
            if (lane < 16) {
                __stcg(gp + lane, make_uint2(0u, 0u));
                tot += __uint_as_float(v.x);
            }
        }
        if (ok && lane < 16) {
            tot += acc;
            const int64_t row = (int64_t)tile * 16 + lane;
            if (row < P.rows) P.y[row] = P.residual ? fmaf(P.alpha, tot, P.residual[row]) : tot;
        }
        return ok;
    };

    if (warp < W) {
        // ===================== compute warps =====================
        bool dead = false;
        LaneConst L;
        L.q_off = 16u * lane;
        L.hdr_off = 16u * g;
        L.x_off = (unsigned)(((g & 1) * 4 + t) * 32);
        L.grp = (unsigned)(g >> 1);
        L.t = (unsigned)t;
        L.g = (unsigned)g;
        L.sh16 = 16u * (t & 1);
        L.zero_s = smem_u32(zero_block);
        const unsigned smem_s = smem_u32(smem);
        while (c_op < n_ops && !dead) {
            // ---------- enter op ----------
            const int o = c_op;
            const ChainOp& P = A.op[o];
            if (lane == 0) prog[warp] = o;
            long long t0 = 0;
            if (o >= kRecDepth) {
                // records and tickets of op o - kRecDepth are reused: every warp must have left it
                for (unsigned i = 1;; i++) {
                    int v = lane < W ? prog[lane] : 0x7fffffff;
#pragma unroll
                    for (int d = 16; d > 0; d >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, d));
                    if (v > o - kRecDepth) break;
                    if (timed_out(t0, i)) {
                        dead = true;
                        break;
                    }
                    __nanosleep(100);
                }
            }
            t0 = 0;
            for (unsigned i = 1; !dead && !tab_ready[P.tab]; i++) {
                if (tab_open[P.tab]) build_some(P.tab);
                else __nanosleep(50);
                if (timed_out(t0, i)) dead = true;
            }
            if (dead) break;
            __threadfence_block();
            const u32 spt = (u32)P.spt;
            const u32 cs = share_lo[o][0], ce = share_lo[o][W];
            const u32 n = ce - cs, s = c_k, e = c_e;
            // lane l: first K-step (block-relative) and first tile of warp l's share; lane W: the end
            const u32 wlo = lane <= W ? share_lo[o][lane] - cs : 0xffffffffu;
            const u32 wtile = lane <= W ? share_tile[o][lane] : 0u;
            const u32 first_tile = share_tile[o][warp];
            const int type = P.type;
            const int64_t rows = P.rows;
            float* const yp = P.y;
            const float* const resid = P.residual;
            const float alpha = P.alpha;
            float* rec = reinterpret_cast<float*>(smem + A.rec_off) + (size_t)(o & (kRecDepth - 1)) * W * 32;
            int* const ticks = &tick[o & (kRecDepth - 1)][0];
            // tables of the op: fragments, then sums
            unsigned xs_s = smem_s + (unsigned)A.tab_off[A.op[P.tab].tslot];
            order_after(xs_s);
            const unsigned sa_s = xs_s + (unsigned)P.chunks * 256u;

            // the warp's share [s, e) of the op, in the arithmetic of one block format
            auto run = [&](auto tag) {
                constexpr int TYPE = decltype(tag)::value;
                constexpr u32 bytes = (u32)step_bytes(TYPE), grp = copy_steps(TYPE);
                constexpr u32 aux_bytes = TYPE == LEV_GGML_Q4_K ? 32u : (TYPE == LEV_GGML_Q6_K ? 128u : 64u);
                u32 tile = first_tile;
                u32 k = s - tile * spt, seg_k0 = k;
                unsigned xk = xs_s + k * 1024u, ak = sa_s + k * aux_bytes;
                float ya = 0.f, yb = 0.f;
                u32 left = e - s;  // K-steps of the share not yet done
                while (left != 0) {
                    // ---------- one bulk copy: one or two K-steps ----------
                    if (!mbar_wait(bar_s + 8 * (c_seq & (kRingBars - 1)), (c_seq >> 3) & 1u)) {
                        if (lane == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
                        abort_flag = 1;
                        dead = true;
                        return;
                    }
                    const u32 grp_n = left < grp ? left : grp;
                    u32 grp_skip = 0;
                    if (c_pos + grp_n * bytes > R) {
                        grp_skip = R - c_pos;
                        c_pos = 0;
                    }
                    unsigned st = ring_s + c_pos;
                    order_after(st);
#pragma unroll 1
                    for (u32 j = 0; j < grp_n; j++) {
                        {
                            chain_step<TYPE>(st, xk, ak, L, ya, yb);
                            if (j + 1 == grp_n) {
                                // every lane has read the copy's bytes: hand them back to the fetch side
                                __syncwarp();
                                c_seq++;
                                c_pos += grp_n * bytes;
                                if (lane == 0) {
                                    in_use -= grp_skip + grp_n * bytes;
                                    try_issue();
                                }
                            }
                            st += bytes;
                            xk += 1024u;
                            ak += aux_bytes;
                            k++;
                            if (k == spt || (j + 1 == grp_n && left == grp_n)) {
                                // ---------- this warp's segment of the tile ends ----------
                                float va = ya, vb = yb;
                                va += __shfl_xor_sync(0xffffffffu, va, 1);
                                vb += __shfl_xor_sync(0xffffffffu, vb, 1);
                                va += __shfl_xor_sync(0xffffffffu, va, 2);
                                vb += __shfl_xor_sync(0xffffffffu, vb, 2);
                                const bool whole = seg_k0 == 0 && k == spt;
                                if (whole) {
                                    if (t == 0) {
                                        const int64_t row = (int64_t)tile * 16 + g;
                                        if (resid) {
                                            if (row < rows) va = fmaf(alpha, va, resid[row]);
                                            if (row + 8 < rows) vb = fmaf(alpha, vb, resid[row + 8]);
                                        }
                                        if (row < rows) yp[row] = va;
                                        if (row + 8 < rows) yp[row + 8] = vb;
                                    }
                                } else {
                                    const int r = tile == first_tile ? 0 : 1;
                                    float* mine_rec = rec + (warp * 2 + r) * 16;
                                    if (t == 0) {
                                        mine_rec[g] = va;
                                        mine_rec[g + 8] = vb;
                                    }
                                    // the tile's K-steps inside this block and the warps that share them: warp l owns
                                    // block-relative K-step j when wlo(l) <= j < wlo(l + 1)
                                    const u32 ta = tile * spt, tb = ta + spt;
                                    const u32 a = (ta > cs ? ta : cs) - cs, b = (tb < ce ? tb : ce) - cs;
                                    const int l_first = __popc(__ballot_sync(0xffffffffu, lane < W && wlo <= a)) - 1;
                                    const int l_last = __popc(__ballot_sync(0xffffffffu, lane < W && wlo <= b - 1u)) - 1;
                                    const int expected = n >= (u32)W ? l_last - l_first + 1 : (int)(b - a);
                                    int* tk = ticks + 2 * l_first + (ta >= cs ? 1 : 0);
                                    __threadfence_block();
                                    __syncwarp();
                                    int old = 0;
                                    if (lane == 0) old = atomicAdd(tk, 1);
                                    old = __shfl_sync(0xffffffffu, old, 0);
                                    if (old == expected - 1) {
                                        // last to arrive: add the warps' records in warp order
                                        if (lane == 0) *tk = 0;
                                        __threadfence_block();
                                        float acc = 0.f;
                                        for (int l = l_first; l <= l_last; l++) {
                                            const u32 lo_l = __shfl_sync(0xffffffffu, wlo, l), hi_l = __shfl_sync(0xffffffffu, wlo, l + 1);
                                            const u32 tile_l = __shfl_sync(0xffffffffu, wtile, l);
                                            if (lo_l == hi_l) continue;  // a warp without a share
                                            if (lane < 16) acc += rec[(l * 2 + (tile == tile_l ? 0 : 1)) * 16 + lane];
                                        }
                                        if (ta >= cs && tb <= ce) {
                                            const int64_t row = (int64_t)tile * 16 + lane;
                                            if (lane < 16 && row < rows) yp[row] = resid ? fmaf(alpha, acc, resid[row]) : acc;
                                        } else {
                                            // shared with other blocks: every sharer but the last leaves its sums as
                                            // (value, flag) pairs; the last one queues its own for the finishing warp,
                                            // which waits for the others' pairs and writes y
                                            const u32 N = (u32)P.nsteps;
                                            const u32 c0 = lev_split_owner<u32>(N, ta, (u32)G), c1 = lev_split_owner<u32>(N, tb - 1u, (u32)G);
                                            if ((u32)cta != c1) {
                                                uint2* gp = A.gpart + ((size_t)(o * G + cta) * 2 + ((u32)cta == c0 ? 1 : 0)) * 16;
                                                if (lane < 16) __stcg(gp + lane, make_uint2(__float_as_uint(acc), 1u));
                                            } else {
                                                u32 at = 0;
                                                if (lane == 0) at = atomicAdd(&fq_tail, 1u);
                                                at = __shfl_sync(0xffffffffu, at, 0);
                                                long long tq = 0;
                                                for (unsigned i = 1; at - fq_head >= (u32)kQueue; i++)
                                                    if (timed_out(tq, i)) {
                                                        dead = true;
                                                        break;
                                                    }
                                                if (!dead) {
                                                    TileEntry& E = fq[at & (kQueue - 1)];
                                                    if (lane < 16) E.v[lane] = acc;
                                                    if (lane == 16) E.op = o;
                                                    if (lane == 17) E.tile = tile;
                                                    __threadfence_block();
                                                    __syncwarp();
                                                    if (lane == 0) E.ready = at + 1u;
                                                }
                                            }
                                        }
                                    }
                                }
                                ya = yb = 0.f;
                                tile++;
                                k = 0;
                                seg_k0 = 0;
                                xk = xs_s;
                                ak = sa_s;
                            }
                        }
                    }
                    left -= grp_n;
                    if (dead) return;
                }
            };
            if (type == LEV_GGML_Q4_K) run(std::integral_constant<int, LEV_GGML_Q4_K>{});
            else if (type == LEV_GGML_Q6_K) run(std::integral_constant<int, LEV_GGML_Q6_K>{});
            else run(std::integral_constant<int, LEV_GGML_Q4_0>{});
            if (dead) break;
            // results of this op are ordered before the warp reports it done (needed where a later op of the
            // launch waits for them; the builder thread that arrives at the grid counter fences at GPU scope)
            if (P.fence) __threadfence_block();
            __syncwarp();
            // next op with a share for this warp
            c_k = c_e;
            while (c_k >= c_e && ++c_op < n_ops) warp_range(c_op, warp, c_k, c_e);
        }
        if (lane == 0 && !dead) prog[warp] = n_ops;
        // copies still in flight (only after a wait ran out): let them land before the block goes
        if (lane == 0)
            for (; dead && c_seq != f_seq; c_seq++) mbar_wait(bar_s + 8 * (c_seq & (kRingBars - 1)), (c_seq >> 3) & 1u);
    } else if (warp == W + kHelperWarps - 1) {
        // ===================== finishing warp: tiles shared with other blocks =====================
        long long t0 = 0;
        for (unsigned i = 1;; i++) {
            const u32 h = fq_head;
            TileEntry& E = fq[h & (kQueue - 1)];
            if (E.ready == h + 1u) {
                __threadfence_block();
                const float acc = lane < 16 ? E.v[lane] : 0.f;
                const int o = E.op;
                const u32 tile = E.tile;
                __syncwarp();
                if (!finish_shared_tile(o, tile, acc)) break;
                __threadfence_block();  // y is written before the queue reads as drained
                __syncwarp();
                if (lane == 0) fq_head = h + 1u;
                t0 = 0;
                i = 0;
                continue;
            }
            // done when every compute warp has finished and the queue is empty
            int v = lane < W ? prog[lane] : 0x7fffffff;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, d));
            if (v >= n_ops && fq_head == *(volatile unsigned*)&fq_tail) break;
            if (timed_out(t0, i)) break;
            // a poll costs issue slots of the compute warps: poll rarely until they are done or an op that waits is near
            __nanosleep(v >= n_ops || fq_hurry ? 20 : 200);
        }
    } else {
        // ===================== table builders =====================
        const int hw = warp - W, htid = threadIdx.x - W * 32;
        auto helpers_sync = [&]() { asm volatile("bar.sync 1, %0;\n" ::"n"(kBuilderWarps * 32) : "memory"); };
        auto wait_prog = [&](int target) -> bool {  // thread 0 of the builders: every compute warp is at op >= target
            long long t0 = 0;
            for (unsigned i = 1;; i++) {
                int v = 0x7fffffff;
                for (int w = 0; w < W; w++) v = min(v, prog[w]);
                if (v >= target) return true;
                if (timed_out(t0, i)) return false;
                __nanosleep(200);
            }
        };
        for (int o = 0; o < n_ops; o++) {
            const ChainOp& P = A.op[o];
            if (P.tab != o) continue;
            if (htid == 0) {
                bool ok = true;
                if (P.free_after >= 0) ok = wait_prog(P.free_after + 1);
                if (ok && P.wait) {
                    // every block has finished (and fenced) all earlier ops before any block reads their results:
                    // this block's compute warps have left them and its queue of shared tiles is empty
                    fq_hurry = 1;
                    ok = wait_prog(o);
                    long long t0 = 0;
                    for (unsigned i = 1; ok && fq_head != *(volatile unsigned*)&fq_tail; i++)
                        if (timed_out(t0, i)) ok = false;
                    fq_hurry = 0;
                    if (ok) {
                        __threadfence();
                        unsigned* arrive = A.sync + 2 * o;
                        atomicAdd(arrive, 1u);
                        t0 = 0;
                        for (unsigned i = 1; ld_acquire(arrive) < (unsigned)G; i++) {
                            if (timed_out(t0, i)) {
                                ok = false;
                                break;
                            }
                        }
                        if (ok && atomicAdd(arrive + 1, 1u) == (unsigned)G - 1) {
                            // last to leave: nobody polls any more
                            arrive[0] = 0u;
                            arrive[1] = 0u;
                        }
                        __threadfence();
                    }
                }
            }
            helpers_sync();
            if (abort_flag) break;
            if (P.norm_on) {
                // inverse RMS of the column: thread-strided partials, warp tree, warps in order
                float ss = 0.f;
                for (int i = htid * 4; i < P.cols; i += kBuilderWarps * 128) {
                    const float4 v = *reinterpret_cast<const float4*>(P.x + i);
                    ss = fmaf(v.x, v.x, ss);
                    ss = fmaf(v.y, v.y, ss);
                    ss = fmaf(v.z, v.z, ss);
                    ss = fmaf(v.w, v.w, ss);
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
                if (lane == 0) hpart[hw] = ss;
                helpers_sync();
                if (htid == 0) {
                    float tot = 0.f;
                    for (int w2 = 0; w2 < kBuilderWarps; w2++) tot += hpart[w2];
                    norm_inv[P.tslot] = 1.0f / sqrtf(tot / (float)P.cols + P.norm_eps);
                }
            } else if (htid == 0) {
                norm_inv[P.tslot] = 1.0f;
            }
            __threadfence_block();
            helpers_sync();
            if (htid == 0) tab_open[o] = 1;
            build_some(o);
            // wait for pieces claimed by compute warps too
            {
                long long t0 = 0;
                for (unsigned i = 1; !tab_ready[o]; i++) {
                    if (timed_out(t0, i)) break;
                    __nanosleep(100);
                }
            }
            if (abort_flag) break;
        }
    }
}

struct ChainPlan {
    int warps, ring_bytes, ring_stride;
    int tab_off[2], rec_off;
    size_t smem;
};

}  // namespace

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

static bool chain_item_ok(const lev_chain_item& it) {
    const lev_weights* w = it.w;
    if (!w || !w->packed || it.row0 % 16 != 0 || ((uintptr_t)it.x & 15) != 0) return false;
    const int64_t chunks = lev_stream_chunks(w), spt = chunks / 4, tiles = (it.rows + 15) / 16;
    if (spt < 1 || spt > 4096 || tiles * spt > (int64_t)lev_split_max_items(160)) return false;
    if (it.fusion && it.fusion->norm_w && ((uintptr_t)it.fusion->norm_w & 15) != 0) return false;
    return true;
}

// Lays the launch out: which op builds tables and in which buffer, ring depth, shared memory.
static bool chain_plan(lev_ctx* ctx, int n_ops, const lev_chain_item* items, ChainArgs* A, ChainPlan* P) {
    if (n_ops < 1 || n_ops > kChainMaxOps) return false;
    size_t tab_bytes[2] = {0, 0};
    int last_builder = -1, last_reader[2] = {-1, -1}, slot_owner[2] = {-1, -1};
    int max_step = 0;  // bytes of the largest bulk copy
    for (int o = 0; o < n_ops; o++) {
        const lev_chain_item& it = items[o];
        if (!chain_item_ok(it)) return false;
        const lev_weights* w = it.w;
        ChainOp& op = A->op[o];
        memset(&op, 0, sizeof op);
        const int64_t chunks = lev_stream_chunks(w), spt = chunks / 4, tiles = (it.rows + 15) / 16;
        const size_t step = step_bytes(w->type);
        op.wp = w->packed + (size_t)(it.row0 / 16) * spt * step;
        op.x = it.x;
        op.y = it.y;
        op.rows = it.rows;
        op.type = w->type;
        op.spt = (int)spt;
        op.nsteps = (int)(tiles * spt);
        op.cols = (int)w->cols;
        op.chunks = (int)chunks;
        op.wait = it.wait;
        op.alpha = 1.0f;
        if (it.fusion) {
            op.norm_on = it.fusion->norm_on;
            op.norm_w = it.fusion->norm_w;
            op.norm_eps = it.fusion->eps;
            op.gelu_inter = it.fusion->gelu_up ? (int)w->cols : 0;
            op.residual = it.fusion->residual;
            op.alpha = it.fusion->alpha;
        }
        if ((int)(step * copy_steps(w->type)) > max_step) max_step = (int)(step * copy_steps(w->type));
        // same activations through the same prologue into the same fragment order: share the tables
        bool same = false;
        if (last_builder >= 0 && !it.wait) {
            const ChainOp& b = A->op[last_builder];
            same = b.x == op.x && b.cols == op.cols && b.norm_on == op.norm_on && b.norm_w == op.norm_w &&
                   b.norm_eps == op.norm_eps && b.gelu_inter == op.gelu_inter && b.type == op.type;
        }
        if (same) {
            op.tab = last_builder;
            op.tslot = A->op[last_builder].tslot;
            op.free_after = -1;
            last_reader[op.tslot] = o;
        } else {
            const int slot = last_builder < 0 ? 0 : 1 - A->op[last_builder].tslot;
            op.tab = o;
            op.tslot = slot;
            op.free_after = slot_owner[slot] >= 0 ? last_reader[slot] : -1;
            slot_owner[slot] = o;
            last_reader[slot] = o;
            last_builder = o;
            const size_t tb = (lev_stream_table_bytes(w, 1, 2, 1, nullptr) + 255) & ~(size_t)255;
            if (tb > tab_bytes[slot]) tab_bytes[slot] = tb;
        }
    }
    A->n_ops = n_ops;
    for (int o = n_ops - 1, later_wait = 0; o >= 0; o--) {
        A->op[o].fence = later_wait;
        later_wait |= A->op[o].wait;
    }
    const size_t cap = ctx->prop.sharedMemPerBlockOptin;
    const size_t fixed_static = 8 * 1024;  // static shared memory of the kernel, rounded up
    // compute warps: with the four helper warps a multiple of four, so that the register file splits evenly
    int warps = ctx->chain_warps == 12 ? 12 : 16;
    for (;; warps = 12) {
        const size_t rec = (size_t)kRecDepth * warps * 32 * sizeof(float);
        const size_t fixed = fixed_static + tab_bytes[0] + tab_bytes[1] + rec;
        size_t ring = fixed < cap ? ((cap - fixed) / warps) & ~(size_t)127 : 0;
        // every warp needs room for at least two of the largest K-steps
        if (ring < (size_t)2 * max_step) {
            if (warps == 12) return false;
            continue;
        }
        if (ring > (size_t)kRingBars * max_step) ring = ((size_t)kRingBars * max_step + 127) & ~(size_t)127;
        if (ctx->chain_depth >= 2 && (size_t)ctx->chain_depth * max_step < ring) ring = ((size_t)ctx->chain_depth * max_step + 127) & ~(size_t)127;
        const size_t stride = ring;
        P->warps = warps;
        P->ring_bytes = (int)ring;
        P->ring_stride = (int)stride;
        const size_t rings = (size_t)warps * stride;
        P->tab_off[0] = (int)rings;
        P->tab_off[1] = (int)(rings + tab_bytes[0]);
        P->rec_off = (int)(rings + tab_bytes[0] + tab_bytes[1]);
        P->smem = rings + tab_bytes[0] + tab_bytes[1] + rec;
        break;
    }
    A->ring_bytes = P->ring_bytes;
    A->ring_stride = P->ring_stride;
    A->tab_off[0] = P->tab_off[0];
    A->tab_off[1] = P->tab_off[1];
    A->rec_off = P->rec_off;
    return true;
}

bool lev_chain_supported(lev_ctx* ctx, int n_ops, const lev_chain_item* items) {
    ChainArgs A;
    ChainPlan P;
    return ctx->chain_off == 0 && chain_plan(ctx, n_ops, items, &A, &P);
}

// Whether a call that did not ask for a list should take the persistent kernel.  A launch of it fills every SM
// and cannot overlap its neighbours in the stream, which costs about 5 us; it pays from roughly 40 MB of weight
// bytes per launch on (the FFN's gate + up pair, its Q6_K down tensor, the vocabulary head).  Below that the half-SM
// one-launch kernel, whose blocks become resident beside the previous kernel's, is the faster one (a 28 MB tensor:
// 9.9 against 12.9 us; the q / k / v and output projections of a decode layer: 9 us per layer less).  The line is
// drawn so that the FFN's two fused launches land on the same side: a persistent launch followed by a half-SM one
// overlaps with nothing and cost 59 us for the pair where two persistent launches cost 44 (a 41 MB Q6_K tensor alone:
// 18.2 against 17.6 us).
static const size_t kChainPreferredBytes = 40000000;
bool lev_chain_preferred(lev_ctx* ctx, int n_ops, const lev_chain_item* items) {
    size_t bytes = 0;
    for (int i = 0; i < n_ops; i++)
        bytes += (size_t)items[i].rows * (size_t)items[i].w->blocks_per_row * (size_t)lev_block_bytes(items[i].w->type);
    return bytes >= kChainPreferredBytes && lev_chain_supported(ctx, n_ops, items);
}

template <int W>
static int chain_launch(lev_ctx* ctx, int grid, size_t smem, const ChainArgs& A) {
    static size_t configured[16] = {};
    if (configured[ctx->device & 15] < smem) {
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_chain<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[ctx->device & 15] = smem;
    }
    LEV_CUDA(ctx, launch_pdl(k_chain<W>, dim3(grid), dim3((W + kHelperWarps) * 32), smem, ctx->stream, A));
    return LEV_OK;
}

int lev_chain_run(lev_ctx* ctx, int n_ops, const lev_chain_item* items) {
    ChainArgs A;
    ChainPlan P;
    if (ctx->chain_off || !chain_plan(ctx, n_ops, items, &A, &P))
        return lev_fail(ctx, LEV_UNSUPPORTED, "persistent matvec kernel: list not served");
    const int grid = ctx->prop.multiProcessorCount;
    if (!ctx->chain_sync) return lev_fail(ctx, LEV_UNSUPPORTED, "persistent matvec kernel: no buffers");
    A.status = ctx->d_status;
    A.sync = (unsigned*)ctx->chain_sync;
    A.gpart = (uint2*)ctx->chain_part;
    int st = P.warps == 16 ? chain_launch<16>(ctx, grid, P.smem, A) : chain_launch<12>(ctx, grid, P.smem, A);
    if (st) return st;
    ctx->launches++;
    ctx->ev.grid = grid;
    ctx->ev.block = (P.warps + kHelperWarps) * 32;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_chain");
}

// counters and flags (left at zero by every launch) and the partial sums of tiles shared by blocks
static size_t chain_buffer_bytes(lev_ctx* ctx, size_t* sync_bytes) {
    const int grid = ctx->prop.multiProcessorCount;
    *sync_bytes = (size_t)(2 * kChainMaxOps) * sizeof(unsigned);
    return *sync_bytes + (size_t)kChainMaxOps * grid * 2 * 16 * sizeof(uint2);
}

int lev_chain_init(lev_ctx* ctx) {
    size_t sync_bytes;
    const size_t total = chain_buffer_bytes(ctx, &sync_bytes);
    LEV_CUDA(ctx, cudaMalloc(&ctx->chain_sync, total));
    LEV_CUDA(ctx, cudaMemsetAsync(ctx->chain_sync, 0, total, ctx->stream));
    ctx->chain_part = (char*)ctx->chain_sync + sync_bytes;
    return LEV_OK;
}

int lev_chain_reset(lev_ctx* ctx) {
    if (!ctx->chain_sync) return LEV_OK;
    size_t sync_bytes;
    const size_t total = chain_buffer_bytes(ctx, &sync_bytes);
    LEV_CUDA(ctx, cudaMemsetAsync(ctx->chain_sync, 0, total, ctx->stream));
    return lev_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "reset of the persistent kernel's counters");
}
