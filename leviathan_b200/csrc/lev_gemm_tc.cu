// Prefill dequant-GEMM on the fifth-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   Y[t][r] = sum_k bf16(W[r][k]) * X[t][k],  f32 accumulate in tensor memory
//
// Same operand rounding as the mma.sync form in lev_gemm.cu (weights decoded bit-exactly
// as the block decoders form them, then one rounding to bf16; activations are bf16 already;
// rust/crates/lev-forge/src/coopmat.rs:236-425, oracle rust/crates/lev-cli/src/main.rs:1201-1217).
//
// One CTA computes a tile of 256 tokens x 176 weight rows over the whole K:
//   * warp 0 (one thread): TMA loads of the activation tile, two boxes of 128 tokens x 64 k
//     (128-byte rows, hardware 128B swizzle) per K-step into a 3-stage ring;
//   * warps 2..12 (352 threads): decode the K-step's 176 x 64 weights from the GGUF blocks in
//     global memory and store them as bf16 into the same K-major 128B-swizzled layout, then
//     publish them to the async proxy (fence.proxy.async) and arrive on the stage's barrier;
//   * warp 1 (one thread): for each K-step 4 x 2 tcgen05.mma (M = 128 tokens, N = 176 rows,
//     K = 16) from shared-memory descriptors into two TMEM accumulators (352 of 512 columns),
//     tcgen05.commit hands the stage back to the producers;
//   * epilogue: warps 2..9 read the accumulators with tcgen05.ld (warp w owns TMEM lanes
//     32*(w%4)...) and store Y rows with 16-byte stores.
// Decode batches (up to 128 tokens) of the 4-bit formats take the STAGED form of the same kernel: the raw
// bytes reach shared memory by cp.async one 256-column group ahead and two threads share a weight row; the
// launch then also splits K over gridDim.z, partial products summed in split order by k_gemm_split_sum.
// The grouped forms further down serve the routed MoE (weights as the MMA's M operand).
// Every wait is bounded by about a second of SM clocks; on a timeout the CTA sets
// LEV_DEV_TIMEOUT, skips the remaining work, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "lev_internal.h"

namespace {

constexpr int TM = 256;      // tokens per CTA tile (two MMA tiles of 128)
constexpr int RN = 176;      // weight rows per CTA tile (MMA N): 12288 rows x 512 tokens -> 140 CTAs on 148 SMs
constexpr int KS = 64;       // k per pipeline stage (one 128-byte swizzle row of bf16)
constexpr int STAGES = 3;
constexpr int kDequantWarps = 11;
constexpr int kThreads = (2 + kDequantWarps) * 32;
constexpr int kXHalfBytes = 128 * KS * 2;             // 16384: one TMA box
constexpr int kXStageBytes = 2 * kXHalfBytes;         // 32768
constexpr int kWStageBytes = RN * KS * 2;             // 24576
constexpr int kStageBytes = kXStageBytes + kWStageBytes;
constexpr int kTmemCols = 512;
constexpr long long kWaitCycles = 2000000000LL;
constexpr int kAhead = 3;  // K-steps of raw weight bytes a decode thread has requested ahead of the one it decodes

struct GemmTcArgs {
    const uint8_t* raw;   // GGUF blocks, row-major
    int type;
    int64_t row_bytes;
    int64_t rows, cols;
    int tokens;
    float* y;             // [tokens][rows]; with a K split: [gridDim.z][tokens][rows] partial products
    int y_vec;            // rows of y start on 16-byte boundaries
    int* status;
    int ksteps_per_split; // K-steps a CTA takes (blockIdx.z picks the range); the whole K without a split
};

__device__ __forceinline__ unsigned s32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait; false on timeout or when another thread of the CTA has already given up.  The polls are spaced by
// the loop's own bookkeeping on purpose: a tight three-instruction poll loop measured 15 % slower on the whole
// kernel (the waiting warps take issue slots from the decode warps of their scheduler).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
    long long t_start = 0;
    for (unsigned i = 1;; i++) {
        unsigned ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 63u) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t_start == 0) t_start = now;
            else if (now - t_start > kWaitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor: D f32, A and B bf16, both K-major, M = 128, N = RN
constexpr unsigned kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(RN >> 3) << 17) | ((unsigned)(128 >> 4) << 24);

__device__ __forceinline__ void umma_bf16(unsigned d_tmem, uint64_t adesc, uint64_t bdesc, unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint4 pack8(const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    return make_uint4(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b), *reinterpret_cast<unsigned*>(&c),
                      *reinterpret_cast<unsigned*>(&d));
}
// byte offset of 16-byte chunk ch (0..7) of row r inside a K-major 128B-swizzled tile
__device__ __forceinline__ unsigned swz(int r, int ch) { return (unsigned)((r >> 3) * 1024 + (r & 7) * 128 + ((ch ^ (r & 7)) << 4)); }

// Loads of weight bytes as volatile asm: they are issued where they are written (one K-step ahead
// of their use) instead of being sunk to the first use.
__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned ldg2(const void* p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];\n" : "=h"(v) : "l"(p));
    return v;
}
// 8 bytes from a 2-byte aligned address
__device__ __forceinline__ uint2 load8_u16(const uint8_t* p) {
    const unsigned a = ldg2(p), b = ldg2(p + 2), c = ldg2(p + 4), d = ldg2(p + 6);
    return make_uint2(a | (b << 16), c | (d << 16));
}
// Eight bytes from a 2-byte aligned address inside a Q6_K block, as the aligned words that cover them: the words
// may reach two bytes before p and two bytes past p + 8, which the callers keep inside the tensor (a block's
// quant bytes end 16 bytes before the block does, and a tensor's first block is 4-byte aligned).
__device__ __forceinline__ uint2 load8_words(const uint8_t* p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const unsigned* w = reinterpret_cast<const unsigned*>(a & ~(uintptr_t)3);
    const unsigned sh = (unsigned)(a & 2u) * 8u;
    const unsigned x0 = __ldg(w), x1 = __ldg(w + 1), x2 = sh ? __ldg(w + 2) : 0u;
    return make_uint2(__funnelshift_r(x0, x1, sh), __funnelshift_r(x1, x2, sh));
}
// float(byte k of w) without the conversion unit: the byte lands in the mantissa of 2^23
__device__ __forceinline__ float byte_f(unsigned w, unsigned k) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u + k)) - 8388608.0f;
}

// asynchronous copies into shared memory (raw weight bytes staged ahead of their decode)
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(unsigned dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_but() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void decode_barrier() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

// What one decode thread needs of one row for one K-step (64 columns): it is thread j = 0..3 of
// the four that share the row and produces two 16-byte chunks (8 bf16 each) of the tile row.
//   Q4_K: K-step = chunk c of block b; bytes qs[32c + 8j ..+8): low nibbles -> chunk j (sub-block
//         2c), high nibbles -> chunk j+4 (sub-block 2c+1); the block header every fourth step.
//   Q4_0: K-step = two blocks; j>>1 picks the block, j&1 the byte half; low nibbles are values
//         0..15, high nibbles 16..31 of the block -> chunks 4*(j>>1) + (j&1) and + 2.
//   Q6_K: K-step = two 32-value groups (2*(it&1), +1) of half c = (it&3)>>1 of block b; thread j
//         takes values 8j..8j+7 of both groups -> chunks j and j+4.
template <int TYPE>
struct RowRaw {
    uint4 hdr;  // Q4_K: d, dmin, 12 scale bytes.  Q4_0: .x = d bits.  Q6_K: .x = d bits, .y = two int8 scales
    uint2 q0;   // nibble bytes (Q6_K: of the first group)
    uint2 q1;   // Q6_K: nibble bytes of the second group
    uint2 qh;   // Q6_K: high-bit bytes
};

template <int TYPE>
__device__ __forceinline__ void load_raw(const uint8_t* row, int it, int j, bool valid, RowRaw<TYPE>& R) {
    if (!valid) return;
    if (TYPE == LEV_GGML_Q4_K) {
        const uint8_t* blk = row + (int64_t)(it >> 2) * LEV_Q4_K_BYTES;
        R.hdr = ldg16(blk);
        R.q0 = ldg8(blk + 16 + 32 * (it & 3) + 8 * j);
    } else if (TYPE == LEV_GGML_Q4_0) {
        const uint8_t* blk = row + (int64_t)(2 * it + (j >> 1)) * LEV_Q4_0_BYTES;
        R.hdr.x = ldg2(blk);
        R.q0 = load8_u16(blk + 2 + 8 * (j & 1));
    } else {
        const uint8_t* blk = row + (int64_t)(it >> 2) * LEV_Q6_K_BYTES;
        const int c = (it & 3) >> 1, g0 = 2 * (it & 1);
        R.q0 = load8_words(blk + 64 * c + 8 * j);
        R.q1 = load8_words(blk + 64 * c + 32 + 8 * j);
        R.qh = load8_words(blk + 128 + 32 * c + 8 * j);
        R.hdr.x = ldg2(blk + 208);
        // int8 scales of the two groups for values 8j..8j+7: index 8c + 2*grp + (j >> 1)
        const unsigned s0 = blk[192 + 8 * c + 2 * g0 + (j >> 1)], s1 = blk[192 + 8 * c + 2 * (g0 + 1) + (j >> 1)];
        R.hdr.y = s0 | (s1 << 8);
    }
}

template <int TYPE>
__device__ __forceinline__ void decode_store(const RowRaw<TYPE>& R, int it, int j, bool valid, unsigned char* wtile, int r) {
    float lo[8], hi[8];
    int ch_lo = j, ch_hi = j + 4;
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 8; i++) lo[i] = hi[i] = 0.f;
        if (TYPE == LEV_GGML_Q4_0) {
            ch_lo = (j >> 1) * 4 + (j & 1);
            ch_hi = ch_lo + 2;
        }
    } else if (TYPE == LEV_GGML_Q4_K) {
        const int c = it & 3;
        const float d = h2f(R.hdr.x & 0xffffu), dmin = h2f(R.hdr.x >> 16);
        // 6-bit scales / mins of sub-blocks 0..3 and 4..7, one byte each
        // (rust/crates/lev-cpu/src/lib.rs:64-74)
        const unsigned sc_w = c < 2 ? (R.hdr.y & 0x3F3F3F3Fu) : ((R.hdr.w & 0x0F0F0F0Fu) | ((R.hdr.y >> 2) & 0x30303030u));
        const unsigned mn_w = c < 2 ? (R.hdr.z & 0x3F3F3F3Fu) : (((R.hdr.w >> 4) & 0x0F0F0F0Fu) | ((R.hdr.z >> 2) & 0x30303030u));
        const unsigned k0 = 2u * (c & 1);
        const float d0 = __fmul_rn(d, byte_f(sc_w, k0)), m0 = __fmul_rn(dmin, byte_f(mn_w, k0));
        const float d1 = __fmul_rn(d, byte_f(sc_w, k0 + 1)), m1 = __fmul_rn(dmin, byte_f(mn_w, k0 + 1));
        const unsigned w[2] = {R.q0.x, R.q0.y};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const unsigned l4 = w[h] & 0x0F0F0F0Fu, h4 = (w[h] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo[4 * h + i] = __fsub_rn(__fmul_rn(d0, byte_f(l4, i)), m0);
                hi[4 * h + i] = __fsub_rn(__fmul_rn(d1, byte_f(h4, i)), m1);
            }
        }
    } else if (TYPE == LEV_GGML_Q4_0) {
        ch_lo = (j >> 1) * 4 + (j & 1);
        ch_hi = ch_lo + 2;
        const float d = h2f(R.hdr.x);
        const unsigned w[2] = {R.q0.x, R.q0.y};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const unsigned l4 = w[h] & 0x0F0F0F0Fu, h4 = (w[h] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo[4 * h + i] = __fmul_rn(d, __uint_as_float(__byte_perm(l4, 0x4B000000u, 0x7650u + i)) - 8388616.0f);
                hi[4 * h + i] = __fmul_rn(d, __uint_as_float(__byte_perm(h4, 0x4B000000u, 0x7650u + i)) - 8388616.0f);
            }
        }
    } else {
        // Q6_K (Sources/LeviathanCore/Q6.swift:10-62): level = nibble | (two high bits << 4), value = d*scale*(level-32)
        const int g0 = 2 * (it & 1);
        const float d = h2f(R.hdr.x);
        const float ds0 = __fmul_rn(d, (float)(int)(signed char)(R.hdr.y & 0xffu));
        const float ds1 = __fmul_rn(d, (float)(int)(signed char)((R.hdr.y >> 8) & 0xffu));
        // four levels per word: the groups of an even K-step take the low nibbles and high-bit pairs 0 and 1, those of
        // an odd one the high nibbles and pairs 2 and 3; level - 32 is exact in f32, and so is its product with d * scale
        const unsigned a[2] = {R.q0.x, R.q0.y}, b[2] = {R.q1.x, R.q1.y}, h[2] = {R.qh.x, R.qh.y};
        const unsigned sh = 2u * (unsigned)g0;  // 0 or 4
#pragma unroll
        for (int wd = 0; wd < 2; wd++) {
            const unsigned hs = h[wd] >> sh;
            const unsigned la = ((a[wd] >> sh) & 0x0F0F0F0Fu) | ((hs << 4) & 0x30303030u);
            const unsigned lb = ((b[wd] >> sh) & 0x0F0F0F0Fu) | ((hs << 2) & 0x30303030u);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo[4 * wd + i] = __fmul_rn(ds0, __uint_as_float(__byte_perm(la, 0x4B000000u, 0x7650u + i)) - 8388640.0f);
                hi[4 * wd + i] = __fmul_rn(ds1, __uint_as_float(__byte_perm(lb, 0x4B000000u, 0x7650u + i)) - 8388640.0f);
            }
        }
    }
    *reinterpret_cast<uint4*>(wtile + swz(r, ch_lo)) = pack8(lo);
    *reinterpret_cast<uint4*>(wtile + swz(r, ch_hi)) = pack8(hi);
}

// ---- staged decode of the dense kernel: two threads per weight row ----
// The raw GGUF bytes of the tile's 176 rows x 256 columns (144 bytes per row for both 4-bit formats) are copied
// to shared memory by cp.async one group ahead; a thread reads its row's bytes with 16-byte shared loads (rows
// 144 bytes apart: eight lanes cover the 32 banks) and produces 32 of the K-step's 64 values, four 16-byte chunks
// of the swizzled tile row.  Thread half h takes the low (0) or the high (1) nibbles, so both halves run the
// same instructions with a shift of 4h.
constexpr int DS_ROW_BYTES = 144;
constexpr int DS_RAW_BYTES = RN * DS_ROW_BYTES;     // 25344 per group
constexpr int kDecodeThreads = kDequantWarps * 32;   // 352 = 2 x RN
static_assert(kDecodeThreads == 2 * RN && DS_RAW_BYTES % 16 == 0, "two decode threads per weight row");
__device__ __forceinline__ void dense_decode_barrier() { asm volatile("bar.sync 1, %0;\n" ::"n"(kDecodeThreads) : "memory"); }

// Q4_K: K-step c of the block whose 144 bytes start at blk; half h = sub-block 2c + h.  value = d1 * q - m1 with
// d1 = d * sc, m1 = dmin * m as the reference forms them (rust/crates/lev-cpu/src/lib.rs:110-130); d1 * q is
// exact in f32 (11 + 6 + 4 bits), so the fused multiply-add gives the bits of its multiply-then-subtract.
__device__ __forceinline__ void q4k_half_store(const unsigned char* blk, int c, unsigned h, unsigned char* wtile, int r) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    const uint4 qa = *reinterpret_cast<const uint4*>(blk + 16 + 32 * c), qb = *reinterpret_cast<const uint4*>(blk + 32 + 32 * c);
    const float d = h2f(hdr.x & 0xffffu), dmin = h2f(hdr.x >> 16);
    const unsigned sc_w = c < 2 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u));
    const unsigned mn_w = c < 2 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u));
    const unsigned sh = 8u * (2u * (unsigned)(c & 1) + h);
    const float d1 = __fmul_rn(d, (float)((sc_w >> sh) & 0xffu)), nm1 = -__fmul_rn(dmin, (float)((mn_w >> sh) & 0xffu));
    const unsigned w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const unsigned n4 = (w[2 * j + k] >> (4u * h)) & 0x0F0F0F0Fu;
#pragma unroll
            for (int i = 0; i < 4; i++) v[4 * k + i] = __fmaf_rn(d1, __uint_as_float(__byte_perm(n4, 0x4B000000u, 0x7650u + i)) - 8388608.0f, nm1);
        }
        *reinterpret_cast<uint4*>(wtile + swz(r, 4 * (int)h + j)) = pack8(v);
    }
}

// Q4_0: K-step S (0..3) of a 256-column group = the two blocks at byte 36 * S of the row's 144; half h takes the
// low or high nibbles of both blocks: values 16h .. 16h + 15 of each, chunks 4b + 2h and 4b + 2h + 1.
// d * (128 + q) - 136 d is exact and equals the reference's d * (q - 8) (Sources/LeviathanCore/Q4.swift:54-69).
template <int S>
__device__ __forceinline__ void q40_half_store(const unsigned char* rowraw, unsigned h, unsigned char* wtile, int r) {
    const uint4* src = reinterpret_cast<const uint4*>(rowraw + ((36 * S) & ~15));
    unsigned L[12];
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const uint4 v4 = src[c];
        L[4 * c] = v4.x; L[4 * c + 1] = v4.y; L[4 * c + 2] = v4.z; L[4 * c + 3] = v4.w;
    }
    const unsigned* w = L + S;   // the 36 bytes start at word S of the window
#pragma unroll
    for (int b = 0; b < 2; b++) {
        unsigned q[4];
        unsigned dbits;
        if (b == 0) {
            dbits = w[0] & 0xffffu;
#pragma unroll
            for (int k = 0; k < 4; k++) q[k] = __funnelshift_r(w[k], w[k + 1], 16);
        } else {
            dbits = w[4] >> 16;
#pragma unroll
            for (int k = 0; k < 4; k++) q[k] = w[5 + k];
        }
        const float d = h2f(dbits), c136 = __fmul_rn(d, -136.0f);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const unsigned n4 = (q[2 * j + k] >> (4u * h)) & 0x0F0F0F0Fu;
#pragma unroll
                for (int i = 0; i < 4; i++) v[4 * k + i] = __fmaf_rn(d, __uint_as_float(__byte_perm(n4, 0x43000000u, 0x7054u + (i << 8))), c136);
            }
            *reinterpret_cast<uint4*>(wtile + swz(r, 4 * b + 2 * (int)h + j)) = pack8(v);
        }
    }
}

template <int TYPE, bool STAGED>
__global__ void __launch_bounds__(kThreads, 1) k_gemm_tc(const __grid_constant__ CUtensorMap xmap, GemmTcArgs A) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_x[STAGES], full_w[STAGES], empty[STAGES], accum_full;
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    const int64_t r0 = (int64_t)blockIdx.x * RN;
    const int t0 = blockIdx.y * TM;
    const int halves = A.tokens - t0 > 128 ? 2 : 1;
    // K split: this CTA's K-steps are [kbase, kbase + kt) of the tensor's, its output slab is blockIdx.z
    const int kt_all = (int)(A.cols / KS);
    const int kbase = (int)blockIdx.z * A.ksteps_per_split;
    const int kt = kt_all - kbase < A.ksteps_per_split ? kt_all - kbase : A.ksteps_per_split;
    float* const yout = A.y + (int64_t)blockIdx.z * A.tokens * A.rows;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(s32(&full_x[s]), 1);
            mbar_init(s32(&full_w[s]), kDequantWarps);
            mbar_init(s32(&empty[s]), 1);
        }
        mbar_init(s32(&accum_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    volatile int* abort_flag = &abort_s;

    if (warp == 0) {
        // ---- activation tiles by TMA ----
        if (lane == 0) {
            for (int it = 0; it < kt; it++) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(s32(&empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag)) break;
                const unsigned dst = s32(smem + (size_t)s * kStageBytes);
                mbar_expect_tx(s32(&full_x[s]), halves * kXHalfBytes);
                tma_load_2d(dst, &xmap, (kbase + it) * KS, t0, s32(&full_x[s]));
                if (halves == 2) tma_load_2d(dst + kXHalfBytes, &xmap, (kbase + it) * KS, t0 + 128, s32(&full_x[s]));
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < kt && ok; it++) {
                const int s = it % STAGES;
                const unsigned ph = (it / STAGES) & 1;
                ok = mbar_wait(s32(&full_x[s]), ph, abort_flag);
                ok = ok && mbar_wait(s32(&full_w[s]), ph, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned xs = s32(smem + (size_t)s * kStageBytes), ws = xs + kXStageBytes;
#pragma unroll
                for (int kk = 0; kk < KS / 16; kk++) {
                    const uint64_t bdesc = umma_desc(ws + kk * 32);
                    for (int h = 0; h < halves; h++)
                        umma_bf16(tmem_base + h * RN, umma_desc(xs + h * kXHalfBytes + kk * 32), bdesc, (it | kk) ? 1u : 0u);
                }
                umma_commit(s32(&empty[s]));  // the stage may be refilled when these MMAs have read it
            }
            umma_commit(s32(&accum_full));
        }
    } else {
        bool ok = true;
        if constexpr (STAGED) {
            // ---- weight staging and decode: thread = (weight row, nibble half) ----
            const int dt = threadIdx.x - 64;
            const int row = dt % RN;
            const unsigned half_h = (unsigned)(dt / RN);
            unsigned char* rawbuf = smem + (size_t)STAGES * kStageBytes;
            const int ngroups = kt >> 2;              // this form serves K in whole 256-column groups
            // decode warp dw stages rows dw, dw + 11, ... (16 rows): lanes 0..26 take three rows at a time, nine
            // 16-byte pieces each
            const int dw = warp - 2;
            const int l9 = lane / 9, p9 = lane - 9 * l9;
            auto stage_group = [&](int g) {
                const unsigned dst0 = s32(rawbuf + (size_t)(g & 1) * DS_RAW_BYTES);
                const uint8_t* src0 = A.raw + r0 * A.row_bytes + (int64_t)((kbase >> 2) + g) * DS_ROW_BYTES;
                if (lane < 27) {
#pragma unroll
                    for (int q = 0; q < 6; q++) {
                        const int m = 3 * q + l9;
                        const int r = dw + kDequantWarps * m;
                        if (m < 16 && r0 + r < A.rows) cp_async16(dst0 + r * DS_ROW_BYTES + p9 * 16, src0 + (int64_t)r * A.row_bytes + p9 * 16);
                    }
                }
            };
            if (ngroups > 0) stage_group(0);
            cp_async_commit();
            for (int g = 0; g < ngroups; g++) {
                cp_async_wait_but<0>();       // this thread's copies of group g have landed
                dense_decode_barrier();       // everyone's have, and everyone is done reading the other slot
                if (g + 1 < ngroups && ok) stage_group(g + 1);
                cp_async_commit();
                const unsigned char* rowraw = rawbuf + (size_t)(g & 1) * DS_RAW_BYTES + row * DS_ROW_BYTES;
                auto kstep = [&](auto s_tag) {
                    constexpr int SK = decltype(s_tag)::value;
                    const int it = 4 * g + SK;
                    if (!ok) return;
                    const int s = it % STAGES;
                    if (it >= STAGES) ok = mbar_wait(s32(&empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag);
                    if (!ok) return;
                    unsigned char* wtile = smem + (size_t)s * kStageBytes + kXStageBytes;
                    if (TYPE == LEV_GGML_Q4_K) q4k_half_store(rowraw, SK, half_h, wtile, row);
                    else q40_half_store<SK>(rowraw, half_h, wtile, row);
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s32(&full_w[s]));
                };
                kstep(std::integral_constant<int, 0>());
                kstep(std::integral_constant<int, 1>());
                kstep(std::integral_constant<int, 2>());
                kstep(std::integral_constant<int, 3>());
            }
            cp_async_wait_but<0>();
        } else {
        // ---- weight decode: thread = (2 rows 88 apart) x (byte group j); the raw bytes of the
        // next K-step are requested before this one is decoded ----
        // lanes 0..7 of a warp take byte group 0 of eight consecutive rows, lanes 8..15 group 1, ...:
        // the eight 16-byte stores of one shared-memory wavefront then fall into eight different
        // bank groups of the swizzled tile
        const int j = lane >> 3, rb = (warp - 2) * 8 + (lane & 7);
        constexpr int kRowStep = kDequantWarps * 8;   // rows covered by one pass of the decode threads
        constexpr int NR = RN / kRowStep;
        static_assert(RN % kRowStep == 0, "decode threads tile the weight rows evenly");
        RowRaw<TYPE> ahead[kAhead][NR];
        const uint8_t* rowp[NR];
        bool valid[NR];
#pragma unroll
        for (int i = 0; i < NR; i++) {
            valid[i] = r0 + rb + kRowStep * i < A.rows;
            rowp[i] = A.raw + (r0 + (valid[i] ? rb + kRowStep * i : 0)) * A.row_bytes;
#pragma unroll
            for (int u = 0; u < kAhead; u++)
                if (u < kt) load_raw<TYPE>(rowp[i], kbase + u, j, valid[i], ahead[u][i]);
        }
        for (int it0 = 0; it0 < kt && ok; it0 += kAhead) {
#pragma unroll
            for (int u = 0; u < kAhead; u++) {
                const int it = it0 + u;
                if (it >= kt || !ok) break;
                const int s = it % STAGES;
                RowRaw<TYPE> cur[NR];
#pragma unroll
                for (int i = 0; i < NR; i++) {
                    cur[i] = ahead[u][i];
                    if (it + kAhead < kt) load_raw<TYPE>(rowp[i], kbase + it + kAhead, j, valid[i], ahead[u][i]);
                }
                if (it >= STAGES) ok = mbar_wait(s32(&empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag);
                if (!ok) break;
                unsigned char* wtile = smem + (size_t)s * kStageBytes + kXStageBytes;
#pragma unroll
                for (int i = 0; i < NR; i++) decode_store<TYPE>(cur[i], kbase + it, j, valid[i], wtile, rb + kRowStep * i);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(s32(&full_w[s]));
            }
        }
        }
        // ---- epilogue: TMEM -> Y ----
        if (ok && warp < 10 && mbar_wait(s32(&accum_full), 0, abort_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int quarter = warp & 3, half = (warp - 2) >> 2;
            if (half < halves) {
                unsigned* stg = reinterpret_cast<unsigned*>(smem) + (warp - 2) * (32 * 36);
#pragma unroll 1
                for (int c = 0; c < RN; c += 32) {
                    unsigned v[32];
                    const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(half * RN + c);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    // transpose through shared memory (the pipeline stages are idle now) so that every
                    // store instruction writes whole 128-byte lines of four token rows
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < 32; q += 4)
                        *reinterpret_cast<uint4*>(stg + lane * 36 + q) = make_uint4(v[q], v[q + 1], v[q + 2], v[q + 3]);
                    __syncwarp();
                    const int col4 = (lane & 7) * 4;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int tl = i * 4 + (lane >> 3);
                        const int tok = t0 + half * 128 + quarter * 32 + tl;
                        const uint4 o = *reinterpret_cast<const uint4*>(stg + tl * 36 + col4);
                        if (tok < A.tokens && c + col4 < RN) {  // the last chunk of a tile may be narrower than 32
                            float* dst = yout + (int64_t)tok * A.rows + r0 + c + col4;
                            if (r0 + c + col4 + 4 <= A.rows && A.y_vec) {
                                *reinterpret_cast<uint4*>(dst) = o;
                            } else {
                                const unsigned ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (int q = 0; q < 4; q++)
                                    if (r0 + c + col4 + q < A.rows) dst[q] = __uint_as_float(ov[q]);
                            }
                        }
                    }
                }
            }
        }
    }
    if (abort_s && threadIdx.x == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Grouped form for the routed MoE at prefill-sized token counts: operands swapped, so that the
// weight rows are the MMA's M (128) and the tokens of one expert its N (16..128 in steps of 16;
// experts rarely see many tokens and a padded M would waste most of the tensor work).
//   job j (device-side table) = up to 128 consecutive grouped positions of one expert;
//   CTA (rt, j): rows [128*rt, +128) of the job's expert slice x the job's tokens, whole K.
//   X rows come from a position-ordered bf16 buffer (TMA, 128 rows per box);
//   D[row][position] is stored as out[out_row(position)][row]: a warp writes 32 consecutive rows.
// ---------------------------------------------------------------------------
// The kernel is bound by the weight decode (an expert's weights are decoded for a few dozen tokens
// only), so three CTAs share an SM: 2 stages x (16 KB weights + 16 KB tokens) and 128 TMEM columns each.
constexpr int GR_STAGES = 2;
constexpr int GR_DECODE_WARPS = 8;
constexpr int GR_THREADS = (2 + GR_DECODE_WARPS) * 32;
constexpr int GR_W_BYTES = 128 * KS * 2;               // 16384
constexpr int GR_STAGE_BYTES = GR_W_BYTES + kXHalfBytes;   // 32768
constexpr int GR_TMEM_COLS = 128;
constexpr int GR_JOB_TOKENS = 64;

struct GroupedArgs {
    const uint8_t* raw;      // expert-stacked tensor, row-major GGUF blocks
    int64_t row_bytes;
    int rows_per_expert;
    int cols;                // K
    const int* njobs;        // [1]
    const int* job_slice;    // [job] local expert
    const int* job_pos;      // [job][GR_JOB_TOKENS] grouped positions (first entry = first position)
    const int* offsets;      // [experts + 1] grouped offsets by global expert id
    int first_expert;        // global id of local expert 0
    const int* out_row;      // [position] row of `out` for that position, NULL: the position itself
    float* out;              // [rows of out][out_ld]
    int64_t out_ld;
    int* status;
};

template <int TYPE>
__global__ void __launch_bounds__(GR_THREADS, 3) k_gemm_tc_grouped(const __grid_constant__ CUtensorMap xmap, GroupedArgs A) {
    const int job = blockIdx.y;
    if (job >= *A.njobs) return;  // whole CTA leaves before touching barriers or tensor memory
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_x[GR_STAGES], full_w[GR_STAGES], empty[GR_STAGES], accum_full;
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    const int e = A.job_slice[job];
    const int pos0 = A.job_pos[(int64_t)job * GR_JOB_TOKENS];
    int cnt = A.offsets[A.first_expert + e + 1] - pos0;
    cnt = cnt > GR_JOB_TOKENS ? GR_JOB_TOKENS : cnt;
    const int n_pad = (cnt + 15) & ~15;           // MMA N
    const int row0 = blockIdx.x * 128;            // first row inside the expert slice
    const int kt = A.cols / KS;
    const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n_pad >> 3) << 17) | ((unsigned)(128 >> 4) << 24);

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < GR_STAGES; s++) {
            mbar_init(s32(&full_x[s]), 1);
            mbar_init(s32(&full_w[s]), GR_DECODE_WARPS);
            mbar_init(s32(&empty[s]), 1);
        }
        mbar_init(s32(&accum_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(GR_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    volatile int* abort_flag = &abort_s;

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < kt; it++) {
                const int s = it % GR_STAGES;
                if (it >= GR_STAGES && !mbar_wait(s32(&empty[s]), ((it / GR_STAGES) & 1) ^ 1, abort_flag)) break;
                const unsigned dst = s32(smem + (size_t)s * GR_STAGE_BYTES + GR_W_BYTES);
                mbar_expect_tx(s32(&full_x[s]), kXHalfBytes);
                tma_load_2d(dst, &xmap, it * KS, pos0, s32(&full_x[s]));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < kt && ok; it++) {
                const int s = it % GR_STAGES;
                const unsigned ph = (it / GR_STAGES) & 1;
                ok = mbar_wait(s32(&full_x[s]), ph, abort_flag) && mbar_wait(s32(&full_w[s]), ph, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned ws = s32(smem + (size_t)s * GR_STAGE_BYTES), xs = ws + GR_W_BYTES;
#pragma unroll
                for (int kk = 0; kk < KS / 16; kk++) {
                    const uint64_t adesc = umma_desc(ws + kk * 32), bdesc = umma_desc(xs + kk * 32);
                    const unsigned acc = (it | kk) ? 1u : 0u;
                    asm volatile(
                        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(
                            tmem_base),
                        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                        : "memory");
                }
                umma_commit(s32(&empty[s]));
            }
            umma_commit(s32(&accum_full));
        }
    } else {
        // ---- weight decode: thread = (2 rows 64 apart) x (byte group j) ----
        const int j = lane >> 3, rb = (warp - 2) * 8 + (lane & 7);
        constexpr int NR = 2;
        RowRaw<TYPE> ahead[kAhead][NR];
        const uint8_t* rowp[NR];
        bool valid[NR];
#pragma unroll
        for (int i = 0; i < NR; i++) {
            const int r = row0 + rb + 64 * i;
            valid[i] = r < A.rows_per_expert;
            rowp[i] = A.raw + ((int64_t)e * A.rows_per_expert + (valid[i] ? r : 0)) * A.row_bytes;
#pragma unroll
            for (int u = 0; u < kAhead; u++)
                if (u < kt) load_raw<TYPE>(rowp[i], u, j, valid[i], ahead[u][i]);
        }
        bool ok = true;
        for (int it0 = 0; it0 < kt && ok; it0 += kAhead) {
#pragma unroll
            for (int u = 0; u < kAhead; u++) {
                const int it = it0 + u;
                if (it >= kt || !ok) break;
                const int s = it % GR_STAGES;
                RowRaw<TYPE> cur[NR];
#pragma unroll
                for (int i = 0; i < NR; i++) {
                    cur[i] = ahead[u][i];
                    if (it + kAhead < kt) load_raw<TYPE>(rowp[i], it + kAhead, j, valid[i], ahead[u][i]);
                }
                if (it >= GR_STAGES) ok = mbar_wait(s32(&empty[s]), ((it / GR_STAGES) & 1) ^ 1, abort_flag);
                if (!ok) break;
                unsigned char* wtile = smem + (size_t)s * GR_STAGE_BYTES;
#pragma unroll
                for (int i = 0; i < NR; i++) decode_store<TYPE>(cur[i], it, j, valid[i], wtile, rb + 64 * i);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(s32(&full_w[s]));
            }
        }
        // ---- epilogue: lane = weight row, TMEM columns = positions ----
        if (ok && mbar_wait(s32(&accum_full), 0, abort_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int quarter = warp & 3, chalf = (warp - 2) >> 2;
            const int row = row0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 32 * chalf; c < n_pad; c += 64) {
                unsigned v[32];
                const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c;
                // n_pad is a multiple of 16: the last chunk may hold 16 columns only
                if (c + 32 <= n_pad) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                } else {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                        : "r"(taddr)
                        : "memory");
#pragma unroll
                    for (int q = 16; q < 32; q++) v[q] = 0u;
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row < A.rows_per_expert) {
#pragma unroll
                    for (int q = 0; q < 32; q++) {
                        if (c + q < cnt) {
                            const int pos = pos0 + c + q;
                            const int orow = A.out_row ? A.out_row[pos] : pos;
                            A.out[(int64_t)orow * A.out_ld + row] = __uint_as_float(v[q]);
                        }
                    }
                }
            }
        }
    }
    if (abort_s && threadIdx.x == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(GR_TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Grouped form for Q4_0 with the raw blocks staged in shared memory.
//
// The kernel above spends most of its instructions on getting 18-byte blocks out of global memory with 2-byte
// loads and on the bookkeeping around 32 values per thread and K-step.  Here the GGUF bytes of 128 rows x 256
// columns (8 blocks = 144 bytes per row) are copied to shared memory asynchronously (cp.async, 16 bytes a copy
// where the tensor's rows are 16-byte aligned, 4 bytes otherwise), one such group ahead of the one being
// decoded; a decode thread owns ONE weight row, reads its two K-steps of the group with 16-byte shared loads
// (rows 144 bytes apart: eight lanes cover the 32 banks) and turns a nibble into its value with two
// instructions: a byte permute puts it into the mantissa of 128.0 (= 128 + q exactly) and one fused
// multiply-add forms d * (128 + q) - 136 d = d * (q - 8), which is exact, so the value equals the reference
// decoder's d * (q - 8) (Sources/LeviathanCore/Q4.swift:54-69) bit for bit; then one rounding to bf16.
// The decoded K-step of a row (64 bf16 = 32 registers) goes straight into tensor memory with one tcgen05.st: the
// MMA takes its A operand (the weights) from tensor memory, lane = weight row, and only the tokens from shared
// memory, so decoded weights never pass through shared memory and need no swizzled stores or proxy fences.
// Decode warps 2..5 take the even K-steps, warps 6..9 the odd ones; jobs hold up to 64 tokens, so two CTAs
// share an SM: 5 x 8 KB tokens, 2 x 18 KB raw bytes, and 256 TMEM columns each (64 accumulator + 4 x 32 weights).
// ---------------------------------------------------------------------------
constexpr int SG_STAGES = 4;      // decoded weight tiles in tensor memory (32 columns each)
constexpr int SG_XSTAGES = 5;    // token tiles (8 KB each): a TMA load takes several K-steps to arrive, so this ring is the deeper one
constexpr int SG_RAW_SLOTS = 2;   // groups of raw bytes in shared memory: one being decoded, the others on their way
constexpr int SG_X_BYTES = GR_JOB_TOKENS * KS * 2;          // 8192: one TMA box of 64 positions x 64 k
constexpr int SG_GROUP_COLS = 256;
constexpr int SG_ROW_BYTES = SG_GROUP_COLS / 32 * LEV_Q4_0_BYTES;   // 144
constexpr int SG_RAW_BYTES = 128 * SG_ROW_BYTES;            // 18432
constexpr int SG_SMEM = SG_XSTAGES * SG_X_BYTES + SG_RAW_SLOTS * SG_RAW_BYTES + 1024;
constexpr int SG_ACC_COLS = 64;                       // accumulator: one column per token of the job
constexpr int SG_A_COLS = KS / 2;                      // a K-step of one row: 64 bf16 = 32 columns
constexpr int SG_TMEM_COLS = 256;
static_assert(GR_JOB_TOKENS <= SG_ACC_COLS && SG_ACC_COLS + SG_STAGES * SG_A_COLS <= SG_TMEM_COLS && SG_ROW_BYTES % 16 == 0,
              "staged grouped form geometry");


// one Q4_0 block (f16 d, 16 nibble bytes in q[4]) -> its 32 values as 16 packed bf16 pairs in column order: low
// nibbles are values 0..15, high nibbles 16..31
__device__ __forceinline__ void q40_block_regs(unsigned dbits, const unsigned* q, unsigned* out) {
    const float d = h2f(dbits);
    const float c = __fmul_rn(d, -136.0f);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const unsigned l4 = q[k] & 0x0F0F0F0Fu, h4 = (q[k] >> 4) & 0x0F0F0F0Fu;
        float lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            lo[i] = __fmaf_rn(d, __uint_as_float(__byte_perm(l4, 0x43000000u, 0x7054u + (i << 8))), c);
            hi[i] = __fmaf_rn(d, __uint_as_float(__byte_perm(h4, 0x43000000u, 0x7054u + (i << 8))), c);
        }
        __nv_bfloat162 a = __floats2bfloat162_rn(lo[0], lo[1]), b = __floats2bfloat162_rn(lo[2], lo[3]);
        __nv_bfloat162 e = __floats2bfloat162_rn(hi[0], hi[1]), f = __floats2bfloat162_rn(hi[2], hi[3]);
        out[2 * k] = *reinterpret_cast<unsigned*>(&a);
        out[2 * k + 1] = *reinterpret_cast<unsigned*>(&b);
        out[8 + 2 * k] = *reinterpret_cast<unsigned*>(&e);
        out[8 + 2 * k + 1] = *reinterpret_cast<unsigned*>(&f);
    }
}

// K-step S (0..3) of a group: the 36 bytes at 36 * S of the row's 144, i.e. words S .. S + 8 of the twelve
// words L loaded from the 16-byte chunk that holds byte 36 * S; out = the row's 64 values as 32 bf16 pairs
template <int S>
__device__ __forceinline__ void q40_kstep_regs(const unsigned* L, unsigned* out) {
    const unsigned* w = L + S;
    unsigned qa[4];
#pragma unroll
    for (int k = 0; k < 4; k++) qa[k] = __funnelshift_r(w[k], w[k + 1], 16);   // block 0: d in the low half of w[0], nibbles from byte 2
    q40_block_regs(w[0] & 0xffffu, qa, out);
    q40_block_regs(w[4] >> 16, w + 5, out + 16);                               // block 1: d in the high half of w[4], nibbles aligned
}

// 32 consecutive 32-bit columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
        "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
        "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

// what a CTA needs to know of tile t = (job, row tile): the job's expert slice, first grouped position, token count
struct SgTile {
    int e, pos0, cnt, row0;
};
__device__ __forceinline__ SgTile sg_tile(const GroupedArgs& A, int t, int row_tiles) {
    SgTile T;
    const int job = t / row_tiles;
    T.row0 = (t - job * row_tiles) * 128;
    T.e = A.job_slice[job];
    T.pos0 = A.job_pos[(int64_t)job * GR_JOB_TOKENS];
    const int c = A.offsets[A.first_expert + T.e + 1] - T.pos0;
    T.cnt = c > GR_JOB_TOKENS ? GR_JOB_TOKENS : c;
    return T;
}

// The CTAs are persistent: CTA c works through tiles c, c + gridDim.x, ... of the job list, so tensor memory, the
// barriers and the first trip to global memory are paid once per CTA, and the staging of a tile's first columns
// runs while the previous tile is still being decoded.  Ring positions count K-steps over all of a CTA's tiles.
template <int CW>
__global__ void __launch_bounds__(GR_THREADS, 2) k_gemm_tc_grouped_q40(const __grid_constant__ CUtensorMap xmap, GroupedArgs A) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_x[SG_XSTAGES], empty_x[SG_XSTAGES], full_w[SG_STAGES], empty[SG_STAGES];
    __shared__ __align__(8) unsigned long long accum_full, accum_empty;
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* xbuf = smem;
    unsigned char* rawbuf = xbuf + SG_XSTAGES * SG_X_BYTES;
    const int row_tiles = (A.rows_per_expert + 127) >> 7;
    const int total_tiles = *A.njobs * row_tiles;
    const int my_tiles = (int)blockIdx.x < total_tiles ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int kt = A.cols / KS;
    const int ngroups = (kt + 3) >> 2;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < SG_STAGES; s++) {
            mbar_init(s32(&full_w[s]), GR_DECODE_WARPS / 2);
            mbar_init(s32(&empty[s]), 1);
        }
        for (int s = 0; s < SG_XSTAGES; s++) {
            mbar_init(s32(&full_x[s]), 1);
            mbar_init(s32(&empty_x[s]), 1);
        }
        mbar_init(s32(&accum_full), 1);
        mbar_init(s32(&accum_empty), GR_DECODE_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(SG_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    volatile int* abort_flag = &abort_s;

    if (warp == 0) {
        // ---- token tiles by TMA ----
        if (lane == 0) {
            bool ok = true;
            for (int k = 0; k < my_tiles && ok; k++) {
                const SgTile T = sg_tile(A, (int)blockIdx.x + k * (int)gridDim.x, row_tiles);
                for (int it = 0; it < kt; it++) {
                    const int n = k * kt + it, s = n % SG_XSTAGES;
                    if (n >= SG_XSTAGES && !mbar_wait(s32(&empty_x[s]), ((n / SG_XSTAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(s32(&full_x[s]), SG_X_BYTES);
                    tma_load_2d(s32(xbuf + (size_t)s * SG_X_BYTES), &xmap, it * KS, T.pos0, s32(&full_x[s]));
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        if (lane == 0) {
            bool ok = true;
            for (int k = 0; k < my_tiles && ok; k++) {
                const SgTile T = sg_tile(A, (int)blockIdx.x + k * (int)gridDim.x, row_tiles);
                const int n_pad = (T.cnt + 15) & ~15;   // MMA N
                const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n_pad >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
                // the accumulator is free again when every decode warp has read tile k - 1 out of it
                if (k > 0 && !mbar_wait(s32(&accum_empty), (k - 1) & 1, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                for (int it = 0; it < kt && ok; it++) {
                    const int n = k * kt + it, s = n % SG_STAGES, sx = n % SG_XSTAGES;
                    ok = mbar_wait(s32(&full_x[sx]), (n / SG_XSTAGES) & 1, abort_flag) && mbar_wait(s32(&full_w[s]), (n / SG_STAGES) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned xs = s32(xbuf + (size_t)sx * SG_X_BYTES);
                    const unsigned at = tmem_base + SG_ACC_COLS + (unsigned)s * SG_A_COLS;   // A: this stage's columns, lane = weight row
#pragma unroll
                    for (int kk = 0; kk < KS / 16; kk++) {
                        const uint64_t bdesc = umma_desc(xs + kk * 32);
                        const unsigned acc = (it | kk) ? 1u : 0u;
                        asm volatile(
                            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(
                                tmem_base),
                            "r"(at + kk * 8), "l"(bdesc), "r"(idesc), "r"(acc)
                            : "memory");
                    }
                    umma_commit(s32(&empty[s]));      // both tiles may be refilled when these MMAs have read them
                    umma_commit(s32(&empty_x[sx]));
                }
                if (ok) umma_commit(s32(&accum_full));
            }
        }
    } else {
        // ---- weight staging and decode: 256 threads; thread = weight row (tid & 127), K-step parity (tid >> 7) ----
        // a warp reaches the 32 tensor-memory lanes 32 * (warp % 4) ..., so those are its weight rows
        const int quarter = warp & 3, par = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        // Copies of group g of the CTA's tile k into raw slot (k * ngroups + g) % SG_RAW_SLOTS.  Decode warp dw stages
        // rows dw, dw + 8, ... (16 rows); nothing below divides by a run-time value.
        //   16-byte pieces: lanes 0..26 take three rows at a time, nine pieces each;
        //   4-byte pieces: a row is 36 words: all lanes take words 0..31 of a row, then the four words left over of
        //   eight rows at once (lane = 4 * row + word).
        const int dw = warp - 2;
        const int l9 = lane / 9, p9 = lane - 9 * l9;          // 16-byte form: row of the triple, piece
        const int l4 = lane >> 2, p4 = 32 + (lane & 3);        // 4-byte form, left-over words: row of the eight, word
        auto stage_group = [&](const SgTile& T, int g, int slot) {
            const int gbytes = min(SG_ROW_BYTES, (int)A.row_bytes - g * SG_ROW_BYTES);
            const unsigned dst0 = s32(rawbuf + (size_t)slot * SG_RAW_BYTES);
            const uint8_t* src0 = A.raw + ((int64_t)T.e * A.rows_per_expert + T.row0) * A.row_bytes + (int64_t)g * SG_ROW_BYTES;
            if (CW == 16) {
                if (lane < 27) {
#pragma unroll
                    for (int q = 0; q < 6; q++) {
                        const int r = dw + 8 * (3 * q + l9);   // rows dw + 8 * (0..15)
                        if (3 * q + l9 < 16 && T.row0 + r < A.rows_per_expert)
                            cp_async16(dst0 + r * SG_ROW_BYTES + p9 * 16, src0 + (int64_t)r * A.row_bytes + p9 * 16);
                    }
                }
            } else {
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    const int r = dw + 8 * q;
                    if (4 * lane < gbytes && T.row0 + r < A.rows_per_expert)
                        cp_async4(dst0 + r * SG_ROW_BYTES + 4 * lane, src0 + (int64_t)r * A.row_bytes + 4 * lane);
                }
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int r = dw + 8 * (8 * q + l4);
                    if (4 * p4 < gbytes && T.row0 + r < A.rows_per_expert)
                        cp_async4(dst0 + r * SG_ROW_BYTES + 4 * p4, src0 + (int64_t)r * A.row_bytes + 4 * p4);
                }
            }
        };
        // Every thread commits one copy group per group of columns (an empty one past the end), so that "all but the
        // newest SG_RAW_SLOTS - 2" always means: group G has landed.  (sk, sg, sslot) is the next group to stage: tile,
        // group inside the tile, raw slot; the staging runs SG_RAW_SLOTS - 1 groups ahead of the decode and so crosses
        // into the next tile before the decode does.
        static_assert(SG_RAW_SLOTS == 2, "the staging below looks at most one tile ahead");
        SgTile T = {0, 0, 0, 0};
        if (my_tiles > 0) {
            T = sg_tile(A, (int)blockIdx.x, row_tiles);
            stage_group(T, 0, 0);
        }
        cp_async_commit();
        int sk = 0, sg = 1, sslot = 1;   // the group after the one just staged
        if (sg == ngroups) { sg = 0; sk = 1; }
        bool ok = true;
        for (int k = 0; k < my_tiles; k++) {
            // the next tile's parameters are fetched a whole tile before the staging needs them
            const SgTile Tnext = k + 1 < my_tiles ? sg_tile(A, (int)blockIdx.x + (k + 1) * (int)gridDim.x, row_tiles) : T;
            for (int g = 0; g < ngroups; g++) {
                const int G = k * ngroups + g;
                cp_async_wait_but<0>();   // this thread's copies of group G have landed
                decode_barrier();         // everyone's have, and everyone is done reading group G - 1's slot
                if (sk < my_tiles && ok) stage_group(sk == k ? T : Tnext, sg, sslot);
                cp_async_commit();
                sslot ^= 1;
                if (++sg == ngroups) { sg = 0; sk++; }
                const unsigned char* rs = rawbuf + (size_t)(G % SG_RAW_SLOTS) * SG_RAW_BYTES + row * SG_ROW_BYTES;
                // K-step sk of the group -> tensor memory; the four forms differ in compile-time word offsets only and
                // each ends in its own tcgen05.st, so no register moves join them.  A row past the end of the expert
                // decodes whatever its slot holds: its accumulator lane is never stored.
                auto kstep = [&](auto sk_tag) {
                    constexpr int SK = decltype(sk_tag)::value;
                    const int it = 4 * g + SK;
                    if (it >= kt || !ok) return;
                    const int n = k * kt + it, s = n % SG_STAGES;
                    unsigned L[12];
                    const uint4* src = reinterpret_cast<const uint4*>(rs + ((36 * SK) & ~15));
#pragma unroll
                    for (int c = 0; c < 3; c++) {
                        const uint4 v4 = src[c];
                        L[4 * c] = v4.x; L[4 * c + 1] = v4.y; L[4 * c + 2] = v4.z; L[4 * c + 3] = v4.w;
                    }
                    if (n >= SG_STAGES) ok = mbar_wait(s32(&empty[s]), ((n / SG_STAGES) & 1) ^ 1, abort_flag);
                    if (!ok) return;
                    unsigned v[32];
                    q40_kstep_regs<SK>(L, v);
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    tmem_st32(tmem_base + lane_addr + SG_ACC_COLS + (unsigned)s * SG_A_COLS, v);
                    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s32(&full_w[s]));
                };
                if (par == 0) {
                    kstep(std::integral_constant<int, 0>());
                    kstep(std::integral_constant<int, 2>());
                } else {
                    kstep(std::integral_constant<int, 1>());
                    kstep(std::integral_constant<int, 3>());
                }
            }
            // ---- epilogue of tile k: lane = weight row, TMEM columns = positions ----
            if (ok) ok = mbar_wait(s32(&accum_full), k & 1, abort_flag);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const int n_pad = (T.cnt + 15) & ~15;
                const int orow_w = T.row0 + row;
                const int c = 32 * par;
                unsigned v[32];
                if (c < n_pad) {
                    const unsigned taddr = tmem_base + lane_addr + (unsigned)c;
                    if (c + 32 <= n_pad) {
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                              "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                              "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                            : "r"(taddr)
                            : "memory");
                    } else {
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                            : "r"(taddr)
                            : "memory");
#pragma unroll
                        for (int q = 16; q < 32; q++) v[q] = 0u;
                    }
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                }
                // the values are in registers: the next tile's first MMA may overwrite the accumulator
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(s32(&accum_empty));
                if (c < n_pad && orow_w < A.rows_per_expert) {
#pragma unroll
                    for (int q = 0; q < 32; q++) {
                        if (c + q < T.cnt) {
                            const int pos = T.pos0 + c + q;
                            const int orow = A.out_row ? A.out_row[pos] : pos;
                            A.out[(int64_t)orow * A.out_ld + orow_w] = __uint_as_float(v[q]);
                        }
                    }
                }
            }
            T = Tnext;
        }
        cp_async_wait_but<0>();
    }
    if (abort_s && threadIdx.x == 0) atomicOr(A.status, LEV_DEV_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(SG_TMEM_COLS) : "memory");
    }
}

// x f32 [tokens][cols] -> position-ordered bf16 rows: row pos = token of pair perm[pos]
__global__ void k_gather_bf16(const float* __restrict__ x, const int* __restrict__ perm, const int* __restrict__ total_pos,
                              int top_k, int cols, __nv_bfloat16* __restrict__ out) {
    const int64_t n = (int64_t)(*total_pos) * (cols / 4);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pos = i / (cols / 4);
        const int c4 = (int)(i - pos * (cols / 4));
        const float4 v = __ldg(reinterpret_cast<const float4*>(x + (int64_t)(perm[pos] / top_k) * cols) + c4);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        reinterpret_cast<uint2*>(out + pos * cols)[c4] = make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
    }
}

// gu f32 [pos][2*inter] -> bf16 [pos][inter] of gelu_tanh(gate) * up
// (Sources/LeviathanCore/Gemma4.swift:4364-4377)
__global__ void k_act_grouped_bf16(const float* __restrict__ gu, const int* __restrict__ total_pos, int inter,
                                   __nv_bfloat16* __restrict__ out) {
    const int64_t n = (int64_t)(*total_pos) * inter;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pos = i / inter;
        const int k = (int)(i - pos * inter);
        const float g = gu[pos * 2 * inter + k], u = gu[pos * 2 * inter + inter + k];
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        const float ex = expf(-2.0f * fabsf(inner));
        const float th = copysignf((1.0f - ex) / (1.0f + ex), inner);
        out[i] = __float2bfloat16_rn(0.5f * g * (1.0f + th) * u);
    }
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// y = sum over the K splits' partial products, in split order (the same bits on every run)
__global__ void __launch_bounds__(256) k_gemm_split_sum(const float4* __restrict__ part, int splits, int64_t n4, float4* __restrict__ y) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 a = part[i];
        for (int z = 1; z < splits; z++) {
            const float4 b = part[(int64_t)z * n4 + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        y[i] = a;
    }
}

template <int TYPE, bool STAGED>
int launch_tc(lev_ctx* ctx, const CUtensorMap& map, const GemmTcArgs& A, dim3 grid, size_t smem) {
    static bool configured[16] = {};
    if (!configured[ctx->device & 15]) {
        LEV_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc<TYPE, STAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[ctx->device & 15] = true;
    }
    k_gemm_tc<TYPE, STAGED><<<grid, kThreads, smem, ctx->stream>>>(map, A);
    return LEV_OK;
}

}  // namespace

// shapes the tensor-memory kernel serves: rows whose K is a multiple of 64,
// 16-byte aligned activations
bool lev_gemm_tc_supported(const lev_weights* w, const void* x_bf16, int64_t tokens) {
    if (w->type != LEV_GGML_Q4_K && w->type != LEV_GGML_Q4_0 && w->type != LEV_GGML_Q6_K) return false;
    if (w->cols % KS != 0 || ((uintptr_t)x_bf16 & 15) != 0 || tokens < 1) return false;
    return encode_tiled() != nullptr;
}

int lev_gemm_tc_run(lev_ctx* ctx, const lev_weights* w, const void* x_bf16, int64_t tokens, float* y) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return lev_fail(ctx, LEV_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)w->cols, (cuuint64_t)tokens};
    const cuuint64_t gstride[1] = {(cuuint64_t)w->cols * 2};
    const cuuint32_t box[2] = {KS, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), gdim, gstride, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return lev_fail(ctx, LEV_KERNEL_FAILED, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
    GemmTcArgs A;
    A.raw = w->raw;
    A.type = w->type;
    A.row_bytes = w->blocks_per_row * lev_block_bytes(w->type);
    A.rows = w->rows;
    A.cols = w->cols;
    A.tokens = (int)tokens;
    A.y = y;
    A.y_vec = ((uintptr_t)y & 15) == 0 && (w->rows & 3) == 0;
    A.status = ctx->d_status;
    A.ksteps_per_split = (int)(w->cols / KS);
    dim3 grid((unsigned)((w->rows + RN - 1) / RN), (unsigned)((tokens + TM - 1) / TM));
    const size_t smem = (size_t)STAGES * kStageBytes + 1024;
    // Up to 128 tokens (decode batches) the kernel is bound by the weight decode: the 4-bit formats then decode from
    // raw bytes staged in shared memory (40 % fewer instructions), when K comes in whole 256-column groups and every
    // row starts on a 16-byte boundary (16-byte asynchronous copies).  Above that the token tiles' trip from L2 is
    // the bound (measured: decode warps wait on the MMA's stage release 45 % of the time) and the register-staged
    // form, which leaves shared memory to the pipeline, is the faster one (73 against 80 us on 512 x 12288 x 4096).
    const bool staged = tokens <= 128 && w->type != LEV_GGML_Q6_K && w->cols % 256 == 0 && A.row_bytes % 16 == 0 &&
                        ((uintptr_t)A.raw & 15) == 0;
    const size_t smem_staged = smem + 2 * (size_t)DS_RAW_BYTES;
    // A decode batch against a tensor of a few thousand rows makes a few dozen tiles, each a serial walk over the
    // whole K: split K over gridDim.z (whole 256-column groups) until the SMs are covered, partial products to
    // scratch, summed in split order by a second launch.
    int splits = 1;
    const int64_t groups = w->cols / 256, tiles = (int64_t)grid.x * grid.y;
    const bool can_sum = ((uintptr_t)y & 15) == 0 && (tokens * w->rows) % 4 == 0;
    if (staged && can_sum && tiles * 2 <= ctx->prop.multiProcessorCount && groups >= 2) {
        int64_t want = ctx->prop.multiProcessorCount / tiles;
        if (want > 8) want = 8;
        if (want > groups) want = groups;
        const int64_t per = (groups + want - 1) / want;          // groups per split
        splits = (int)((groups + per - 1) / per);
        A.ksteps_per_split = (int)(4 * per);
    }
    float* y_final = y;
    if (splits > 1) {
        void* scr;
        LEV_TRY(lev_scratch(ctx, LEV_SCR_GEMM, (size_t)splits * tokens * w->rows * sizeof(float), &scr));
        A.y = (float*)scr;
        grid.z = (unsigned)splits;
    }
    int st = w->type == LEV_GGML_Q6_K ? launch_tc<LEV_GGML_Q6_K, false>(ctx, map, A, grid, smem)
             : w->type == LEV_GGML_Q4_K
                 ? (staged ? launch_tc<LEV_GGML_Q4_K, true>(ctx, map, A, grid, smem_staged) : launch_tc<LEV_GGML_Q4_K, false>(ctx, map, A, grid, smem))
                 : (staged ? launch_tc<LEV_GGML_Q4_0, true>(ctx, map, A, grid, smem_staged) : launch_tc<LEV_GGML_Q4_0, false>(ctx, map, A, grid, smem));
    if (st) return st;
    ctx->launches++;
    LEV_TRY(lev_cuda_check(ctx, cudaGetLastError(), "k_gemm_tc"));
    if (splits > 1) {
        const int64_t n4 = tokens * w->rows / 4;
        int64_t blocks = (n4 + 255) / 256, cap = (int64_t)ctx->prop.multiProcessorCount * 4;
        k_gemm_split_sum<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>((const float4*)A.y, splits, n4, (float4*)y_final);
        ctx->launches++;
        return lev_cuda_check(ctx, cudaGetLastError(), "k_gemm_split_sum");
    }
    return LEV_OK;
}

// ---------------------------------------------------------------------------
// grouped form: host side
// ---------------------------------------------------------------------------
bool lev_gemm_grouped_supported(const lev_weights* w, int rows_per_expert) {
    if (w->type != LEV_GGML_Q4_K && w->type != LEV_GGML_Q4_0 && w->type != LEV_GGML_Q6_K) return false;
    if (w->cols % KS != 0 || rows_per_expert < 1 || !w->raw) return false;
    return encode_tiled() != nullptr;
}

int lev_gemm_grouped_job_tokens(void) { return GR_JOB_TOKENS; }

// xg: bf16 [capacity_rows][w->cols], rows in grouped-position order.
int lev_gemm_grouped_run(lev_ctx* ctx, const lev_weights* w, int rows_per_expert, const void* xg_bf16, int64_t capacity_rows,
                         int max_jobs, const int* njobs, const int* job_slice, const int* job_pos, const int* offsets,
                         int first_expert, const int* out_row, float* out, int64_t out_ld) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return lev_fail(ctx, LEV_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
    if (((uintptr_t)xg_bf16 & 15) != 0) return lev_fail(ctx, LEV_BAD_ARGUMENT, "grouped activations must be 16-byte aligned");
    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)w->cols, (cuuint64_t)capacity_rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)w->cols * 2};
    // the staged Q4_0 kernel takes one box of GR_JOB_TOKENS positions per K-step, the general one a box of 128
    const bool staged = w->type == LEV_GGML_Q4_0;
    const cuuint32_t box[2] = {KS, staged ? (cuuint32_t)GR_JOB_TOKENS : 128u};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(xg_bf16), gdim, gstride, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return lev_fail(ctx, LEV_KERNEL_FAILED, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
    GroupedArgs A;
    A.raw = w->raw;
    A.row_bytes = w->blocks_per_row * lev_block_bytes(w->type);
    A.rows_per_expert = rows_per_expert;
    A.cols = (int)w->cols;
    A.njobs = njobs;
    A.job_slice = job_slice;
    A.job_pos = job_pos;
    A.offsets = offsets;
    A.first_expert = first_expert;
    A.out_row = out_row;
    A.out = out;
    A.out_ld = out_ld;
    A.status = ctx->d_status;
    dim3 grid((unsigned)((rows_per_expert + 127) / 128), (unsigned)max_jobs);
    if (staged) {
        // 16-byte copies need every row of the tensor to start on a 16-byte boundary
        const bool wide = A.row_bytes % 16 == 0 && w->cols % SG_GROUP_COLS == 0 && ((uintptr_t)A.raw & 15) == 0;
        static bool configured_q40[2][16] = {};
        if (!configured_q40[wide][ctx->device & 15]) {
            if (wide) LEV_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc_grouped_q40<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SG_SMEM));
            else LEV_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc_grouped_q40<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SG_SMEM));
            configured_q40[wide][ctx->device & 15] = true;
        }
        // persistent CTAs, two per SM, each taking every gridDim.x-th tile of the device-side job list
        int64_t ctas = 2 * (int64_t)ctx->prop.multiProcessorCount, most = (int64_t)grid.x * max_jobs;
        const dim3 pgrid((unsigned)(ctas < most ? ctas : most));
        if (wide) k_gemm_tc_grouped_q40<16><<<pgrid, GR_THREADS, SG_SMEM, ctx->stream>>>(map, A);
        else k_gemm_tc_grouped_q40<4><<<pgrid, GR_THREADS, SG_SMEM, ctx->stream>>>(map, A);
        ctx->launches++;
        return lev_cuda_check(ctx, cudaGetLastError(), "k_gemm_tc_grouped_q40");
    }
    const size_t smem = (size_t)GR_STAGES * GR_STAGE_BYTES + 1024;
    static bool configured[3][16] = {};
    const int ti = w->type == LEV_GGML_Q4_K ? 0 : (w->type == LEV_GGML_Q6_K ? 1 : 2);
    if (!configured[ti][ctx->device & 15]) {
        if (ti == 0) LEV_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc_grouped<LEV_GGML_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (ti == 1) LEV_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc_grouped<LEV_GGML_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (ti == 2) LEV_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc_grouped<LEV_GGML_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[ti][ctx->device & 15] = true;
    }
    if (ti == 0) k_gemm_tc_grouped<LEV_GGML_Q4_K><<<grid, GR_THREADS, smem, ctx->stream>>>(map, A);
    if (ti == 1) k_gemm_tc_grouped<LEV_GGML_Q6_K><<<grid, GR_THREADS, smem, ctx->stream>>>(map, A);
    if (ti == 2) k_gemm_tc_grouped<LEV_GGML_Q4_0><<<grid, GR_THREADS, smem, ctx->stream>>>(map, A);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_gemm_tc_grouped");
}

int lev_gather_bf16(lev_ctx* ctx, const float* x, const int* perm, const int* total_pos, int64_t max_pos, int top_k, int cols,
                    void* out_bf16) {
    int64_t g = (max_pos * (cols / 4) + 255) / 256, cap = (int64_t)ctx->prop.multiProcessorCount * 8;
    k_gather_bf16<<<(unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), 256, 0, ctx->stream>>>(x, perm, total_pos, top_k, cols,
                                                                                        (__nv_bfloat16*)out_bf16);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_gather_bf16");
}

int lev_act_grouped_bf16(lev_ctx* ctx, const float* gu, const int* total_pos, int64_t max_pos, int inter, void* out_bf16) {
    int64_t g = (max_pos * inter + 255) / 256, cap = (int64_t)ctx->prop.multiProcessorCount * 8;
    k_act_grouped_bf16<<<(unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), 256, 0, ctx->stream>>>(gu, total_pos, inter,
                                                                                              (__nv_bfloat16*)out_bf16);
    ctx->launches++;
    return lev_cuda_check(ctx, cudaGetLastError(), "k_act_grouped_bf16");
}
