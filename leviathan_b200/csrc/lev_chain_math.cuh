// One K-step of the one-column decode matvec in column-group arithmetic, shared by the persistent kernel
// (lev_chain.cu) and the one-launch kernel's single-column form (lev_dense.cu).
//
// The eight columns of an mma.m16n8k16 are four sub-block groups x two activation terms: the B fragments of
// 64-column chunk c are non-zero only in column group c, so one accumulator per lane collects four sub-blocks at
// once and the block scales are applied once per K-step by the lane that owns the sub-block.  Operands are
// shared-memory addresses: the step's packed bytes (see lev_stream.cu for the layout), the fragments of its four
// chunks ([term][quad lane][32 B] per chunk, 1 KB per K-step) and the sums that go with them.
#pragma once
#include "lev_stream_math.cuh"

namespace {

constexpr float kTerm1 = 4.8828125e-4f;  // 2^-11: weight of the second activation term

// Shared-memory loads and the tensor-core product as plain (non-volatile) asm: the compiler may
// interleave them freely inside a K-step.  What orders them against the waits is a data dependency: the
// caller passes every base address through order_after() once the wait that guards the bytes is over.
__device__ __forceinline__ void order_after(unsigned& addr) { asm volatile("" : "+r"(addr)::"memory"); }
__device__ __forceinline__ uint4 lds128(unsigned a) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(unsigned a) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ unsigned lds32(unsigned a) {
    unsigned v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ unsigned lds16(unsigned a) {
    unsigned short v;
    asm("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void mma(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first product of a chain: the accumulator input is the zero register
__device__ __forceinline__ void mma0(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// what a lane needs of itself in every K-step, computed once
struct LaneConst {
    unsigned q_off;      // 16 * lane: this lane's 16 bytes of a chunk's weights
    unsigned hdr_off;    // 16 * g: header / scale row of row g
    unsigned x_off;      // fragments (term, t) inside a chunk's 256 bytes
    unsigned grp;        // the chunk whose fragments this lane supplies (column group g / 2)
    unsigned t, g;
    unsigned sh16;       // 16 * (t & 1)
    unsigned zero_s;     // 32 zero bytes in shared memory
};

// ---------------------------------------------------------------------------
// one K-step, one activation column.  The eight mma columns are (sub-block group s = 0..3) x (term):
// the B fragments of chunk c are non-zero in group c only, so after the K-step lane (g, t) holds, in
// accumulator columns 2t and 2t+1, the two terms of what chunk t contributed to rows g and g + 8.
// st / xk / ak: shared-memory addresses of the step's bytes, of the fragments and of the sums of its
// four chunks.  Lanes outside group c read the zero block instead of chunk c's fragments.
// ---------------------------------------------------------------------------
template <int TYPE>
__device__ __forceinline__ void chain_step(unsigned st, unsigned xk, unsigned ak, const LaneConst& L, float& ya, float& yb) {
    const unsigned t = L.t;
    const unsigned mine = xk + L.x_off;
    if (TYPE == LEV_GGML_Q4_K) {
        const uint4 h0 = lds128(st + L.hdr_off), h1 = lds128(st + 128 + L.hdr_off);
        // four accumulator chains (low / high nibbles x even / odd chunks): chunks write disjoint columns,
        // so the pairs are simply added afterwards
        float lo[4], hi[4], lo2[4], hi2[4];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint4 q = lds128(st + 256 + c * 512 + L.q_off);
            const unsigned xa = L.grp == (unsigned)c ? mine + c * 256 : L.zero_s;
            const uint4 x0 = lds128(xa), x1 = lds128(xa + 16);
            const unsigned w0 = q.x, w1 = q.y, w2 = q.z, w3 = q.w;
            const unsigned w0s = w0 >> 8, w1s = w1 >> 8, w2s = w2 >> 8, w3s = w3 >> 8;
            float* Lo = c & 1 ? lo2 : lo;
            float* Hi = c & 1 ? hi2 : hi;
            if (c < 2) {
                mma0(Lo, w0 & 0x000F000Fu, w2 & 0x000F000Fu, w0s & 0x000F000Fu, w2s & 0x000F000Fu, x0.x, x0.y);
                mma0(Hi, w0 & 0x00F000F0u, w2 & 0x00F000F0u, w0s & 0x00F000F0u, w2s & 0x00F000F0u, x1.x, x1.y);
            } else {
                mma(Lo, w0 & 0x000F000Fu, w2 & 0x000F000Fu, w0s & 0x000F000Fu, w2s & 0x000F000Fu, x0.x, x0.y);
                mma(Hi, w0 & 0x00F000F0u, w2 & 0x00F000F0u, w0s & 0x00F000F0u, w2s & 0x00F000F0u, x1.x, x1.y);
            }
            mma(Lo, w1 & 0x000F000Fu, w3 & 0x000F000Fu, w1s & 0x000F000Fu, w3s & 0x000F000Fu, x0.z, x0.w);
            mma(Hi, w1 & 0x00F000F0u, w3 & 0x00F000F0u, w1s & 0x00F000F0u, w3s & 0x00F000F0u, x1.z, x1.w);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            lo[j] += lo2[j];
            hi[j] += hi2[j];
        }
        // this lane owns sub-blocks 2t (low nibbles of chunk t) and 2t+1 (high nibbles) of its two rows:
        // 6-bit scales and mins (rust/crates/lev-cpu/src/lib.rs:64-74)
        const unsigned sa = t < 2 ? (h0.y & 0x3F3F3F3Fu) : ((h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u));
        const unsigned sb = t < 2 ? (h1.y & 0x3F3F3F3Fu) : ((h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u));
        const unsigned ma = t < 2 ? (h0.z & 0x3F3F3F3Fu) : (((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u));
        const unsigned mb = t < 2 ? (h1.z & 0x3F3F3F3Fu) : (((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u));
        const unsigned sab = sa >> L.sh16, sbb = sb >> L.sh16, mab = ma >> L.sh16, mbb = mb >> L.sh16;
        const float dA = h2f_bits(h0.x & 0xffffu) * 16777216.0f, dB = h2f_bits(h1.x & 0xffffu) * 16777216.0f;  // d * 2^24
        const float dminA = h2f_bits(h0.x >> 16), dminB = h2f_bits(h1.x >> 16);
        const uint2 sxb = lds64(ak + 8 * t);  // activation sums of sub-blocks 2t, 2t+1
        const float sx0 = __uint_as_float(sxb.x), sx1 = __uint_as_float(sxb.y);
        const float pa = fmaf(byte_to_float(sab, 0), fmaf(lo[1], kTerm1, lo[0]), byte_to_float(sab, 1) * fmaf(hi[1], kTerm1, hi[0]));
        const float pb = fmaf(byte_to_float(sbb, 0), fmaf(lo[3], kTerm1, lo[2]), byte_to_float(sbb, 1) * fmaf(hi[3], kTerm1, hi[2]));
        const float qa = fmaf(byte_to_float(mab, 0), sx0, byte_to_float(mab, 1) * sx1);
        const float qb = fmaf(byte_to_float(mbb, 0), sx0, byte_to_float(mbb, 1) * sx1);
        ya = fmaf(dA, pa, fmaf(-dminA, qa, ya));
        yb = fmaf(dB, pb, fmaf(-dminB, qb, yb));
    } else if (TYPE == LEV_GGML_Q6_K) {
        // accumulator m: 16-value sub-block m of every chunk, starting at -32 * 2^-24 * (sum the tensor core sees)
        const uint4 k01 = lds128(ak + 32 * t), k23 = lds128(ak + 32 * t + 16);
        float acc[4][4] = {{__uint_as_float(k01.x), __uint_as_float(k01.y), __uint_as_float(k01.x), __uint_as_float(k01.y)},
                           {__uint_as_float(k01.z), __uint_as_float(k01.w), __uint_as_float(k01.z), __uint_as_float(k01.w)},
                           {__uint_as_float(k23.x), __uint_as_float(k23.y), __uint_as_float(k23.x), __uint_as_float(k23.y)},
                           {__uint_as_float(k23.z), __uint_as_float(k23.w), __uint_as_float(k23.z), __uint_as_float(k23.w)}};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint4 q = lds128(st + 288 + c * 512 + L.q_off);
            const uint2 hq = lds64(st + 2336 + c * 256 + (L.q_off >> 1));
            const unsigned xa = L.grp == (unsigned)c ? mine + c * 256 : L.zero_s;
            const uint4 x0 = lds128(xa), x1 = lds128(xa + 16);
            const unsigned w0 = q.x, w1 = q.y, w2 = q.z, w3 = q.w;
            const unsigned w0s = w0 >> 8, w1s = w1 >> 8, w2s = w2 >> 8, w3s = w3 >> 8;
            const unsigned ha = hq.x, hb = hq.y;
            const unsigned ha_r2 = ha >> 2, ha_l2 = ha << 2, ha_l4 = ha << 4, ha_r4 = ha >> 4, ha_r6 = ha >> 6;
            const unsigned hb_r2 = hb >> 2, hb_l2 = hb << 2, hb_l4 = hb << 4, hb_r4 = hb >> 4, hb_r6 = hb >> 6;
            mma(acc[0], (w0 & 0x000F000Fu) | (ha & 0x00300030u), (w2 & 0x000F000Fu) | (hb & 0x00300030u),
                (w0s & 0x000F000Fu) | (ha_r2 & 0x00300030u), (w2s & 0x000F000Fu) | (hb_r2 & 0x00300030u), x0.x, x0.y);
            mma(acc[1], (w1 & 0x000F000Fu) | (ha_l2 & 0x00300030u), (w3 & 0x000F000Fu) | (hb_l2 & 0x00300030u),
                (w1s & 0x000F000Fu) | (ha_l4 & 0x00300030u), (w3s & 0x000F000Fu) | (hb_l4 & 0x00300030u), x0.z, x0.w);
            mma(acc[2], (w0 & 0x00F000F0u) | (ha & 0x03000300u), (w2 & 0x00F000F0u) | (hb & 0x03000300u),
                (w0s & 0x00F000F0u) | (ha_r2 & 0x03000300u), (w2s & 0x00F000F0u) | (hb_r2 & 0x03000300u), x1.x, x1.y);
            mma(acc[3], (w1 & 0x00F000F0u) | (ha_r4 & 0x03000300u), (w3 & 0x00F000F0u) | (hb_r4 & 0x03000300u),
                (w1s & 0x00F000F0u) | (ha_r6 & 0x03000300u), (w3s & 0x00F000F0u) | (hb_r6 & 0x03000300u), x1.z, x1.w);
        }
        // this lane owns sub-blocks 4t .. 4t+3 (chunk t) of its two rows: int8 scales = word t of the row's 16
        const unsigned scA = lds32(st + L.hdr_off + 4 * t) ^ 0x80808080u;
        const unsigned scB = lds32(st + 128 + L.hdr_off + 4 * t) ^ 0x80808080u;
        const float dA = h2f_bits(lds16(st + 256 + 2 * L.g)) * 16777216.0f, dB = h2f_bits(lds16(st + 272 + 2 * L.g)) * 16777216.0f;
        float pa = 0.f, pb = 0.f;
#pragma unroll
        for (int m = 0; m < 4; m++) {
            // float(byte + 128) - 128 without the conversion unit
            const float sA = __uint_as_float(__byte_perm(scA, 0x4B000000u, 0x7650u + m)) - 8388736.0f;
            const float sB = __uint_as_float(__byte_perm(scB, 0x4B000000u, 0x7650u + m)) - 8388736.0f;
            pa = fmaf(sA, fmaf(acc[m][1], kTerm1, acc[m][0]), pa);
            pb = fmaf(sB, fmaf(acc[m][3], kTerm1, acc[m][2]), pb);
        }
        ya = fmaf(dA, pa, ya);
        yb = fmaf(dB, pb, yb);
    } else {
        // Q4_0: accumulator b = 32-value block b of every chunk, starting at -8 * 2^-24 * (sum seen)
        const uint4 kk = lds128(ak + 16 * t);
        float a0[4] = {__uint_as_float(kk.x), __uint_as_float(kk.y), __uint_as_float(kk.x), __uint_as_float(kk.y)};
        float a1[4] = {__uint_as_float(kk.z), __uint_as_float(kk.w), __uint_as_float(kk.z), __uint_as_float(kk.w)};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint4 q = lds128(st + c * 576 + 64 + L.q_off);
            const unsigned xa = L.grp == (unsigned)c ? mine + c * 256 : L.zero_s;
            const uint4 x0 = lds128(xa), x1 = lds128(xa + 16);
            const unsigned w0 = q.x, w1 = q.y, w2 = q.z, w3 = q.w;
            const unsigned w0s = w0 >> 8, w1s = w1 >> 8, w2s = w2 >> 8, w3s = w3 >> 8;
            mma(a0, w0 & 0x000F000Fu, w2 & 0x000F000Fu, w0s & 0x000F000Fu, w2s & 0x000F000Fu, x0.x, x0.y);
            mma(a1, w1 & 0x000F000Fu, w3 & 0x000F000Fu, w1s & 0x000F000Fu, w3s & 0x000F000Fu, x1.x, x1.y);
            mma(a0, w0 & 0x00F000F0u, w2 & 0x00F000F0u, w0s & 0x00F000F0u, w2s & 0x00F000F0u, x0.z, x0.w);
            mma(a1, w1 & 0x00F000F0u, w3 & 0x00F000F0u, w1s & 0x00F000F0u, w3s & 0x00F000F0u, x1.z, x1.w);
        }
        // this lane owns the two blocks of chunk t: fp16 d of (row g, blk 0 | blk 1), (row g+8, ...)
        const uint2 sc = lds64(st + t * 576 + 8 * L.g);
        const float dA0 = h2f_bits(sc.x & 0xffffu) * 16777216.0f, dA1 = h2f_bits(sc.x >> 16) * 16777216.0f;
        const float dB0 = h2f_bits(sc.y & 0xffffu) * 16777216.0f, dB1 = h2f_bits(sc.y >> 16) * 16777216.0f;
        ya = fmaf(dA0, fmaf(a0[1], kTerm1, a0[0]), fmaf(dA1, fmaf(a1[1], kTerm1, a1[0]), ya));
        yb = fmaf(dB0, fmaf(a0[3], kTerm1, a0[2]), fmaf(dB1, fmaf(a1[3], kTerm1, a1[2]), yb));
    }
}

}  // namespace
