/*
 * CPU oracle for the quantized-weight hot path.  TEST INFRASTRUCTURE ONLY:
 * see lev_oracle.h for what each group follows and how it is pinned.
 *
 * Build with -ffp-contract=off: the reference's f32 loops are a separate
 * multiply and add per term, and a fused multiply-add would change bits.
 */
#include "lev_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#define Q4_0_VALUES 32
#define Q4_0_BYTES 18
#define QK_K 256
#define Q4_K_BYTES 144
#define Q6_K_BYTES 210
#define MAX_DIM (1L << 22) /* Sources/LeviathanCore/Q4.swift:8-15 */

/* ------------------------------------------------------------------ */
/* half / bfloat                                                       */
/* ------------------------------------------------------------------ */

/* rust/crates/lev-cpu/src/lib.rs:14-25 */
double lev_or_f16_to_f64(uint16_t h) {
    double sign = (h & 0x8000) ? -1.0 : 1.0;
    int exp = (h >> 10) & 0x1f;
    double mant = (double)(h & 0x3ff);
    if (exp == 0) return sign * mant * ldexp(1.0, -24);
    if (exp == 31) return mant == 0.0 ? sign * INFINITY : NAN;
    return sign * (1.0 + mant / 1024.0) * ldexp(1.0, exp - 15);
}

/* rust/crates/lev-cpu/src/lib.rs:58-60 (every half is exact in f32) */
float lev_or_f16_to_f32(uint16_t h) { return (float)lev_or_f16_to_f64(h); }

/* rust/crates/lev-cpu/src/lib.rs:28-55: round to nearest even, overflow -> inf */
uint16_t lev_or_f32_to_f16_bits(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
    int exp = (int)((b >> 23) & 0xff);
    uint32_t mant = b & 0x7fffff;
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00 | (mant ? 0x200 : 0));
    int e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00);
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = mant | 0x800000;
        unsigned shift = (unsigned)(14 - e);
        uint16_t half = (uint16_t)(m >> shift);
        uint32_t rem = m & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        unsigned round = (rem > mid || (rem == mid && (half & 1))) ? 1 : 0;
        return (uint16_t)(sign | (uint16_t)(half + round));
    }
    uint32_t half = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fff;
    unsigned round = (rem > 0x1000 || (rem == 0x1000 && (half & 1))) ? 1 : 0;
    return (uint16_t)(sign | (uint16_t)(half + round));
}

uint16_t lev_or_f32_to_bf16_bits(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    if ((b & 0x7f800000u) == 0x7f800000u) { /* inf / nan: keep class */
        uint16_t hi = (uint16_t)(b >> 16);
        if ((b & 0x7fffffu) && !(hi & 0x7f)) hi |= 0x40;
        return hi;
    }
    uint32_t lsb = (b >> 16) & 1u;
    b += 0x7fffu + lsb;
    return (uint16_t)(b >> 16);
}

float lev_or_bf16_to_f32(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float f;
    memcpy(&f, &b, 4);
    return f;
}

/* ------------------------------------------------------------------ */
/* SplitMix64                                                          */
/* ------------------------------------------------------------------ */

/* Sources/LeviathanCore/RNG.swift:11-17 */
uint64_t lev_or_splitmix_next(uint64_t* state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Sources/LeviathanCore/RNG.swift:20-23 */
float lev_or_splitmix_uniform_swift(uint64_t* state) {
    uint64_t u = lev_or_splitmix_next(state) >> 11;
    return (float)((double)u / 9007199254740992.0) * 2.0f - 1.0f;
}

/* rust/crates/lev-cpu/src/lib.rs:369-372 */
float lev_or_splitmix_signed_unit_rust(uint64_t* state) {
    float u = (float)(lev_or_splitmix_next(state) >> 40) / (float)(1ull << 24);
    return u * 2.0f - 1.0f;
}

/* ------------------------------------------------------------------ */
/* shared shape checks                                                 */
/* ------------------------------------------------------------------ */

static int check_geometry(long out_dim, long in_dim, long values_per_block,
                          long bytes_per_block, size_t w_bytes, long x_count) {
    if (in_dim <= 0 || out_dim <= 0 || in_dim % values_per_block != 0 || in_dim > MAX_DIM ||
        out_dim > MAX_DIM)
        return LEV_OR_BAD_DIMENSIONS;
    size_t need = (size_t)out_dim * (size_t)(in_dim / values_per_block) * (size_t)bytes_per_block;
    if (w_bytes != need) return LEV_OR_BAD_DIMENSIONS;
    if (x_count != in_dim) return 2; /* wrong input count */
    return LEV_OR_OK;
}

static int f16_is_nonfinite(uint16_t bits) { return (bits & 0x7C00) == 0x7C00; }

/* ------------------------------------------------------------------ */
/* Q4_0                                                                */
/* ------------------------------------------------------------------ */

/* Sources/LeviathanCore/Q4.swift:43-69 */
int lev_or_q4_0_decode_block(const uint8_t* blk, float* out) {
    uint16_t bits = (uint16_t)(blk[0] | (blk[1] << 8));
    if (f16_is_nonfinite(bits)) return LEV_OR_NONFINITE_SCALE;
    float d = lev_or_f16_to_f32(bits);
    for (int l = 0; l < 16; l++) {
        uint8_t byte = blk[2 + l];
        out[l] = d * ((float)(byte & 0xF) - 8.0f);
        out[16 + l] = d * ((float)(byte >> 4) - 8.0f);
    }
    return LEV_OR_OK;
}

/* Sources/LeviathanCore/Q4.swift:73-113: per block an f32 partial over the
 * 32 decoded values in element order, then the row sum adds the partial. */
int lev_or_q4_0_matvec_f32(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, float* y) {
    int st = check_geometry(out_dim, in_dim, Q4_0_VALUES, Q4_0_BYTES, w_bytes, x_count);
    if (st) return st;
    long bpr = in_dim / Q4_0_VALUES;
    float v[32];
    for (long row = 0; row < out_dim; row++) {
        float sum = 0.0f;
        for (long b = 0; b < bpr; b++) {
            const uint8_t* blk = w + ((size_t)row * bpr + b) * Q4_0_BYTES;
            st = lev_or_q4_0_decode_block(blk, v);
            if (st) return st;
            float s = 0.0f;
            for (int j = 0; j < 32; j++) {
                float xi = x[b * 32 + j];
                if (!isfinite(xi)) return LEV_OR_NONFINITE_INPUT;
                s += v[j] * xi;
            }
            sum += s;
        }
        if (!isfinite(sum)) return LEV_OR_NONFINITE_OUTPUT;
        y[row] = sum;
    }
    return LEV_OR_OK;
}

/* Sources/LeviathanCore/Q4Lowering.swift:676-711 */
int lev_or_q4_0_matvec_f64(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, double* y) {
    if (in_dim <= 0 || out_dim <= 0 || in_dim % Q4_0_VALUES != 0) return LEV_OR_BAD_DIMENSIONS;
    long bpr = in_dim / Q4_0_VALUES;
    if (w_bytes != (size_t)out_dim * bpr * Q4_0_BYTES || x_count != in_dim)
        return LEV_OR_BAD_DIMENSIONS;
    for (long i = 0; i < in_dim; i++)
        if (!isfinite(x[i])) return LEV_OR_NONFINITE_INPUT;
    for (long row = 0; row < out_dim; row++) {
        double sum = 0.0;
        for (long b = 0; b < bpr; b++) {
            const uint8_t* blk = w + ((size_t)row * bpr + b) * Q4_0_BYTES;
            uint16_t bits = (uint16_t)(blk[0] | (blk[1] << 8));
            if (f16_is_nonfinite(bits)) return LEV_OR_NONFINITE_SCALE;
            double d = lev_or_f16_to_f64(bits);
            for (int l = 0; l < 16; l++) {
                uint8_t q = blk[2 + l];
                sum += d * ((double)(q & 0xF) - 8.0) * (double)x[b * 32 + l];
                sum += d * ((double)(q >> 4) - 8.0) * (double)x[b * 32 + 16 + l];
            }
        }
        if (!isfinite(sum)) return LEV_OR_NONFINITE_OUTPUT;
        y[row] = sum;
    }
    return LEV_OR_OK;
}

/* Sources/LeviathanCore/Gemma4.swift:3931-3953: one running f32 sum, low
 * nibble term then high nibble term per byte, no per-block partial. */
int lev_or_q4_0_matvec_f32_interleaved(const uint8_t* w, size_t w_bytes, long out_dim,
                                       long in_dim, const float* x, long x_count, float* y) {
    int st = check_geometry(out_dim, in_dim, Q4_0_VALUES, Q4_0_BYTES, w_bytes, x_count);
    if (st) return st;
    long bpr = in_dim / Q4_0_VALUES;
    for (long row = 0; row < out_dim; row++) {
        float sum = 0.0f;
        for (long b = 0; b < bpr; b++) {
            const uint8_t* blk = w + ((size_t)row * bpr + b) * Q4_0_BYTES;
            float d = lev_or_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int l = 0; l < 16; l++) {
                uint8_t q = blk[2 + l];
                sum += d * ((float)(q & 0x0F) - 8.0f) * x[b * 32 + l];
                sum += d * ((float)(q >> 4) - 8.0f) * x[b * 32 + 16 + l];
            }
        }
        y[row] = sum;
    }
    return LEV_OR_OK;
}

/* Sources/LeviathanCore/MoESIMDLowering.swift:934-977 */
int lev_or_q4_0_matvec_f64_dx(const uint8_t* w, size_t w_bytes, size_t byte_offset,
                              long out_dim, long in_dim, const double* x, long x_count,
                              double* y) {
    if (out_dim <= 0 || in_dim <= 0 || in_dim % 32 != 0 || x_count != in_dim)
        return LEV_OR_BAD_DIMENSIONS;
    for (long i = 0; i < in_dim; i++)
        if (!isfinite(x[i])) return LEV_OR_NONFINITE_INPUT;
    long bpr = in_dim / 32;
    size_t row_bytes = (size_t)bpr * 18;
    size_t needed = (size_t)out_dim * row_bytes;
    if (byte_offset + needed > w_bytes) return LEV_OR_BAD_DIMENSIONS;
    for (long row = 0; row < out_dim; row++) {
        size_t row_base = byte_offset + (size_t)row * row_bytes;
        double sum = 0.0;
        for (long b = 0; b < bpr; b++) {
            size_t o = row_base + (size_t)b * 18;
            uint16_t bits = (uint16_t)(w[o] | (w[o + 1] << 8));
            if (f16_is_nonfinite(bits)) return LEV_OR_NONFINITE_SCALE;
            double d = lev_or_f16_to_f64(bits);
            long xb = b * 32;
            for (int l = 0; l < 16; l++) {
                uint8_t q = w[o + 2 + l];
                sum += d * (double)((int)(q & 0x0F) - 8) * x[xb + l];
                sum += d * (double)((int)(q >> 4) - 8) * x[xb + 16 + l];
            }
        }
        if (!isfinite(sum)) return LEV_OR_NONFINITE_OUTPUT;
        y[row] = sum;
    }
    return LEV_OR_OK;
}

/* ------------------------------------------------------------------ */
/* Q4_K                                                                */
/* ------------------------------------------------------------------ */

/* rust/crates/lev-cpu/src/lib.rs:64-74 */
void lev_or_q4_k_unpack_scale_min(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* rust/crates/lev-cpu/src/lib.rs:380-395 (the encoder side used by the
 * reference's own round-trip test) */
void lev_or_q4_k_pack_scale_min(const uint8_t* sc, const uint8_t* mn, uint8_t* s) {
    memset(s, 0, 12);
    for (int j = 0; j < 8; j++) {
        uint8_t ls = sc[j], lm = mn[j];
        if (j < 4) {
            s[j] |= ls;
            s[j + 4] |= lm;
        } else {
            s[j + 4] = (uint8_t)((ls & 0x0F) | ((lm & 0x0F) << 4));
            s[j - 4] |= (uint8_t)((ls >> 4) << 6);
            s[j] |= (uint8_t)((lm >> 4) << 6);
        }
    }
}

/* rust/crates/lev-cpu/src/lib.rs:110-130 */
void lev_or_q4_k_dequant_block_f32(const uint8_t* block, float* out) {
    float d = lev_or_f16_to_f32((uint16_t)(block[0] | (block[1] << 8)));
    float dmin = lev_or_f16_to_f32((uint16_t)(block[2] | (block[3] << 8)));
    const uint8_t* scales = block + 4;
    const uint8_t* qs = block + 16;
    int is = 0;
    for (int chunk = 0; chunk < 4; chunk++) {
        const uint8_t* q = qs + chunk * 32;
        uint8_t sc1, m1, sc2, m2;
        lev_or_q4_k_unpack_scale_min(is, scales, &sc1, &m1);
        lev_or_q4_k_unpack_scale_min(is + 1, scales, &sc2, &m2);
        float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
        float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
        int o = chunk * 64;
        for (int l = 0; l < 32; l++) {
            out[o + l] = d1 * (float)(q[l] & 0x0F) - mm1;
            out[o + 32 + l] = d2 * (float)(q[l] >> 4) - mm2;
        }
        is += 2;
    }
}

/* rust/crates/lev-cpu/src/lib.rs:133-154 */
void lev_or_q4_k_dequant_block_f64(const uint8_t* block, double* out) {
    double d = lev_or_f16_to_f64((uint16_t)(block[0] | (block[1] << 8)));
    double dmin = lev_or_f16_to_f64((uint16_t)(block[2] | (block[3] << 8)));
    const uint8_t* scales = block + 4;
    const uint8_t* qs = block + 16;
    int is = 0;
    for (int chunk = 0; chunk < 4; chunk++) {
        const uint8_t* q = qs + chunk * 32;
        uint8_t sc1, m1, sc2, m2;
        lev_or_q4_k_unpack_scale_min(is, scales, &sc1, &m1);
        lev_or_q4_k_unpack_scale_min(is + 1, scales, &sc2, &m2);
        double d1 = d * (double)sc1, mm1 = dmin * (double)m1;
        double d2 = d * (double)sc2, mm2 = dmin * (double)m2;
        int o = chunk * 64;
        for (int l = 0; l < 32; l++) {
            out[o + l] = d1 * (double)(q[l] & 0x0F) - mm1;
            out[o + 32 + l] = d2 * (double)(q[l] >> 4) - mm2;
        }
        is += 2;
    }
}

/* rust/crates/lev-cpu/src/lib.rs:95-108: 1 cols, 2 weight bytes, 3 input length */
static int check_shape_k(size_t w_bytes, long rows, long cols, long x_len, long block_bytes) {
    if (cols <= 0 || cols % QK_K != 0) return LEV_OR_BAD_DIMENSIONS;
    size_t row_bytes = (size_t)(cols / QK_K) * (size_t)block_bytes;
    if (rows < 0 || w_bytes != (size_t)rows * row_bytes) return LEV_OR_BAD_DIMENSIONS;
    if (x_len != cols) return 2;
    return LEV_OR_OK;
}

/* rust/crates/lev-cpu/src/lib.rs:158-175 */
int lev_or_q4_k_matvec_f32(const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, long x_count, float* y) {
    int st = check_shape_k(w_bytes, rows, cols, x_count, Q4_K_BYTES);
    if (st) return st;
    long bpr = cols / QK_K;
    float tmp[QK_K];
    for (long r = 0; r < rows; r++) {
        float sum = 0.0f;
        for (long b = 0; b < bpr; b++) {
            lev_or_q4_k_dequant_block_f32(w + ((size_t)r * bpr + b) * Q4_K_BYTES, tmp);
            const float* xs = x + b * QK_K;
            for (int i = 0; i < QK_K; i++) sum += tmp[i] * xs[i];
        }
        y[r] = sum;
    }
    return LEV_OR_OK;
}

/* rust/crates/lev-cpu/src/lib.rs:178-195 */
int lev_or_q4_k_matvec_f64(const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, long x_count, double* y) {
    int st = check_shape_k(w_bytes, rows, cols, x_count, Q4_K_BYTES);
    if (st) return st;
    long bpr = cols / QK_K;
    double tmp[QK_K];
    for (long r = 0; r < rows; r++) {
        double sum = 0.0;
        for (long b = 0; b < bpr; b++) {
            lev_or_q4_k_dequant_block_f64(w + ((size_t)r * bpr + b) * Q4_K_BYTES, tmp);
            const float* xs = x + b * QK_K;
            for (int i = 0; i < QK_K; i++) sum += tmp[i] * (double)xs[i];
        }
        y[r] = sum;
    }
    return LEV_OR_OK;
}

/* ------------------------------------------------------------------ */
/* Q6_K                                                                */
/* ------------------------------------------------------------------ */

/* Sources/LeviathanCore/Q6.swift:24-62 */
int lev_or_q6_k_decode_block(const uint8_t* u8, float* out) {
    uint16_t dbits = (uint16_t)(u8[208] | (u8[209] << 8));
    if (f16_is_nonfinite(dbits)) return LEV_OR_NONFINITE_SCALE;
    float d = lev_or_f16_to_f32(dbits);
    int scales[16];
    for (int i = 0; i < 16; i++) scales[i] = (int)(int8_t)u8[192 + i];
    for (int c = 0; c < 2; c++) {
        int ql = c * 64, qh = 128 + c * 32, sc = c * 8, base = c * 128;
        for (int l = 0; l < 32; l++) {
            int isub = l / 16;
            uint8_t b = u8[qh + l];
            int l0 = ((int)(u8[ql + l] & 0xF) | ((int)((b >> 0) & 3) << 4)) - 32;
            int l1 = ((int)(u8[ql + 32 + l] & 0xF) | ((int)((b >> 2) & 3) << 4)) - 32;
            int l2 = ((int)(u8[ql + l] >> 4) | ((int)((b >> 4) & 3) << 4)) - 32;
            int l3 = ((int)(u8[ql + 32 + l] >> 4) | ((int)((b >> 6) & 3) << 4)) - 32;
            out[base + l] = d * (float)scales[sc + isub + 0] * (float)l0;
            out[base + 32 + l] = d * (float)scales[sc + isub + 2] * (float)l1;
            out[base + 64 + l] = d * (float)scales[sc + isub + 4] * (float)l2;
            out[base + 96 + l] = d * (float)scales[sc + isub + 6] * (float)l3;
        }
    }
    return LEV_OR_OK;
}

/* rust/crates/lev-cpu/src/lib.rs:203-215 */
void lev_or_q6_k_unpack(const uint8_t* block, int8_t* q) {
    const uint8_t* ql0 = block;
    const uint8_t* qh0 = block + 128;
    for (int half = 0; half < 2; half++) {
        const uint8_t* ql = ql0 + half * 64;
        const uint8_t* qh = qh0 + half * 32;
        for (int l = 0; l < 32; l++) {
            uint8_t h = qh[l];
            q[half * 128 + l] = (int8_t)((int)((ql[l] & 0x0F) | ((h & 3) << 4)) - 32);
            q[half * 128 + l + 32] = (int8_t)((int)((ql[l + 32] & 0x0F) | (((h >> 2) & 3) << 4)) - 32);
            q[half * 128 + l + 64] = (int8_t)((int)((ql[l] >> 4) | (((h >> 4) & 3) << 4)) - 32);
            q[half * 128 + l + 96] = (int8_t)((int)((ql[l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32);
        }
    }
}

/* rust/crates/lev-cpu/src/lib.rs:225-233 */
void lev_or_q6_k_dequant_block_f32(const uint8_t* block, float* out) {
    int8_t q[QK_K];
    lev_or_q6_k_unpack(block, q);
    float d = (float)lev_or_f16_to_f64((uint16_t)(block[208] | (block[209] << 8)));
    for (int e = 0; e < QK_K; e++) out[e] = d * (float)(int8_t)block[192 + e / 16] * (float)q[e];
}

/* rust/crates/lev-cpu/src/lib.rs:235-242 */
void lev_or_q6_k_dequant_block_f64(const uint8_t* block, double* out) {
    int8_t q[QK_K];
    lev_or_q6_k_unpack(block, q);
    double d = lev_or_f16_to_f64((uint16_t)(block[208] | (block[209] << 8)));
    for (int e = 0; e < QK_K; e++) out[e] = d * (double)(int8_t)block[192 + e / 16] * (double)q[e];
}

/* Sources/LeviathanCore/Q6.swift:65-108: Double accumulation, Float at the end */
int lev_or_q6_k_matvec_ref(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, float* y) {
    int st = check_geometry(out_dim, in_dim, QK_K, Q6_K_BYTES, w_bytes, x_count);
    if (st) return st;
    long bpr = in_dim / QK_K;
    float v[QK_K];
    for (long row = 0; row < out_dim; row++) {
        double sum = 0.0;
        for (long b = 0; b < bpr; b++) {
            st = lev_or_q6_k_decode_block(w + ((size_t)row * bpr + b) * Q6_K_BYTES, v);
            if (st) return st;
            for (int j = 0; j < QK_K; j++) {
                float xi = x[b * QK_K + j];
                if (!isfinite(xi)) return LEV_OR_NONFINITE_INPUT;
                sum += (double)v[j] * (double)xi;
            }
        }
        float f = (float)sum;
        if (!isfinite(f)) return LEV_OR_NONFINITE_OUTPUT;
        y[row] = f;
    }
    return LEV_OR_OK;
}

/* Sources/LeviathanCore/Q6.swift:113-145 */
int lev_or_q6_k_matvec_f64(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, double* y) {
    int st = check_geometry(out_dim, in_dim, QK_K, Q6_K_BYTES, w_bytes, x_count);
    if (st) return st;
    for (long i = 0; i < in_dim; i++)
        if (!isfinite(x[i])) return LEV_OR_NONFINITE_INPUT;
    long bpr = in_dim / QK_K;
    float v[QK_K];
    for (long row = 0; row < out_dim; row++) {
        double sum = 0.0;
        for (long b = 0; b < bpr; b++) {
            st = lev_or_q6_k_decode_block(w + ((size_t)row * bpr + b) * Q6_K_BYTES, v);
            if (st) return st;
            for (int j = 0; j < QK_K; j++) sum += (double)v[j] * (double)x[b * QK_K + j];
        }
        if (!isfinite(sum)) return LEV_OR_NONFINITE_OUTPUT;
        y[row] = sum;
    }
    return LEV_OR_OK;
}

/* rust/crates/lev-cpu/src/lib.rs:261-276 */
int lev_or_q6_k_matvec_f32(const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, long x_count, float* y) {
    int st = check_shape_k(w_bytes, rows, cols, x_count, Q6_K_BYTES);
    if (st) return st;
    long bpr = cols / QK_K;
    float tmp[QK_K];
    for (long r = 0; r < rows; r++) {
        float sum = 0.0f;
        for (long b = 0; b < bpr; b++) {
            lev_or_q6_k_dequant_block_f32(w + ((size_t)r * bpr + b) * Q6_K_BYTES, tmp);
            for (int i = 0; i < QK_K; i++) sum += tmp[i] * x[b * QK_K + i];
        }
        y[r] = sum;
    }
    return LEV_OR_OK;
}

/* ------------------------------------------------------------------ */
/* error metric, q8 activations                                        */
/* ------------------------------------------------------------------ */

/* rust/crates/lev-cpu/src/lib.rs:341-353;
 * Sources/LeviathanCore/MoESIMDLowering.swift:1034-1043 */
double lev_or_max_rel_err(const float* got, long n_got, const double* ref, long n_ref) {
    if (n_got != n_ref || n_got <= 0) return INFINITY;
    double worst = 0.0;
    for (long i = 0; i < n_got; i++) {
        double g = (double)got[i];
        if (!isfinite(g) || !isfinite(ref[i])) return INFINITY;
        double den = fabs(ref[i]) > 1.0 ? fabs(ref[i]) : 1.0;
        double e = fabs(g - ref[i]) / den;
        if (e > worst) worst = e;
    }
    return worst;
}

/* rust/crates/lev-cpu/src/lib.rs:306-322 */
void lev_or_quantize_q8(const float* x, long n, int8_t* q, float* d, float* s) {
    for (long g = 0; g < n / 32; g++) {
        const float* xs = x + g * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xs[i]));
        float dd = amax > 0.0f ? amax / 127.0f : 0.0f;
        float id = amax > 0.0f ? 127.0f / amax : 0.0f;
        int sum = 0;
        for (int i = 0; i < 32; i++) {
            int qi = (int)nearbyintf(xs[i] * id); /* ties to even in the default mode */
            sum += qi;
            q[g * 32 + i] = (int8_t)qi;
        }
        d[g] = dd;
        s[g] = dd * (float)sum;
    }
}

/* ------------------------------------------------------------------ */
/* RMSNorm                                                             */
/* ------------------------------------------------------------------ */

/* g4_rmsnorm, Sources/LeviathanCore/Gemma4.swift:4247-4268: one serial f32 sum in index order,
 * inv = 1 / sqrt(ms / n + eps), y = x * inv * w (w NULL: no scale) */
void lev_or_rmsnorm_f32(const float* x, long n, long vectors, const float* w, float eps, float* y) {
    for (long v = 0; v < vectors; v++) {
        const float* xv = x + v * n;
        float ms = 0.0f;
        for (long i = 0; i < n; i++) ms += xv[i] * xv[i];
        ms = ms / (float)n + eps;
        float inv = 1.0f / sqrtf(ms);
        for (long i = 0; i < n; i++) y[v * n + i] = xv[i] * inv * (w ? w[i] : 1.0f);
    }
}

/* the f64 statistic of rust/crates/lev-model/src/lib.rs:110-114, kept in f64 to the end */
void lev_or_rmsnorm_f64(const float* x, long n, long vectors, const float* w, float eps, double* y) {
    for (long v = 0; v < vectors; v++) {
        const float* xv = x + v * n;
        double ms = 0.0;
        for (long i = 0; i < n; i++) ms += (double)xv[i] * (double)xv[i];
        double inv = 1.0 / sqrt(ms / (double)n + (double)eps);
        for (long i = 0; i < n; i++) y[v * n + i] = (double)xv[i] * inv * (w ? (double)w[i] : 1.0);
    }
}

/* per-head RMSNorm then rotary, in f64: g4_rmsnorm over each head (Gemma4.swift:4247-4268) followed by
 * g4_rope (Gemma4.swift:4390-4410): pairs (i, i + hd/2) turned by inv_freq[i] * pos.  w NULL: no scale;
 * inv_freq NULL: no rotary.  x, out [heads][hd]. */
void lev_or_head_norm_rope_f64(const float* x, long heads, long hd, const float* w, float eps, const float* inv_freq, long pos,
                               double* out) {
    long half = hd / 2;
    for (long h = 0; h < heads; h++) {
        const float* xv = x + h * hd;
        double ms = 0.0;
        for (long i = 0; i < hd; i++) ms += (double)xv[i] * (double)xv[i];
        double inv = 1.0 / sqrt(ms / (double)hd + (double)eps);
        double* o = out + h * hd;
        for (long i = 0; i < hd; i++) o[i] = (double)xv[i] * inv * (w ? (double)w[i] : 1.0);
        if (!inv_freq) continue;
        for (long i = 0; i < half; i++) {
            /* the kernel forms the angle in f32 (inv[i] * float(pos)); so does the oracle, then f64 */
            float f = inv_freq[i] * (float)pos;
            double cs = cos((double)f), sn = sin((double)f);
            double a = o[i], b = o[i + half];
            o[i] = a * cs - b * sn;
            o[i + half] = a * sn + b * cs;
        }
    }
}

/* ------------------------------------------------------------------ */
/* Decode attention                                                    */
/* ------------------------------------------------------------------ */

/* fp64Attention, Sources/LeviathanCore/AttentionLowering.swift:358-388, with the score scale of
 * attn_decode_paged (rust/crates/lev-forge/src/ops.rs:1072) as a parameter (1.0 in the Swift model).
 * q [q_heads][hd]; k, v [tokens][kv_heads][hd]; the query sits at position tokens - 1. */
int lev_or_attention_f64(const float* q, const float* k, const float* v, long q_heads, long kv_heads, long hd, long tokens,
                         long window, double scale, double* out) {
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || hd <= 0 || tokens <= 0 || window < 0) return 1;
    long qpos = tokens - 1;
    long lo = (window != 0 && qpos + 1 > window) ? qpos + 1 - window : 0;
    long group = q_heads / kv_heads;
    double* s = (double*)malloc((size_t)tokens * sizeof(double));
    if (!s) return 2;
    for (long h = 0; h < q_heads; h++) {
        long kvh = h / group;
        double m = -INFINITY;
        for (long t = lo; t <= qpos; t++) {
            const float* kt = k + (t * kv_heads + kvh) * hd;
            double d = 0.0;
            for (long i = 0; i < hd; i++) d += (double)q[h * hd + i] * (double)kt[i];
            s[t] = d * scale;
            if (s[t] > m) m = s[t];
        }
        double l = 0.0;
        for (long t = lo; t <= qpos; t++) {
            s[t] = exp(s[t] - m);
            l += s[t];
        }
        for (long i = 0; i < hd; i++) out[h * hd + i] = 0.0;
        for (long t = lo; t <= qpos; t++) {
            double w = s[t] / l;
            const float* vt = v + (t * kv_heads + kvh) * hd;
            for (long i = 0; i < hd; i++) out[h * hd + i] += w * (double)vt[i];
        }
    }
    free(s);
    return 0;
}

/* ------------------------------------------------------------------ */
/* MoE region                                                          */
/* ------------------------------------------------------------------ */

/* Sources/LeviathanCore/MoESIMDLowering.swift:981-984 */
double lev_or_gelu_tanh_up(double g, double u) {
    double inner = 0.7978845608028654 * (g + 0.044715 * g * g * g);
    return 0.5 * g * (1.0 + tanh(inner)) * u;
}

/* Sources/LeviathanCore/Gemma4.swift:4364-4377 */
float lev_or_gelu_tanh_up_f32(float g, float u) {
    float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    float e = expf(-2.0f * fabsf(inner));
    float t = copysignf((1.0f - e) / (1.0f + e), inner);
    float gelu = 0.5f * g * (1.0f + t);
    return gelu * u;
}

/* Sources/LeviathanCore/MoESIMDLowering.swift:989-1030 */
int lev_or_moe_region_f64(long hidden, long inter, long top_k, const uint8_t* gu,
                          size_t gu_bytes, const uint8_t* dn, size_t dn_bytes, const float* x,
                          double* gate, double* up, double* act, double* dn_out) {
    if (hidden <= 0 || inter <= 0 || top_k <= 0 || hidden % 32 || inter % 32)
        return LEV_OR_BAD_DIMENSIONS;
    for (long i = 0; i < hidden; i++)
        if (!isfinite(x[i])) return LEV_OR_NONFINITE_INPUT;
    long gu_rows = 2 * inter;
    size_t gu_stride = (size_t)gu_rows * (size_t)(hidden / 32) * 18;
    size_t dn_stride = (size_t)hidden * (size_t)(inter / 32) * 18;
    if (gu_bytes != gu_stride * (size_t)top_k || dn_bytes != dn_stride * (size_t)top_k)
        return LEV_OR_BAD_DIMENSIONS;
    double* xd = (double*)malloc(sizeof(double) * (size_t)hidden);
    double* guv = (double*)malloc(sizeof(double) * (size_t)gu_rows);
    double* a = (double*)malloc(sizeof(double) * (size_t)inter);
    double* d = (double*)malloc(sizeof(double) * (size_t)hidden);
    int st = LEV_OR_OK;
    for (long i = 0; i < hidden; i++) xd[i] = (double)x[i];
    for (long slot = 0; slot < top_k && !st; slot++) {
        st = lev_or_q4_0_matvec_f64_dx(gu, gu_bytes, (size_t)slot * gu_stride, gu_rows, hidden,
                                       xd, hidden, guv);
        if (st) break;
        for (long i = 0; i < inter; i++) {
            a[i] = lev_or_gelu_tanh_up(guv[i], guv[inter + i]);
            if (!isfinite(a[i])) {
                st = LEV_OR_NONFINITE_OUTPUT;
                break;
            }
        }
        if (st) break;
        st = lev_or_q4_0_matvec_f64_dx(dn, dn_bytes, (size_t)slot * dn_stride, hidden, inter, a,
                                       inter, d);
        if (st) break;
        if (gate) memcpy(gate + slot * inter, guv, sizeof(double) * (size_t)inter);
        if (up) memcpy(up + slot * inter, guv + inter, sizeof(double) * (size_t)inter);
        if (act) memcpy(act + slot * inter, a, sizeof(double) * (size_t)inter);
        if (dn_out) memcpy(dn_out + slot * hidden, d, sizeof(double) * (size_t)hidden);
    }
    free(xd);
    free(guv);
    free(a);
    free(d);
    return st;
}

/* ------------------------------------------------------------------ */
/* router                                                              */
/* ------------------------------------------------------------------ */

/* Logits of Sources/LeviathanCore/Gemma4.swift:4160-4172 (an f32 GPU kernel
 * with no CPU statement) in the summation order fixed in lev_oracle.h. */
void lev_or_router_logits(const float* router_w, long experts, long hidden, const float* x,
                          float* scores) {
    for (long e = 0; e < experts; e++) {
        const float* w = router_w + (size_t)e * (size_t)hidden;
        double p[32];
        for (int l = 0; l < 32; l++) {
            double acc = 0.0;
            for (long i = l; i < hidden; i += 32) acc = fma((double)w[i], (double)x[i], acc);
            p[l] = acc;
        }
        for (int dist = 16; dist >= 1; dist >>= 1) {
            double q[32];
            for (int l = 0; l < 32; l++) q[l] = p[l] + p[l ^ dist];
            memcpy(p, q, sizeof p);
        }
        scores[e] = (float)p[0];
    }
}

/* Sources/LeviathanCore/Gemma4.swift:3797-3810 */
int lev_or_router_topk(const float* scores, long experts, long top_k,
                       const float* expert_scale, int32_t* idx_out, float* weights) {
    if (experts <= 0 || top_k <= 0 || top_k > experts) return LEV_OR_BAD_DIMENSIONS;
    for (long i = 0; i < experts; i++)
        if (!isfinite(scores[i])) return LEV_OR_NONFINITE_INPUT;
    float max_score = scores[0];
    for (long i = 1; i < experts; i++)
        if (scores[i] > max_score) max_score = scores[i];
    double* probs = (double*)malloc(sizeof(double) * (size_t)experts);
    int32_t* idx = (int32_t*)malloc(sizeof(int32_t) * (size_t)experts);
    double sum_exp = 0.0;
    for (long i = 0; i < experts; i++) {
        probs[i] = exp((double)(scores[i] - max_score)); /* f32 subtraction first */
        sum_exp += probs[i];
    }
    for (long i = 0; i < experts; i++) {
        probs[i] /= sum_exp;
        idx[i] = (int32_t)i;
    }
    /* stable insertion sort: probability descending, ties to the lower index */
    for (long i = 1; i < experts; i++) {
        int32_t k = idx[i];
        long j = i - 1;
        while (j >= 0 && (probs[idx[j]] < probs[k])) {
            idx[j + 1] = idx[j];
            j--;
        }
        idx[j + 1] = k;
    }
    double prob_sum = 0.0;
    for (long k = 0; k < top_k; k++) prob_sum += probs[idx[k]];
    for (long k = 0; k < top_k; k++) {
        idx_out[k] = idx[k];
        float sc = expert_scale ? expert_scale[idx[k]] : 1.0f;
        weights[k] = (float)(probs[idx[k]] / prob_sum) * sc;
    }
    free(probs);
    free(idx);
    return LEV_OR_OK;
}

/* ------------------------------------------------------------------ */
/* grouping and combine                                                */
/* ------------------------------------------------------------------ */

void lev_or_group_tokens(const int32_t* idx, long tokens, long top_k, long experts,
                         int32_t* counts, int32_t* offsets, int32_t* perm) {
    long n = tokens * top_k;
    for (long e = 0; e < experts; e++) counts[e] = 0;
    for (long i = 0; i < n; i++) counts[idx[i]]++;
    offsets[0] = 0;
    for (long e = 0; e < experts; e++) offsets[e + 1] = offsets[e] + counts[e];
    int32_t* cursor = (int32_t*)malloc(sizeof(int32_t) * (size_t)experts);
    for (long e = 0; e < experts; e++) cursor[e] = offsets[e];
    /* pair id = token*top_k + rank, visited ascending: stable by (token, rank) */
    for (long i = 0; i < n; i++) perm[cursor[idx[i]]++] = (int32_t)i;
    free(cursor);
}

/* Sources/LeviathanCore/Gemma4.swift:4459-4466, one call per slot in rank
 * order starting from a zeroed accumulator (:3841, :3878) */
void lev_or_combine(const float* y_slots, const float* weights, long top_k, long hidden,
                    float* out) {
    for (long i = 0; i < hidden; i++) out[i] = 0.0f;
    for (long k = 0; k < top_k; k++) {
        float c = weights[k];
        const float* ys = y_slots + k * hidden;
        for (long i = 0; i < hidden; i++) out[i] += c * ys[i];
    }
}

int lev_or_moe_token(long hidden, long inter, long experts, long top_k, const float* router_w,
                     const uint8_t* gu_all, const uint8_t* dn_all, const float* x,
                     int32_t* idx, float* weights, float* out, double* out_f64) {
    float* scores = (float*)malloc(sizeof(float) * (size_t)experts);
    lev_or_router_logits(router_w, experts, hidden, x, scores);
    int st = lev_or_router_topk(scores, experts, top_k, NULL, idx, weights);
    free(scores);
    if (st) return st;
    size_t gu_stride = (size_t)(2 * inter) * (size_t)(hidden / 32) * 18;
    size_t dn_stride = (size_t)hidden * (size_t)(inter / 32) * 18;
    uint8_t* gu = (uint8_t*)malloc(gu_stride * (size_t)top_k);
    uint8_t* dn = (uint8_t*)malloc(dn_stride * (size_t)top_k);
    for (long k = 0; k < top_k; k++) {
        memcpy(gu + (size_t)k * gu_stride, gu_all + (size_t)idx[k] * gu_stride, gu_stride);
        memcpy(dn + (size_t)k * dn_stride, dn_all + (size_t)idx[k] * dn_stride, dn_stride);
    }
    double* y64 = (double*)malloc(sizeof(double) * (size_t)(top_k * hidden));
    st = lev_or_moe_region_f64(hidden, inter, top_k, gu, gu_stride * (size_t)top_k, dn,
                               dn_stride * (size_t)top_k, x, NULL, NULL, NULL, y64);
    if (!st) {
        float* y32 = (float*)malloc(sizeof(float) * (size_t)(top_k * hidden));
        for (long i = 0; i < top_k * hidden; i++) y32[i] = (float)y64[i];
        lev_or_combine(y32, weights, top_k, hidden, out);
        free(y32);
        if (out_f64) {
            for (long i = 0; i < hidden; i++) {
                double acc = 0.0;
                for (long k = 0; k < top_k; k++) acc += (double)weights[k] * y64[k * hidden + i];
                out_f64[i] = acc;
            }
        }
    }
    free(gu);
    free(dn);
    free(y64);
    return st;
}

/* ------------------------------------------------------------------ */
/* dequantize rows, prefill GEMM oracle                                */
/* ------------------------------------------------------------------ */

static long block_values(int t) { return t == 2 ? 32 : QK_K; }
static long block_bytes(int t) { return t == 2 ? Q4_0_BYTES : (t == 12 ? Q4_K_BYTES : Q6_K_BYTES); }

static int dequant_block_any(int t, const uint8_t* blk, float* out) {
    if (t == 2) return lev_or_q4_0_decode_block(blk, out);
    if (t == 12) {
        lev_or_q4_k_dequant_block_f32(blk, out);
        return LEV_OR_OK;
    }
    if (t == 14) return lev_or_q6_k_decode_block(blk, out);
    return LEV_OR_BAD_DIMENSIONS;
}

int lev_or_dequantize_rows(int t, const uint8_t* w, long rows, long cols, float* out) {
    if (t != 2 && t != 12 && t != 14) return LEV_OR_BAD_DIMENSIONS;
    long bv = block_values(t), bb = block_bytes(t);
    if (cols <= 0 || cols % bv) return LEV_OR_BAD_DIMENSIONS;
    long bpr = cols / bv;
    for (long r = 0; r < rows; r++)
        for (long b = 0; b < bpr; b++) {
            int st = dequant_block_any(t, w + ((size_t)r * bpr + b) * bb, out + (size_t)r * cols + b * bv);
            if (st) return st;
        }
    return LEV_OR_OK;
}

/* rust/crates/lev-cli/src/main.rs:1201-1217 (operand rounding) and
 * :1266-1275 (f64 accumulation over every row_step-th row, all tokens) */
int lev_or_gemm_rounded_f64(int t, const uint8_t* w, long rows, long cols, const float* x,
                            long tokens, int input_type, long r0, long row_step, double* y) {
    if (t != 2 && t != 12 && t != 14) return LEV_OR_BAD_DIMENSIONS;
    long bv = block_values(t), bb = block_bytes(t);
    if (cols <= 0 || cols % bv || row_step <= 0) return LEV_OR_BAD_DIMENSIONS;
    long bpr = cols / bv;
    double* xr = (double*)malloc(sizeof(double) * (size_t)(tokens * cols));
    double* wr = (double*)malloc(sizeof(double) * (size_t)cols);
    float tmp[QK_K];
    for (long i = 0; i < tokens * cols; i++)
        xr[i] = input_type == 0 ? (double)lev_or_bf16_to_f32(lev_or_f32_to_bf16_bits(x[i]))
                                : lev_or_f16_to_f64(lev_or_f32_to_f16_bits(x[i]));
    long n_sampled = 0;
    for (long r = r0; r < rows; r += row_step) n_sampled++;
    long si = 0;
    int st = LEV_OR_OK;
    for (long r = r0; r < rows && !st; r += row_step, si++) {
        for (long b = 0; b < bpr; b++) {
            st = dequant_block_any(t, w + ((size_t)r * bpr + b) * bb, tmp);
            if (st) break;
            for (long i = 0; i < bv; i++)
                wr[b * bv + i] = input_type == 0
                                     ? (double)lev_or_bf16_to_f32(lev_or_f32_to_bf16_bits(tmp[i]))
                                     : lev_or_f16_to_f64(lev_or_f32_to_f16_bits(tmp[i]));
        }
        if (st) break;
        for (long tk = 0; tk < tokens; tk++) {
            double acc = 0.0;
            const double* xs = xr + (size_t)tk * cols;
            for (long c = 0; c < cols; c++) acc += wr[c] * xs[c];
            y[(size_t)tk * n_sampled + si] = acc;
        }
    }
    free(xr);
    free(wr);
    return st;
}

/* ------------------------------------------------------------------ */
/* threaded CPU baseline driver                                        */
/* ------------------------------------------------------------------ */

typedef struct {
    int type;
    const uint8_t* w;
    size_t w_bytes;
    long rows, cols;
    const float* x;
    float* y;
    int status;
} chunk_job;

static void* chunk_main(void* arg) {
    chunk_job* j = (chunk_job*)arg;
    if (j->type == 2)
        j->status = lev_or_q4_0_matvec_f32(j->w, j->w_bytes, j->rows, j->cols, j->x, j->cols, j->y);
    else if (j->type == 12)
        j->status = lev_or_q4_k_matvec_f32(j->w, j->w_bytes, j->rows, j->cols, j->x, j->cols, j->y);
    else
        j->status = lev_or_q6_k_matvec_ref(j->w, j->w_bytes, j->rows, j->cols, j->x, j->cols, j->y);
    return NULL;
}

/* rust/crates/lev-model/src/lib.rs:184-199: contiguous row chunks, one
 * thread per chunk, results concatenated in row order. */
int lev_or_matvec_threaded(int type, const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, float* y, int threads) {
    if (type != 2 && type != 12 && type != 14) return LEV_OR_BAD_DIMENSIONS;
    long bv = block_values(type), bb = block_bytes(type);
    if (cols <= 0 || cols % bv || rows <= 0) return LEV_OR_BAD_DIMENSIONS;
    size_t row_bytes = (size_t)(cols / bv) * (size_t)bb;
    if (w_bytes != row_bytes * (size_t)rows) return LEV_OR_BAD_DIMENSIONS;
    if (threads < 1) threads = 1;
    if (threads > rows) threads = (int)rows;
    long per = (rows + threads - 1) / threads;
    pthread_t* tid = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    chunk_job* jobs = (chunk_job*)malloc(sizeof(chunk_job) * (size_t)threads);
    int n = 0;
    for (long r0 = 0; r0 < rows; r0 += per, n++) {
        long nr = rows - r0 < per ? rows - r0 : per;
        jobs[n] = (chunk_job){type, w + (size_t)r0 * row_bytes, (size_t)nr * row_bytes, nr, cols, x, y + r0, 0};
        pthread_create(&tid[n], NULL, chunk_main, &jobs[n]);
    }
    int st = LEV_OR_OK;
    for (int i = 0; i < n; i++) {
        pthread_join(tid[i], NULL);
        if (jobs[i].status && !st) st = jobs[i].status;
    }
    free(tid);
    free(jobs);
    return st;
}

int lev_or_hardware_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
