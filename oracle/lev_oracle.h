/*
 * CPU oracle for the quantized-weight hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the CPU reference code of dhihm/leviathan
 * for the GGUF Q4_0 / Q4_K / Q6_K block formats, their streaming matvecs,
 * the routed-MoE region and the router decision.  The reference is Swift and
 * Rust and cannot be compiled where this library is built, so every function
 * follows a cited reference file:line by hand and is pinned by the
 * reference's own known-answer tests (tests/test_oracle_known_answers.py).
 *
 * Parity status per function group:
 *   - f16 conversions, Q4_0, Q4_K, Q6_K decode and matvec, the MoE region,
 *     gelu and the error metric: pinned by the reference's hand-computed
 *     vectors.
 *   - router logits / softmax / top-k: PARITY UNPINNED (the reference holds
 *     no known-answer test for it); follows Gemma4.swift:3797-3810 literally,
 *     with the logit summation order fixed below because the reference only
 *     states it as a GPU kernel.
 *   - token->expert grouping and the weight encoders have no reference
 *     counterpart at all.
 *
 * Nothing outside tests/, the smoke check and the CPU-baseline leg of the
 * benchmark may link or load this library; the product never falls back to
 * it.
 */
#ifndef LEV_ORACLE_H
#define LEV_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes shared by all oracle functions */
enum {
    LEV_OR_OK = 0,
    LEV_OR_BAD_DIMENSIONS = 1,
    LEV_OR_NONFINITE_INPUT = 3,
    LEV_OR_NONFINITE_SCALE = 4,
    LEV_OR_NONFINITE_OUTPUT = 5
};

/* ---- half / bfloat conversions (rust/crates/lev-cpu/src/lib.rs:14-60) ---- */
double lev_or_f16_to_f64(uint16_t h);
float lev_or_f16_to_f32(uint16_t h);
uint16_t lev_or_f32_to_f16_bits(float v);
uint16_t lev_or_f32_to_bf16_bits(float v); /* round to nearest even */
float lev_or_bf16_to_f32(uint16_t h);

/* ---- SplitMix64 streams (Sources/LeviathanCore/RNG.swift:4-24,
 *      rust/crates/lev-cpu/src/lib.rs:357-373) ---- */
uint64_t lev_or_splitmix_next(uint64_t* state);
float lev_or_splitmix_uniform_swift(uint64_t* state);   /* 53-bit, [-1,1) */
float lev_or_splitmix_signed_unit_rust(uint64_t* state); /* 24-bit, [-1,1) */

/* ---- Q4_0 (Sources/LeviathanCore/Q4.swift:38-113) ---- */
int lev_or_q4_0_decode_block(const uint8_t* block18, float* out32);
int lev_or_q4_0_matvec_f32(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, float* y);
/* f64 gate reference (Sources/LeviathanCore/Q4Lowering.swift:676-711) */
int lev_or_q4_0_matvec_f64(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, double* y);
/* incumbent GPU term order in f32 (Sources/LeviathanCore/Gemma4.swift:3931-3953) */
int lev_or_q4_0_matvec_f32_interleaved(const uint8_t* w, size_t w_bytes, long out_dim,
                                       long in_dim, const float* x, long x_count, float* y);
/* double-input form over a byte extent
 * (Sources/LeviathanCore/MoESIMDLowering.swift:934-977) */
int lev_or_q4_0_matvec_f64_dx(const uint8_t* w, size_t w_bytes, size_t byte_offset,
                              long out_dim, long in_dim, const double* x, long x_count,
                              double* y);

/* ---- Q4_K (rust/crates/lev-cpu/src/lib.rs:64-195) ---- */
void lev_or_q4_k_unpack_scale_min(int j, const uint8_t* scales12, uint8_t* sc, uint8_t* mn);
void lev_or_q4_k_pack_scale_min(const uint8_t* sc8, const uint8_t* mn8, uint8_t* scales12);
void lev_or_q4_k_dequant_block_f32(const uint8_t* block144, float* out256);
void lev_or_q4_k_dequant_block_f64(const uint8_t* block144, double* out256);
int lev_or_q4_k_matvec_f32(const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, long x_count, float* y);
int lev_or_q4_k_matvec_f64(const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, long x_count, double* y);

/* ---- Q6_K (Sources/LeviathanCore/Q6.swift:10-145,
 *      rust/crates/lev-cpu/src/lib.rs:203-294) ---- */
int lev_or_q6_k_decode_block(const uint8_t* block210, float* out256);      /* Swift form */
void lev_or_q6_k_unpack(const uint8_t* block210, int8_t* q256);            /* Rust form */
void lev_or_q6_k_dequant_block_f32(const uint8_t* block210, float* out256);
void lev_or_q6_k_dequant_block_f64(const uint8_t* block210, double* out256);
/* Swift oracle: f64 accumulate, rounded to f32 at the end */
int lev_or_q6_k_matvec_ref(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, float* y);
int lev_or_q6_k_matvec_f64(const uint8_t* w, size_t w_bytes, long out_dim, long in_dim,
                           const float* x, long x_count, double* y);
/* Rust f32 ascending form */
int lev_or_q6_k_matvec_f32(const uint8_t* w, size_t w_bytes, long rows, long cols,
                           const float* x, long x_count, float* y);

/* ---- error metric (rust/crates/lev-cpu/src/lib.rs:341-353) ----
 * returns the worst |got-ref|/max(1,|ref|); +inf on NaN/Inf/empty/mismatch */
double lev_or_max_rel_err(const float* got, long n_got, const double* ref, long n_ref);

/* ---- int8 activation quantizer (rust/crates/lev-cpu/src/lib.rs:298-322) ---- */
void lev_or_quantize_q8(const float* x, long n, int8_t* q, float* d, float* s);

/* ---- MoE region (Sources/LeviathanCore/MoESIMDLowering.swift:981-1030) ---- */
/* Gemma4.swift:4247-4268 (serial f32) and lev-model/src/lib.rs:110-114 (f64 statistic) */
void lev_or_rmsnorm_f32(const float* x, long n, long vectors, const float* w, float eps, float* y);
void lev_or_rmsnorm_f64(const float* x, long n, long vectors, const float* w, float eps, double* y);
/* Gemma4.swift:4247-4268 per head, then Gemma4.swift:4390-4410 */
void lev_or_head_norm_rope_f64(const float* x, long heads, long hd, const float* w, float eps, const float* inv_freq, long pos,
                               double* out);
/* AttentionLowering.swift:358-388 */
int lev_or_attention_f64(const float* q, const float* k, const float* v, long q_heads, long kv_heads, long hd, long tokens,
                         long window, double scale, double* out);
double lev_or_gelu_tanh_up(double gate, double up);
float lev_or_gelu_tanh_up_f32(float gate, float up); /* Gemma4.swift:4364-4377 */
/* gu: [top_k][2*inter rows][hidden/32 blocks], dn: [top_k][hidden rows][inter/32 blocks].
 * outputs slot-major: gate/up/act [top_k][inter], dn_out [top_k][hidden]; any may be NULL */
int lev_or_moe_region_f64(long hidden, long inter, long top_k,
                          const uint8_t* gu, size_t gu_bytes,
                          const uint8_t* dn, size_t dn_bytes,
                          const float* x, double* gate, double* up, double* act,
                          double* dn_out);

/* ---- router (Sources/LeviathanCore/Gemma4.swift:3797-3810; logits kernel
 *      Gemma4.swift:4160-4172) ----
 * Logit summation order is FIXED here: partial p[l] (l = 0..31) accumulates
 * elements l, l+32, l+64, ... in ascending order with a correctly rounded
 * double fma; the 32 partials are then combined by an xor butterfly
 * (distance 16, 8, 4, 2, 1) of double adds and the result is rounded once
 * to f32.  */
void lev_or_router_logits(const float* router_w, long experts, long hidden,
                          const float* x, float* scores);
/* softmax in f64, sort by probability descending with ties to the lower
 * index, first top_k, weights renormalised over the selected experts and
 * multiplied by expert_scale[idx] (NULL = 1.0) */
int lev_or_router_topk(const float* scores, long experts, long top_k,
                       const float* expert_scale, int32_t* idx, float* weights);

/* ---- grouping (no reference counterpart: stable counting sort of the
 *      (token, rank) pairs by expert) ---- */
void lev_or_group_tokens(const int32_t* idx, long tokens, long top_k, long experts,
                         int32_t* counts, int32_t* offsets /* experts+1 */,
                         int32_t* perm /* tokens*top_k */);

/* ---- combine (Sources/LeviathanCore/Gemma4.swift:4459-4466 applied once
 *      per slot in rank order, :3878) ---- */
void lev_or_combine(const float* y_slots /* [top_k][hidden] */, const float* weights,
                    long top_k, long hidden, float* out);

/* Whole layer for one token in the reference's own arithmetic classes:
 * f64 region outputs rounded to f32, then the f32 ordered combine.  */
int lev_or_moe_token(long hidden, long inter, long experts, long top_k,
                     const float* router_w, const uint8_t* gu_all, const uint8_t* dn_all,
                     const float* x, int32_t* idx, float* weights, float* out,
                     double* out_f64 /* nullable: f64 combine of f64 slots */);

/* ---- prefill GEMM oracle (rust/crates/lev-cli/src/main.rs:1201-1217,
 *      :1266-1275): both operands rounded to the tensor-core input type,
 *      f64 accumulate.  ggml_type: 2 = Q4_0, 12 = Q4_K, 14 = Q6_K.
 *      input_type: 0 = bf16, 1 = f16.  Computes rows r0, r0+row_step, ...
 *      y[token][sampled_row]. */
int lev_or_gemm_rounded_f64(int ggml_type, const uint8_t* w, long rows, long cols,
                            const float* x, long tokens, int input_type,
                            long r0, long row_step, double* y);

/* ---- generic dequantize of whole rows (f32), any of the three types ---- */
int lev_or_dequantize_rows(int ggml_type, const uint8_t* w, long rows, long cols, float* out);

/* ---- threaded drivers for the timed CPU baseline: rows are split into
 *      contiguous chunks, one thread per chunk
 *      (rust/crates/lev-model/src/lib.rs:184-199) ---- */
int lev_or_matvec_threaded(int ggml_type, const uint8_t* w, size_t w_bytes, long rows,
                           long cols, const float* x, float* y, int threads);
int lev_or_hardware_threads(void);

#ifdef __cplusplus
}
#endif
#endif
