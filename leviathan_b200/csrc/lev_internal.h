// Internal declarations shared by the translation units of libleviathan_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "leviathan_cuda.h"

#define LEV_Q4_0_VALUES 32
#define LEV_Q4_0_BYTES 18
#define LEV_QK_K 256
#define LEV_Q4_K_BYTES 144
#define LEV_Q6_K_BYTES 210

// device status word bits (finite checks, bounded waits)
#define LEV_DEV_NONFINITE_INPUT 1
#define LEV_DEV_NONFINITE_SCALE 2
#define LEV_DEV_NONFINITE_OUTPUT 4
#define LEV_DEV_TIMEOUT 8
#define LEV_DEV_BAD_INDEX 16  // a slot, position or block-table entry outside the cache layout

// Row (in units of rows of head_dim elements) of (block, position inside the block, KV head) in a paged cache pool.
#ifdef LEV_KV_HEAD_MAJOR
#define LEV_KV_ROW(block, in_page, kvh, page, kv_heads) (((int64_t)(block) * (kv_heads) + (kvh)) * (page) + (in_page))
#else
#define LEV_KV_ROW(block, in_page, kvh, page, kv_heads) (((int64_t)(block) * (page) + (in_page)) * (kv_heads) + (kvh))
#endif
// ints after the status word: counters that kernels leave at zero (ctx->d_status + LEV_COUNTER_OFFSET)
#define LEV_COUNTER_OFFSET 64
#define LEV_COUNTERS 65536

struct lev_dist_state;

struct lev_ctx {
    int device;
    cudaStream_t own_stream;
    cudaStream_t stream;
    cudaDeviceProp prop;
    char err[512];
    int64_t launches;
    lev_evidence ev;
    // scratch owned by the context, grown on demand, reused across calls
    void* scratch[12];
    size_t scratch_bytes[12];
    int* d_status;   // device status word
    int* h_status;   // pinned mirror
    cudaEvent_t ev0, ev1;
    lev_dist_state* dist;
    // persistent matvec kernel (lev_chain.cu): counters it leaves at zero and partial sums of tiles
    // shared by thread blocks; tuning read once at lev_cuda_init
    void* chain_sync;
    void* chain_part;
    int chain_off, chain_warps, chain_depth;
};

// Scratch slots (each one buffer; a call may use several at once).
enum {
    LEV_SCR_X = 0,       // staged activations (host io) / prepared activations
    LEV_SCR_Y = 1,       // staged outputs (host io)
    LEV_SCR_MOE_A = 2,   // router scores, idx, weights
    LEV_SCR_MOE_B = 3,   // grouping tables
    LEV_SCR_MOE_C = 4,   // gathered activations / expert intermediates
    LEV_SCR_MOE_D = 5,   // expert outputs per (token, rank)
    LEV_SCR_XPREP = 6,   // split activations for the stream schedule
    LEV_SCR_DIST = 7,
    LEV_SCR_ATTN = 8,    // attention partials per position range
    LEV_SCR_GEMM = 9,    // partial products of a K-split prefill GEMM
    LEV_SCR_SLOTS = 12
};

struct lev_weights {
    int type;
    int64_t rows, cols;
    int64_t blocks_per_row;
    size_t gguf_bytes;    // rows * blocks_per_row * block bytes
    uint8_t* raw;         // GGUF block bytes, row-major (device)
    // fragment-major repack for the stream schedule (device); NULL if absent
    uint8_t* packed;
    size_t packed_bytes;
    int64_t packed_rows;  // rows rounded up to the 16-row tile
    int owns_raw;
};

struct lev_moe_weights {
    int experts, hidden, inter;
    int local_first, local_count;
    float* router_w;          // [experts][hidden]
    lev_weights* gate_up;     // [local_count * 2*inter][hidden] Q4_0
    lev_weights* down;        // [local_count * hidden][inter]  Q4_0
};

static inline int lev_block_values(int type) { return type == LEV_GGML_Q4_0 ? 32 : 256; }
static inline int lev_block_bytes(int type) {
    return type == LEV_GGML_Q4_0 ? LEV_Q4_0_BYTES : (type == LEV_GGML_Q4_K ? LEV_Q4_K_BYTES : LEV_Q6_K_BYTES);
}
static inline bool lev_type_ok(int type) {
    return type == LEV_GGML_Q4_0 || type == LEV_GGML_Q4_K || type == LEV_GGML_Q6_K;
}

int lev_fail(lev_ctx* ctx, int status, const char* fmt, ...);
int lev_cuda_check(lev_ctx* ctx, cudaError_t e, const char* what);
int lev_scratch(lev_ctx* ctx, int slot, size_t bytes, void** out);
// like lev_scratch, and the buffer is zero-filled whenever it is (re)allocated
// reads the device status word (synchronizes the stream) and clears it
int lev_read_status(lev_ctx* ctx, int* bits);

#define LEV_CUDA(ctx, call)                                         \
    do {                                                            \
        int _st = lev_cuda_check((ctx), (call), #call);             \
        if (_st) return _st;                                        \
    } while (0)

#define LEV_TRY(call)                \
    do {                             \
        int _st = (call);            \
        if (_st) return _st;         \
    } while (0)

// ---- launchers implemented in the kernel translation units ----
int lev_launch_scale_check(lev_ctx* ctx, const lev_weights* w);
int lev_launch_finite_check(lev_ctx* ctx, const float* v, int64_t n, int bit);
int lev_launch_dequantize(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, float* out);
int lev_launch_matvec_plain(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows,
                            const float* x, int n_cols, float* y);
int lev_repack_weights(lev_ctx* ctx, lev_weights* w);
bool lev_stream_supported(const lev_weights* w, int64_t row0, int64_t rows, int n_cols);
int lev_launch_matvec_stream(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows,
                             const float* x, int n_cols, float* y);

int lev_weights_create(lev_ctx* ctx, const void* bytes, size_t n_bytes, int type, int64_t rows,
                       int64_t cols, int on_device, bool repack, lev_weights** out);

// device-pointer stages of the MoE composite (lev_moe.cu), shared with the expert-parallel layer
int lev_moe_route_dev(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k, int32_t* idx,
                      float* weights, float* scores);
int lev_moe_experts_dev(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                        const int32_t* idx, float* y_pairs, float* act_out);
int lev_moe_combine_dev(lev_ctx* ctx, const float* y, const float* wts, int64_t tokens, int top_k, int hidden, float* out);
int lev_moe_combine_resident_dev(lev_ctx* ctx, const float* y, const float* wts, int64_t tokens, int top_k, int hidden,
                                 float* out, const int32_t* idx, int first, int count);
int lev_moe_combine_residual_dev(lev_ctx* ctx, const float* y, const float* wts, int64_t tokens, int top_k, int hidden,
                                 float* out, const int32_t* idx, int first, int count, const float* residual, float alpha);
