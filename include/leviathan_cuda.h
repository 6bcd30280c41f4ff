/*
 * libleviathan_cuda.so -- C ABI of the B200 (sm_100a) quantized-weight hot
 * path of Leviathan: GGUF Q4_0 / Q4_K / Q6_K dequant-fused matvec (decode),
 * dequant-GEMM (prefill) and the routed-MoE composite.
 *
 * Conventions
 *   - every entry point returns a lev_status; LEV_OK is 0.  Nothing aborts,
 *     traps or falls back silently.  lev_last_error(ctx) holds the message
 *     of the most recent failure on that context.
 *   - shapes are validated on the host before any device work, in the order
 *     the reference validates them (dimensions, byte counts, input counts,
 *     finiteness).
 *   - the caller owns host arrays and the device buffers it passes; the
 *     library owns what it allocates behind opaque handles.  Weights are
 *     uploaded once and stay resident, addressed by (handle, row offset)
 *     the way the reference addresses one resident buffer by byte offset
 *     (Sources/LeviathanCore/Gemma4.swift:2622-2631).
 *   - a context is not thread-safe; all work of a context is issued on one
 *     CUDA stream (lev_cuda_set_stream).  Entry points given device
 *     pointers are asynchronous on that stream; entry points given host
 *     pointers (LEV_FLAG_HOST_IO, the *_host conveniences) copy in, run,
 *     copy out and synchronize before returning.
 *   - no torch types appear anywhere in this header.
 */
#ifndef LEVIATHAN_CUDA_H
#define LEVIATHAN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LEV_CUDA_ABI_VERSION 1

/* Status codes.  The first group keeps the names of the reference's typed
 * errors (Sources/LeviathanCore/Q4.swift:17-31; rust ShapeError,
 * rust/crates/lev-cpu/src/lib.rs:76-81). */
typedef enum lev_status {
    LEV_OK = 0,
    LEV_BAD_DIMENSIONS = 1,
    LEV_WRONG_INPUT_COUNT = 2,
    LEV_NONFINITE_INPUT = 3,
    LEV_NONFINITE_SCALE = 4,
    LEV_NONFINITE_OUTPUT = 5,
    LEV_EXCEEDS_WORKLOAD = 6,
    LEV_INTEGER_OVERFLOW = 7,
    LEV_DEVICE_UNAVAILABLE = 8,
    LEV_KERNEL_FAILED = 9,
    LEV_TIMEOUT = 10,
    LEV_NCCL_ERROR = 11,
    LEV_BAD_ARGUMENT = 12,
    LEV_OUT_OF_MEMORY = 13,
    LEV_BAD_OP_SPEC = 14,
    LEV_UNSUPPORTED = 15,
    /* container errors, named after GGUFError (Sources/LeviathanCore/GGUF.swift:3-35);
     * its integerOverflow case is LEV_INTEGER_OVERFLOW */
    LEV_GGUF_BAD_MAGIC = 16,
    LEV_GGUF_UNSUPPORTED_VERSION = 17,
    LEV_GGUF_TRUNCATED = 18,
    LEV_GGUF_UNKNOWN_VALUE_TYPE = 19,
    LEV_GGUF_BAD_TENSOR = 20,
    LEV_GGUF_DATA_BEYOND_EOF = 21,
    LEV_GGUF_MISSING = 22, /* missingMetadata / missingTensor */
    LEV_GGUF_UNSUPPORTED_TENSOR_TYPE = 23
} lev_status;

/* ggml tensor type ids of the block formats on the path
 * (Sources/LeviathanCore/GGUF.swift:58-93, rust/crates/lev-gguf/src/lib.rs:94-112) */
typedef enum lev_ggml_type {
    LEV_GGML_F32 = 0,
    LEV_GGML_Q4_0 = 2,  /* 32 values / 18 bytes  */
    LEV_GGML_Q4_K = 12, /* 256 values / 144 bytes */
    LEV_GGML_Q6_K = 14  /* 256 values / 210 bytes */
} lev_ggml_type;

/* Limits restated from Sources/LeviathanCore/Q4.swift:8-15.  The byte cap is
 * raised from 32 GiB to what one B200 holds; the overflow checks stay. */
#define LEV_MAX_DIM (1 << 22)
#define LEV_MAX_WEIGHT_BYTES (160ull << 30)
#define LEV_MAX_COLUMNS 8    /* activation columns per matvec call */
#define LEV_MAX_TOP_K 64     /* Sources/LeviathanCore/MoELowering.swift region bound */
#define LEV_MAX_EXPERTS 1024

/* flags */
#define LEV_FLAG_CHECK_FINITE 1u /* reject non-finite x and y (synchronizes) */
#define LEV_FLAG_HOST_IO 2u      /* x / y (and idx, w) are host pointers */

/* Kernel schedules: named, enumerable, shape- and device-derived candidates
 * with candidate 0 the plain kernel, after Q4ScheduleDeriver.derive
 * (Sources/LeviathanCore/Q4Lowering.swift:283-362). */
typedef enum lev_schedule {
    LEV_SCHEDULE_AUTO = -1,
    LEV_SCHEDULE_PLAIN = 0,  /* one warp per row, reference block order */
    LEV_SCHEDULE_STREAM = 1  /* repacked fragment-major stream, tensor-core dot */
} lev_schedule;

typedef struct lev_ctx lev_ctx;
typedef struct lev_weights lev_weights;
typedef struct lev_moe_weights lev_moe_weights;
typedef struct lev_op lev_op;
typedef struct lev_gguf lev_gguf;

/* CUDA analogue of ForgeHardwareProfile (Sources/LeviathanCore/Forge.swift:17-30) */
typedef struct lev_hw_profile {
    char device_name[128];
    int sm_count;
    int max_threads_per_block;
    int warp_width;
    int cc_major, cc_minor;
    size_t total_memory;
    size_t free_memory;
    size_t shared_memory_per_block_optin;
    size_t l2_bytes;
} lev_hw_profile;

/* Evidence of one run, after Q4MatvecEvidence
 * (Sources/LeviathanCore/Q4.swift:117-124) */
typedef struct lev_evidence {
    char device_name[128];
    char kernel_name[64];
    int64_t out_dim, in_dim;
    int n_cols;
    int grid, block;
    size_t weight_bytes;
    float gpu_us;        /* device time of the kernel(s), CUDA events */
    int status;          /* "completed" == LEV_OK */
} lev_evidence;

/* ---- context ---------------------------------------------------------- */
int lev_cuda_abi_version(void);
const char* lev_status_name(int status);
/* Replaces MTLCreateSystemDefaultDevice + makeCommandQueue
 * (Sources/LeviathanCore/Q4.swift:193-196). */
int lev_cuda_init(int device, lev_ctx** out_ctx);
int lev_cuda_destroy(lev_ctx* ctx);
const char* lev_last_error(const lev_ctx* ctx);
int lev_cuda_hardware_profile(lev_ctx* ctx, lev_hw_profile* out);
/* cuda_stream is a cudaStream_t; NULL restores the context's own stream (pass
 * cudaStreamLegacy, not 0, to name the legacy default stream). */
int lev_cuda_set_stream(lev_ctx* ctx, void* cuda_stream);
/* waits for the stream; LEV_TIMEOUT if a kernel's bounded wait ran out, LEV_BAD_DIMENSIONS if a
 * cache index lay outside its layout (kernels record these instead of faulting) */
int lev_cuda_synchronize(lev_ctx* ctx);
/* Launch counter: kernels launched by this context since creation. */
int64_t lev_cuda_launch_count(const lev_ctx* ctx);
int lev_cuda_last_evidence(const lev_ctx* ctx, lev_evidence* out);

/* ---- resident weights --------------------------------------------------
 * Replaces the resident weightsBuffer + per-tensor byte offsets
 * (Sources/LeviathanCore/Gemma4.swift:2583-2631).  `bytes` are raw GGUF
 * block bytes, row-major [rows][cols/block][block bytes]; the byte count is
 * validated against the geometry (Sources/LeviathanCore/Q4.swift:176-186).
 * Block scales are checked finite at upload (Q4.swift:43-50, Q6.swift:33-37).
 * bytes_on_device != 0 means `bytes` is a device pointer. */
int lev_weights_upload(lev_ctx* ctx, const void* bytes, size_t n_bytes, int ggml_type,
                       int64_t rows, int64_t cols, int bytes_on_device, lev_weights** out);
int lev_weights_free(lev_ctx* ctx, lev_weights* w);
int lev_weights_info(const lev_weights* w, int* ggml_type, int64_t* rows, int64_t* cols,
                     size_t* gguf_bytes);
/* A resident tensor is held twice: in GGUF order (read by lev_dequantize, the plain schedule and the
 * prefill GEMM) and repacked in tile order for the stream schedule (the same bytes, permuted).  A
 * decode-only host can release the GGUF-order copy, as the reference keeps one resident buffer per
 * model (Sources/LeviathanCore/Gemma4.swift:2622-2631); the entry points that read it then return
 * LEV_UNSUPPORTED for this tensor. */
int lev_weights_release_gguf(lev_ctx* ctx, lev_weights* w);

/* Block dequantization of rows [row0, row0+rows) to f32 [rows][cols],
 * bit-exact with Q4_0.decodeBlock (Q4.swift:54-69), Q6_K.decodeBlock
 * (Q6.swift:24-62) and dequant_block_f32
 * (rust/crates/lev-cpu/src/lib.rs:110-130). */
int lev_dequantize(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, float* out,
                   unsigned flags);

/* ---- decode matvec -----------------------------------------------------
 * y[c][r] = sum_k W[row0 + r][k] * x[c][k], c < n_cols <= LEV_MAX_COLUMNS.
 * x is [n_cols][cols], y is [n_cols][rows] (column-major over tokens like
 * the reference's nb-column kernels, rust/crates/lev-forge/src/q8.rs:196).
 * Replaces Gemma4Runner.matvec(tensor:extraOffset:x:xCount:y:yCapacity:)
 * (Sources/LeviathanCore/Gemma4.swift:2583-2638) and Builder::matvec
 * (rust/crates/lev-model/src/gpu.rs:334-370).  x_count and y_capacity are
 * element counts and are checked like xCount / yCapacity there. */
int lev_matvec(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x,
               int64_t x_count, int n_cols, float* y, int64_t y_capacity, int schedule,
               unsigned flags);

/* One-shot host conveniences: upload, run, read back, report.  Replace
 * Q4MetalBackend.matvecReporting (Sources/LeviathanCore/Q4.swift:165-167),
 * Q6MetalBackend.matvecReporting (Sources/LeviathanCore/Q6.swift:199-201)
 * and VulkanContext::run_matvec for Q4_K
 * (rust/crates/lev-vulkan/src/lib.rs:571-582).  Finite checks always on. */
int lev_q4_0_matvec_host(lev_ctx* ctx, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                         int64_t in_dim, const float* x, int64_t x_count, float* y,
                         lev_evidence* evidence);
int lev_q4_k_matvec_host(lev_ctx* ctx, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                         int64_t in_dim, const float* x, int64_t x_count, float* y,
                         lev_evidence* evidence);
int lev_q6_k_matvec_host(lev_ctx* ctx, const uint8_t* blocks, size_t n_bytes, int64_t out_dim,
                         int64_t in_dim, const float* x, int64_t x_count, float* y,
                         lev_evidence* evidence);

/* No counterpart in the reference.  The same matvec as lev_matvec on the stream
 * schedule, for callers that cannot allocate device memory when they call:
 * loops whose memory budget was fixed at start-up, processes whose own
 * allocator holds the whole device, threads that must not take the driver's
 * allocation lock.  x and y are device pointers; all work buffers sit in a
 * fixed array inside the library (lev_static_scratch_bytes() bytes on every GPU
 * that loads it, until the process ends), so nothing is allocated or freed.
 * Calls whose buffers would not fit return LEV_EXCEEDS_WORKLOAD; tensors the
 * stream schedule does not serve return LEV_UNSUPPORTED.  All calls on a
 * device share the array: do not let two of them overlap on the GPU.  The
 * first call on a device resolves the array's address and configures the
 * kernel; make it before any stream capture begins. */
int lev_matvec_static_scratch(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows,
                              const float* x, int64_t x_count, int n_cols, float* y,
                              int64_t y_capacity);
size_t lev_static_scratch_bytes(void);

/* No single counterpart in the reference: n_ops (1...4) resident tensors against the same
 * activations in one call -- gate and up of an FFN, q/k/v of attention (the reference issues one
 * matvec dispatch per tensor, Sources/LeviathanCore/Gemma4.swift:3747-3750; its expert tensors
 * are stored gate/up-fused for the same reason, MoESIMDLowering.swift:106-107).  Whole tensors
 * (no row window); y[i] is [n_cols][rows of tensor i] with y_capacity[i] elements.  Tensors of
 * one format and inDim run as ONE launch; any other mix runs one matvec per tensor. */
int lev_matvec_multi(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x,
                     int64_t x_count, int n_cols, float* const* y, const int64_t* y_capacity,
                     unsigned flags);

/* ---- prefill dequant-GEMM ----------------------------------------------
 * Y[t][r] = sum_k bf16(W[r][k]) * X[t][k], f32 accumulate; X is bf16
 * [tokens][cols], Y is f32 [tokens][rows].  Replaces the act_f16 +
 * q4k/q6k_gemm_blocked_tokens program of
 * rust/crates/lev-forge/src/coopmat.rs:49-58, :236-425. */
int lev_gemm_prefill(lev_ctx* ctx, const lev_weights* w, const void* x_bf16, int64_t tokens,
                     float* y, unsigned flags);
/* f32 activations -> bf16 (round to nearest even); emit_act_f16's role
 * (rust/crates/lev-forge/src/coopmat.rs:49-58). */
int lev_act_bf16(lev_ctx* ctx, const float* x, int64_t n, void* out_bf16);

/* ---- the steps either side of a decode matvec ----------------------------
 * Device pointers; asynchronous on the context's stream.
 * lev_rmsnorm: y[v] = x[v] * (1 / sqrt(mean(x[v]^2) + eps)) * weight (weight NULL: no scale), g4_rmsnorm
 * (Sources/LeviathanCore/Gemma4.swift:4247-4268; tiled form :4323-4358).  x == y is allowed.
 * inverse_out (optional) receives 1 / sqrt(...) per vector for lev_rmsnorm_cached, the cached apply
 * of a statistics group (Sources/LeviathanCore/RMSStatisticsKernels.swift:42-130).
 * lev_gelu_up: out[v][e] = gelu_tanh(gate_up[v][e]) * gate_up[v][inter + e], g4_gelu_up
 * (Gemma4.swift:4364-4377).  lev_axpy: y = r + alpha * x, r may be y (g4_axpy, Gemma4.swift:4459). */
int lev_rmsnorm(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n, const float* weight,
                float eps, float* y, float* inverse_out);
int lev_rmsnorm_cached(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n,
                       const float* weight, const float* inverse, float* y);
int lev_gelu_up(lev_ctx* ctx, const float* gate_up, int64_t vectors, int64_t inter, float* out);
int lev_axpy(lev_ctx* ctx, float alpha, const float* x, const float* r, int64_t n, float* y);
/* The per-head steps between the q / k / v projections and the cache append of a local layer
 * (Sources/LeviathanCore/Gemma4.swift:3662-3687) in one launch, in place on rows laid out as
 * [q_heads | kv_heads (k) | kv_heads (v)] x head_dim: q heads RMSNorm(q_weight) then rotary, k heads
 * RMSNorm(k_weight) then rotary, v heads the scale-free RMSNorm.  Rotary as g4_rope
 * (Gemma4.swift:4390-4410): pairs (i, i + head_dim / 2) turned by inv_freq[i] * pos[column]; inv_freq
 * NULL leaves rotary out.  Weights NULL: no scale.  kv_heads may be 0 (q only). */
int lev_qkv_norm_rope(lev_ctx* ctx, float* qkv, int n_cols, int q_heads, int kv_heads, int head_dim,
                      const float* q_weight, const float* k_weight, float eps,
                      const float* inv_freq, const int32_t* pos);
/* Greedy token choice: out_index[v] = index of the maximum of x[v][0..n) (lowest index on ties, NaN
 * never wins), out_margin[v] (optional) = best - second best; argmax of
 * rust/crates/lev-forge/src/ops.rs:478-517.  Device pointers, no host synchronisation. */
int lev_argmax(lev_ctx* ctx, const float* x, int64_t vectors, int64_t n, int32_t* out_index,
               float* out_margin);
/* The two ends of a decode step.  lev_embed_rows: y[t][0..cols) = value(w[tokens[t]][.]) * scale, the
 * embedding-row decoder g4_q6_embed_row (Sources/LeviathanCore/Gemma4.swift:4210-4245; the caller at
 * :3560-3578 passes scale = sqrt(hidden)); a Q6_K value is ((d * s) * level) * scale with every product
 * rounded to f32, as there.  Q4_0 and Q4_K tensors are read the same way (decoded value * scale).
 * tokens is DEVICE memory, so the id lev_argmax wrote feeds the next step without a host round trip; an
 * id outside [0, rows) leaves a zero row and the next lev_cuda_synchronize returns LEV_BAD_DIMENSIONS.  Reads
 * the tensor's GGUF-order copy: refused after lev_weights_release_gguf.
 * lev_softcap: x = cap * tanh(x / cap) in place (g4_softcap, Gemma4.swift:4496-4503; tanh through
 * exp(-2|x|), :4360-4367).  Asynchronous on the context's stream. */
int lev_embed_rows(lev_ctx* ctx, const lev_weights* w, const int32_t* tokens, int64_t n_tokens,
                   float scale, float* y);
int lev_softcap(lev_ctx* ctx, float* x, int64_t n, float cap);

/* The same steps folded into the matvec launch: the prologue is applied while the kernel builds
 * its activation tables (the norm's statistic is reduced by every thread block for itself), the
 * residual where output rows are stored.  y[c][r] = residual[c][r] + alpha * sum_k W[row0+r][k] *
 * a[c][k] with a = x, rmsnorm(x) or gelu_up(x); with LEV_PROLOGUE_GELU_UP x is
 * [n_cols][2 * cols] (gate then up).  Replaces the rmsnorm -> matvec, gelu_up -> matvec and
 * matvec -> axpy dispatch pairs of the layer loop (Gemma4.swift:3740-3760, :3878).  Shapes the
 * one-launch kernel does not serve run the same steps as separate launches. */
enum { LEV_PROLOGUE_NONE = 0, LEV_PROLOGUE_RMSNORM = 1, LEV_PROLOGUE_GELU_UP = 2 };
typedef struct lev_fusion {
    int prologue;
    const float* norm_weight; /* RMSNORM: device [cols], NULL = no scale */
    float eps;                /* RMSNORM */
    const float* residual;    /* device, y's layout, may be y itself; NULL: y = W a */
    float alpha;              /* used with residual */
} lev_fusion;
int lev_matvec_fused(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x,
                     int64_t x_count, int n_cols, const lev_fusion* fusion, float* y,
                     int64_t y_capacity);
/* several tensors of one inDim behind one prologue (no residual) */
int lev_matvec_multi_fused(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x,
                           int64_t x_count, int n_cols, const lev_fusion* fusion, float* const* y,
                           const int64_t* y_capacity);

/* A recorded list of one-column products in one submission: the decode loop of the Rust runtime
 * records its matvec steps and runs them together (Builder::matvec,
 * rust/crates/lev-model/src/gpu.rs:334-370; Program::run, rust/crates/lev-vulkan/src/engine.rs:87-153),
 * and the Swift layer loop issues matvec(gate), matvec(up), geluUp, matvec(down), axpy back to back
 * (Sources/LeviathanCore/Gemma4.swift:3741-3753).  Ops take effect as if executed in order.  An op
 * whose input (or residual) is written by an earlier op of the list, or whose output an earlier op
 * reads, starts only after every earlier op has finished; the library detects this from the
 * pointers, `depends` forces it.  Where the persistent kernel serves the list it is ONE launch and
 * the weight stream does not pause between ops; otherwise each op runs as lev_matvec_fused.
 * Device pointers; x has w->cols floats (2 * cols with LEV_PROLOGUE_GELU_UP), y has rows floats.
 * With LEV_FLAG_HOST_IO every x and y is a host buffer (independent plain or gelu-up products only):
 * distinct inputs are brought in once (those in pinned, device-mapped host memory by one small kernel that
 * reads them over the bus, the others by a queued copy each), outputs are copied back (an output in pinned,
 * device-mapped host memory is stored by the kernel itself and needs no copy) and the call synchronises;
 * LEV_FLAG_CHECK_FINITE then checks inputs and outputs on the host like the one-shot entry points. */
#define LEV_MAX_CHAIN_OPS 32
typedef struct lev_chain_op {
    const lev_weights* w;
    int64_t row0, rows;
    const float* x;
    float* y;
    int depends;
    lev_fusion fusion; /* prologue LEV_PROLOGUE_NONE and residual NULL: a plain product */
} lev_chain_op;
int lev_matvec_chain(lev_ctx* ctx, int n_ops, const lev_chain_op* ops, unsigned flags);

/* ---- decode attention over a paged KV cache ------------------------------
 * Single-query attention of g4_attn (Sources/LeviathanCore/Gemma4.swift:4412-4457; f64 oracle
 * Sources/LeviathanCore/AttentionLowering.swift:358-388): column c, at query position pos[c] of
 * sequence slot[c], attends to positions [lo, pos[c]] (lo = pos + 1 - window when window > 0),
 * weights softmax(scale * q.k), query head h reads KV head h / (q_heads / kv_heads).  The cache is
 * the paged pool of attn_decode_paged (rust/crates/lev-forge/src/ops.rs:1038-1101;
 * rust/crates/lev-model/src/kv.rs:36-85): pools [blocks][page][kv_heads][head_dim], block table
 * [slots][max_blocks] (int32).  All pointers are device pointers; slot and pos are read on the
 * device, so a decode step needs no host synchronisation.  A slot, position or table entry outside
 * the layout is not followed: the column's output is NaN and the context's next status read
 * reports it.  head_dim 128 or 256; q_heads / kv_heads 1, 2 or 4.
 * lev_kv_append stores each column's new K and V rows (f32 [n_cols][kv_heads][head_dim]) at its
 * position (attn_prep_paged's store, ops.rs:972-1036; the cache append of Gemma4.swift:3690-3698). */
enum { LEV_KV_F32 = 0, LEV_KV_F16 = 1 };
typedef struct lev_kv_layout {
    int kv_type;    /* LEV_KV_F16 or LEV_KV_F32 */
    int page;       /* positions per block (16 in the reference) */
    int kv_heads;
    int head_dim;
    int64_t blocks; /* blocks in each pool */
    int max_blocks; /* entries per row of the block table */
    int slots;      /* rows of the block table */
} lev_kv_layout;
int lev_kv_append(lev_ctx* ctx, const lev_kv_layout* layout, void* k_pool, void* v_pool,
                  const int32_t* block_table, const int32_t* slot, const int32_t* pos, int n_cols,
                  const float* k, const float* v);
int lev_attn_decode(lev_ctx* ctx, const lev_kv_layout* layout, const void* k_pool,
                    const void* v_pool, const int32_t* block_table, const int32_t* slot,
                    const int32_t* pos, int n_cols, int q_heads, const float* q, int window,
                    float scale, float* out);
/* lev_attn_decode with the columns' query rows q_ld elements apart (even, at least
 * q_heads * head_dim; q 8-byte aligned): q may be the leading part of each row of a fused
 * [n_cols][(q_heads + 2 kv_heads) * head_dim] projection output, as lev_qkv_norm_rope_append leaves it. */
int lev_attn_decode_ld(lev_ctx* ctx, const lev_kv_layout* layout, const void* k_pool,
                       const void* v_pool, const int32_t* block_table, const int32_t* slot,
                       const int32_t* pos, int n_cols, int q_heads, const float* q, int64_t q_ld,
                       int window, float scale, float* out);
/* lev_qkv_norm_rope whose launch also stores the finished k and v heads at pos[column] of sequence
 * slot[column] of the cache (lev_kv_append without a launch of its own); kv_heads and head_dim come
 * from the layout. */
int lev_qkv_norm_rope_append(lev_ctx* ctx, float* qkv, int n_cols, int q_heads, int head_dim,
                             const float* q_weight, const float* k_weight, float eps,
                             const float* inv_freq, const int32_t* pos, const lev_kv_layout* layout,
                             void* k_pool, void* v_pool, const int32_t* block_table,
                             const int32_t* slot);
/* The same with q [n_cols][q_heads * head_dim], k and v [n_cols][kv_heads * head_dim] as three
 * matrices, the form the projections of several sequences leave them in. */
int lev_qkv_norm_rope_append_split(lev_ctx* ctx, float* q, float* k, float* v, int n_cols,
                                   int q_heads, int head_dim, const float* q_weight,
                                   const float* k_weight, float eps, const float* inv_freq,
                                   const int32_t* pos, const lev_kv_layout* layout, void* k_pool,
                                   void* v_pool, const int32_t* block_table, const int32_t* slot);

/* ---- routed MoE composite ----------------------------------------------
 * Expert weights are the fused gate_up tensor [experts][2*inter][hidden] and
 * the down tensor [experts][hidden][inter], both Q4_0
 * (Sources/LeviathanCore/MoESIMDLowering.swift:106-107); router weight is
 * f32 [experts][hidden].  local_first/local_count select the experts
 * resident on this GPU (expert parallel); pass 0/experts for all. */
int lev_moe_weights_upload(lev_ctx* ctx, const float* router_w, const uint8_t* gate_up_q4_0,
                           size_t gate_up_bytes, const uint8_t* down_q4_0, size_t down_bytes,
                           int experts, int hidden, int inter, int local_first,
                           int local_count, int bytes_on_device, lev_moe_weights** out);
int lev_moe_weights_free(lev_ctx* ctx, lev_moe_weights* w);
/* lev_weights_release_gguf for both expert tensors of a layer: a decode-only host keeps one copy of the
 * experts (the repacked one).  Calls the tensor-core form would serve (from 512 token-slot pairs on, where the
 * job-list form no longer applies; it reads the GGUF-order bytes) then run on the multi-column stream kernels. */
int lev_moe_weights_release_gguf(lev_ctx* ctx, lev_moe_weights* w);

/* Router decision for `tokens` rows of x [tokens][hidden]: logits in the
 * fixed order documented in lev_moe.cu, softmax in f64, top_k by
 * probability (ties to the lower index), renormalised f32 weights.
 * Replaces the readback + CPU block of
 * Sources/LeviathanCore/Gemma4.swift:3794-3810.  scores may be NULL. */
int lev_moe_route(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens,
                  int top_k, int32_t* idx, float* weights, float* scores, unsigned flags);
/* Token->expert grouping: histogram, exclusive scan, stable permutation of
 * pair ids (token*top_k + rank).  No reference counterpart (the reference
 * batch is one token; closest analogue MoEModelBinding.offsets,
 * Sources/LeviathanCore/MoEModelBinding.swift:174-195). */
int lev_moe_group(lev_ctx* ctx, const int32_t* idx, int64_t tokens, int top_k, int experts,
                  int32_t* counts, int32_t* offsets, int32_t* perm, unsigned flags);
/* Expert FFN for every (token, rank): y_slots [tokens][top_k][hidden];
 * act_out [tokens][top_k][inter] may be NULL.  One grouped launch per stage
 * driven by the device-side offsets.  Replaces runMoeBatchedRouted
 * (Sources/LeviathanCore/Gemma4.swift:2073-2176) and
 * MoEEmittedKernels.runComponent (MoELowering.swift:975). */
int lev_moe_experts(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens,
                    int top_k, const int32_t* idx, float* y_slots, float* act_out,
                    unsigned flags);
/* out[t] = sum_k weights[t][k] * y_slots[t][k], f32, rank order, from zero
 * (g4_axpy per slot, Sources/LeviathanCore/Gemma4.swift:4459-4466, :3878). */
int lev_moe_combine(lev_ctx* ctx, const float* y_slots, const float* weights, int64_t tokens,
                    int top_k, int hidden, float* out, unsigned flags);
/* The whole layer.  idx_out / w_out may be NULL. */
int lev_moe_layer(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens,
                  int top_k, float* out, int32_t* idx_out, float* w_out, unsigned flags);
/* out = residual + alpha * layer(x): the whole layer with the decoder loop's residual step (g4_axpy,
 * Sources/LeviathanCore/Gemma4.swift:3878, :4459-4466) folded into the combine launch; the bits are those of
 * lev_moe_layer followed by lev_axpy.  Device pointers, no flags; out may be residual, not x. */
int lev_moe_layer_residual(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens, int top_k,
                           const float* residual, float alpha, float* out, unsigned flags);

/* ---- Forge op-spec surface ---------------------------------------------
 * Accepts the op JSON of Q4OpIR (Sources/LeviathanCore/Q4Lowering.swift:50-145,
 * producer tools/q4_lower/q4_op_model.py:76-124) extended with
 * quant "q4_k" / "q6_k", `columns` and op "<quant>.gemm"; and the region JSON
 * of MoERegionIR (Sources/LeviathanCore/MoELowering.swift:176-283): scalar
 * fields, graphSha256 over the canonical node lines (:66-168), and the
 * structural re-derivation of the region from its graph
 * (MoERegionGraphWalk.walk, :300-571: three placeholders, per slot select ->
 * linear -> split -> getitem 0/1 -> gelu(tanh) * up -> linear over the slot's
 * down slice, one stack, static f32 shapes, no node shared between slots, the
 * exact ATen census), whose dims the declared ones must equal.  Unknown fields
 * are rejected.  Replaces installQ4GeneratedKernel / uninstall
 * (Sources/LeviathanCore/Gemma4.swift:1022-1110). */
int lev_op_install_json(lev_ctx* ctx, const char* json, size_t json_len, lev_op** out);
int lev_op_uninstall(lev_ctx* ctx, lev_op* op);
/* identity = SHA-256 hex of the sorted-keys JSON (Q4Lowering.swift:176-181) */
int lev_op_describe(const lev_op* op, char* kind /*32*/, int64_t* in_dim, int64_t* out_dim,
                    int* ggml_type, int* columns, char* identity_hex /*65*/,
                    char* kernel_name /*64*/);
/* does this installed op serve a weights handle of that geometry?
 * (q4GeneratedServesTensor, Sources/LeviathanCore/Gemma4.swift:989-1012) */
int lev_op_serves(const lev_op* op, const lev_weights* w, int64_t rows);

/* ---- GGUF container ------------------------------------------------------
 * Replaces GGUFFile(path:) / GGUFFile.parse and its tensor directory
 * (Sources/LeviathanCore/GGUF.swift:96-406; rust/crates/lev-gguf/src/lib.rs):
 * versions 2 and 3, little-endian, the same caps on counts, string and array
 * lengths and header size, `general.alignment` (default 32), and every tensor
 * validated at open: known type, whole blocks, aligned offset, inside the
 * file, no overlap, no duplicate name.  lev_gguf_open maps the file read-only;
 * lev_gguf_parse reads caller-owned bytes that must outlive the handle.
 * `err` (optional) receives the reason of a failure. */
int lev_gguf_open(const char* path, lev_gguf** out, char* err, size_t err_len);
int lev_gguf_parse(const void* bytes, size_t n_bytes, lev_gguf** out, char* err, size_t err_len);
void lev_gguf_close(lev_gguf* g);
int lev_gguf_summary(const lev_gguf* g, uint32_t* version, int64_t* n_tensors,
                     int64_t* n_metadata, uint64_t* alignment, uint64_t* data_offset);
/* index of a tensor by name, -1 when absent (GGUF.swift:384-389) */
int64_t lev_gguf_find_tensor(const lev_gguf* g, const char* name);
/* dims4 are innermost-first as stored; file_offset is absolute */
int lev_gguf_tensor_info(const lev_gguf* g, int64_t index, const char** name, int* ggml_type,
                         int* n_dims, int64_t* dims4, uint64_t* file_offset, uint64_t* n_bytes);
const void* lev_gguf_tensor_data(const lev_gguf* g, int64_t index);
/* metadata getters (metadataUInt / metadataFloat / metadataString, GGUF.swift:366-382) */
int lev_gguf_meta_u64(const lev_gguf* g, const char* key, uint64_t* out);
int lev_gguf_meta_f64(const lev_gguf* g, const char* key, double* out);
int lev_gguf_meta_string(const lev_gguf* g, const char* key, const char** out, size_t* len);
/* array metadata (GGUFValue.array, GGUF.swift:37-56): element value type and count, then one
 * element at a time as its payload in the file (little-endian scalar, or a string's characters) */
int lev_gguf_meta_array(const lev_gguf* g, const char* key, int* elem_type, uint64_t* count);
int lev_gguf_meta_array_item(const lev_gguf* g, const char* key, uint64_t index,
                             const void** payload, size_t* n_bytes);
/* upload a Q4_0 / Q4_K / Q6_K tensor from the file: dims[0] = cols, dims[1] = rows;
 * a third dimension (expert tensors [in, out, experts]) stacks the experts' rows */
int lev_gguf_upload(lev_ctx* ctx, const lev_gguf* g, const char* name, lev_weights** out);
/* one layer's routed-expert weights from a model file, with the checks of
 * MoEModelBinding.bind (Sources/LeviathanCore/MoEModelBinding.swift:93-166): shape metadata
 * under `<general.architecture>.` (block_count, expert_count, expert_used_count,
 * embedding_length, expert_feed_forward_length), blk.<layer>.ffn_gate_up_exps.weight Q4_0
 * [hidden, 2*inter, experts], blk.<layer>.ffn_down_exps.weight Q4_0 [inter, hidden, experts],
 * blk.<layer>.ffn_gate_inp.weight f32 [hidden, experts].  local_count <= 0 keeps every expert
 * resident; top_k (optional) receives expert_used_count. */
int lev_gguf_moe_upload(lev_ctx* ctx, const lev_gguf* g, int layer, int local_first,
                        int local_count, lev_moe_weights** out, int* top_k);

/* ---- multi-GPU (one process per GPU on one NVSwitch box) -----------------
 * The reference has no multi-GPU path (its expert loop runs slots one after another on one device,
 * Sources/LeviathanCore/Gemma4.swift:3856-3880); these entry points shard that path where it splits.
 * lev_dist_init creates an NCCL communicator and, where CUDA IPC allows, maps every rank's work heap
 * into every other rank (LEV_DIST_HEAP_MB, default 96, read once at init): the data paths then run as
 * plain peer stores with bounded flag waits, and NCCL is the fallback.  Every rank must make the same
 * sequence of these calls.  Device pointers only; LEV_FLAG_CHECK_FINITE is refused (a check that fails
 * on one rank would leave its peers waiting). */
#define LEV_NCCL_ID_BYTES 128
int lev_dist_unique_id(void* id128);
int lev_dist_init(lev_ctx* ctx, int rank, int world, const void* id128);
int lev_dist_destroy(lev_ctx* ctx);
/* 1 when the ranks' peer-memory heaps are mapped (the fast forms run), 0 when the entry points fall back to NCCL */
int lev_dist_peer_memory(const lev_ctx* ctx);
/* rows of W are split across ranks; each rank computes its slice into
 * y_full[c][rank*rows_local ...] and the slices are all-gathered. */
int lev_matvec_rowsplit_allgather(lev_ctx* ctx, const lev_weights* w_local, const float* x,
                                  int64_t x_count, int n_cols, float* y_full,
                                  int64_t y_capacity, unsigned flags);
/* a list of row-split products (lev_matvec_chain over this rank's rows of every tensor): ops[i].w is the
 * local slice (whole 16-row tiles), ops[i].y receives all rows_local * world outputs on every rank;
 * independent ops, at most eight */
int lev_matvec_chain_rowsplit(lev_ctx* ctx, int n_ops, const lev_chain_op* ops);
int lev_gemm_prefill_rowsplit_allgather(lev_ctx* ctx, const lev_weights* w_local,
                                        const void* x_bf16, int64_t tokens, float* y_full,
                                        unsigned flags);
/* expert-parallel layer: tokens are data-parallel (this rank's x rows, the same count on every rank),
 * experts are sharded as uploaded.  Dispatch: every rank pushes its token rows, indices and weights to
 * all ranks; each rank runs the pairs of its resident experts; combine: every pair's unweighted output
 * row is stored to the token's rank, which adds its slots in rank order (the ordered axpy of
 * Gemma4.swift:3878, :2171-2175), so the result equals the single-GPU layer bit for bit.  Without peer
 * memory: NCCL all-gather + reduce-scatter, equal to f32 rounding. */
int lev_moe_layer_ep(lev_ctx* ctx, const lev_moe_weights* w, const float* x, int64_t tokens,
                     int top_k, float* out, int32_t* idx_out, float* w_out, unsigned flags);

#ifdef __cplusplus
}
#endif
#endif /* LEVIATHAN_CUDA_H */
