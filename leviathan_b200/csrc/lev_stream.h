// Interface of the stream schedule shared by the dense matvec and the
// grouped expert FFN.
#pragma once

#include "lev_internal.h"

// where the activation columns of a call come from
struct lev_stream_source {
    const float* x;        // source rows
    int64_t ld;            // elements between source rows
    const int* rowmap;     // [job][cmax] source row per column (-1 = empty); NULL: row = column
    const int* njobs_dev;  // device count of jobs; NULL: all `jobs` given to lev_stream_prepare
    int gelu_inter;        // > 0: value = gelu_tanh(x[e]) * x[gelu_inter + e]
    float* act_out;        // optional [row][cols] copy of the source values
};

// which weight rows a call streams and where results go
struct lev_stream_job {
    int64_t row0;          // dense: first row (multiple of 16); grouped: 0
    int64_t rows;          // rows per job
    int64_t out_ld;        // elements between output columns
    int max_jobs;          // dense: 1; grouped: upper bound of the device job count
    const int* njobs_dev;  // grouped: device count of jobs
    const int* job_slice;  // grouped: [job] slice index (slice = rows consecutive rows of the tensor)
    const int* outmap;     // grouped: [job][cmax] output column index (-1 = none)
};

int lev_stream_terms(int n_cols);
int64_t lev_stream_chunks(const lev_weights* w);
size_t lev_stream_table_bytes(const lev_weights* w, int cmax, int terms, int jobs, size_t* frag_bytes);
int lev_stream_prepare(lev_ctx* ctx, const lev_weights* w, const lev_stream_source& src, int cmax, int terms, int jobs,
                       void* tables);
// tables: what lev_stream_prepare wrote for the same (weights, cmax, terms, jobs)
int lev_stream_run(lev_ctx* ctx, const lev_weights* w, const lev_stream_job& job, const void* tables, int cmax,
                   int terms, float* y);

// steps fused into the one-launch kernel either side of the product
struct lev_dense_fusion {
    int norm_on;            // activations = x * inv_rms(x) * norm_w
    const float* norm_w;    // [cols] or NULL
    float eps;
    int gelu_up;            // x rows are [gate(cols) | up(cols)]; activations = gelu_tanh(gate) * up
    const float* residual;  // y = residual + alpha * (W x); same layout as y, may be y itself
    float alpha;
};

// one-launch dense matvec (lev_dense.cu): n_cols <= 4 and tables that fit shared memory
bool lev_dense_supported(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols);
int lev_dense_run(lev_ctx* ctx, const lev_weights* w, int64_t row0, int64_t rows, const float* x, int n_cols, float* y,
                  const lev_dense_fusion* fusion = nullptr);

// sliced form of the one-launch kernel: a device-side job list, cmax (1 or 4) activation columns per job
bool lev_dense_jobs_supported(lev_ctx* ctx, const lev_weights* w, int64_t rows_per_job, int max_jobs, int cmax,
                              const float* x, int64_t x_ld);
int lev_dense_jobs_run(lev_ctx* ctx, const lev_weights* w, int64_t rows_per_job, int max_jobs, int cmax, const int* njobs_dev,
                       const int* job_slice, const int* job_src, const int* job_out, const float* x, int64_t x_ld,
                       int gelu_inter, float* y, int64_t out_ld);

// multi form: several whole tensors of one format and K against the same activations, one launch
bool lev_dense_multi_supported(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x, int n_cols);
int lev_dense_multi_run(lev_ctx* ctx, int n_ops, const lev_weights* const* w, const float* x, int n_cols, float* const* y,
                        const lev_dense_fusion* fusion = nullptr);

// persistent form (lev_chain.cu): a list of one-column products in one launch, with the fused steps
// of lev_dense_fusion per op; `wait`: the op reads what earlier ops of the list write
struct lev_chain_item {
    const lev_weights* w;
    int64_t row0, rows;
    const float* x;
    float* y;
    int wait;
    const lev_dense_fusion* fusion;
};
constexpr int kLevChainMaxOps = 32;
bool lev_chain_supported(lev_ctx* ctx, int n_ops, const lev_chain_item* items);
bool lev_chain_preferred(lev_ctx* ctx, int n_ops, const lev_chain_item* items);
int lev_chain_run(lev_ctx* ctx, int n_ops, const lev_chain_item* items);
// buffers of the persistent kernel, allocated with the context
int lev_chain_init(lev_ctx* ctx);
// puts them back to zero (after a kernel gave up on a bounded wait)
int lev_chain_reset(lev_ctx* ctx);
