// C++ host side above the C ABI (leviathan_cuda.h): header-only, exceptions instead of status
// codes, RAII handles.  The shapes follow the reference's own host interfaces for this path so
// that a caller (and its tests) read like the reference's:
//
//   lev::Q4Backend::matvecReporting   Q4MetalBackend.matvecReporting   Sources/LeviathanCore/Q4.swift:165-167
//   lev::Q6Backend::matvecReporting   Q6MetalBackend.matvecReporting   Sources/LeviathanCore/Q6.swift:199-201
//   lev::Context::run_matvec          VulkanContext::run_matvec        rust/crates/lev-vulkan/src/lib.rs:571-582
//   lev::Runner::matvec               Gemma4Runner.matvec / Builder::matvec
//                                     Sources/LeviathanCore/Gemma4.swift:2583-2638, rust/crates/lev-model/src/gpu.rs:334-370
//   lev::MoE::forward                 runMoeBatchedRouted              Sources/LeviathanCore/Gemma4.swift:2073-2176
//   lev::Error (case names)           Q4Error                          Sources/LeviathanCore/Q4.swift:17-31
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "leviathan_cuda.h"

namespace lev {

// One exception type; `name()` is the reference's error-case name (badDimensions, wrongInputCount,
// nonFiniteInput, nonFiniteScale, nonFiniteOutput, exceedsModelWorkload, ...).
class Error : public std::runtime_error {
  public:
    Error(int status, const std::string& message)
        : std::runtime_error(std::string(lev_status_name(status)) + ": " + message), status_(status) {}
    int status() const { return status_; }
    const char* name() const { return lev_status_name(status_); }

  private:
    int status_;
};

struct MatvecEvidence {  // Q4MatvecEvidence, Sources/LeviathanCore/Q4.swift:117-124
    std::string deviceName, kernelName;
    int64_t outDim = 0, inDim = 0;
    float gpuUs = 0.f;
    std::string commandStatus;
};

struct RunResult {  // rust/crates/lev-vulkan/src/lib.rs:533-545
    std::vector<float> y;
    std::vector<double> gpu_us;
};

class Context {
  public:
    explicit Context(int device = 0) {
        int st = lev_cuda_init(device, &ctx_);
        if (st != LEV_OK) throw Error(st, "no usable sm_100 device");
    }
    ~Context() {
        if (ctx_) lev_cuda_destroy(ctx_);
    }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;

    lev_ctx* raw() const { return ctx_; }
    void check(int st) const {
        if (st != LEV_OK) throw Error(st, lev_last_error(ctx_));
    }
    lev_hw_profile hardwareProfile() const {  // ForgeHardwareProfile, Sources/LeviathanCore/Forge.swift:17-30
        lev_hw_profile p;
        check(lev_cuda_hardware_profile(ctx_, &p));
        return p;
    }
    void synchronize() const { check(lev_cuda_synchronize(ctx_)); }

    // One-shot Q4_K matvec from host memory: `warmups` untimed and `timed` timed runs, like the
    // reference's Vulkan entry point; y is the last run's output.
    RunResult run_matvec(const std::vector<uint8_t>& weights, int64_t rows, int64_t cols, const std::vector<float>& x,
                         int warmups, int timed) const {
        RunResult r;
        r.y.assign((size_t)(rows > 0 ? rows : 0), 0.f);
        for (int i = 0; i < warmups + (timed > 0 ? timed : 1); i++) {
            lev_evidence ev;
            check(lev_q4_k_matvec_host(ctx_, weights.data(), weights.size(), rows, cols, x.data(), (int64_t)x.size(), r.y.data(), &ev));
            if (i >= warmups && timed > 0) r.gpu_us.push_back(ev.gpu_us);
        }
        return r;
    }

  private:
    lev_ctx* ctx_ = nullptr;
};

namespace detail {
typedef int (*HostMatvec)(lev_ctx*, const uint8_t*, size_t, int64_t, int64_t, const float*, int64_t, float*, lev_evidence*);
inline std::pair<std::vector<float>, MatvecEvidence> reporting(const Context& c, HostMatvec fn, const std::vector<uint8_t>& blocks,
                                                               int64_t outDim, int64_t inDim, const std::vector<float>& x) {
    std::vector<float> y((size_t)(outDim > 0 ? outDim : 0));
    lev_evidence ev;
    c.check(fn(c.raw(), blocks.data(), blocks.size(), outDim, inDim, x.data(), (int64_t)x.size(), y.data(), &ev));
    MatvecEvidence e;
    e.deviceName = ev.device_name;
    e.kernelName = ev.kernel_name;
    e.outDim = ev.out_dim;
    e.inDim = ev.in_dim;
    e.gpuUs = ev.gpu_us;
    e.commandStatus = ev.status == LEV_OK ? "completed" : lev_status_name(ev.status);
    return {std::move(y), std::move(e)};
}
}  // namespace detail

struct Q4Backend {
    static std::pair<std::vector<float>, MatvecEvidence> matvecReporting(const Context& c, const std::vector<uint8_t>& blocks,
                                                                         int64_t outDim, int64_t inDim, const std::vector<float>& x) {
        return detail::reporting(c, lev_q4_0_matvec_host, blocks, outDim, inDim, x);
    }
};
struct Q6Backend {
    static std::pair<std::vector<float>, MatvecEvidence> matvecReporting(const Context& c, const std::vector<uint8_t>& blocks,
                                                                         int64_t outDim, int64_t inDim, const std::vector<float>& x) {
        return detail::reporting(c, lev_q6_k_matvec_host, blocks, outDim, inDim, x);
    }
};

// GGUFFile (Sources/LeviathanCore/GGUF.swift:96-178): a validated container; `path` is mapped read-only.
struct GGUFTensorInfo {
    std::string name;
    std::vector<int64_t> dims;  // innermost first
    int ggmlType = 0;
    uint64_t fileOffset = 0, byteCount = 0;
};

class GGUFFile {
  public:
    explicit GGUFFile(const std::string& path) {
        char err[256] = {0};
        int st = lev_gguf_open(path.c_str(), &g_, err, sizeof err);
        if (st != LEV_OK) throw Error(st, err);
        lev_gguf_summary(g_, &version, &tensorCount, &metadataCount, &alignment, &dataOffset);
    }
    ~GGUFFile() { lev_gguf_close(g_); }
    GGUFFile(const GGUFFile&) = delete;
    GGUFFile& operator=(const GGUFFile&) = delete;
    lev_gguf* raw() const { return g_; }
    GGUFTensorInfo tensor(const std::string& name) const {
        int64_t i = lev_gguf_find_tensor(g_, name.c_str());
        if (i < 0) throw Error(LEV_GGUF_MISSING, "tensor " + name);
        return tensor(i);
    }
    GGUFTensorInfo tensor(int64_t index) const {
        const char* name = nullptr;
        int type = 0, nd = 0;
        int64_t dims[4];
        GGUFTensorInfo t;
        int st = lev_gguf_tensor_info(g_, index, &name, &type, &nd, dims, &t.fileOffset, &t.byteCount);
        if (st != LEV_OK) throw Error(st, "tensor index " + std::to_string(index));
        t.name = name;
        t.ggmlType = type;
        t.dims.assign(dims, dims + nd);
        return t;
    }
    uint64_t metadataUInt(const std::string& key) const {
        uint64_t v = 0;
        int st = lev_gguf_meta_u64(g_, key.c_str(), &v);
        if (st != LEV_OK) throw Error(st, "metadata " + key);
        return v;
    }
    double metadataFloat(const std::string& key) const {
        double v = 0;
        int st = lev_gguf_meta_f64(g_, key.c_str(), &v);
        if (st != LEV_OK) throw Error(st, "metadata " + key);
        return v;
    }
    std::string metadataString(const std::string& key) const {
        const char* p = nullptr;
        size_t n = 0;
        int st = lev_gguf_meta_string(g_, key.c_str(), &p, &n);
        if (st != LEV_OK) throw Error(st, "metadata " + key);
        return std::string(p, n);
    }
    uint32_t version = 0;
    int64_t tensorCount = 0, metadataCount = 0;
    uint64_t alignment = 0, dataOffset = 0;

  private:
    lev_gguf* g_ = nullptr;
};

// A resident quantized tensor, addressed by (handle, row offset) like the runner's weights buffer.
class Weights {
  public:
    // a Q4_0 / Q4_K / Q6_K tensor of a container, uploaded from the mapping
    Weights(const Context& c, const GGUFFile& file, const std::string& name) : c_(&c) {
        c.check(lev_gguf_upload(c.raw(), file.raw(), name.c_str(), &w_));
        lev_weights_info(w_, nullptr, &rows_, &cols_, nullptr);
    }
    Weights(const Context& c, const std::vector<uint8_t>& ggufBytes, int ggmlType, int64_t rows, int64_t cols) : c_(&c) {
        c.check(lev_weights_upload(c.raw(), ggufBytes.data(), ggufBytes.size(), ggmlType, rows, cols, 0, &w_));
        rows_ = rows;
        cols_ = cols;
    }
    ~Weights() {
        if (w_) lev_weights_free(c_->raw(), w_);
    }
    Weights(const Weights&) = delete;
    Weights& operator=(const Weights&) = delete;
    lev_weights* raw() const { return w_; }
    int64_t rows() const { return rows_; }
    int64_t cols() const { return cols_; }

  private:
    const Context* c_;
    lev_weights* w_ = nullptr;
    int64_t rows_ = 0, cols_ = 0;
};

struct Runner {
    // y[nb][rows] = W[rowOffset .. rowOffset + rows) * x[nb][cols]; host vectors in and out.
    static std::vector<float> matvec(const Context& c, const Weights& w, int64_t rowOffset, int64_t rows, const std::vector<float>& x,
                                     int nb = 1, bool checkFinite = true) {
        std::vector<float> y((size_t)nb * (size_t)(rows > 0 ? rows : 0));
        unsigned flags = LEV_FLAG_HOST_IO | (checkFinite ? LEV_FLAG_CHECK_FINITE : 0u);
        c.check(lev_matvec(c.raw(), w.raw(), rowOffset, rows, x.data(), (int64_t)x.size(), nb, y.data(), (int64_t)y.size(),
                           LEV_SCHEDULE_AUTO, flags));
        return y;
    }
    static std::vector<float> dequantize(const Context& c, const Weights& w, int64_t row0, int64_t rows) {
        std::vector<float> out((size_t)rows * (size_t)w.cols());
        c.check(lev_dequantize(c.raw(), w.raw(), row0, rows, out.data(), LEV_FLAG_HOST_IO));
        return out;
    }
};

// Routed MoE layer over resident Q4_0 experts.
class MoE {
  public:
    MoE(const Context& c, const std::vector<float>& routerW, const std::vector<uint8_t>& gateUp, const std::vector<uint8_t>& down,
        int experts, int hidden, int inter)
        : c_(&c), hidden_(hidden) {
        c.check(lev_moe_weights_upload(c.raw(), routerW.data(), gateUp.data(), gateUp.size(), down.data(), down.size(), experts, hidden,
                                       inter, 0, experts, 0, &w_));
    }
    ~MoE() {
        if (w_) lev_moe_weights_free(c_->raw(), w_);
    }
    MoE(const MoE&) = delete;
    MoE& operator=(const MoE&) = delete;

    struct Output {
        std::vector<float> out;       // [tokens][hidden]
        std::vector<int32_t> topIdx;  // [tokens][topK]
        std::vector<float> weights;   // [tokens][topK]
    };
    Output forward(const std::vector<float>& x, int64_t tokens, int topK) const {
        Output o;
        o.out.resize((size_t)tokens * hidden_);
        o.topIdx.resize((size_t)tokens * topK);
        o.weights.resize((size_t)tokens * topK);
        c_->check(lev_moe_layer(c_->raw(), w_, x.data(), tokens, topK, o.out.data(), o.topIdx.data(), o.weights.data(),
                                LEV_FLAG_HOST_IO | LEV_FLAG_CHECK_FINITE));
        return o;
    }

  private:
    const Context* c_;
    lev_moe_weights* w_ = nullptr;
    int hidden_;
};

}  // namespace lev
