// Forge op-spec surface: parses and validates the op JSON of the matvec
// operator (Q4OpIR, Sources/LeviathanCore/Q4Lowering.swift:50-181; producer
// tools/q4_lower/q4_op_model.py:76-124) and the routed-MoE region JSON
// (MoERegionIR, Sources/LeviathanCore/MoELowering.swift:66-283), and installs
// them as named operators that say which resident tensors they serve
// (q4GeneratedServesTensor, Sources/LeviathanCore/Gemma4.swift:989-1012).
//
// Extensions over the reference schema: quant "q4_k" / "q6_k" with layouts
// "row-major-q4_k-blocks" / "row-major-q6_k-blocks", an optional `columns`
// (1..8), and ops "<quant>.gemm" for prefill.  Unknown fields are rejected.
// Identity is the SHA-256 of the sorted-keys compact JSON (Q4Lowering.swift:
// 176-181); for a region it is the graph digest over the canonical node lines
// (MoELowering.swift:66-168), which must equal the document's graphSha256.
// The region's dataflow is re-derived from the graph itself (RegionWalk below,
// the checks of MoERegionGraphWalk.walk, MoELowering.swift:300-571): the
// document's declared dims must agree with what the graph says.
#include <stdlib.h>

#include <map>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "lev_internal.h"

namespace {

// ---- SHA-256 (FIPS 180-4) ----
struct Sha256 {
    uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    uint8_t buf[64];
    uint64_t len = 0;
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t* p) {
        static const uint32_t K[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
            0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
            0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
            0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
            0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
            0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
            0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; i++) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + w[i];
            uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const void* data, size_t n) {
        const uint8_t* p = (const uint8_t*)data;
        while (n) {
            size_t off = len % 64, take = 64 - off < n ? 64 - off : n;
            memcpy(buf + off, p, take);
            len += take; p += take; n -= take;
            if (len % 64 == 0) block(buf);
        }
    }
    std::string hex() {
        uint64_t bits = len * 8;
        uint8_t pad = 0x80;
        update(&pad, 1);
        uint8_t z = 0;
        while (len % 64 != 56) update(&z, 1);
        uint8_t lb[8];
        for (int i = 0; i < 8; i++) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(lb, 8);
        char out[65];
        for (int i = 0; i < 8; i++) snprintf(out + 8 * i, 9, "%08x", h[i]);
        return std::string(out, 64);
    }
};

// ---- minimal JSON ----
struct JVal;
typedef std::shared_ptr<JVal> JP;
struct JVal {
    enum Kind { Null, Bool, Int, Real, Str, Arr, Obj } kind = Null;
    bool b = false;
    int64_t i = 0;
    std::string s;
    std::vector<JP> arr;
    std::vector<std::pair<std::string, JP>> obj;  // document order
    const JP* get(const std::string& k) const {
        for (auto& kv : obj) if (kv.first == k) return &kv.second;
        return nullptr;
    }
};
struct JParser {
    const char* p; const char* end; std::string err; int depth = 0;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool fail(const char* m) { if (err.empty()) err = m; return false; }
    bool str(std::string& out) {
        if (p >= end || *p != '"') return fail("expected string");
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("bad escape");
                switch (*p) {
                    case '"': out += '"'; break; case '\\': out += '\\'; break; case '/': out += '/'; break;
                    case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) return fail("bad \\u");
                        unsigned cp = (unsigned)strtoul(std::string(p + 1, 4).c_str(), nullptr, 16);
                        p += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 63)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 63)); out += (char)(0x80 | (cp & 63)); }
                        break;
                    }
                    default: return fail("bad escape");
                }
                p++;
            } else out += *p++;
        }
        if (p >= end) return fail("unterminated string");
        p++;
        return true;
    }
    bool value(JP& out) {
        if (++depth > 64) return fail("nesting too deep");
        ws();
        out = std::make_shared<JVal>();
        if (p >= end) return fail("unexpected end");
        bool ok = true;
        if (*p == '{') {
            out->kind = JVal::Obj; p++; ws();
            if (p < end && *p == '}') p++;
            else for (;;) {
                ws(); std::string k;
                if (!str(k)) { ok = false; break; }
                if (out->get(k)) { ok = fail("duplicate key"); break; }
                ws(); if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
                p++; JP v;
                if (!value(v)) { ok = false; break; }
                out->obj.push_back({k, v}); ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; break; }
                ok = fail("expected ',' or '}'"); break;
            }
        } else if (*p == '[') {
            out->kind = JVal::Arr; p++; ws();
            if (p < end && *p == ']') p++;
            else for (;;) {
                JP v;
                if (!value(v)) { ok = false; break; }
                out->arr.push_back(v); ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; break; }
                ok = fail("expected ',' or ']'"); break;
            }
        } else if (*p == '"') { out->kind = JVal::Str; ok = str(out->s); }
        else if (end - p >= 4 && !strncmp(p, "true", 4)) { out->kind = JVal::Bool; out->b = true; p += 4; }
        else if (end - p >= 5 && !strncmp(p, "false", 5)) { out->kind = JVal::Bool; out->b = false; p += 5; }
        else if (end - p >= 4 && !strncmp(p, "null", 4)) { out->kind = JVal::Null; p += 4; }
        else if (*p == '-' || (*p >= '0' && *p <= '9')) {
            const char* q = p; if (*q == '-') q++;
            while (q < end && *q >= '0' && *q <= '9') q++;
            if (q < end && (*q == '.' || *q == 'e' || *q == 'E')) {
                while (q < end && (strchr("+-.eE", *q) || (*q >= '0' && *q <= '9'))) q++;
                out->kind = JVal::Real; out->s.assign(p, q);
            } else {
                if (q - p > 18) ok = fail("integer too long");
                out->kind = JVal::Int; out->i = strtoll(std::string(p, q).c_str(), nullptr, 10);
            }
            p = q;
        } else ok = fail("unexpected character");
        depth--;
        return ok;
    }
};

std::string json_quote(const std::string& s) {  // JSONEncoder escapes: quote, backslash, slash, control characters
    std::string o = "\"";
    for (unsigned char c : s) {
        if (c == '"') o += "\\\""; else if (c == '\\') o += "\\\\"; else if (c == '/') o += "\\/";
        else if (c == '\n') o += "\\n"; else if (c == '\t') o += "\\t"; else if (c == '\r') o += "\\r";
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += (char)c;
    }
    return o + "\"";
}

bool ends_with(const std::string& s, const char* suf) {
    size_t n = strlen(suf);
    return s.size() >= n && !s.compare(s.size() - n, n, suf);
}
bool is_attn_output_name(const std::string& n) {  // Q4Lowering.swift:85-91
    const std::string pre = "blk.", suf = ".attn_output.weight";
    if (n.size() <= pre.size() + suf.size() || n.compare(0, pre.size(), pre) || !ends_with(n, suf.c_str())) return false;
    for (size_t i = pre.size(); i < n.size() - suf.size(); i++) if (n[i] < '0' || n[i] > '9') return false;
    return true;
}

// canonical strings of the region graph (MoELowering.swift:66-168)
bool canon_val(const JVal& v, std::string& o) {
    switch (v.kind) {
        case JVal::Null: o += "n"; return true;
        case JVal::Bool: o += v.b ? "b:1" : "b:0"; return true;
        case JVal::Int: o += "i:" + std::to_string(v.i); return true;
        case JVal::Str: o += "s:" + v.s; return true;
        case JVal::Obj:
            if (v.obj.size() == 1 && v.obj[0].first == "__node__" && v.obj[0].second->kind == JVal::Str) { o += "@" + v.obj[0].second->s; return true; }
            return false;
        case JVal::Arr: {
            o += "l<";
            for (size_t i = 0; i < v.arr.size(); i++) { if (i) o += ","; if (!canon_val(*v.arr[i], o)) return false; }
            o += ">"; return true;
        }
        default: return false;
    }
}
bool canon_meta(const JVal& m, std::string& o) {
    if (m.kind != JVal::Obj) return false;
    const JP* dt = m.get("dtype"); const JP* sh = m.get("shape"); const JP* it = m.get("items");
    if (!dt || (*dt)->kind != JVal::Str) return false;
    o += "d<dtype:s:" + (*dt)->s;
    if (it && (*it)->kind == JVal::Arr) {
        o += ",items:l<";
        for (size_t i = 0; i < (*it)->arr.size(); i++) { if (i) o += ","; if (!canon_meta(*(*it)->arr[i], o)) return false; }
        o += ">";
    }
    o += ",shape:";
    if (sh && (*sh)->kind == JVal::Arr) {
        o += "l<";
        for (size_t i = 0; i < (*sh)->arr.size(); i++) { if ((*sh)->arr[i]->kind != JVal::Int) return false; if (i) o += ","; o += "i:" + std::to_string((*sh)->arr[i]->i); }
        o += ">";
    } else o += "n";
    o += ">";
    return true;
}


// ---- structural re-derivation of the routed region from its graph ----
// The supported graph is, for every slot s of topK:
//   select(gu_weights, 0, s) -> linear(x, .) -> split(., inter, -1) -> getitem 0 / 1 -> gelu(tanh) * up
//   -> linear(., select(down_weights, 0, s)), and one stack of the slots' outputs.
// Every node is looked up by name from the consumer's operands, its operator, arity, constants and
// static f32 shape are checked, and it is claimed for its slot; a node claimed twice, left unclaimed,
// or of another operator fails the walk.  The dims the walk returns come from the placeholders' and the
// splits' metadata only, never from the document's scalar fields.
struct RegionDims { int64_t hidden = 0, inter = 0, top_k = 0, gate_up_out = 0; };

class RegionWalk {
  public:
    std::string err;
    bool run(const JVal& graph, RegionDims* out);

  private:
    static constexpr int64_t kDimCap = 4 * 8192;  // 4 * MoERegionIR.maxDim
    std::map<std::string, const JVal*> by_name_;
    std::map<std::string, int> claimed_;

    bool fail(const std::string& m) { if (err.empty()) err = m; return false; }
    static const std::string& str(const JVal& n, const char* k) {
        static const std::string none;
        const JP* v = n.get(k);
        return v && (*v)->kind == JVal::Str ? (*v)->s : none;
    }
    static const std::vector<JP>& args(const JVal& n) { return (*n.get("args"))->arr; }
    static const JVal& kwargs(const JVal& n) { return **n.get("kwargs"); }
    // the node an operand {"__node__": name} names
    const JVal* deref(const JVal& v) const {
        if (v.kind != JVal::Obj || v.obj.size() != 1 || v.obj[0].first != "__node__" || v.obj[0].second->kind != JVal::Str) return nullptr;
        auto it = by_name_.find(v.obj[0].second->s);
        return it == by_name_.end() ? nullptr : it->second;
    }
    static bool is_int(const JVal& v, int64_t want) { return v.kind == JVal::Int && v.i == want; }
    // operands of a call: exactly `n`, a trailing null (an absent bias) dropped first when allowed
    static bool arity(const JVal& n, size_t want, bool drop_null = false) {
        size_t have = args(n).size();
        if (drop_null && have == want + 1 && args(n)[want]->kind == JVal::Null) have = want;
        return have == want;
    }
    // node is a call of `target` without keyword operands
    bool plain_call(const JVal& n, const char* target) const {
        return str(n, "op") == "call_function" && str(n, "target") == target && kwargs(n).obj.empty();
    }
    // static f32 metadata of exactly this shape
    static bool f32_shape(const JVal& meta, const std::vector<int64_t>& want) {
        if (meta.kind != JVal::Obj) return false;
        const JP* dt = meta.get("dtype"); const JP* sh = meta.get("shape");
        if (!dt || (*dt)->kind != JVal::Str || (*dt)->s != "float32" || !sh || (*sh)->kind != JVal::Arr || (*sh)->arr.size() != want.size()) return false;
        for (size_t i = 0; i < want.size(); i++) if (!is_int(*(*sh)->arr[i], want[i])) return false;
        return true;
    }
    static bool has_f32_shape(const JVal& n, const std::vector<int64_t>& want) {
        const JP* m = n.get("meta");
        return m && f32_shape(**m, want);
    }
    // the bounded dims of a placeholder of this rank
    bool placeholder_dims(const JVal& n, size_t rank, std::vector<int64_t>* dims) {
        const JP* m = n.get("meta");
        if (!m || (*m)->kind != JVal::Obj) return fail("input " + str(n, "name") + ": missing static meta");
        const JP* dt = (*m)->get("dtype"); const JP* sh = (*m)->get("shape");
        if (!dt || (*dt)->kind != JVal::Str || !sh || (*sh)->kind != JVal::Arr) return fail("input " + str(n, "name") + ": missing static meta");
        if ((*dt)->s != "float32") return fail("input " + str(n, "name") + " dtype " + (*dt)->s + " != float32");
        if ((*sh)->arr.size() != rank) return fail("input " + str(n, "name") + ": rank " + std::to_string((*sh)->arr.size()) + " != " + std::to_string(rank));
        for (auto& d : (*sh)->arr) {
            if (d->kind != JVal::Int || d->i < 0 || d->i > kDimCap) return fail("input " + str(n, "name") + ": dims out of bounds");
            dims->push_back(d->i);
        }
        return true;
    }
    bool claim(const JVal& n, int slot, const char* what) {
        if (!claimed_.emplace(str(n, "name"), slot).second)
            return fail("slot " + std::to_string(slot) + " " + what + " (" + str(n, "name") + ") is reused or shared across slots");
        return true;
    }
    bool slot(int s, const JVal& fin, const JVal& x, const JVal& gu, const JVal& dn, const RegionDims& D, int64_t dn_in, int64_t* inter);
};

bool RegionWalk::slot(int s, const JVal& fin, const JVal& x, const JVal& gu, const JVal& dn, const RegionDims& D, int64_t dn_in, int64_t* inter) {
    const std::string S = "slot " + std::to_string(s) + ": ";
    // down projection: linear(activation, select(down_weights, 0, s)), no bias
    if (!plain_call(fin, "aten.linear.default") || !arity(fin, 2, true)) return fail(S + "final op must be aten.linear.default (input, weight) without bias");
    const JVal* act = deref(*args(fin)[0]);
    const JVal* dsel = deref(*args(fin)[1]);
    if (!act || !dsel) return fail(S + "down linear operands must be node references");
    if (!plain_call(*dsel, "aten.select.int") || !arity(*dsel, 3) || deref(*args(*dsel)[0]) != &dn || !is_int(*args(*dsel)[1], 0) || !is_int(*args(*dsel)[2], s))
        return fail(S + "down weight select must be " + str(dn, "name") + "[0, " + std::to_string(s) + "]");
    if (!has_f32_shape(fin, {1, D.hidden})) return fail(S + "down output meta malformed");
    if (!has_f32_shape(*dsel, {D.hidden, dn_in})) return fail(S + "down slice meta malformed");
    // activation: gelu(gate, tanh) * up, gate and up the two items of one split
    if (!plain_call(*act, "aten.mul.Tensor") || !arity(*act, 2)) return fail(S + "activation must be aten.mul.Tensor");
    const JVal* gelu = deref(*args(*act)[0]);
    const JVal* up = deref(*args(*act)[1]);
    if (!gelu || !up) return fail(S + "activation operands must be node references");
    const JVal& gkw = kwargs(*gelu);
    if (str(*gelu, "op") != "call_function" || str(*gelu, "target") != "aten.gelu.default" || !arity(*gelu, 1) || gkw.obj.size() != 1 ||
        gkw.obj[0].first != "approximate" || gkw.obj[0].second->kind != JVal::Str || gkw.obj[0].second->s != "tanh")
        return fail(S + "gelu must be approximate='tanh' only");
    const JVal* gate = deref(*args(*gelu)[0]);
    if (!gate) return fail(S + "gelu operand must be a node reference");
    if (!plain_call(*gate, "operator.getitem") || !plain_call(*up, "operator.getitem") || !arity(*gate, 2) || !arity(*up, 2) ||
        !is_int(*args(*gate)[1], 0) || !is_int(*args(*up)[1], 1) || !deref(*args(*gate)[0]) || deref(*args(*gate)[0]) != deref(*args(*up)[0]))
        return fail(S + "gate/up must be getitems 0/1 of the SAME split");
    const JVal& split = *deref(*args(*gate)[0]);
    if (!plain_call(split, "aten.split.Tensor") || !arity(split, 3) || !is_int(*args(split)[2], -1)) return fail(S + "split must be (tensor, size, -1) with no kwargs");
    const JVal& sz = *args(split)[1];
    if (sz.kind != JVal::Int || sz.i <= 0 || sz.i > kDimCap) return fail(S + "split size must be a positive bounded int");
    if (*inter && *inter != sz.i) return fail(S + "split size " + std::to_string(sz.i) + " != " + std::to_string(*inter));
    *inter = sz.i;
    const JP* sm = split.get("meta");
    const JP* items = sm && (*sm)->kind == JVal::Obj ? (*sm)->get("items") : nullptr;
    const JP* sdt = sm && (*sm)->kind == JVal::Obj ? (*sm)->get("dtype") : nullptr;
    if (!items || !sdt || (*sdt)->kind != JVal::Str || (*sdt)->s != "seq" || (*items)->kind != JVal::Arr || (*items)->arr.size() != 2 ||
        !f32_shape(*(*items)->arr[0], {1, sz.i}) || !f32_shape(*(*items)->arr[1], {1, sz.i}))
        return fail(S + "split item metas must be 2x f32 [1, " + std::to_string(sz.i) + "]");
    if (!has_f32_shape(*gate, {1, sz.i}) || !has_f32_shape(*up, {1, sz.i}) || !has_f32_shape(*act, {1, sz.i})) return fail(S + "gate / up / activation meta malformed");
    // gate_up projection: linear(x, select(gu_weights, 0, s)), no bias, on the SHARED input
    const JVal* lin = deref(*args(split)[0]);
    if (!lin || !plain_call(*lin, "aten.linear.default") || !arity(*lin, 2, true) || deref(*args(*lin)[0]) != &x)
        return fail(S + "GU linear must take the SHARED x placeholder, no bias");
    const JVal* gsel = deref(*args(*lin)[1]);
    if (!gsel || !plain_call(*gsel, "aten.select.int") || !arity(*gsel, 3) || deref(*args(*gsel)[0]) != &gu || !is_int(*args(*gsel)[1], 0) || !is_int(*args(*gsel)[2], s))
        return fail(S + "GU weight select must be " + str(gu, "name") + "[0, " + std::to_string(s) + "]");
    if (!has_f32_shape(*lin, {1, D.gate_up_out})) return fail(S + "GU output meta malformed");
    if (!has_f32_shape(*gsel, {D.gate_up_out, D.hidden})) return fail(S + "GU slice meta malformed");
    return claim(fin, s, "down linear") && claim(*dsel, s, "down select") && claim(*act, s, "activation") && claim(*gelu, s, "gelu") &&
           claim(*gate, s, "gate") && claim(*up, s, "up") && claim(split, s, "split") && claim(*lin, s, "GU linear") && claim(*gsel, s, "GU select");
}

bool RegionWalk::run(const JVal& graph, RegionDims* out) {
    const std::vector<JP>& nodes = (*graph.get("nodes"))->arr;
    const std::vector<JP>& inputs = (*graph.get("inputs"))->arr;
    const std::vector<JP>& outputs = (*graph.get("outputs"))->arr;
    std::vector<const JVal*> placeholders, outs;
    for (auto& np : nodes) {
        const JVal& n = *np;
        const std::string& kind = str(n, "op");
        if (kind != "placeholder" && kind != "call_function" && kind != "output") return fail("unsupported node kind " + kind + " (" + str(n, "name") + ")");
        if (kind != "call_function" && !kwargs(n).obj.empty()) return fail(kind + " node " + str(n, "name") + " must carry no kwargs");
        if (!by_name_.emplace(str(n, "name"), &n).second) return fail("node name " + str(n, "name") + " appears twice");
        if (kind == "placeholder") placeholders.push_back(&n);
        if (kind == "output") outs.push_back(&n);
    }
    if (placeholders.size() != 3 || inputs.size() != 3) return fail("graph inputs must be the 3 placeholders");
    for (int i = 0; i < 3; i++)
        if (inputs[i]->kind != JVal::Str || inputs[i]->s != str(*placeholders[i], "name")) return fail("graph inputs must be the 3 placeholders");
    const JVal &x = *placeholders[0], &gu = *placeholders[1], &dn = *placeholders[2];
    std::vector<int64_t> xd, gd, dd;
    if (!placeholder_dims(x, 2, &xd) || !placeholder_dims(gu, 3, &gd) || !placeholder_dims(dn, 3, &dd)) return false;
    if (xd[0] != 1) return fail("x batch dim must be 1");
    RegionDims D;
    D.hidden = xd[1]; D.top_k = gd[0]; D.gate_up_out = gd[1];
    const int64_t dn_in = dd[2];
    if (gd[2] != D.hidden || dd[0] != D.top_k || dd[1] != D.hidden) return fail("input dims inconsistent with region");
    // one output packing one value: the stack of the slots
    if (outs.size() != 1 || outputs.empty() || outputs[0]->kind != JVal::Str || outputs[0]->s != str(*outs[0], "name") || args(*outs[0]).size() != 1 ||
        args(*outs[0])[0]->kind != JVal::Arr || args(*outs[0])[0]->arr.size() != 1)
        return fail("output must pack exactly one value");
    const JVal* stack = deref(*args(*outs[0])[0]->arr[0]);
    if (!stack || str(*stack, "op") != "call_function" || str(*stack, "target") != "aten.stack.default") return fail("output must be aten.stack.default");
    // stack(list, dim = 0): dim left out, second operand, or keyword
    const std::vector<JP>& sa = args(*stack);
    const JVal& skw = kwargs(*stack);
    const bool dim_ok = (sa.size() == 1 && skw.obj.empty()) || (sa.size() == 2 && skw.obj.empty() && is_int(*sa[1], 0)) ||
                        (sa.size() == 1 && skw.obj.size() == 1 && skw.obj[0].first == "dim" && is_int(*skw.obj[0].second, 0));
    if (!dim_ok || sa[0]->kind != JVal::Arr) return fail("stack must be (list of slots, dim 0)");
    const std::vector<JP>& slots = sa[0]->arr;
    if ((int64_t)slots.size() != D.top_k) return fail("stack has " + std::to_string(slots.size()) + " inputs != topK " + std::to_string(D.top_k));
    if (!has_f32_shape(*stack, {D.top_k, 1, D.hidden})) return fail("stack output meta malformed");
    claimed_.emplace(str(x, "name"), -1); claimed_.emplace(str(gu, "name"), -1); claimed_.emplace(str(dn, "name"), -1);
    if (!claim(*stack, -1, "stack") || !claim(*outs[0], -1, "output")) return false;
    int64_t inter = 0;
    for (size_t s = 0; s < slots.size(); s++) {
        const JVal* fin = deref(*slots[s]);
        if (!fin) return fail("slot " + std::to_string(s) + " final: expected a node reference");
        if (!slot((int)s, *fin, x, gu, dn, D, dn_in, &inter)) return false;
    }
    // exact census: every call is one the pattern claimed, in the pattern's counts
    std::map<std::string, int64_t> census;
    for (auto& np : nodes) {
        if (str(*np, "op") != "call_function") continue;
        census[str(*np, "target")]++;
        if (!claimed_.count(str(*np, "name"))) return fail("unconsumed/extra graph node " + str(*np, "target") + " (" + str(*np, "name") + ")");
    }
    const int64_t K = D.top_k;
    const std::map<std::string, int64_t> want = {{"aten.select.int", 2 * K}, {"aten.linear.default", 2 * K}, {"aten.split.Tensor", K},
                                                 {"aten.gelu.default", K}, {"aten.mul.Tensor", K}, {"aten.stack.default", 1}, {"operator.getitem", 2 * K}};
    if (census != want) return fail("ATen census does not match topK slots of select/linear/split/getitem/gelu/mul/linear");
    if (inter == 0) return fail("no slots");
    if (2 * inter != D.gate_up_out || dn_in != inter) return fail("inter " + std::to_string(inter) + " inconsistent with the expert tensors");
    D.inter = inter;
    *out = D;
    return true;
}

}  // namespace

struct lev_op {
    std::string kind, identity, kernel, tensor, view;
    int64_t in_dim = 0, out_dim = 0;
    int type = 0, columns = 1;
    int hidden = 0, inter = 0, top_k = 0;
};

static int bad(lev_ctx* ctx, const std::string& m) { return lev_fail(ctx, LEV_BAD_OP_SPEC, "%s", m.c_str()); }

static int parse_matvec(lev_ctx* ctx, const JVal& d, lev_op* op) {
    static const char* allowed[] = {"schema", "op", "semantics", "inDim", "outDim", "layout", "quant", "accumulate",
                                    "inputPrecision", "tensor", "view", "representativeRows", "columns"};
    for (auto& kv : d.obj) {
        bool ok = false;
        for (const char* a : allowed) ok |= kv.first == a;
        if (!ok) return bad(ctx, "unknown field " + kv.first);
    }
    auto S = [&](const char* k, std::string& out, bool optional) -> int {
        const JP* v = d.get(k);
        if (!v || (*v)->kind == JVal::Null) return optional ? 0 : 1;
        if ((*v)->kind != JVal::Str) return 1;
        out = (*v)->s; return 0;
    };
    auto I = [&](const char* k, int64_t& out, bool optional) -> int {
        const JP* v = d.get(k);
        if (!v || (*v)->kind == JVal::Null) return optional ? 2 : 1;
        if ((*v)->kind != JVal::Int) return 1;
        out = (*v)->i; return 0;
    };
    int64_t schema = 0, in_dim = 0, out_dim = 0, rep = 0, columns = 1;
    std::string opn, sem, layout, quant, acc, prec, tensor, view;
    if (I("schema", schema, false) || S("op", opn, false) || S("semantics", sem, false) || I("inDim", in_dim, false) ||
        I("outDim", out_dim, false) || S("layout", layout, false) || S("quant", quant, false) || S("accumulate", acc, false) ||
        S("inputPrecision", prec, false) || S("tensor", tensor, true) || S("view", view, true))
        return bad(ctx, "op JSON decode: a required field is missing or has the wrong type");
    if (schema != 1) return bad(ctx, "schema " + std::to_string(schema) + " != 1");
    int type = quant == "q4_0" ? LEV_GGML_Q4_0 : quant == "q4_k" ? LEV_GGML_Q4_K : quant == "q6_k" ? LEV_GGML_Q6_K : -1;
    bool gemm = opn == quant + ".gemm";
    if (type < 0 || (opn != quant + ".matvec" && !gemm) || sem != "dot(W_row, x)")
        return bad(ctx, "unsupported op/semantics " + opn + "/" + sem);
    if (layout != "row-major-" + quant + "-blocks") return bad(ctx, "unsupported layout/quant " + layout + "/" + quant);
    const std::string want_prec = gemm ? "bf16" : "f32";
    if (acc != "f32" || prec != want_prec) return bad(ctx, "unsupported accumulate/inputPrecision");
    if (!view.empty() && view != "expert-row-slice" && view != "attention-output-family") return bad(ctx, "unsupported view " + view);
    if (view == "expert-row-slice" && !(ends_with(tensor, ".ffn_gate_up_exps.weight") || ends_with(tensor, ".ffn_down_exps.weight")))
        return bad(ctx, "expert-row-slice binds a blk.<L>.ffn_{gate_up,down}_exps.weight tensor");
    if (view == "attention-output-family" && !is_attn_output_name(tensor))
        return bad(ctx, "attention-output-family binds a strict blk.<digits>.attn_output.weight tensor, got " + (tensor.empty() ? "nil" : tensor));
    if (in_dim <= 0 || out_dim <= 0 || in_dim % lev_block_values(type) || in_dim > LEV_MAX_DIM || out_dim > LEV_MAX_DIM)
        return bad(ctx, "bad dims inDim " + std::to_string(in_dim) + " outDim " + std::to_string(out_dim));
    int r = I("representativeRows", rep, true);
    if (r == 1 || (r == 0 && (rep <= 0 || rep > out_dim || rep > 4096))) return bad(ctx, "representativeRows " + std::to_string(rep) + " out of bounds");
    int c = I("columns", columns, true);
    if (c == 1 || (c == 0 && (columns < 1 || (!gemm && columns > LEV_MAX_COLUMNS)))) return bad(ctx, "columns " + std::to_string(columns) + " out of bounds");
    // identity: sorted keys, compact, absent optionals omitted
    std::map<std::string, std::string> enc;
    for (auto& kv : d.obj) {
        if (kv.second->kind == JVal::Null) continue;
        enc[kv.first] = kv.second->kind == JVal::Str ? json_quote(kv.second->s) : std::to_string(kv.second->i);
    }
    std::string canon = "{";
    for (auto& kv : enc) { if (canon.size() > 1) canon += ","; canon += json_quote(kv.first) + ":" + kv.second; }
    canon += "}";
    Sha256 h; h.update(canon.data(), canon.size());
    op->kind = opn; op->identity = h.hex(); op->in_dim = in_dim; op->out_dim = out_dim; op->type = type;
    op->columns = (int)columns; op->tensor = tensor; op->view = view;
    op->kernel = gemm ? "lev_gemm_prefill" : (type == LEV_GGML_Q6_K ? "lev_matvec_plain" : "lev_matvec_stream");
    return LEV_OK;
}

static int parse_region(lev_ctx* ctx, const JVal& d, lev_op* op) {
    static const char* allowed[] = {"schema", "region", "hidden", "expertIntermediate", "topK", "gateUpOut", "geluApprox",
                                    "stackOutputs", "slotOps", "guTensor", "dnTensor", "graph", "graphSha256", "torch"};
    for (auto& kv : d.obj) {
        bool ok = false;
        for (const char* a : allowed) ok |= kv.first == a;
        if (!ok) return bad(ctx, "unknown field " + kv.first);
    }
    auto geti = [&](const char* k, int64_t& o) { const JP* v = d.get(k); if (!v || (*v)->kind != JVal::Int) return false; o = (*v)->i; return true; };
    auto gets = [&](const char* k, std::string& o) { const JP* v = d.get(k); if (!v || (*v)->kind != JVal::Str) return false; o = (*v)->s; return true; };
    int64_t schema, hidden, inter, topk, guo;
    std::string region, gelu, gu, dn, sha;
    if (!geti("schema", schema) || !gets("region", region) || !geti("hidden", hidden) || !geti("expertIntermediate", inter) ||
        !geti("topK", topk) || !geti("gateUpOut", guo) || !gets("geluApprox", gelu) || !gets("guTensor", gu) || !gets("dnTensor", dn) ||
        !gets("graphSha256", sha))
        return bad(ctx, "region JSON decode: a required field is missing or has the wrong type");
    if (schema != 1 || region != "gemma4.moe.routed-region") return bad(ctx, "unsupported schema/region " + region);
    if (hidden <= 0 || inter <= 0 || hidden % 32 || inter % 32 || hidden > 8192 || inter > 8192) return bad(ctx, "region dims out of bounds");
    if (topk <= 0 || topk > LEV_MAX_TOP_K) return bad(ctx, "topK out of bounds");
    if (guo != 2 * inter) return bad(ctx, "gateUpOut must be 2 * expertIntermediate");
    if (gelu != "tanh") return bad(ctx, "geluApprox must be tanh");
    const JP* so = d.get("stackOutputs");
    if (!so || (*so)->kind != JVal::Bool || !(*so)->b) return bad(ctx, "stackOutputs must be true");
    static const char* slot_ops[3] = {"q4_0.expert-slice-linear-gate-up", "gelu-tanh-split-mul", "q4_0.expert-slice-linear-down"};
    const JP* sl = d.get("slotOps");
    if (!sl || (*sl)->kind != JVal::Arr || (*sl)->arr.size() != 3) return bad(ctx, "slotOps must name the three slot operators");
    for (int i = 0; i < 3; i++) if ((*sl)->arr[i]->kind != JVal::Str || (*sl)->arr[i]->s != slot_ops[i]) return bad(ctx, "slotOps must name the three slot operators");
    if (!ends_with(gu, ".ffn_gate_up_exps.weight") || !ends_with(dn, ".ffn_down_exps.weight")) return bad(ctx, "expert tensor names");
    const JP* g = d.get("graph");
    if (!g || (*g)->kind != JVal::Obj) return bad(ctx, "graph missing");
    const JP* nodes = (*g)->get("nodes"); const JP* ins = (*g)->get("inputs"); const JP* outs = (*g)->get("outputs");
    if (!nodes || !ins || !outs || (*nodes)->kind != JVal::Arr || (*ins)->kind != JVal::Arr || (*outs)->kind != JVal::Arr)
        return bad(ctx, "graph needs nodes, inputs, outputs");
    if ((*nodes)->arr.size() > 512) return bad(ctx, "graph exceeds 512 nodes");
    std::string payload;
    for (auto& n : (*nodes)->arr) {
        if (n->kind != JVal::Obj) return bad(ctx, "graph node is not an object");
        const JP* name = n->get("name"); const JP* nop = n->get("op"); const JP* tgt = n->get("target");
        const JP* args = n->get("args"); const JP* kw = n->get("kwargs"); const JP* meta = n->get("meta");
        if (!name || !nop || !tgt || !args || !kw || (*name)->kind != JVal::Str || (*nop)->kind != JVal::Str ||
            (*tgt)->kind != JVal::Str || (*args)->kind != JVal::Arr || (*kw)->kind != JVal::Obj)
            return bad(ctx, "graph node fields");
        std::string line = (*name)->s + "|" + (*nop)->s + "|" + (*tgt)->s + "|";
        if (!canon_val(**args, line)) return bad(ctx, "unsupported operand kind");
        line += "|d<";
        std::map<std::string, JP> sorted((*kw)->obj.begin(), (*kw)->obj.end());
        bool first = true;
        for (auto& kv : sorted) { if (!first) line += ","; first = false; line += kv.first + ":"; if (!canon_val(*kv.second, line)) return bad(ctx, "unsupported operand kind"); }
        line += ">|";
        if (meta && (*meta)->kind != JVal::Null) { if (!canon_meta(**meta, line)) return bad(ctx, "node meta"); } else line += "n";
        payload += line + "\n";
    }
    auto strlist = [&](const JVal& a, std::string& o) { o += "l<"; for (size_t i = 0; i < a.arr.size(); i++) { if (i) o += ","; o += "s:" + a.arr[i]->s; } o += ">"; };
    payload += "inputs|"; strlist(**ins, payload);
    payload += "\noutputs|"; strlist(**outs, payload);
    Sha256 h; h.update(payload.data(), payload.size());
    std::string digest = h.hex();
    if (digest != sha) return bad(ctx, "graphSha256 does not match the graph (" + digest + ")");
    const int K = (int)topk;
    // re-derive the region from the graph; the declared dims must agree with it
    RegionWalk walk;
    RegionDims D;
    if (!walk.run(**g, &D)) return bad(ctx, "region graph: " + walk.err);
    if (D.hidden != hidden || D.inter != inter || D.top_k != topk || D.gate_up_out != guo)
        return bad(ctx, "declared dims disagree with the graph-derived hidden " + std::to_string(D.hidden) + " inter " + std::to_string(D.inter) +
                            " topK " + std::to_string(D.top_k) + " gateUpOut " + std::to_string(D.gate_up_out));
    op->kind = "moe.routed-region"; op->identity = digest; op->in_dim = hidden; op->out_dim = hidden; op->type = LEV_GGML_Q4_0;
    op->columns = 1; op->hidden = (int)hidden; op->inter = (int)inter; op->top_k = K; op->tensor = gu; op->kernel = "lev_moe_experts";
    return LEV_OK;
}

extern "C" int lev_op_install_json(lev_ctx* ctx, const char* json, size_t json_len, lev_op** out) {
    if (!json || !out) return LEV_BAD_ARGUMENT;
    *out = nullptr;
    JParser P{json, json + json_len};
    JP root;
    if (!P.value(root)) return bad(ctx, "op JSON decode: " + P.err);
    P.ws();
    if (P.p != P.end) return bad(ctx, "op JSON decode: trailing characters");
    if (root->kind != JVal::Obj) return bad(ctx, "op JSON decode: not an object");
    lev_op* op = new (std::nothrow) lev_op();
    if (!op) return lev_fail(ctx, LEV_OUT_OF_MEMORY, "host allocation");
    int st;
    if (root->get("region")) {
        st = json_len > (512u << 10) ? bad(ctx, "region JSON exceeds 512 KiB") : parse_region(ctx, *root, op);
    } else {
        st = json_len > (1u << 16) ? bad(ctx, "op JSON exceeds 64 KiB") : parse_matvec(ctx, *root, op);
    }
    if (st) { delete op; return st; }
    *out = op;
    return LEV_OK;
}

extern "C" int lev_op_uninstall(lev_ctx* ctx, lev_op* op) {
    (void)ctx;
    if (!op) return LEV_BAD_ARGUMENT;
    delete op;
    return LEV_OK;
}

extern "C" int lev_op_describe(const lev_op* op, char* kind, int64_t* in_dim, int64_t* out_dim, int* type, int* columns,
                               char* identity_hex, char* kernel_name) {
    if (!op) return LEV_BAD_ARGUMENT;
    if (kind) snprintf(kind, 32, "%s", op->kind.c_str());
    if (in_dim) *in_dim = op->in_dim;
    if (out_dim) *out_dim = op->out_dim;
    if (type) *type = op->type;
    if (columns) *columns = op->columns;
    if (identity_hex) snprintf(identity_hex, 65, "%s", op->identity.c_str());
    if (kernel_name) snprintf(kernel_name, 64, "%s", op->kernel.c_str());
    return LEV_OK;
}

// An op serves a resident tensor of its quant and inDim whose row window is
// its outDim; under the expert view the tensor is a stack of outDim-row slices.
extern "C" int lev_op_serves(const lev_op* op, const lev_weights* w, int64_t rows) {
    if (!op || !w || op->kind == "moe.routed-region") return 0;
    if (w->type != op->type || w->cols != op->in_dim || rows != op->out_dim) return 0;
    if (op->view == "expert-row-slice") return w->rows % op->out_dim == 0;
    return w->rows == op->out_dim || !op->view.empty() ? 1 : 0;
}
