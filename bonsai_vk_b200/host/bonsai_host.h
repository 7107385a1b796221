// bonsai_host.h - C++17 host above the C ABI: GGUF reader, model plan with the prism.hadamard contract, loader.
//
// Mirrors the reference host's behaviour for the decode path (all paths relative to the reference tree):
//   gguf_load            runtime_vk/bonsai_gguf.h:72-155      v3 header, KV types 0-12, tensor table, data start
//   model_plan_hparams   runtime_vk/bonsai_model.h:642-760    hyper-parameters only from GGUF metadata
//   model_plan_contract  runtime_vk/bonsai_model.h:773-912    prism.hadamard.* gate (refuse before any GPU work)
//   model_plan_build     runtime_vk/bonsai_model.h:1013-1078  dtype 143 (PTQ1_0) / 0 (f32) only, K % 128 == 0
//   load_ptq_weights     runtime_vk/bonsai_weights.h:502-558  file -> staging -> device, here without any repack
// Written from the documented behaviour; no reference source text is reproduced.
#pragma once

#include "../../include/bonsai_cuda.h"

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <vector>

namespace bh {

struct Tensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t d[4] = {1, 1, 1, 1};
    uint32_t dtype = 0;
    uint64_t off = 0;        // relative to data_start
    uint64_t bytes = 0;
};

struct Gguf {
    uint32_t version = 0, alignment = 32;
    uint64_t data_start = 0;
    std::map<std::string, int64_t> ki;
    std::map<std::string, double> kf;
    std::map<std::string, std::string> ks;
    std::map<std::string, std::vector<int64_t>> ai;       // numeric arrays
    std::map<std::string, std::vector<std::string>> as;   // string arrays
    std::vector<Tensor> tensors;
};

class Reader {
public:
    explicit Reader(FILE *f) : f_(f) {}
    bool ok() const { return ok_; }
    template <class T> T get() { T v{}; if (fread(&v, sizeof v, 1, f_) != 1) ok_ = false; return v; }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok_ || n > (1ull << 30)) { ok_ = false; return {}; }
        std::string s(n, '\0');
        if (n && fread(&s[0], 1, n, f_) != n) ok_ = false;
        return s;
    }
private:
    FILE *f_;
    bool ok_ = true;
};

// One GGUF metadata value. The fixed-width kinds are described by a table (bytes, signed, floating) and read in one
// place; strings are length-prefixed. Type numbers are the GGUF specification's (0..12, 9 = array).
struct Value { int64_t i = 0; double f = 0; std::string s; bool is_float = false, is_string = false; };
inline bool read_value(Reader &r, uint32_t ty, Value &v) {
    struct Kind { int bytes; bool sign, flt; };
    static const Kind kinds[13] = {{1, false, false}, {1, true, false}, {2, false, false}, {2, true, false}, {4, false, false}, {4, true, false},
                                   {4, true, true}, {1, false, false}, {0, false, false}, {-1, false, false}, {8, false, false}, {8, true, false},
                                   {8, true, true}};
    if (ty > 12 || kinds[ty].bytes < 0) return false;
    v = Value();
    if (ty == 8) { v.s = r.str(); v.is_string = true; return r.ok(); }
    const Kind k = kinds[ty];
    uint64_t raw = 0;
    for (int b = 0; b < k.bytes; ++b) raw |= uint64_t(r.get<uint8_t>()) << (8 * b);      // little endian
    if (k.flt) {
        v.is_float = true;
        if (k.bytes == 4) { uint32_t w = uint32_t(raw); float x; memcpy(&x, &w, 4); v.f = x; } else memcpy(&v.f, &raw, 8);
    } else if (k.sign && k.bytes < 8) {
        const int sh = 64 - 8 * k.bytes;
        v.i = int64_t(raw << sh) >> sh;
    } else v.i = int64_t(raw);
    return r.ok();
}

inline uint64_t tensor_bytes(const Tensor &t, std::string &why) {
    uint64_t n = 1;
    for (uint32_t i = 0; i < t.n_dims; ++i) n *= t.d[i];
    if (t.dtype == 0) return n * 4;
    if (t.dtype == 143) {
        if (t.d[0] % 128) { why = "tensor " + t.name + ": PTQ1_0 needs d0 (the reduction length) to be a multiple of 128"; return 0; }
        return n / 128 * 28;
    }
    why = "tensor " + t.name + ": dtype " + std::to_string(t.dtype) + " is neither PTQ1_0 (143) nor f32 (0)";
    return 0;
}

inline bool gguf_load(const char *path, Gguf &g, std::string &why) {
    FILE *f = fopen(path, "rb");
    if (!f) { why = std::string("cannot open ") + path; return false; }
    struct Closer { FILE *f; ~Closer() { fclose(f); } } closer{f};
    fseek(f, 0, SEEK_END);
    const uint64_t file_size = uint64_t(ftell(f));
    fseek(f, 0, SEEK_SET);
    Reader r(f);
    char magic[4] = {};
    if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "GGUF", 4) != 0) { why = std::string(path) + " is not a GGUF file"; return false; }
    g.version = r.get<uint32_t>();
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok() || n_tensors > (1u << 20) || n_kv > (1u << 20)) { why = "truncated or implausible GGUF header"; return false; }
    // metadata: scalars by kind into ki / kf / ks, arrays into ai / as. An array cannot hold more elements than the file
    // has bytes left: a corrupt count is refused before anything is allocated for it.
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = r.str();
        const uint32_t ty = r.get<uint32_t>();
        if (!r.ok()) { why = "truncated GGUF metadata"; return false; }
        if (ty == 9) {
            const uint32_t et = r.get<uint32_t>();
            const uint64_t n = r.get<uint64_t>();
            if (!r.ok() || n > file_size - std::min<uint64_t>(file_size, uint64_t(ftell(f)))) { why = "array " + key + " is longer than the file"; return false; }
            if (et == 8) {
                std::vector<std::string> &dst = g.as[key];
                dst.reserve(n);
                for (uint64_t k = 0; k < n && r.ok(); ++k) dst.push_back(r.str());
            } else {
                std::vector<int64_t> &dst = g.ai[key];
                dst.reserve(n);
                Value v;
                for (uint64_t k = 0; k < n; ++k) {
                    if (!read_value(r, et, v) || v.is_string) { why = "bad array element type in " + key; return false; }
                    dst.push_back(v.is_float ? int64_t(v.f) : v.i);
                }
            }
        } else {
            Value v;
            if (!read_value(r, ty, v)) { why = "bad value type for key " + key; return false; }
            if (v.is_string) g.ks[key] = v.s; else if (v.is_float) g.kf[key] = v.f; else g.ki[key] = v.i;
        }
        if (!r.ok()) { why = "truncated GGUF metadata at key " + key; return false; }
    }
    g.tensors.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        Tensor t;
        t.name = r.str();
        t.n_dims = r.get<uint32_t>();
        if (!r.ok() || t.n_dims > 4) { why = "tensor table: entry " + std::to_string(i) + " (" + t.name + ") is truncated or has more than 4 dims"; return false; }
        for (uint32_t k = 0; k < t.n_dims; ++k) t.d[k] = r.get<uint64_t>();
        t.dtype = r.get<uint32_t>();
        t.off = r.get<uint64_t>();
        if (!r.ok()) { why = "truncated GGUF tensor table"; return false; }
        t.bytes = tensor_bytes(t, why);
        if (!t.bytes) return false;
        g.tensors.push_back(t);
    }
    const auto al = g.ki.find("general.alignment");
    if (al != g.ki.end() && al->second > 0) g.alignment = uint32_t(al->second);
    const uint64_t table_end = uint64_t(ftell(f));
    g.data_start = (table_end + g.alignment - 1) / g.alignment * g.alignment;
    // every tensor's bytes must lie inside the file (a truncated download otherwise shows up as a short read mid-load)
    for (const Tensor &t : g.tensors)
        if (t.off > file_size || t.bytes > file_size - t.off || g.data_start > file_size - t.off - t.bytes) {
            why = "tensor " + t.name + " lies outside the file (" + std::to_string(file_size) + " bytes): truncated GGUF";
            return false;
        }
    return true;
}

// ---- layer typing -------------------------------------------------------------------------------------------------
// Which blocks are softmax-attention blocks and which are gated-delta-net blocks, from every spelling the reference
// loader accepts (contract: bonsai_model.h:432-472): S1 an explicit per-layer list, S2 the interval key, S3 counts
// (cross-check only), S4 the tensor table (always computed). Every spelling that answers must give the same mask.
inline bool is_attn_block(const bn_hparams &h, int b) {
    return h.attn_interval > 0 ? (b % h.attn_interval) == h.attn_interval - 1
                               : (((uint64_t(h.attn_mask_hi) << 32 | h.attn_mask_lo) >> b) & 1ull) != 0;
}
// 1 = attention, 0 = recurrent, -1 = a kind this engine has no kernels for (refused, never remapped), -2 = unknown word
inline int layer_token_kind(std::string t) {
    while (!t.empty() && (t.back() == ' ' || t.back() == ',' || t.back() == ';')) t.pop_back();
    while (!t.empty() && t.front() == ' ') t.erase(t.begin());
    for (char &c : t) if (c >= 'A' && c <= 'Z') c = char(c - 'A' + 'a');
    static const char *attn[] = {"full_attention", "attention", "attn", "full", "softmax", "self", "1"};
    static const char *rec[] = {"ssm", "gdn", "gated_delta", "gated_delta_net", "linear_attention", "linear", "recurrent", "mamba", "none", "0"};
    static const char *refused[] = {"sliding_attention", "sliding_window", "window", "windowed", "chunked", "moe", "hybrid"};
    for (const char *w : attn) if (t == w) return 1;
    for (const char *w : rec) if (t == w) return 0;
    for (const char *w : refused) if (t == w) return -1;
    return -2;
}
inline bool layer_mask_from_tokens(const std::vector<std::string> &tok, int n_layer, const std::string &key, uint64_t &mask, std::string &why) {
    if (int(tok.size()) != n_layer) { why = key + " has " + std::to_string(tok.size()) + " entries, block_count is " + std::to_string(n_layer); return false; }
    mask = 0;
    for (int b = 0; b < n_layer; ++b) {
        const int k = layer_token_kind(tok[b]);
        if (k == -1) { why = key + ": block " + std::to_string(b) + " is '" + tok[b] + "', a layer kind this engine has no kernels for"; return false; }
        if (k == -2) { why = key + ": block " + std::to_string(b) + " has the unknown layer type '" + tok[b] + "'"; return false; }
        if (k == 1) mask |= 1ull << b;
    }
    return true;
}
// rc 0: h.attn_interval / h.attn_mask_* set. rc 2: refused, `why` says which spellings disagree or what is malformed.
inline int resolve_layer_types(const Gguf &g, const std::string &arch, bn_hparams &h, std::string &why) {
    const int n = h.n_layer;
    if (n < 1 || n > 64) { why = "block_count " + std::to_string(n) + " is outside [1, 64] (the layer mask is 64 bits)"; return 2; }
    const std::string prefixes[] = {arch + ".", "prism."};
    struct Answer { std::string from; uint64_t mask; };
    std::vector<Answer> answers;
    // S1 explicit list
    static const char *sufs[] = {"attention.layer_types", "layer_types", "layers.types"};
    for (const std::string &P : prefixes) for (const char *s : sufs) {
        const std::string key = P + s;
        std::vector<std::string> tok;
        bool have = false;
        if (auto it = g.as.find(key); it != g.as.end()) { tok = it->second; have = true; }
        else if (auto it2 = g.ai.find(key); it2 != g.ai.end()) { for (int64_t v : it2->second) tok.push_back(std::to_string(v)); have = true; }
        else if (auto it3 = g.ks.find(key); it3 != g.ks.end()) {
            std::string cur;
            for (char c : it3->second + " ") {
                if (c == ' ' || c == ',' || c == ';') { if (!cur.empty()) tok.push_back(cur); cur.clear(); } else cur.push_back(c);
            }
            have = true;
        }
        if (!have) continue;
        uint64_t m = 0;
        if (!layer_mask_from_tokens(tok, n, key, m, why)) return 2;
        answers.push_back({key, m});
    }
    const bool have_list = !answers.empty();
    // S2 interval
    int interval = 0;
    for (const std::string &P : prefixes) {
        auto it = g.ki.find(P + "full_attention_interval");
        if (it == g.ki.end()) continue;
        if (it->second < 1) { why = P + "full_attention_interval = " + std::to_string(it->second) + ": must be >= 1 (a file whose layers are all attention says so with a layer list)"; return 2; }
        if (interval && interval != int(it->second)) { why = "two full_attention_interval keys disagree"; return 2; }
        interval = int(it->second);
        uint64_t m = 0;
        for (int b = 0; b < n; ++b) if ((b + 1) % interval == 0) m |= 1ull << b;
        answers.push_back({P + "full_attention_interval", m});
    }
    const bool have_rule = have_list || interval > 0;
    // S4 tensor table
    {
        std::set<std::string> names;
        for (const Tensor &t : g.tensors) names.insert(t.name);
        uint64_t m = 0;
        for (int b = 0; b < n; ++b) {
            const std::string B = "blk." + std::to_string(b) + ".";
            const bool a = names.count(B + "attn_q.weight") || names.count(B + "attn_k.weight") || names.count(B + "attn_v.weight");
            const bool r = names.count(B + "attn_qkv.weight") != 0;
            if (a && r) { why = "block " + std::to_string(b) + " carries both attention (attn_q/k/v) and recurrent (attn_qkv) tensors"; return 2; }
            if (!a && !r) { why = "block " + std::to_string(b) + " carries neither attn_q/k/v nor attn_qkv: it cannot be typed (a draft/MTP block has no path here)"; return 2; }
            if (a) m |= 1ull << b;
        }
        answers.push_back({"the tensor table", m});
    }
    // S3 counts: cross-checks only
    auto popcount = [](uint64_t v) { int c = 0; for (; v; v &= v - 1) ++c; return c; };
    static const char *rec_counts[] = {"ssm_layer_count", "linear_attention_layer_count", "recurrent_layer_count", "gdn_layer_count"};
    static const char *attn_counts[] = {"attn_layer_count", "full_attention_layer_count"};
    for (const std::string &P : prefixes) {
        for (int kind = 0; kind < 2; ++kind) {
            const char *const *keys = kind ? attn_counts : rec_counts;
            const int nkeys = kind ? 2 : 4;
            for (int i = 0; i < nkeys; ++i) {
                auto it = g.ki.find(P + keys[i]);
                if (it == g.ki.end()) continue;
                if (!have_rule) { why = P + keys[i] + " is present but neither a layer list nor full_attention_interval: a count cannot say where the layers are"; return 2; }
                const int want = kind ? popcount(answers[0].mask) : n - popcount(answers[0].mask);
                if (it->second != want) { why = P + keys[i] + " = " + std::to_string(it->second) + " but " + answers[0].from + " gives " + std::to_string(want); return 2; }
            }
        }
    }
    // agreement
    for (size_t i = 1; i < answers.size(); ++i)
        if (answers[i].mask != answers[0].mask) {
            char buf[64];
            snprintf(buf, sizeof buf, "%016llx vs %016llx", (unsigned long long)answers[0].mask, (unsigned long long)answers[i].mask);
            why = "layer typing disagrees: " + answers[0].from + " and " + answers[i].from + " give different attention masks (" + buf + ")";
            return 2;
        }
    const uint64_t mask = answers[0].mask;
    h.attn_mask_lo = uint32_t(mask); h.attn_mask_hi = uint32_t(mask >> 32);
    h.attn_interval = (interval > 0 && !have_list) ? interval : 0;
    // an explicit list that happens to be an interval pattern stays a list: both forms give the same schedule
    return 0;
}

struct Plan {
    bn_hparams hp = {};
    std::vector<int32_t> signs;
    int64_t hat_version = 0;
};

// hyper-parameters and the rotation contract; `why` explains a refusal. rc: 0 ok, 2 contract/metadata, 6 rotation refusal
inline int plan_build(const Gguf &g, Plan &p, int cap, std::string &why) {
    auto arch_it = g.ks.find("general.architecture");
    if (arch_it == g.ks.end()) { why = "general.architecture is missing"; return 2; }
    const std::string A = arch_it->second + ".";
    auto I = [&](const std::string &k, int64_t &out) { auto it = g.ki.find(A + k); if (it == g.ki.end()) { why = "metadata key " + A + k + " is missing"; return false; } out = it->second; return true; };
    auto F = [&](const std::string &k, double &out) { auto it = g.kf.find(A + k); if (it == g.kf.end()) { why = "metadata key " + A + k + " is missing"; return false; } out = it->second; return true; };
    int64_t v = 0; double d = 0;
    bn_hparams &h = p.hp;
    if (!I("block_count", v)) return 2; h.n_layer = int(v);
    if (!I("embedding_length", v)) return 2; h.hidden = int(v);
    if (!I("feed_forward_length", v)) return 2; h.ffn = int(v);
    if (!I("attention.head_count", v)) return 2; h.n_head = int(v);
    if (!I("attention.head_count_kv", v)) return 2; h.n_kv = int(v);
    if (!I("attention.key_length", v)) return 2; h.head_dim = int(v);
    int64_t vl = 0;
    if (!I("attention.value_length", vl)) return 2;
    if (vl != h.head_dim) { why = "attention.value_length differs from key_length"; return 2; }
    if (!I("rope.dimension_count", v)) return 2; h.n_rot = int(v);
    if (int rc = resolve_layer_types(g, arch_it->second, h, why)) return rc;
    if (!I("ssm.conv_kernel", v)) return 2; if (v != 4) { why = "ssm.conv_kernel must be 4"; return 2; }
    if (!I("ssm.state_size", v)) return 2; h.gdn_dim = int(v);
    if (!I("ssm.group_count", v)) return 2; h.gdn_qk_heads = int(v);
    if (!I("ssm.time_step_rank", v)) return 2; h.gdn_heads = int(v);
    if (!I("ssm.inner_size", v)) return 2; if (v != int64_t(h.gdn_heads) * h.gdn_dim) { why = "ssm.inner_size != time_step_rank * state_size"; return 2; }
    if (!F("attention.layer_norm_rms_epsilon", d)) return 2; h.rms_eps = float(d);
    if (!F("rope.freq_base", d)) return 2; h.rope_base = float(d);
    auto tok = g.as.find("tokenizer.ggml.tokens");
    if (tok == g.as.end() || tok->second.empty()) { why = "tokenizer.ggml.tokens is missing (its length is the vocabulary size)"; return 2; }
    h.vocab = int(tok->second.size());
    if (int64_t(h.n_head) * h.head_dim != h.hidden) { why = "head_count * key_length != embedding_length"; return 2; }
    h.cap = cap; h.act_mode = 0; h.k_mode = 0; h.v_mode = 0;
    // ---- prism.hadamard.* (absent / 0 = no rotation -> this forward refuses; > 1 refused)
    auto hv = g.ki.find("prism.hadamard.version");
    p.hat_version = hv == g.ki.end() ? 0 : hv->second;
    if (p.hat_version == 0) { why = "prism.hadamard.version = 0: the file declares no activation rotation, but this forward applies signs + Hadamard before every ternary projection; refusing instead of rotating a model that was never rotated"; return 6; }
    if (p.hat_version != 1) { why = "prism.hadamard.version = " + std::to_string(p.hat_version) + ": only version 1 (normalized Sylvester-Walsh block transform) is implemented"; return 2; }
    auto tx = g.ks.find("prism.hadamard.transform");
    if (tx == g.ks.end() || tx->second != "normalized-sylvester-walsh-hadamard") { why = "prism.hadamard.transform must be normalized-sylvester-walsh-hadamard"; return 2; }
    auto bs = g.ki.find("prism.hadamard.block_size");
    if (bs == g.ki.end()) { why = "prism.hadamard.block_size is missing"; return 2; }
    h.hat_block = int(bs->second);
    if (h.hat_block < 16 || h.hat_block > 4096 || (h.hat_block & (h.hat_block - 1)) || h.hidden % h.hat_block || h.ffn % h.hat_block) { why = "prism.hadamard.block_size must be a power of two in [16, 4096] dividing hidden and ffn"; return 2; }
    auto sw = g.ai.find("prism.hadamard.sign_widths"), sv = g.ai.find("prism.hadamard.sign_values");
    if (sw == g.ai.end() || sv == g.ai.end()) { why = "prism.hadamard.sign_widths / sign_values are missing"; return 2; }
    int64_t sum = 0;
    for (int64_t w : sw->second) { if (w != h.hidden && w != h.ffn) { why = "prism.hadamard.sign_widths must be a subset of {hidden, ffn}"; return 2; } sum += w; }
    if (sum != int64_t(sv->second.size()) || sum != int64_t(h.hidden) + h.ffn) { why = "prism.hadamard.sign_values length must equal the sum of sign_widths = hidden + ffn"; return 2; }
    p.signs.resize(sv->second.size());
    for (size_t i = 0; i < p.signs.size(); ++i) { const int64_t s = sv->second[i]; if (s != 1 && s != -1) { why = "prism.hadamard.sign_values must be +-1"; return 2; } p.signs[i] = int32_t(s); }
    return 0;
}

struct Engine {
    bn_ctx *ctx = nullptr;
    bn_buf *weights = nullptr;
    bn_model *model = nullptr;
    Plan plan;
    double load_ms = 0;
};

// Device order of the weights: projections that read the same input are placed back to back (qkv|gate, q|k|v,
// ffn_gate|ffn_up) whatever their order in the file, so that the token schedule can run each group as one launch.
inline long layout_rank(const std::string &n) {
    static const char *order[] = {"attn_norm.weight", "attn_qkv.weight", "attn_gate.weight", "attn_q.weight", "attn_k.weight",
                                  "attn_v.weight", "attn_output.weight", "ssm_out.weight", "post_attention_norm.weight",
                                  "ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"};
    if (n.rfind("blk.", 0) != 0) return n == "token_embd.weight" ? -2 : (n == "output.weight" ? 1L << 40 : -1);
    const long b = strtol(n.c_str() + 4, nullptr, 10);
    const size_t dot = n.find('.', 4);
    const std::string suffix = dot == std::string::npos ? "" : n.substr(dot + 1);
    long r = 63;
    for (int i = 0; i < int(sizeof order / sizeof *order); ++i) if (suffix == order[i]) r = i;
    return b * 64 + r;
}

// Upload every tensor (native bytes; 256-byte aligned starts) and register it by name. rc 3 = load error.
inline int engine_load(Engine &e, const char *path, const Gguf &g, size_t chunk_bytes, std::string &why) {
    auto al = [](uint64_t n) { return (n + 255) & ~uint64_t(255); };
    std::vector<const Tensor *> order;
    for (const Tensor &t : g.tensors) order.push_back(&t);
    std::stable_sort(order.begin(), order.end(), [](const Tensor *a, const Tensor *b) { return layout_rank(a->name) < layout_rank(b->name); });
    uint64_t total = al(e.plan.signs.size() * 4);
    for (const Tensor &t : g.tensors) total += al(t.bytes);
    if (bn_alloc(e.ctx, total, &e.weights)) { why = bn_last_error(); return 3; }
    if (bn_model_create(e.ctx, &e.plan.hp, &e.model)) { why = bn_last_error(); return 2; }
    FILE *f = fopen(path, "rb");
    if (!f) { why = "cannot reopen the GGUF"; return 3; }
    // Two page-locked staging buffers: while the copy of one piece runs on the device's copy engine, the next piece
    // is read from the file into the other buffer. bn_sync before a buffer is queued confirms that the copy queued one
    // step earlier (out of the other buffer) is done, so a buffer is never overwritten while it is still being copied.
    void *stage[2] = {nullptr, nullptr};
    auto drop = [&]() { for (void *&s : stage) if (s) { bn_host_free(s); s = nullptr; } fclose(f); };
    for (void *&s : stage) if (bn_host_alloc(chunk_bytes, &s)) { why = bn_last_error(); drop(); return 3; }
    uint64_t off = 0;
    int cur = 0;
    for (const Tensor *tp : order) {
        const Tensor &t = *tp;
        if (fseeko(f, off_t(g.data_start + t.off), SEEK_SET) != 0) { why = "seek failed for " + t.name; bn_sync(e.ctx); drop(); return 3; }
        for (uint64_t done = 0; done < t.bytes; done += chunk_bytes) {
            const size_t n = size_t(std::min<uint64_t>(chunk_bytes, t.bytes - done));
            if (fread(stage[cur], 1, n, f) != n) { why = "short read in " + t.name; bn_sync(e.ctx); drop(); return 3; }
            if (bn_sync(e.ctx) || bn_upload_async(e.ctx, e.weights, off + done, stage[cur], n)) { why = bn_last_error(); bn_sync(e.ctx); drop(); return 3; }
            cur ^= 1;
        }
        if (bn_model_set_tensor(e.model, t.name.c_str(), e.weights, off, t.bytes)) { why = bn_last_error(); bn_sync(e.ctx); drop(); return 3; }
        off += al(t.bytes);
    }
    if (bn_sync(e.ctx)) { why = bn_last_error(); drop(); return 3; }
    drop();
    if (bn_upload(e.ctx, e.weights, off, e.plan.signs.data(), e.plan.signs.size() * 4)) { why = bn_last_error(); return 3; }
    if (bn_model_set_signs(e.model, e.weights, off, int(e.plan.signs.size()))) { why = bn_last_error(); return 2; }
    if (bn_model_finalize(e.model)) { why = bn_last_error(); return 2; }
    return 0;
}

}  // namespace bh
