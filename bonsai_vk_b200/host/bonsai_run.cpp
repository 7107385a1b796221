// bonsai_run - command-line host for the decode path on one B200.
//
//   bonsai_run run [model.gguf] [chunk_MiB=32] [n_tokens=24] [-- "prompt"]     the reference's own grammar
//                                                (bonsai_vk.exe run ..., runtime_vk/bonsai_forward.h:3086-3093)
//   bonsai_run info [model.gguf]                 metadata, contract and tensor census; no GPU work
//   bonsai_run <model.gguf> info | run [n_gen]   the earlier spelling, kept
//
// chunk_MiB is the size of the pinned staging buffers of the loader (the reference's upload chunk). The prompt is
// taken as token ids from BONSAI_PROMPT_IDS: the tokenizer and the chat template stay on the reference's side of
// the boundary (its Bpe / chat::render feed ids into bn_model_token unchanged), so a text prompt given after "--" or
// in BONSAI_PROMPT is refused with that explanation unless BONSAI_PROMPT_IDS accompanies it.
//
// Behaviour mirrors the reference engine's `run` mode (runtime_vk/bonsai_forward.h:2645-3000 fwd_run,
// :3240-3300 fwd_main): hyper-parameters only from GGUF metadata, the rotation gate before any GPU work
// (exit 6), capacity checks (exit 4), context-fit guard (exit 7), the bitwise lineage gate behind
// BONSAI_QCHECK=1 (exit 6, "REFUSING TO GENERATE"), and the same report lines
// ("... generated tokens in ... ms  ->  ... tok/s", "steady-state: ... ms/token", "gate: PASS (bitmask 0 = ...)").
//
// Environment: BONSAI_PROMPT_IDS (comma separated ids; default "1,2,3,4,5,6,7,8"), BONSAI_CAP (KV capacity in
// positions, even; default 4096), BONSAI_QCHECK=1 (run the gate after the prefill), BONSAI_DEVICE (CUDA ordinal),
// BONSAI_STEPWISE=1 (one host call per generated token instead of the device-chained loop), BONSAI_PREFILL_BLOCK (prompt
// tokens per prefill pass, default 16; 0 = token by token; the lineage gate always prefills token by token).
#include "bonsai_host.h"
#include "bonsai_sampler.h"

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace {

double now_ms() {
    using namespace std::chrono;
    return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

std::vector<int> parse_ids(const char *s) {
    std::vector<int> out;
    while (s && *s) {
        char *end = nullptr;
        const long v = strtol(s, &end, 10);
        if (end == s) break;
        out.push_back(int(v));
        s = *end == ',' ? end + 1 : end;
    }
    return out;
}

int fail(int rc, const std::string &why) {
    fprintf(stderr, "bonsai_run: %s (exit %d)\n", why.c_str(), rc);
    return rc;
}

// Two kernel lineages of the same forward (fused phase kernels vs one stand-alone kernel per reference dispatch)
// must leave bit-identical logits, residual, KV bytes and recurrent state after the same prompt. Extra
// invariants: cache slots beyond the prompt are still zero bytes; every logit is finite.
int lineage_gate(bh::Engine &e, const bh::Gguf &g, const char *path, const std::vector<int> &prompt, std::string &why) {
    bh::Engine ref;
    ref.ctx = e.ctx;
    ref.plan = e.plan;
    setenv("BONSAI_NO_FUSE", "1", 1);
    const int rc = bh::engine_load(ref, path, g, 64u << 20, why);
    unsetenv("BONSAI_NO_FUSE");
    if (rc) return -1;
    for (size_t i = 0; i < prompt.size(); ++i)
        if (bn_model_token(ref.model, prompt[i], int(i), -1, nullptr)) { why = bn_last_error(); return -1; }
    const bn_hparams &h = e.plan.hp;
    int n_attn = 0, n_gdn = 0;
    for (int b = 0; b < h.n_layer; ++b) (bh::is_attn_block(h, b) ? n_attn : n_gdn)++;
    int mask = 0;
    std::vector<uint8_t> a, b;
    auto same = [&](int what, int index, size_t bytes, int bit) {
        a.resize(bytes); b.resize(bytes);
        if (bn_model_read(e.model, what, index, a.data(), bytes) || bn_model_read(ref.model, what, index, b.data(), bytes)) { mask |= 1 << 7; return; }
        if (memcmp(a.data(), b.data(), bytes) != 0) mask |= 1 << bit;
    };
    same(BN_READ_LOGITS, 0, size_t(h.vocab) * 4, 0);
    {
        const float *l = reinterpret_cast<const float *>(a.data());
        for (int i = 0; i < h.vocab; ++i) if (!std::isfinite(l[i])) { mask |= 1 << 5; break; }
    }
    same(BN_READ_RESIDUAL, 0, size_t(h.hidden) * 4, 1);
    const size_t kvn = size_t(h.cap) * h.n_kv * h.head_dim, row = size_t(h.n_kv) * h.head_dim;
    for (int l = 0; l < n_attn; ++l) {
        same(BN_READ_K_DATA, l, kvn, 2);
        for (size_t i = prompt.size() * row; i < kvn; ++i) if (a[i]) { mask |= 1 << 4; break; }
        same(BN_READ_K_SCALE, l, kvn / 32 * 2, 2);
        same(BN_READ_V_DATA, l, kvn, 2);
        for (size_t i = prompt.size() * row; i < kvn; ++i) if (a[i]) { mask |= 1 << 4; break; }
        same(BN_READ_V_SCALE, l, kvn / 32 * 2, 2);
    }
    const size_t state = size_t(h.gdn_heads) * h.gdn_dim * h.gdn_dim * 4;
    const size_t taps = size_t(2 * h.gdn_qk_heads * h.gdn_dim + h.gdn_heads * h.gdn_dim) * 3 * 4;
    for (int l = 0; l < n_gdn; ++l) { same(BN_READ_GDN_STATE, l, state, 3); same(BN_READ_CONV_HIST, l, taps, 3); }
    bn_model_destroy(ref.model);
    bn_free(e.ctx, ref.weights);
    return mask;
}

}  // namespace

int main(int argc, char **argv) {
    if (argc < 2) {
        fprintf(stderr, "usage: %s run [model.gguf] [chunk_MiB] [n_tokens] [-- \"prompt\"] | info [model.gguf] | <model.gguf> info | <model.gguf> run [n_gen]\n", argv[0]);
        return 2;
    }
    if (!strcmp(argv[1], "sampler-check")) {
        // No GPU: read cases from stdin and print the pick and the generator state of each (the knobs come from the
        // environment as in `run`). A case is: n, then n logits, then m, then m history ids (text, whitespace separated).
        bh::Sampler sp;
        sp.from_env();
        unsigned n = 0;
        while (scanf("%u", &n) == 1 && n > 0 && n < (1u << 24)) {
            std::vector<float> lg(n);
            for (unsigned i = 0; i < n; ++i) if (scanf("%f", &lg[i]) != 1) return 2;
            unsigned m = 0;
            if (scanf("%u", &m) != 1 || m > (1u << 24)) return 2;
            std::vector<int> hist(m);
            for (unsigned i = 0; i < m; ++i) if (scanf("%d", &hist[i]) != 1) return 2;
            const int t = sp.pick(lg.data(), n, hist);
            printf("%d %llu\n", t, (unsigned long long)sp.rng);
        }
        return 0;
    }
    // everything after "--" is the prompt text and not a positional argument
    int npos = argc;
    std::string text_prompt;
    for (int i = 1; i < argc; ++i) if (!strcmp(argv[i], "--")) { npos = i; if (i + 1 < argc) text_prompt = argv[i + 1]; break; }
    if (const char *p = getenv("BONSAI_PROMPT")) text_prompt = p;
    const bool ref_grammar = !strcmp(argv[1], "run") || !strcmp(argv[1], "info");
    const char *path = ref_grammar ? (npos > 2 ? argv[2] : "models/Ternary-Bonsai-2-9B-PTQ1_0.gguf") : argv[1];
    if (!ref_grammar && npos < 3) { fprintf(stderr, "usage: %s <model.gguf> info | run [n_gen]\n", argv[0]); return 2; }
    const std::string mode = ref_grammar ? argv[1] : argv[2];
    const long chunk_mib = ref_grammar && npos > 3 ? atol(argv[3]) : (ref_grammar ? 32 : 64);
    const int n_default = ref_grammar ? (npos > 4 ? atoi(argv[4]) : 24) : (npos > 3 ? atoi(argv[3]) : 48);
    std::string why;
    bh::Gguf g;
    double t0 = now_ms();
    if (!bh::gguf_load(path, g, why)) return fail(3, why);
    const char *cap_s = getenv("BONSAI_CAP");
    const int cap = cap_s ? atoi(cap_s) : 4096;
    bh::Engine e;
    const int prc = bh::plan_build(g, e.plan, cap, why);
    uint64_t n_ptq = 0, b_ptq = 0, n_f32 = 0, b_f32 = 0;
    for (const bh::Tensor &t : g.tensors) { if (t.dtype == 143) { ++n_ptq; b_ptq += t.bytes; } else { ++n_f32; b_f32 += t.bytes; } }
    if (mode == "info") {
        printf("gguf v%u, %zu tensors: %llu PTQ1_0 (%.3f GB) + %llu f32 (%.1f MB), data at %llu, alignment %u\n", g.version,
               g.tensors.size(), (unsigned long long)n_ptq, b_ptq / 1e9, (unsigned long long)n_f32, b_f32 / 1e6,
               (unsigned long long)g.data_start, g.alignment);
        if (prc) return fail(prc, why);
        const bn_hparams &h = e.plan.hp;
        printf("n_layer %d hidden %d ffn %d vocab %d heads %d/%d x %d rot %d interval %d gdn %d/%d x %d hat_block %d signs %zu\n", h.n_layer,
               h.hidden, h.ffn, h.vocab, h.n_head, h.n_kv, h.head_dim, h.n_rot, h.attn_interval, h.gdn_heads, h.gdn_qk_heads, h.gdn_dim,
               h.hat_block, e.plan.signs.size());
        std::string kinds;
        for (int b = 0; b < h.n_layer; ++b) kinds.push_back(bh::is_attn_block(h, b) ? 'A' : 'R');
        printf("layer types %s (A = attention, R = gated delta net)\n", kinds.c_str());
        return 0;
    }
    if (mode != "run") return fail(2, "unknown mode " + mode);
    if (prc) return fail(prc, why);                       // rotation gate and contract: before any GPU work
    if (cap <= 0 || (cap & 1)) return fail(4, "BONSAI_CAP must be a positive even number of positions");
    const int n_gen = n_default;
    if (n_gen < 1) return fail(2, "n_tokens must be >= 1");
    if (chunk_mib < 1 || chunk_mib > 4096) return fail(2, "chunk_MiB must be between 1 and 4096");
    const char *ids_s = getenv("BONSAI_PROMPT_IDS");
    if (!ids_s && !text_prompt.empty())
        return fail(2, "a text prompt needs the tokenizer, which stays on the host side of the boundary: pass the prompt's token ids in BONSAI_PROMPT_IDS");
    const std::vector<int> prompt = parse_ids(ids_s ? ids_s : "1,2,3,4,5,6,7,8");
    if (prompt.empty()) return fail(2, "BONSAI_PROMPT_IDS holds no token id");
    for (int id : prompt) if (id < 0 || id >= e.plan.hp.vocab) return fail(2, "prompt id " + std::to_string(id) + " is outside the vocabulary");
    if (int(prompt.size()) + n_gen > cap)
        return fail(7, "prompt (" + std::to_string(prompt.size()) + ") + generation (" + std::to_string(n_gen) + ") does not fit the KV capacity " + std::to_string(cap));

    // BONSAI_PREFILL_BLOCK: prompt tokens per prefill pass (default 16; 0 or 1 = token by token as the reference does)
    const char *pb_s = getenv("BONSAI_PREFILL_BLOCK");
    const int prefill_want = pb_s ? atoi(pb_s) : 16;
    if (prefill_want < 0 || prefill_want > 32) return fail(2, "BONSAI_PREFILL_BLOCK must be between 0 and 32");
    // BONSAI_TEMP above zero: tokens are sampled on the host from the logits, as the reference's `run` does
    // (bonsai_forward.h:2657-2664, 2892); the prompt is then fed token by token so that the logits read back are its last
    // token's. Without it the device's greedy pick is used.
    bh::Sampler sampler;
    const bool sampling = sampler.from_env() && !getenv("BONSAI_QCHECK");
    const int prefill_block = (getenv("BONSAI_QCHECK") || sampling) ? 0 : prefill_want;
    if (prefill_block > 1) e.plan.hp.batch_cols = prefill_block;
    const char *dev_s = getenv("BONSAI_DEVICE");
    if (bn_init(dev_s ? atoi(dev_s) : 0, &e.ctx)) return fail(3, bn_last_error());
    int rc = bh::engine_load(e, path, g, size_t(chunk_mib) << 20, why);
    if (rc) return fail(rc, why);
    e.load_ms = now_ms() - t0;
    printf("loaded %zu tensors (%.3f GB) in %.1f ms\n", g.tensors.size(), (b_ptq + b_f32) / 1e9, e.load_ms);

    t0 = now_ms();
    int next = -1;
    if (prefill_block > 1) {
        // the prompt in blocks: one pass per block reads every projection's weights once (bn_model_prefill)
        for (size_t i = 0; i < prompt.size(); i += size_t(prefill_block)) {
            const int n = int(std::min(prompt.size() - i, size_t(prefill_block)));
            if (bn_model_prefill(e.model, prompt.data() + i, n, int(i), i + n == prompt.size() ? &next : nullptr)) return fail(3, bn_last_error());
        }
    } else {
        for (size_t i = 0; i < prompt.size(); ++i)
            if (bn_model_token(e.model, prompt[i], int(i), -1, i + 1 == prompt.size() ? &next : nullptr)) return fail(3, bn_last_error());
    }
    if (bn_sync(e.ctx)) return fail(3, bn_last_error());
    const double prefill_ms = now_ms() - t0;
    if (prefill_block > 1) printf("prefill: %zu tokens in %.1f ms (%.2f ms/token, blocks of %d)\n", prompt.size(), prefill_ms, prefill_ms / prompt.size(), prefill_block);
    else printf("prefill: %zu tokens in %.1f ms (%.2f ms/token, token-serial)\n", prompt.size(), prefill_ms, prefill_ms / prompt.size());

    if (getenv("BONSAI_QCHECK")) {
        const int mask = lineage_gate(e, g, path, prompt, why);
        if (mask < 0) return fail(3, "gate could not run: " + why);
        printf("gate: %s (bitmask %d = A logits, A2 residual, A3 KV bytes, A4 recurrent state, B dead slots, C finite)\n", mask ? "FAIL" : "PASS", mask);
        if (mask) { fprintf(stderr, "REFUSING TO GENERATE\n"); return 6; }
    }

    std::vector<int> out(n_gen);
    out[0] = next;
    t0 = now_ms();
    double t_first = 0;
    if (sampling) {
        std::vector<float> logits(size_t(e.plan.hp.vocab));
        std::vector<int> gen;
        for (int i = 0; i < n_gen; ++i) {
            if (i > 0 && bn_model_token(e.model, out[i - 1], int(prompt.size()) + i - 1, -1, nullptr)) return fail(3, bn_last_error());
            if (bn_model_read(e.model, BN_READ_LOGITS, 0, logits.data(), logits.size() * sizeof(float))) return fail(3, bn_last_error());
            out[i] = sampler.pick(logits.data(), uint32_t(logits.size()), gen);
            gen.push_back(out[i]);
            if (i == 1) t_first = now_ms() - t0;
        }
        printf("sampled: temp %.2f top_k %d top_p %.2f repetition %.2f presence %.2f frequency %.2f\n", sampler.temp, sampler.top_k, sampler.top_p,
               sampler.rep_penalty, sampler.presence_penalty, sampler.freq_penalty);
    } else if (getenv("BONSAI_STEPWISE")) {
        for (int i = 1; i < n_gen; ++i) {
            if (bn_model_token(e.model, out[i - 1], int(prompt.size()) + i - 1, -1, &out[i])) return fail(3, bn_last_error());
            if (i == 1) t_first = now_ms() - t0;
        }
    } else if (n_gen > 1) {
        // one warm call captures the token graph; it also produces the second token
        if (bn_model_decode(e.model, out[0], int(prompt.size()), 1, &out[1])) return fail(3, bn_last_error());
        t_first = now_ms() - t0;
        if (n_gen > 2 && bn_model_decode(e.model, out[1], int(prompt.size()) + 1, n_gen - 2, &out[2])) return fail(3, bn_last_error());
    }
    const double gen_ms = now_ms() - t0;
    printf("ids:");
    for (int id : out) printf(" %d", id);
    printf("\n");
    printf("%d generated tokens in %.1f ms  ->  %.2f tok/s\n", n_gen, gen_ms + prefill_ms / prompt.size(), n_gen * 1e3 / (gen_ms + prefill_ms / prompt.size()));
    if (n_gen > 2) printf("steady-state: %.3f ms/token\n", (gen_ms - t_first) / (n_gen - 2));
    printf("launches: %llu\n", (unsigned long long)bn_launch_count(e.ctx));
    bn_model_destroy(e.model);
    bn_free(e.ctx, e.weights);
    bn_destroy(e.ctx);
    return 0;
}
