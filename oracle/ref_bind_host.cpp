// ref_bind_host.cpp - TEST INFRASTRUCTURE. The reference's own host headers (GGUF reader, model plan + rotation
// contract, byte-level BPE tokenizer, chat template), compiled unmodified from where they lie in the reference tree
// (-I$(REF)/runtime_vk), driving this repository's C ABI: what a maintainer of the reference writes when the Vulkan
// backend is swapped for libbonsai_cuda.so. Built by oracle/Makefile into oracle/_ref/ref_bind_run; only tests run it.
//
//   ref_bind_run <model.gguf> <n_tokens> -- "prompt text"
//
// Reference code used as is: gguf_load (bonsai_gguf.h:72), model_plan_build incl. model_plan_contract
// (bonsai_model.h:1013, :773), Bpe::load / Bpe::encode / Bpe::decode_ids (bonsai_tok.h:159, :367, :397),
// chat::render_ids (bonsai_chat.h:76, only with BONSAI_CHAT=1 - it needs the 9B's control-token ids).
// Prints "prompt ids: ...", then "ids: ..." for the generated tokens, then their text.
#include "bonsai_gguf.h"
#include "bonsai_model.h"
#include "bonsai_tok.h"
#include "bonsai_chat.h"

#include "../include/bonsai_cuda.h"

#include <cstdlib>

static uint64_t tensor_bytes(const GgufTensor &t) {
    uint64_t n = 1;
    for (uint32_t k = 0; k < t.n_dims; ++k) n *= t.d[k];
    if (t.dtype == 143) return n / 128 * 28;      // PTQ1_0: 28 bytes per 128 weights along dim 0
    if (t.dtype == 0) return n * 4;               // f32
    return 0;
}

int main(int argc, char **argv) {
    if (argc < 3) { fprintf(stderr, "usage: %s <model.gguf> <n_tokens> [-- \"prompt\"]\n", argv[0]); return 2; }
    const char *path = argv[1];
    const int n_gen = atoi(argv[2]);
    std::string prompt = "hello";
    for (int i = 1; i < argc - 1; ++i) if (!strcmp(argv[i], "--")) prompt = argv[i + 1];

    GgufHeader h;
    if (!gguf_load(path, h)) return 3;
    ModelPlan p;
    if (!model_plan_build(h, p)) return 6;         // the reference's own contract refusal
    Bpe tok;
    if (!tok.load(h)) return 3;
    std::vector<int> ids;
    if (getenv("BONSAI_CHAT") && atoi(getenv("BONSAI_CHAT"))) ids = chat::render_ids(tok, "", prompt, false);
    else ids = tok.encode(prompt, true, false);
    printf("prompt ids:");
    for (int id : ids) printf(" %d", id);
    printf("\n");
    if (ids.empty()) return 2;

    bn_hparams hp = {};
    hp.n_layer = p.n_layer; hp.hidden = p.hidden; hp.ffn = p.ffn; hp.vocab = p.vocab;
    hp.n_head = p.n_head; hp.n_kv = p.n_head_kv; hp.head_dim = p.head_dim; hp.n_rot = p.n_rot;
    hp.attn_interval = p.full_attn_interval;
    hp.gdn_heads = p.ts_rank; hp.gdn_qk_heads = p.group_count; hp.gdn_dim = p.state_size;
    hp.hat_block = int(p.hat_block);
    hp.rms_eps = p.rms_eps; hp.rope_base = p.rope_base;
    hp.cap = getenv("BONSAI_CAP") ? atoi(getenv("BONSAI_CAP")) : 256;
    if (!p.layer_kind.empty()) {                   // explicit layer list resolved by the reference: pass it as the mask
        hp.attn_interval = 0;
        unsigned long long mask = 0;
        for (size_t b = 0; b < p.layer_kind.size() && b < 64; ++b) if (p.layer_kind[b] == 1) mask |= 1ull << b;
        hp.attn_mask_lo = uint32_t(mask); hp.attn_mask_hi = uint32_t(mask >> 32);
    }

    bn_ctx *ctx = nullptr;
    if (bn_init(0, &ctx)) { fprintf(stderr, "%s\n", bn_last_error()); return 3; }
    bn_model *m = nullptr;
    if (bn_model_create(ctx, &hp, &m)) { fprintf(stderr, "%s\n", bn_last_error()); return 4; }
    FILE *f = fopen(path, "rb");
    if (!f) return 3;
    std::vector<bn_buf *> bufs;
    std::vector<unsigned char> host;
    for (const GgufTensor &t : h.t) {
        const uint64_t nb = tensor_bytes(t);
        if (!nb) continue;
        host.resize(nb);
        fseek(f, long(h.data_start + t.off), SEEK_SET);
        if (fread(host.data(), 1, nb, f) != nb) { fprintf(stderr, "short read of %s\n", t.name.c_str()); return 3; }
        bn_buf *b = nullptr;
        if (bn_alloc(ctx, nb, &b) || bn_upload(ctx, b, 0, host.data(), nb) || bn_model_set_tensor(m, t.name.c_str(), b, 0, nb)) {
            fprintf(stderr, "%s\n", bn_last_error()); return 3;
        }
        bufs.push_back(b);
    }
    fclose(f);
    {
        const std::string key = p.sign_values_key.empty() ? std::string("prism.hadamard.sign_values") : p.sign_values_key;
        auto sv = h.kv_a.find(key);
        if (sv == h.kv_a.end()) { fprintf(stderr, "no sign values under %s\n", key.c_str()); return 6; }
        std::vector<int32_t> sg(sv->second.size());
        for (size_t i = 0; i < sg.size(); ++i) sg[i] = int32_t(atoi(sv->second[i].c_str()));
        bn_buf *b = nullptr;
        if (bn_alloc(ctx, sg.size() * 4, &b) || bn_upload(ctx, b, 0, sg.data(), sg.size() * 4) || bn_model_set_signs(m, b, 0, int(sg.size()))) {
            fprintf(stderr, "%s\n", bn_last_error()); return 6;
        }
        bufs.push_back(b);
    }
    if (bn_model_finalize(m)) { fprintf(stderr, "%s\n", bn_last_error()); return 4; }
    int next = -1;
    for (size_t i = 0; i < ids.size(); ++i)
        if (bn_model_token(m, ids[i], int(i), -1, i + 1 == ids.size() ? &next : nullptr)) { fprintf(stderr, "%s\n", bn_last_error()); return 3; }
    std::vector<int> out(n_gen);
    out[0] = next;
    if (n_gen > 1 && bn_model_decode(m, out[0], int(ids.size()), n_gen - 1, &out[1])) { fprintf(stderr, "%s\n", bn_last_error()); return 3; }
    printf("ids:");
    for (int id : out) printf(" %d", id);
    printf("\n");
    printf("text: %s\n", tok.decode_ids(out).c_str());
    bn_model_destroy(m);
    for (bn_buf *b : bufs) bn_free(ctx, b);
    bn_destroy(ctx);
    return 0;
}
