// model.cu - the whole-token schedule (reference: fwd_token, runtime_vk/bonsai_forward.h:664-758, with
// gdn_block :509-573, attn_block :581-645, ffn_block :489-506) over tensors registered by GGUF name.
#include "ops.cuh"

#include "phase_gemv.cuh"
#include "gemm_tc.cuh"
#include "token_kernel.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

struct bn_tensor_ref { const bn_buf *buf; size_t off, bytes; };

struct bn_model {
    bn_ctx *ctx;
    bn_hparams hp;
    std::map<std::string, bn_tensor_ref> tensors;
    const int32_t *signs = nullptr;
    bool finalized = false;
    int n_gdn = 0, n_attn = 0;
    // activation arena (one allocation), carved into named regions
    char *arena = nullptr;
    size_t arena_bytes = 0;
    float *RES, *AN, *X1, *X2, *QKV, *Z, *CONV, *L2, *O, *KBUF, *VBUF, *Q16F, *GATEB, *GOUT, *FG, *FU, *FS, *D, *LOGITS;
    float *ALPHA, *BETA, *G, *BT, *SCORE, *P16F, *ESUM, *PVPART, *AMV;
    float *XROT = nullptr, *F32ACT = nullptr;   // act_mode 1: the rotated fp32 input of a projection and the split partial sums
    int *AMI, *TOK, *POS, *NEXT, *HIST, *STEP;
    cudaGraphExec_t token_graph = nullptr;   // one whole token + advance, captured on first use
    std::vector<cudaGraphExec_t> stage_graphs;   // pipeline stage: one captured schedule per stream (its state pointers are baked in)
    uint32_t *PACK_H, *PACK_F;
    int *SWCNT = nullptr;                 // arrival counters of swiglu_pack (one per Hadamard block of the FFN width)
    float *GEMV_SCRATCH;
    // persistent state
    float *gdn_state = nullptr, *conv_hist = nullptr, *conv_hist2 = nullptr;   // conv taps: two buffers (position parity)
    int next_pos = 0;
    int cur = 0;              // stream whose state the next enqueue works on
    int b0 = 0, b1 = 0;       // local block range [b0, b1): a pipeline stage owns a contiguous run of blocks
    size_t gdn_stream_stride = 0, conv_stream_stride = 0;
    char *kv = nullptr;
    size_t kv_layer_bytes = 0, kv_k_scale_off = 0, kv_v_off = 0, kv_v_scale_off = 0;
    int pv_splits = 1;
    int graph_launches = 0;
    bool fused = true;        // phase kernels (false: one kernel per reference dispatch, env BONSAI_NO_FUSE=1)
    bool phases_only = false; // measurement: enqueue only the projection kernels of the fused schedule
    bool mixers_only = false; // measurement: enqueue only what runs between a block's projections (recurrent core / attention)
    bool use_pdl = true;      // programmatic dependent launch between phases (env BONSAI_NO_PDL=1 turns it off)
    cudaError_t launch_err = cudaSuccess;
    unsigned long long *stamps = nullptr;   // profiling aid: 8 time stamps per phase kernel of one token
    int stamp_idx = 0;
    unsigned long long *graph_stamps = nullptr;
    // resolved per-layer weights
    struct Layer {
        bool attn;
        const float *attn_norm, *post_norm;
        const uint32_t *ffn_gate, *ffn_up, *ffn_down;
        // gdn
        const uint32_t *qkv, *gate_w, *ssm_out;
        const float *alpha_w, *beta_w, *dt_bias, *ssm_a, *conv_w, *ssm_norm;
        // attn
        const uint32_t *q_w, *k_w, *v_w, *o_w;
        const float *q_norm, *k_norm;
        int idx;   // index among its kind
    };
    std::vector<Layer> layers;
    // multi-sequence pass (bn_model_stage_batch): per-column arenas, shared activation images, tile-major weights
    int ncols = 1;
    uint8_t *IMG_H = nullptr, *IMG_F = nullptr;
    uint8_t *IMG_HD = nullptr;            // sharded head: its own activation image, so that the head may run beside a stage pass
    float *GROUPS = nullptr;              // group sums of the projections that are split over K (gemm_tc.cuh)
    uint8_t *tiled = nullptr;
    struct TiledLayer { const uint8_t *in = nullptr, *out = nullptr, *ffn_in = nullptr, *ffn_down = nullptr; };
    std::vector<TiledLayer> tl;
    const uint8_t *t_head = nullptr;
    int head_r0 = 0, head_r1 = 0;         // rows of the output head this model holds for the multi-sequence pass
    bool head_sharded = false;            // bn_model_set_head_rows: the head runs through bn_model_head_batch, not in the last stage
    float *CAND = nullptr;                // [batch_cols][2] candidates of a head shard
    std::map<long, cudaGraphExec_t> batch_graphs;   // key = stream0 * 64 + ncol
    int batch_graph_launches = 0;
    const uint32_t *embd = nullptr, *out_w = nullptr;
    const float *out_norm = nullptr;
    // whole-token kernel (one launch per token or per run of tokens): the phase list and where each block ends in it
    bool use_token = false;
    std::vector<bnk::TokOp> tok_ops;
    std::vector<int> tok_block_end;          // tok_block_end[b] = number of phases up to and including block b
    unsigned *tok_bar = nullptr;             // grid barrier counter
    uintptr_t tok_serial = 0;                // identifies this model's phase list in the constant bank
    unsigned long long *tok_stamps = nullptr; // profiling aid (env BONSAI_TOKEN_STAMPS): 4 time stamps per phase of CTA 0
    float *CANDV = nullptr; int *CANDI = nullptr;
};

namespace {

template <class T>
const T *tensor_ptr(bn_model *m, const std::string &name, size_t want_bytes, int *rc) {
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) { bn_set_error("bn_model_finalize: tensor '%s' was not registered", name.c_str()); *rc = BN_ERR_STATE; return nullptr; }
    if (it->second.bytes != want_bytes) {
        bn_set_error("bn_model_finalize: tensor '%s' has %zu bytes, the shape needs %zu", name.c_str(), it->second.bytes, want_bytes);
        *rc = BN_ERR_ARG; return nullptr;
    }
    return bn_ptr<T>(it->second.buf, it->second.off);
}

size_t ptq_bytes(size_t M, size_t K) { return M * (K / 128) * 28; }

bnk::AttnDims attn_dims(const bn_model *m) {
    const bn_hparams &h = m->hp;
    return bnk::AttnDims{h.n_head, h.n_kv, h.head_dim, h.n_rot, h.cap, h.rms_eps, h.rope_base, h.k_mode, h.v_mode};
}

float *gdn_state_of(const bn_model *m, int idx) {
    const bn_hparams &h = m->hp;
    return m->gdn_state + size_t(m->cur) * m->gdn_stream_stride + size_t(idx) * h.gdn_heads * h.gdn_dim * h.gdn_dim;
}
float *conv_of(const bn_model *m, int which, int idx) {
    const bn_hparams &h = m->hp;
    const size_t C = size_t(2 * h.gdn_qk_heads + h.gdn_heads) * h.gdn_dim;
    return (which ? m->conv_hist2 : m->conv_hist) + size_t(m->cur) * m->conv_stream_stride + size_t(idx) * C * 3;
}
bnk::KvLayer kv_layer(const bn_model *m, int li) {
    char *base = m->kv + (size_t(m->cur) * m->n_attn + size_t(li)) * m->kv_layer_bytes;
    bnk::KvLayer k;
    k.k_data = base;
    k.k_scale = m->hp.k_mode == 0 ? reinterpret_cast<uint16_t *>(base + m->kv_k_scale_off) : nullptr;
    k.v_data = base + m->kv_v_off;
    k.v_scale = m->hp.v_mode == 0 ? reinterpret_cast<uint16_t *>(base + m->kv_v_scale_off) : nullptr;
    return k;
}

// ---- stand-alone kernel path (one kernel per reference dispatch; kept as the A/B control) ------------
// The stand-alone lineage's projection in the model's activation mode (gemv_ptq, runtime_vk/bonsai_forward.h:409-422):
// act_mode 0 = q8_1 codes x trits with integer block dots, act_mode 1 = the reference engine's own arithmetic, the
// rotated fp32 vector against the dequantised trits with its split rule (gemv_ternary.comp:74-93).
void rotate_in(bn_model *m, const float *x, const int32_t *sg, int K, uint32_t *pack) {
    bnk::rotate_quant(m->ctx->stream, x, sg, K, m->hp.hat_block, m->hp.act_mode == 1 ? m->XROT : nullptr, pack);
}
void project(bn_model *m, const uint32_t *W, int M, int K, const uint32_t *pack, float *out) {
    cudaStream_t st = m->ctx->stream;
    if (m->hp.act_mode == 1)
        bnk::gemv_f32act(st, reinterpret_cast<const uint8_t *>(W), M, K, m->XROT, bn_gemv_f32act_splits(M, K), out, m->F32ACT);
    else bnk::gemv_q81(st, m->ctx->sm_count, W, M, K, pack, out, m->GEMV_SCRATCH, nullptr);
}
void rot_project(bn_model *m, const float *x, const int32_t *sg, int K, uint32_t *pack, const uint32_t *W, int M, float *out) {
    rotate_in(m, x, sg, K, pack);
    project(m, W, M, K, pack, out);
}

void ffn_plain(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    bnk::rms_norm(st, m->RES, L.post_norm, 1, h.hidden, h.rms_eps, m->AN);
    rotate_in(m, m->AN, m->signs, h.hidden, m->PACK_H);
    project(m, L.ffn_gate, h.ffn, h.hidden, m->PACK_H, m->FG);
    project(m, L.ffn_up, h.ffn, h.hidden, m->PACK_H, m->FU);
    bnk::swiglu(st, m->FG, m->FU, h.ffn, m->FS);
    rot_project(m, m->FS, m->signs + h.hidden, h.ffn, m->PACK_F, L.ffn_down, h.hidden, m->D);
    bnk::add_inplace(st, m->RES, m->D, h.hidden);
}

void gdn_core(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D;
    const bnk::GdnDims gd{NH, NQ, D};
    bnk::conv_silu(st, m->QKV, L.conv_w, conv_of(m, 0, L.idx), C, m->CONV);
    bnk::l2_norm_rows(st, m->CONV, 2 * NQ, 1e-12f, m->L2);
    bnk::gdn_delta(st, gd, m->L2, m->L2 + NQ * D, m->CONV + 2 * NQ * D, m->G, m->BT,
                   gdn_state_of(m, L.idx), m->O);
}

void gdn_plain(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    const bnk::GdnDims gd{NH, NQ, D};
    bnk::rms_norm(st, m->RES, L.attn_norm, 1, h.hidden, h.rms_eps, m->AN);
    bnk::gemv_f32_small(st, L.alpha_w, NH, h.hidden, m->AN, m->ALPHA);
    bnk::gemv_f32_small(st, L.beta_w, NH, h.hidden, m->AN, m->BETA);
    bnk::gdn_gates(st, m->ALPHA, m->BETA, L.dt_bias, L.ssm_a, NH, m->G, m->BT);
    rotate_in(m, m->AN, m->signs, h.hidden, m->PACK_H);
    project(m, L.qkv, C, h.hidden, m->PACK_H, m->QKV);
    project(m, L.gate_w, IN, h.hidden, m->PACK_H, m->Z);
    gdn_core(m, L);
    bnk::gdn_out(st, gd, m->O, m->Z, L.ssm_norm, h.rms_eps, m->X1);
    rot_project(m, m->X1, m->signs, IN, m->PACK_H, L.ssm_out, h.hidden, m->D);
    bnk::add_inplace(st, m->RES, m->D, h.hidden);
}

void attn_plain(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    const bnk::AttnDims a = attn_dims(m);
    const bnk::KvLayer kv = kv_layer(m, L.idx);
    bnk::rms_norm(st, m->RES, L.attn_norm, 1, h.hidden, h.rms_eps, m->AN);
    rotate_in(m, m->AN, m->signs, h.hidden, m->PACK_H);
    project(m, L.q_w, 2 * QD, h.hidden, m->PACK_H, m->QKV);
    project(m, L.k_w, KD, h.hidden, m->PACK_H, m->KBUF);
    project(m, L.v_w, KD, h.hidden, m->PACK_H, m->VBUF);
    bnk::attn_prep(st, a, m->QKV, m->KBUF, m->VBUF, L.q_norm, L.k_norm, m->POS, kv, m->Q16F, m->GATEB);
    bnk::attn_decode(st, a, m->Q16F, m->GATEB, m->POS, kv, m->SCORE, m->P16F, m->ESUM, m->PVPART, m->pv_splits, nullptr, m->GOUT, true);
    rot_project(m, m->GOUT, m->signs, QD, m->PACK_H, L.o_w, h.hidden, m->D);
    bnk::add_inplace(st, m->RES, m->D, h.hidden);
}

// ---- fused path: one "phase" kernel per projection group (phase_gemv.cu) -------------------------------
// Projections that read the same rotated input and lie back to back in device memory run as one matrix.
bnk::PhaseArgs phase_base(bn_model *m, const uint32_t *W, int M, int K, const int32_t *sg) {
    bnk::PhaseArgs a = {};
    a.W = reinterpret_cast<const uint8_t *>(W); a.M = M; a.K = K;
    a.signs = sg; a.hat_block = m->hp.hat_block; a.hat_inv = 1.0f / sqrtf(float(m->hp.hat_block)); a.eps = m->hp.rms_eps;
    a.err = m->ctx->err_dev;
    if (m->stamps && m->stamp_idx < 256) a.stamps = m->stamps + 8 * (m->stamp_idx++);
    return a;
}
void launch(bn_model *m, const bnk::PhaseArgs &a) {
    if (m->mixers_only) return;
    cudaError_t e = bnk::launch_phase(m->ctx->stream, m->ctx->sm_count, a, m->use_pdl);
    if (e != cudaSuccess && m->launch_err == cudaSuccess) m->launch_err = e;
}
bool adjacent(const uint32_t *a, size_t a_bytes, const uint32_t *b) {
    return reinterpret_cast<const uint8_t *>(a) + a_bytes == reinterpret_cast<const uint8_t *>(b);
}

void ffn_fused(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    bnk::PhaseArgs a = phase_base(m, L.ffn_gate, h.ffn, h.hidden, m->signs);
    a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.post_norm;
    if (adjacent(L.ffn_gate, ptq_bytes(h.ffn, h.hidden), L.ffn_up)) { a.M = 2 * h.ffn; a.out = m->FG; launch(m, a); }
    else { a.out = m->FG; launch(m, a); a.W = reinterpret_cast<const uint8_t *>(L.ffn_up); a.out = m->FU; launch(m, a); }
    bnk::PhaseArgs d = phase_base(m, L.ffn_down, h.hidden, h.ffn, m->signs + h.hidden);
    // silu needs a double-precision exp per element: computed once by a small kernel, not by every CTA. (Measured: folding it
    // into the gate / up projection's epilogue costs that launch 2.8 us and saves nothing - the small kernel overlaps the
    // neighbouring launches under programmatic dependent launch.)
    // The same small kernel also prepares the down projection's input (signs, three Hadamard blocks, q8_1): its three blocks
    // in parallel, once, instead of one after the other in every CTA of the projection (8.2 -> 2.5 us of prologue there,
    // 3.5 us more in the small kernel).
    if (bnk::swiglu_pack_supported(h.ffn, h.hat_block)) {
        if (!m->phases_only) bnk::swiglu_pack(m->ctx->stream, m->FG, m->FU, h.ffn, m->signs + h.hidden, d.hat_inv, m->FS, m->PACK_F, m->SWCNT);
        d.pro = bnk::PRO_PACKED; d.pack = m->PACK_F;
    } else {
        if (!m->phases_only) bnk::swiglu(m->ctx->stream, m->FG, m->FU, h.ffn, m->FS);
        d.pro = bnk::PRO_PLAIN; d.x0 = m->FS;
    }
    d.resid_in = m->RES; d.resid_out = m->RES;
    launch(m, d);
}

void gdn_fused(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    bnk::PhaseArgs a = phase_base(m, L.qkv, C, h.hidden, m->signs);
    a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.attn_norm;
    a.inv_out = m->G + 48;      // the norm factor, for the layer core's two small projections
    if (adjacent(L.qkv, ptq_bytes(C, h.hidden), L.gate_w)) { a.M = C + IN; a.out = m->QKV; launch(m, a); }
    else {
        a.out = m->QKV; launch(m, a);
        a.inv_out = nullptr; a.W = reinterpret_cast<const uint8_t *>(L.gate_w); a.M = IN; a.out = m->Z; launch(m, a);
    }
    if (!m->phases_only) {
        const bnk::GdnDims gd{NH, NQ, D};
        float *h0 = conv_of(m, 0, L.idx), *h1 = conv_of(m, 1, L.idx);
        // one sequence: heads x 4 CTAs in clusters of 4 (fills the GPU); several sequences: one CTA per head and sequence
        if (D == 128 && getenv("BONSAI_GDN_ONE_CTA_PER_HEAD") == nullptr)
            bnk::gdn_core_split(m->ctx->stream, gd, h.hidden, m->QKV, L.conv_w, h0, h1, m->POS, m->RES, m->G + 48, L.attn_norm, L.alpha_w,
                                L.beta_w, L.dt_bias, L.ssm_a, gdn_state_of(m, L.idx), m->Z, L.ssm_norm, h.rms_eps, m->X1);
        else
            bnk::gdn_core_fused(m->ctx->stream, gd, h.hidden, m->QKV, L.conv_w, h0, h1, m->POS, m->RES, m->G + 48, L.attn_norm,
                                L.alpha_w, L.beta_w, L.dt_bias, L.ssm_a, gdn_state_of(m, L.idx), m->Z, L.ssm_norm, h.rms_eps, m->X1);
    }
    bnk::PhaseArgs o = phase_base(m, L.ssm_out, h.hidden, IN, m->signs);
    o.pro = bnk::PRO_PLAIN; o.x0 = m->X1;
    o.resid_in = m->RES; o.resid_out = m->RES;
    launch(m, o);
}

void attn_fused(bn_model *m, const bn_model::Layer &L) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    const bnk::AttnDims ad = attn_dims(m);
    const bnk::KvLayer kv = kv_layer(m, L.idx);
    bnk::PhaseArgs a = phase_base(m, L.q_w, 2 * QD, h.hidden, m->signs);
    a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.attn_norm;
    if (adjacent(L.q_w, ptq_bytes(2 * QD, h.hidden), L.k_w) && adjacent(L.k_w, ptq_bytes(KD, h.hidden), L.v_w)) {
        a.M = 2 * QD + 2 * KD; a.out = m->QKV; launch(m, a);
    } else {
        a.out = m->QKV; launch(m, a);
        a.W = reinterpret_cast<const uint8_t *>(L.k_w); a.M = KD; a.out = m->KBUF; launch(m, a);
        a.W = reinterpret_cast<const uint8_t *>(L.v_w); a.out = m->VBUF; launch(m, a);
    }
    if (!m->phases_only) {
        bnk::attn_prep(st, ad, m->QKV, m->KBUF, m->VBUF, L.q_norm, L.k_norm, m->POS, kv, m->Q16F, m->GATEB);
        bnk::attn_decode(st, ad, m->Q16F, m->GATEB, m->POS, kv, m->SCORE, m->P16F, m->ESUM, m->PVPART, m->pv_splits, nullptr, m->GOUT, true);
    }
    bnk::PhaseArgs o = phase_base(m, L.o_w, h.hidden, QD, m->signs);
    o.pro = bnk::PRO_PLAIN; o.x0 = m->GOUT;
    o.resid_in = m->RES; o.resid_out = m->RES;
    launch(m, o);
}

// enqueue one token: TOK[0], POS[0] hold the token id and its absolute position
void enqueue_token(bn_model *m, int stop_after, bool want_logits) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    if (m->b0 == 0) {
        bnk::embed_row(st, m->embd, h.hidden, m->TOK, m->X1);
        bnk::rotate_inv(st, m->X1, m->signs, h.hidden, h.hat_block, m->RES);
    }
    for (int b = m->b0; b < m->b1; ++b) {
        const bn_model::Layer &L = m->layers[b];
        if (m->fused) { if (L.attn) attn_fused(m, L); else gdn_fused(m, L); ffn_fused(m, L); }
        else { if (L.attn) attn_plain(m, L); else gdn_plain(m, L); ffn_plain(m, L); }
        if (b == stop_after) return;
    }
    if (!want_logits || m->b1 != h.n_layer) return;
    if (m->fused) {
        bnk::PhaseArgs a = phase_base(m, m->out_w, h.vocab, h.hidden, m->signs);
        a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = m->out_norm; a.out = m->LOGITS;
        launch(m, a);
    } else {
        bnk::rms_norm(st, m->RES, m->out_norm, 1, h.hidden, h.rms_eps, m->AN);
        rot_project(m, m->AN, m->signs, h.hidden, m->PACK_H, m->out_w, h.vocab, m->LOGITS);
    }
    if (!m->phases_only) bnk::argmax_first(st, m->LOGITS, h.vocab, m->NEXT, m->AMV, m->AMI);
}

// ---- whole-token kernel: the token as a list of phases (token_kernel.cu) ------------------------------------------------
// Built once per model for sequence 0 of a whole model. Returns false when a shape falls outside what the kernel
// covers (the launch-per-phase schedule above is used then).
bool build_token_ops(bn_model *m) {
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    const int sm = m->ctx->sm_count;
    // Opt-in (BONSAI_TOKEN_KERNEL=1): measured on the 9B shape the one-launch token is slower than the launch-per-phase
    // schedule with programmatic dependent launch (3.1 ms against 2.2 ms per token) - every phase pays a grid barrier and
    // nothing overlaps across phases - so the default stays the captured graph.
    if (!getenv("BONSAI_TOKEN_KERNEL")) return false;
    if (!m->fused || m->b0 != 0 || m->b1 != h.n_layer) return false;
    if (!bnk::token_supported(sm, h.hat_block, h.hidden)) return false;
    if (h.hidden > 4096 || h.ffn % 16 || D != 128) return false;               // swiglu pairs need one chunk of K
    if (h.n_head != 4 * h.n_kv) return false;                                   // its attention phases are written for four query heads per kv head
    if ((h.cap + m->pv_splits - 1) / m->pv_splits > 512) return false;         // probabilities of one split in shared memory
    if (((h.hidden + 15) / 16 + sm - 1) / sm > 64) return false;               // multi-chunk running sums: 64 tiles per CTA
    m->cur = 0;
    std::vector<bnk::TokOp> ops;
    auto gemv = [&](const uint32_t *W, int M, int K, const int32_t *sg, int wait) -> bnk::PhaseArgs & {
        bnk::TokOp op;
        memset(&op, 0, sizeof op);
        op.kind = bnk::TOP_GEMV; op.wait = wait;
        bnk::PhaseArgs &a = op.ph;
        a.W = reinterpret_cast<const uint8_t *>(W); a.M = M; a.K = K;
        a.signs = sg; a.hat_block = h.hat_block; a.hat_inv = 1.0f / sqrtf(float(h.hat_block)); a.eps = h.rms_eps;
        a.err = m->ctx->err_dev;
        ops.push_back(op);
        return ops.back().ph;
    };
    auto other = [&](int kind) -> bnk::TokOp & {
        bnk::TokOp op;
        memset(&op, 0, sizeof op);
        op.kind = kind; op.wait = 1;
        ops.push_back(op);
        return ops.back();
    };
    m->tok_block_end.assign(h.n_layer, 0);
    for (int b = 0; b < h.n_layer; ++b) {
        const bn_model::Layer &L = m->layers[b];
        const int first_wait = b == 0 ? 0 : 1;        // block 0 reads the residual this CTA wrote itself (embedding) or the host copied in
        if (L.attn) {
            if (adjacent(L.q_w, ptq_bytes(2 * QD, h.hidden), L.k_w) && adjacent(L.k_w, ptq_bytes(KD, h.hidden), L.v_w)) {
                bnk::PhaseArgs &a = gemv(L.q_w, 2 * QD + 2 * KD, h.hidden, m->signs, first_wait);
                a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.attn_norm; a.out = m->QKV;
            } else {
                bnk::PhaseArgs &a = gemv(L.q_w, 2 * QD, h.hidden, m->signs, first_wait);
                a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.attn_norm; a.out = m->QKV;
                bnk::PhaseArgs &k = gemv(L.k_w, KD, h.hidden, m->signs, 0);
                k.pro = bnk::PRO_NORM; k.x0 = m->RES; k.w = L.attn_norm; k.out = m->KBUF;
                bnk::PhaseArgs &v = gemv(L.v_w, KD, h.hidden, m->signs, 0);
                v.pro = bnk::PRO_NORM; v.x0 = m->RES; v.w = L.attn_norm; v.out = m->VBUF;
            }
            bnk::AttnOp at;
            memset(&at, 0, sizeof at);
            at.d = attn_dims(m); at.kv = kv_layer(m, L.idx);
            at.qg = m->QKV; at.kin = m->KBUF; at.vin = m->VBUF; at.qn_w = L.q_norm; at.kn_w = L.k_norm;
            at.q16f = m->Q16F; at.gate = m->GATEB; at.score = m->SCORE; at.pe = m->P16F; at.esum = m->ESUM; at.pv_part = m->PVPART;
            at.gated = m->GOUT; at.splits = m->pv_splits;
            for (int kind : {bnk::TOP_ATTN_PREP, bnk::TOP_ATTN_SCORES, bnk::TOP_ATTN_EXPSUM, bnk::TOP_ATTN_PV, bnk::TOP_ATTN_COMBINE}) other(kind).at = at;
            bnk::PhaseArgs &o = gemv(L.o_w, h.hidden, QD, m->signs, 1);
            o.pro = bnk::PRO_PLAIN; o.x0 = m->GOUT; o.resid_in = m->RES; o.resid_out = m->RES;
        } else {
            if (adjacent(L.qkv, ptq_bytes(C, h.hidden), L.gate_w)) {
                bnk::PhaseArgs &a = gemv(L.qkv, C + IN, h.hidden, m->signs, first_wait);
                a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.attn_norm; a.out = m->QKV;
                a.epi = bnk::EPI_SILU_FROM; a.epi_arg = C;                     // the z rows leave the projection as silu(z)
            } else {
                bnk::PhaseArgs &a = gemv(L.qkv, C, h.hidden, m->signs, first_wait);
                a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = L.attn_norm; a.out = m->QKV;
                bnk::PhaseArgs &z = gemv(L.gate_w, IN, h.hidden, m->signs, 0);
                z.pro = bnk::PRO_NORM; z.x0 = m->RES; z.w = L.attn_norm; z.out = m->Z;
                z.epi = bnk::EPI_SILU_FROM; z.epi_arg = 0;
            }
            bnk::GdnOp &g = other(bnk::TOP_GDN).gdn;
            g.heads = NH; g.qk_heads = NQ; g.hidden = h.hidden;
            g.qkv = m->QKV; g.conv_w = L.conv_w; g.hist0 = conv_of(m, 0, L.idx); g.hist1 = conv_of(m, 1, L.idx);
            g.x = m->RES; g.norm_w = L.attn_norm; g.alpha_w = L.alpha_w; g.beta_w = L.beta_w; g.dt_bias = L.dt_bias; g.ssm_a = L.ssm_a;
            g.state = gdn_state_of(m, L.idx); g.o = m->O; g.scale = 1.0f / sqrtf(float(D));
            bnk::PhaseArgs &o = gemv(L.ssm_out, h.hidden, IN, m->signs, 1);
            o.pro = bnk::PRO_GDN_OUT_SZ; o.x0 = m->O; o.x1 = m->Z; o.w = L.ssm_norm; o.gdn_heads = NH; o.gdn_qk_heads = NQ;
            o.resid_in = m->RES; o.resid_out = m->RES;
        }
        if (!adjacent(L.ffn_gate, ptq_bytes(h.ffn, h.hidden), L.ffn_up)) return false;
        bnk::PhaseArgs &f = gemv(L.ffn_gate, 2 * h.ffn, h.hidden, m->signs, 1);
        f.pro = bnk::PRO_NORM; f.x0 = m->RES; f.w = L.post_norm; f.epi = bnk::EPI_SWIGLU; f.out2 = m->FS;
        bnk::PhaseArgs &d = gemv(L.ffn_down, h.hidden, h.ffn, m->signs + h.hidden, 1);
        d.pro = bnk::PRO_PLAIN; d.x0 = m->FS; d.resid_in = m->RES; d.resid_out = m->RES;
        m->tok_block_end[b] = int(ops.size());
    }
    bnk::PhaseArgs &hd = gemv(m->out_w, h.vocab, h.hidden, m->signs, 1);
    hd.pro = bnk::PRO_NORM; hd.x0 = m->RES; hd.w = m->out_norm; hd.out = m->LOGITS;
    hd.epi = bnk::EPI_ARGMAX; hd.cand_val = m->CANDV; hd.cand_idx = m->CANDI;
    if (int(ops.size()) > bnk::TOKEN_MAX_OPS) return false;
    m->tok_ops.swap(ops);
    static uintptr_t serial = 0;
    m->tok_serial = ++serial;
    return true;
}

// run n_steps tokens from (tok, pos0) in one launch; stop_after >= 0: one token, phases up to that block only
int run_token_kernel(bn_model *m, int tok, int pos0, int n_steps, int stop_after) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    bnk::TokenArgs ta;
    memset(&ta, 0, sizeof ta);
    ta.n_ops = stop_after >= 0 ? m->tok_block_end[stop_after] : int(m->tok_ops.size());
    ta.pick = stop_after >= 0 ? 0 : 1;
    ta.first_tok = tok; ta.pos0 = pos0; ta.n_steps = n_steps;
    ta.embd = m->embd; ta.signs = m->signs; ta.hidden = h.hidden; ta.hat_block = h.hat_block; ta.vocab = h.vocab;
    ta.res = m->RES; ta.cand_val = m->CANDV; ta.cand_idx = m->CANDI; ta.hist = m->HIST; ta.next = m->NEXT; ta.pos_out = m->POS;
    ta.bar = m->tok_bar; ta.err = m->ctx->err_dev; ta.stamps = m->tok_stamps;
    BN_CUDA(bnk::token_upload_ops(st, m->tok_ops.data(), int(m->tok_ops.size()), reinterpret_cast<const void *>(m->tok_serial)));
    BN_CUDA(cudaMemsetAsync(m->tok_bar, 0, 4, st));
    BN_CUDA(bnk::launch_token(st, m->ctx->sm_count, ta));
    return BN_OK;
}

// ---- multi-sequence pass ---------------------------------------------------------------------------------
// Tile-major copies of the local projection weights (one allocation). Projections that read the same input are
// stacked into one matrix whatever their placement in memory: every part is a whole number of 128-row tiles.
int build_batch_side(bn_model *m) {
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    BN_REQUIRE(h.batch_cols <= bnk::GEMM_MAX_COLS, BN_ERR_ARG, "bn_model_finalize: batch_cols %d exceeds %d", h.batch_cols, bnk::GEMM_MAX_COLS);
    BN_REQUIRE(h.hidden % 1024 == 0 && h.ffn % 1024 == 0, BN_ERR_ARG, "bn_model_finalize: the multi-sequence pass needs hidden and ffn to be multiples of 1024");
    BN_REQUIRE(C % 128 == 0 && IN % 128 == 0 && (2 * QD) % 128 == 0 && KD % 128 == 0 && h.ffn % 128 == 0 && h.hidden % 128 == 0, BN_ERR_ARG,
               "bn_model_finalize: the multi-sequence pass needs every projection height to be a multiple of 128");
    struct Part { const uint32_t *w; int M; };
    struct Group { std::vector<Part> parts; int K; const uint8_t **dst; };
    std::vector<Group> groups;
    m->tl.assign(h.n_layer, bn_model::TiledLayer());
    for (int b = m->b0; b < m->b1; ++b) {
        const bn_model::Layer &L = m->layers[b];
        bn_model::TiledLayer &T = m->tl[b];
        if (L.attn) {
            groups.push_back({{{L.q_w, 2 * QD}, {L.k_w, KD}, {L.v_w, KD}}, h.hidden, &T.in});
            groups.push_back({{{L.o_w, h.hidden}}, QD, &T.out});
        } else {
            groups.push_back({{{L.qkv, C}, {L.gate_w, IN}}, h.hidden, &T.in});
            groups.push_back({{{L.ssm_out, h.hidden}}, IN, &T.out});
        }
        groups.push_back({{{L.ffn_gate, h.ffn}, {L.ffn_up, h.ffn}}, h.hidden, &T.ffn_in});
        groups.push_back({{{L.ffn_down, h.hidden}}, h.ffn, &T.ffn_down});
    }
    if (m->head_sharded) groups.push_back({{{m->out_w + size_t(m->head_r0) * (h.hidden / 128) * 7, m->head_r1 - m->head_r0}}, h.hidden, &m->t_head});
    else if (m->b1 == h.n_layer) { groups.push_back({{{m->out_w, h.vocab}}, h.hidden, &m->t_head}); m->head_r0 = 0; m->head_r1 = h.vocab; }
    size_t total = 0;
    for (const Group &g : groups) for (const Part &p : g.parts) total += bnk::gemm_tiled_bytes(p.M, g.K);
    BN_CUDA(cudaMalloc(&m->tiled, total));
    size_t off = 0;
    for (const Group &g : groups) {
        *g.dst = m->tiled + off;
        for (const Part &p : g.parts) {
            bnk::repack_tiles(m->ctx->stream, p.w, p.M, g.K, reinterpret_cast<uint32_t *>(m->tiled + off));
            off += bnk::gemm_tiled_bytes(p.M, g.K);
        }
    }
    BN_CUDA(cudaMalloc(&m->IMG_H, bnk::gemm_image_bytes(h.hidden, h.batch_cols)));
    BN_CUDA(cudaMalloc(&m->IMG_F, bnk::gemm_image_bytes(h.ffn, h.batch_cols)));
    {
        size_t need = 0;
        for (const Group &g : groups) {
            int M = 0;
            for (const Part &p : g.parts) M += p.M;
            if (bnk::gemm_wants_split(m->ctx->sm_count, M, g.K, 1) || bnk::gemm_wants_split(m->ctx->sm_count, M, g.K, h.batch_cols))
                need = std::max(need, bnk::gemm_group_floats(M, g.K, h.batch_cols));
        }
        if (need) BN_CUDA(cudaMalloc(&m->GROUPS, need * 4));
    }
    if (m->head_sharded) {
        BN_CUDA(cudaMalloc(&m->CAND, size_t(h.batch_cols) * 8));
        BN_CUDA(cudaMalloc(&m->IMG_HD, bnk::gemm_image_bytes(h.hidden, h.batch_cols)));
    }
    BN_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return BN_OK;
}

struct ColInit { int tok[bnk::GEMM_MAX_COLS]; int pos[bnk::GEMM_MAX_COLS]; };
// A token id that arrives through device memory (the message from the last pipeline stage) is checked here, before any
// kernel forms an address from it: outside [0, vocab) sets the context's error word (code 3) and id 0 is used instead.
__device__ __forceinline__ int checked_tok(int t, int vocab, int *err) {
    if (t >= 0 && t < vocab) return t;
    atomicExch(err, 3);
    return 0;
}
__global__ void k_set_cols(int *tok, int *pos, size_t arena, int n, ColInit ci, const int *tok_src, int vocab, int *err) {
    const int c = threadIdx.x;
    if (c >= n) return;
    bnk::colp(tok, c * arena)[0] = tok_src ? checked_tok(tok_src[c], vocab, err) : ci.tok[c];
    bnk::colp(pos, c * arena)[0] = ci.pos[c];
}

// the token schedule for ncol sequences at once; m->cur = first sequence.
// one_sequence (batched prefill): the columns are ncol consecutive positions of ONE sequence (m->cur). Projections,
// norms, the embedding and the FFN treat them like independent sequences; the recurrent mixer walks the columns in
// order on the one state (a launch per position: the delta rule is sequential in time); attention inserts every
// column's K/V row first and then lets column c attend to the prefix that ends at its own position (causal), all
// columns at once against the one cache. Every column's result is bit-identical to the token-serial schedule.
void enqueue_batch(bn_model *m, int ncol, bool one_sequence = false) {
    const bn_hparams &h = m->hp;
    cudaStream_t st = m->ctx->stream;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    const size_t AS = m->arena_bytes / 4;       // column stride in floats
    bnk::Cols cols;
    cols.n = ncol; cols.arena = m->arena_bytes; cols.gdn = m->gdn_stream_stride * 4; cols.conv = m->conv_stream_stride * 4;
    cols.kv = m->kv_layer_bytes * m->n_attn;
    if (one_sequence) { cols.gdn = 0; cols.conv = 0; cols.kv = 0; }
    auto prep = [&](int mode, const float *x, const float *w, const int32_t *sg, int K, uint8_t *img, float *inv_out) {
        bnk::PrepArgs a = {};
        a.x = x; a.x_stride = AS; a.w = w; a.signs = sg; a.K = K; a.hat_block = h.hat_block; a.eps = h.rms_eps; a.ncol = ncol;
        a.image = img; a.inv_out = inv_out; a.inv_stride = AS; a.mode = mode;
        bnk::prep_cols(st, a);
    };
    auto gemm = [&](const uint8_t *Wt, int M, int K, const uint8_t *img, float *out, const float *resid) {
        bnk::GemmArgs a = {};
        a.W = Wt; a.M = M; a.K = K; a.tiled = 1; a.image = img; a.ncol = ncol; a.out = out; a.out_stride = AS;
        a.resid = resid; a.resid_stride = AS; a.err = m->ctx->err_dev;
        if (m->GROUPS && bnk::gemm_wants_split(m->ctx->sm_count, M, K, ncol)) a.groups = m->GROUPS;
        cudaError_t e = bnk::launch_gemm(st, m->ctx->sm_count, a, m->use_pdl);
        if (e != cudaSuccess && m->launch_err == cudaSuccess) m->launch_err = e;
    };
    if (m->b0 == 0) {
        bnk::embed_row(st, m->embd, h.hidden, m->TOK, m->X1, cols);
        bnk::rotate_inv(st, m->X1, m->signs, h.hidden, h.hat_block, m->RES, cols);
    }
    for (int b = m->b0; b < m->b1; ++b) {
        const bn_model::Layer &L = m->layers[b];
        const bn_model::TiledLayer &T = m->tl[b];
        if (L.attn) {
            const bnk::AttnDims ad = attn_dims(m);
            const bnk::KvLayer kv = kv_layer(m, L.idx);
            prep(bnk::PREP_NORM, m->RES, L.attn_norm, m->signs, h.hidden, m->IMG_H, nullptr);
            gemm(T.in, 2 * QD + 2 * KD, h.hidden, m->IMG_H, m->QKV, nullptr);
            bnk::attn_prep(st, ad, m->QKV, m->KBUF, m->VBUF, L.q_norm, L.k_norm, m->POS, kv, m->Q16F, m->GATEB, cols);
            bnk::attn_decode(st, ad, m->Q16F, m->GATEB, m->POS, kv, m->SCORE, m->P16F, m->ESUM, m->PVPART, m->pv_splits, nullptr, m->GOUT, true, cols);
            prep(bnk::PREP_PLAIN, m->GOUT, nullptr, m->signs, QD, m->IMG_H, nullptr);
            gemm(T.out, h.hidden, QD, m->IMG_H, m->RES, m->RES);
        } else {
            prep(bnk::PREP_NORM, m->RES, L.attn_norm, m->signs, h.hidden, m->IMG_H, m->G + 48);
            gemm(T.in, C + IN, h.hidden, m->IMG_H, m->QKV, nullptr);
            const bnk::GdnDims gd{NH, NQ, D};
            if (one_sequence) {
                // position after position on the one recurrent state. The kernel requests its state and conv taps before
                // its dependency wait (in the decode schedule its predecessor never writes them); here the predecessor is
                // the previous position's kernel, which does - so from the second position on the launch is a plain,
                // fully serialised one.
                const bool pdl_was = bnk::g_pdl;
                for (int c = 0; c < ncol; ++c) {
                    if (c == 1) bnk::g_pdl = false;
                    bnk::gdn_core_fused(st, gd, h.hidden, m->QKV + c * AS, L.conv_w, conv_of(m, 0, L.idx), conv_of(m, 1, L.idx), m->POS + c * AS,
                                        m->RES + c * AS, m->G + 48 + c * AS, L.attn_norm, L.alpha_w, L.beta_w, L.dt_bias, L.ssm_a,
                                        gdn_state_of(m, L.idx), m->Z + c * AS, L.ssm_norm, h.rms_eps, m->X1 + c * AS, bnk::Cols());
                }
                bnk::g_pdl = pdl_was;
            } else
            bnk::gdn_core_fused(st, gd, h.hidden, m->QKV, L.conv_w, conv_of(m, 0, L.idx), conv_of(m, 1, L.idx), m->POS, m->RES, m->G + 48,
                                L.attn_norm, L.alpha_w, L.beta_w, L.dt_bias, L.ssm_a, gdn_state_of(m, L.idx), m->Z, L.ssm_norm, h.rms_eps, m->X1, cols);
            prep(bnk::PREP_PLAIN, m->X1, nullptr, m->signs, IN, m->IMG_H, nullptr);
            gemm(T.out, h.hidden, IN, m->IMG_H, m->RES, m->RES);
        }
        prep(bnk::PREP_NORM, m->RES, L.post_norm, m->signs, h.hidden, m->IMG_H, nullptr);
        gemm(T.ffn_in, 2 * h.ffn, h.hidden, m->IMG_H, m->FG, nullptr);
        bnk::swiglu(st, m->FG, m->FU, h.ffn, m->FS, cols);
        prep(bnk::PREP_PLAIN, m->FS, nullptr, m->signs + h.hidden, h.ffn, m->IMG_F, nullptr);
        gemm(T.ffn_down, h.hidden, h.ffn, m->IMG_F, m->RES, m->RES);
    }
    if (m->b1 != h.n_layer || m->head_sharded || one_sequence) return;      // (a prefill block picks from its last column only)
    prep(bnk::PREP_NORM, m->RES, m->out_norm, m->signs, h.hidden, m->IMG_H, nullptr);
    gemm(m->t_head, h.vocab, h.hidden, m->IMG_H, m->LOGITS, nullptr);
    bnk::argmax_first(st, m->LOGITS, h.vocab, m->NEXT, m->AMV, m->AMI, cols);
}

// feed the greedy pick back as the next input, on the device
__global__ void k_advance(int *tok, int *pos, const int *next, int *hist, int *step) {
    bnk::pdl_sync();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const int s = step[0];
    hist[s] = next[0];
    tok[0] = next[0];
    pos[0] = pos[0] + 1;
    step[0] = s + 1;
}

__global__ void k_set_tok_pos(int *tok, int *pos, int t, int p, const int *tok_src, int vocab, int *err) {
    bnk::pdl_sync();
    if (threadIdx.x == 0) { tok[0] = tok_src ? checked_tok(tok_src[0], vocab, err) : t; pos[0] = p; }
}
__global__ void k_check_signs(const int32_t *sg, int n, int *bad) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && sg[i] != 1 && sg[i] != -1) atomicAdd(bad, 1);
}
__global__ void k_fill_u16(uint16_t *p, size_t n, uint16_t v) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) p[i] = v;
}

// the whole token (schedule + hand-over of the pick to TOK / POS / HIST) as one CUDA graph, captured on first use
int ensure_token_graph(bn_model *m) {
    if (m->token_graph) return BN_OK;
    cudaStream_t st = m->ctx->stream;
    cudaGraph_t g = nullptr;
    const unsigned long long before = g_bn_launches;
    if (getenv("BONSAI_STAMP_GRAPH")) {      // profiling aid: the captured kernels keep writing their time stamps
        BN_CUDA(cudaMalloc(&m->stamps, 256 * 8 * sizeof(unsigned long long)));
        BN_CUDA(cudaMemset(m->stamps, 0, 256 * 8 * sizeof(unsigned long long)));
        m->stamp_idx = 0;
    }
    BN_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    enqueue_token(m, -1, true);
    m->graph_stamps = m->stamps;
    m->stamps = nullptr;
    bnk::launch(k_advance, dim3(1), dim3(32), 0, st, m->TOK, m->POS, m->NEXT, m->HIST, m->STEP);
    cudaError_t e = cudaStreamEndCapture(st, &g);
    if (e != cudaSuccess) return bn_cuda_fail(e, "cudaStreamEndCapture(token)");
    m->graph_launches = int(g_bn_launches - before);
    g_bn_launches = before;               // captured, not launched
    e = cudaGraphInstantiate(&m->token_graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return bn_cuda_fail(e, "cudaGraphInstantiate(token)");
    return BN_OK;
}

}  // namespace

extern "C" {

int bn_model_create(bn_ctx *ctx, const bn_hparams *hp, bn_model **out) {
    BN_REQUIRE(ctx && hp && out, BN_ERR_ARG, "bn_model_create: null argument");
    const bn_hparams &h = *hp;
    BN_REQUIRE(h.n_layer > 0 && h.hidden > 0 && h.ffn > 0 && h.vocab > 0, BN_ERR_ARG, "bn_model_create: bad sizes");
    BN_REQUIRE(h.hat_block >= 16 && h.hat_block <= 4096 && (h.hat_block & (h.hat_block - 1)) == 0, BN_ERR_ARG,
               "bn_model_create: hadamard block %d must be a power of two in [16, 4096]", h.hat_block);   // the reference's range, bonsai_model.h:853-858
    BN_REQUIRE(h.hidden % h.hat_block == 0 && h.ffn % h.hat_block == 0, BN_ERR_ARG,
               "bn_model_create: hadamard block %d must divide hidden %d and ffn %d", h.hat_block, h.hidden, h.ffn);
    BN_REQUIRE(h.head_dim == 256 && h.gdn_dim == 128, BN_ERR_ARG, "bn_model_create: head_dim must be 256 and gdn_dim 128");
    BN_REQUIRE(h.n_kv > 0 && h.n_head % h.n_kv == 0 && h.n_head <= 256, BN_ERR_ARG, "bn_model_create: n_head must be a multiple of n_kv");
    { const int g = h.n_head / h.n_kv; BN_REQUIRE(g == 1 || g == 2 || g == 4 || g == 8, BN_ERR_ARG, "bn_model_create: %d query heads per kv head (1, 2, 4 or 8 are built)", g); }
    BN_REQUIRE(h.n_head * h.head_dim == h.hidden, BN_ERR_ARG, "bn_model_create: n_head * head_dim must equal hidden");
    BN_REQUIRE(h.gdn_heads * h.gdn_dim == h.hidden, BN_ERR_ARG, "bn_model_create: gdn inner size must equal hidden");
    BN_REQUIRE(h.gdn_heads <= 64 && h.gdn_heads % h.gdn_qk_heads == 0, BN_ERR_ARG, "bn_model_create: bad gdn head counts");
    BN_REQUIRE(h.n_rot > 0 && h.n_rot <= h.head_dim && h.n_rot % 2 == 0, BN_ERR_ARG, "bn_model_create: bad rope dims");
    BN_REQUIRE(h.cap > 0 && h.cap % 2 == 0, BN_ERR_ARG, "bn_model_create: cap %d must be positive and even", h.cap);
    BN_REQUIRE(h.attn_interval >= 1 || (h.attn_interval == 0 && h.n_layer <= 64), BN_ERR_ARG,
               "bn_model_create: attn_interval %d must be >= 1, or 0 with an explicit layer mask over at most 64 blocks (have %d)",
               h.attn_interval, h.n_layer);
    BN_REQUIRE(h.act_mode == 0 || h.act_mode == 1, BN_ERR_ARG, "bn_model_create: act_mode is 0 (q8_1 activations) or 1 (fp32 activations, the reference engine's arithmetic)");
    BN_REQUIRE(h.act_mode == 0 || (h.batch_cols == 0 && h.n_streams <= 1 && h.block_begin == 0 && (h.block_end == 0 || h.block_end == h.n_layer)), BN_ERR_ARG,
               "bn_model_create: act_mode 1 runs the whole model for one sequence through the stand-alone kernels (no stages, no multi-sequence pass)");
    BN_REQUIRE((h.k_mode | 1) == 1 && (h.v_mode | 1) == 1, BN_ERR_ARG, "bn_model_create: kv modes are 0 (q8_0) or 1 (fp16)");
    BN_REQUIRE(h.n_streams >= 0 && h.n_streams <= 1024, BN_ERR_ARG, "bn_model_create: n_streams %d out of range", h.n_streams);
    BN_REQUIRE(h.block_begin >= 0 && h.block_begin < h.n_layer && (h.block_end == 0 || (h.block_end > h.block_begin && h.block_end <= h.n_layer)),
               BN_ERR_ARG, "bn_model_create: block range [%d, %d) is not inside [0, %d)", h.block_begin, h.block_end, h.n_layer);
    bn_model *m = new bn_model();
    m->ctx = ctx;
    m->hp = h;
    *out = m;
    return BN_OK;
}

int bn_model_set_tensor(bn_model *m, const char *name, const bn_buf *buf, size_t off, size_t bytes) {
    BN_REQUIRE(m && name, BN_ERR_ARG, "bn_model_set_tensor: null argument");
    BN_REQUIRE(!m->finalized, BN_ERR_STATE, "bn_model_set_tensor: model already finalized");
    BN_RANGE(buf, off, bytes, 16, "bn_model_set_tensor");
    m->tensors[name] = bn_tensor_ref{buf, off, bytes};
    return BN_OK;
}

int bn_model_set_signs(bn_model *m, const bn_buf *buf, size_t off, int count) {
    BN_REQUIRE(m, BN_ERR_ARG, "bn_model_set_signs: null model");
    BN_REQUIRE(count == m->hp.hidden + m->hp.ffn, BN_ERR_ARG,
               "bn_model_set_signs: %d sign values, need hidden + ffn = %d", count, m->hp.hidden + m->hp.ffn);
    BN_RANGE(buf, off, size_t(count) * 4, 16, "bn_model_set_signs");
    m->signs = bn_ptr<int32_t>(buf, off);
    {   // the kernels apply a sign by flipping the sign bit: every value must be +1 or -1 (prism.hadamard.sign_values)
        int *bad = nullptr;
        BN_CUDA(cudaMalloc(&bad, 4));
        BN_CUDA(cudaMemsetAsync(bad, 0, 4, m->ctx->stream));
        k_check_signs<<<(count + 255) / 256, 256, 0, m->ctx->stream>>>(m->signs, count, bad);
        int h_bad = 0;
        BN_CUDA(cudaMemcpyAsync(&h_bad, bad, 4, cudaMemcpyDeviceToHost, m->ctx->stream));
        BN_CUDA(cudaStreamSynchronize(m->ctx->stream));
        cudaFree(bad);
        BN_REQUIRE(h_bad == 0, BN_ERR_ARG, "bn_model_set_signs: %d sign values are neither +1 nor -1", h_bad);
    }
    return BN_OK;
}

int bn_model_finalize(bn_model *m) {
    BN_REQUIRE(m, BN_ERR_ARG, "bn_model_finalize: null model");
    BN_REQUIRE(!m->finalized, BN_ERR_STATE, "bn_model_finalize: already finalized");
    BN_REQUIRE(m->signs, BN_ERR_STATE, "bn_model_finalize: sign values were not registered");
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    int rc = BN_OK;
    m->layers.resize(h.n_layer);
    m->n_gdn = m->n_attn = 0;
    m->b0 = h.block_begin;
    m->b1 = h.block_end > 0 ? h.block_end : h.n_layer;
    const int S = h.n_streams > 0 ? h.n_streams : 1;
    for (int b = m->b0; b < m->b1 && rc == BN_OK; ++b) {
        bn_model::Layer &L = m->layers[b];
        const std::string B = "blk." + std::to_string(b) + ".";
        L.attn = h.attn_interval > 0 ? (b % h.attn_interval) == h.attn_interval - 1
                                     : (((uint64_t(h.attn_mask_hi) << 32 | h.attn_mask_lo) >> b) & 1ull) != 0;
        L.attn_norm = tensor_ptr<float>(m, B + "attn_norm.weight", size_t(h.hidden) * 4, &rc);
        L.post_norm = tensor_ptr<float>(m, B + "post_attention_norm.weight", size_t(h.hidden) * 4, &rc);
        L.ffn_gate = tensor_ptr<uint32_t>(m, B + "ffn_gate.weight", ptq_bytes(h.ffn, h.hidden), &rc);
        L.ffn_up = tensor_ptr<uint32_t>(m, B + "ffn_up.weight", ptq_bytes(h.ffn, h.hidden), &rc);
        L.ffn_down = tensor_ptr<uint32_t>(m, B + "ffn_down.weight", ptq_bytes(h.hidden, h.ffn), &rc);
        if (L.attn) {
            L.idx = m->n_attn++;
            L.q_w = tensor_ptr<uint32_t>(m, B + "attn_q.weight", ptq_bytes(2 * QD, h.hidden), &rc);
            L.k_w = tensor_ptr<uint32_t>(m, B + "attn_k.weight", ptq_bytes(KD, h.hidden), &rc);
            L.v_w = tensor_ptr<uint32_t>(m, B + "attn_v.weight", ptq_bytes(KD, h.hidden), &rc);
            L.o_w = tensor_ptr<uint32_t>(m, B + "attn_output.weight", ptq_bytes(h.hidden, QD), &rc);
            L.q_norm = tensor_ptr<float>(m, B + "attn_q_norm.weight", size_t(h.head_dim) * 4, &rc);
            L.k_norm = tensor_ptr<float>(m, B + "attn_k_norm.weight", size_t(h.head_dim) * 4, &rc);
        } else {
            L.idx = m->n_gdn++;
            L.qkv = tensor_ptr<uint32_t>(m, B + "attn_qkv.weight", ptq_bytes(C, h.hidden), &rc);
            L.gate_w = tensor_ptr<uint32_t>(m, B + "attn_gate.weight", ptq_bytes(IN, h.hidden), &rc);
            L.ssm_out = tensor_ptr<uint32_t>(m, B + "ssm_out.weight", ptq_bytes(h.hidden, IN), &rc);
            L.alpha_w = tensor_ptr<float>(m, B + "ssm_alpha.weight", size_t(NH) * h.hidden * 4, &rc);
            L.beta_w = tensor_ptr<float>(m, B + "ssm_beta.weight", size_t(NH) * h.hidden * 4, &rc);
            L.dt_bias = tensor_ptr<float>(m, B + "ssm_dt.bias", size_t(NH) * 4, &rc);
            L.ssm_a = tensor_ptr<float>(m, B + "ssm_a", size_t(NH) * 4, &rc);
            L.conv_w = tensor_ptr<float>(m, B + "ssm_conv1d.weight", size_t(C) * 4 * 4, &rc);
            L.ssm_norm = tensor_ptr<float>(m, B + "ssm_norm.weight", size_t(D) * 4, &rc);
        }
    }
    if (rc == BN_OK && m->b0 == 0) m->embd = tensor_ptr<uint32_t>(m, "token_embd.weight", ptq_bytes(h.vocab, h.hidden), &rc);
    if (rc == BN_OK && (m->b1 == h.n_layer || m->head_sharded)) {
        m->out_w = tensor_ptr<uint32_t>(m, "output.weight", ptq_bytes(h.vocab, h.hidden), &rc);
        if (rc == BN_OK) m->out_norm = tensor_ptr<float>(m, "output_norm.weight", size_t(h.hidden) * 4, &rc);
    }
    if (rc != BN_OK) return rc;

    // activation arena
    m->pv_splits = h.cap >= 16384 ? 256 : (h.cap >= 4096 ? 64 : (h.cap >= 512 ? 8 : 1));
    const int maxM = std::max(std::max(h.vocab, h.ffn), std::max(C, 2 * QD));
    const int maxG = (std::max(h.ffn, h.hidden) / 128 + 3) / 4;
    size_t off = 0;
    auto carve = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~size_t(255); return o; };
    struct Slot { void **p; size_t o; };
    std::vector<Slot> slots;
    auto F = [&](float *&p, size_t n) { slots.push_back({reinterpret_cast<void **>(&p), carve(n * 4)}); };
    F(m->RES, h.hidden); F(m->AN, h.hidden); F(m->X1, h.hidden); F(m->X2, h.hidden);
    F(m->QKV, std::max(C + IN, 2 * QD + 2 * KD)); m->Z = nullptr; F(m->CONV, C); F(m->L2, 2 * NQ * D); F(m->O, IN);
    F(m->Q16F, QD); F(m->GATEB, QD); F(m->GOUT, QD);
    F(m->FG, 2 * size_t(h.ffn)); F(m->FS, h.ffn); F(m->D, h.hidden); F(m->LOGITS, h.vocab);
    F(m->ALPHA, 64); F(m->BETA, 64); F(m->G, 64); F(m->BT, 64);
    F(m->SCORE, size_t(h.n_head) * h.cap); F(m->P16F, size_t(h.n_head) * h.cap); F(m->ESUM, size_t(h.n_head) * 1026);
    F(m->PVPART, size_t(m->pv_splits) * QD); F(m->AMV, 64);
    if (h.act_mode == 1) { F(m->XROT, size_t(std::max(h.hidden, h.ffn))); F(m->F32ACT, 1024 + size_t(16) * maxM); }
    F(m->GEMV_SCRATCH, size_t(maxG) * std::max(maxM, 1));
    slots.push_back({reinterpret_cast<void **>(&m->AMI), carve(64 * 4)});
    slots.push_back({reinterpret_cast<void **>(&m->CANDV), carve(1024 * 4)});
    slots.push_back({reinterpret_cast<void **>(&m->CANDI), carve(1024 * 4)});
    slots.push_back({reinterpret_cast<void **>(&m->TOK), carve(256)});
    slots.push_back({reinterpret_cast<void **>(&m->POS), carve(256)});
    slots.push_back({reinterpret_cast<void **>(&m->NEXT), carve(256)});
    slots.push_back({reinterpret_cast<void **>(&m->STEP), carve(256)});
    slots.push_back({reinterpret_cast<void **>(&m->HIST), carve(size_t(h.cap) * 4)});
    slots.push_back({reinterpret_cast<void **>(&m->PACK_H), carve(bnk::act_pack_bytes(h.hidden))});
    slots.push_back({reinterpret_cast<void **>(&m->PACK_F), carve(bnk::act_pack_bytes(h.ffn))});
    m->arena_bytes = off;
    m->ncols = h.batch_cols > 0 ? h.batch_cols : 1;
    BN_CUDA(cudaSetDevice(m->ctx->device));
    BN_CUDA(cudaMalloc(&m->arena, m->arena_bytes * m->ncols));
    BN_CUDA(cudaMalloc(&m->SWCNT, 64 * sizeof(int)));
    BN_CUDA(cudaMemset(m->SWCNT, 0, 64 * sizeof(int)));
    for (auto &s : slots) *s.p = m->arena + s.o;
    m->Z = m->QKV + C;               // [qkv | gate] of a GDN block, [q | k | v] of an attention block
    m->KBUF = m->QKV + 2 * QD;
    m->VBUF = m->KBUF + KD;
    m->FU = m->FG + h.ffn;           // [gate | up]
    m->fused = h.act_mode == 0 && getenv("BONSAI_NO_FUSE") == nullptr && bnk::phase_supported(h.hidden, h.hidden, h.hat_block) &&
               bnk::phase_supported(h.hidden, h.ffn, h.hat_block);
    m->use_pdl = getenv("BONSAI_NO_PDL") == nullptr;
    bnk::g_pdl = m->use_pdl;
    // persistent state
    if (m->n_gdn) {
        m->gdn_stream_stride = size_t(m->n_gdn) * NH * D * D;
        m->conv_stream_stride = size_t(m->n_gdn) * C * 3;
        BN_CUDA(cudaMalloc(&m->gdn_state, m->gdn_stream_stride * S * 4));
        BN_CUDA(cudaMalloc(&m->conv_hist, m->conv_stream_stride * S * 4 * 2));
        m->conv_hist2 = m->conv_hist + m->conv_stream_stride * S;
    }
    if (m->n_attn) {
        const size_t n = size_t(h.cap) * KD;
        size_t o = 0;
        auto al = [&](size_t b) { size_t r = o; o += (b + 255) & ~size_t(255); return r; };
        al(h.k_mode == 0 ? n : n * 2);
        m->kv_k_scale_off = al(h.k_mode == 0 ? n / 32 * 2 : 0);
        m->kv_v_off = al(h.v_mode == 0 ? n : n * 2);
        m->kv_v_scale_off = al(h.v_mode == 0 ? n / 32 * 2 : 0);
        m->kv_layer_bytes = o;
        BN_CUDA(cudaMalloc(&m->kv, m->kv_layer_bytes * m->n_attn * S));
    }
    if (h.batch_cols > 0) {
        rc = build_batch_side(m);
        if (rc != BN_OK) return rc;
    }
    if (m->ctx->sm_count <= 1024) {
        BN_CUDA(cudaMalloc(&m->tok_bar, 256));
        if (getenv("BONSAI_TOKEN_STAMPS")) {
            BN_CUDA(cudaMalloc(&m->tok_stamps, size_t(bnk::TOKEN_MAX_OPS + 64) * 8 * sizeof(unsigned long long)));
            BN_CUDA(cudaMemset(m->tok_stamps, 0, size_t(bnk::TOKEN_MAX_OPS + 64) * 8 * sizeof(unsigned long long)));
        }
        m->use_token = build_token_ops(m);
    }
    m->finalized = true;
    return bn_model_reset(m);
}

int bn_model_reset(bn_model *m) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_reset: model not finalized");
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D;
    cudaStream_t st = m->ctx->stream;
    BN_CUDA(cudaMemsetAsync(m->arena, 0, m->arena_bytes * m->ncols, st));
    BN_CUDA(cudaMemsetAsync(m->SWCNT, 0, 64 * sizeof(int), st));       // (a launch that gave up may have left a count behind)
    if (m->n_gdn) {
        const int S = h.n_streams > 0 ? h.n_streams : 1;
        BN_CUDA(cudaMemsetAsync(m->gdn_state, 0, m->gdn_stream_stride * S * 4, st));
        BN_CUDA(cudaMemsetAsync(m->conv_hist, 0, m->conv_stream_stride * S * 4 * 2, st));
    }
    if (m->n_attn) BN_CUDA(cudaMemsetAsync(m->kv, 0, m->kv_layer_bytes * m->n_attn * (h.n_streams > 0 ? h.n_streams : 1), st));
    return BN_OK;
}

int bn_model_reset_stream(bn_model *m, int stream) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_reset_stream: model not finalized");
    const bn_hparams &h = m->hp;
    const int S = h.n_streams > 0 ? h.n_streams : 1;
    BN_REQUIRE(stream >= 0 && stream < S, BN_ERR_ARG, "bn_model_reset_stream: sequence %d outside [0, %d)", stream, S);
    cudaStream_t st = m->ctx->stream;
    if (m->n_gdn) {
        BN_CUDA(cudaMemsetAsync(m->gdn_state + size_t(stream) * m->gdn_stream_stride, 0, m->gdn_stream_stride * 4, st));
        BN_CUDA(cudaMemsetAsync(m->conv_hist + size_t(stream) * m->conv_stream_stride, 0, m->conv_stream_stride * 4, st));
        BN_CUDA(cudaMemsetAsync(m->conv_hist2 + size_t(stream) * m->conv_stream_stride, 0, m->conv_stream_stride * 4, st));
    }
    if (m->n_attn) BN_CUDA(cudaMemsetAsync(m->kv + size_t(stream) * m->n_attn * m->kv_layer_bytes, 0, m->kv_layer_bytes * m->n_attn, st));
    return BN_OK;
}

void bn_model_destroy(bn_model *m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    if (m->arena) cudaFree(m->arena);
    if (m->gdn_state) cudaFree(m->gdn_state);
    if (m->conv_hist) cudaFree(m->conv_hist);
    if (m->kv) cudaFree(m->kv);
    if (m->token_graph) cudaGraphExecDestroy(m->token_graph);
    for (cudaGraphExec_t g : m->stage_graphs) if (g) cudaGraphExecDestroy(g);
    for (auto &kv : m->batch_graphs) cudaGraphExecDestroy(kv.second);
    if (m->tiled) cudaFree(m->tiled);
    if (m->tok_bar) cudaFree(m->tok_bar);
    if (m->tok_stamps) cudaFree(m->tok_stamps);
    if (m->IMG_H) cudaFree(m->IMG_H);
    if (m->IMG_HD) cudaFree(m->IMG_HD);
    if (m->IMG_F) cudaFree(m->IMG_F);
    if (m->GROUPS) cudaFree(m->GROUPS);
    if (m->SWCNT) cudaFree(m->SWCNT);
    if (m->CAND) cudaFree(m->CAND);
    delete m;
}

int bn_model_token(bn_model *m, int tok, int pos, int stop_after_block, int *next_tok) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_token: model not finalized");
    const bn_hparams &h = m->hp;
    BN_REQUIRE(m->b0 == 0 && m->b1 == h.n_layer, BN_ERR_STATE, "bn_model_token: this model holds blocks [%d, %d) only; use bn_model_stage", m->b0, m->b1);
    m->cur = 0;
    BN_REQUIRE(tok >= 0 && tok < h.vocab, BN_ERR_ARG, "bn_model_token: token %d outside vocab %d", tok, h.vocab);
    BN_REQUIRE(pos >= 0 && pos < h.cap, BN_ERR_BOUNDS, "bn_model_token: position %d does not fit the KV capacity %d", pos, h.cap);
    cudaStream_t st = m->ctx->stream;
    BN_REQUIRE(stop_after_block < h.n_layer, BN_ERR_ARG, "bn_model_token: stop_after_block %d outside the %d blocks", stop_after_block, h.n_layer);
    m->next_pos = pos + 1;
    if (m->use_token) {
        // one launch for the whole token: id and position travel as kernel arguments, nothing is uploaded
        int rc = run_token_kernel(m, tok, pos, 1, stop_after_block);
        if (rc != BN_OK) return rc;
        if (next_tok) {
            BN_CUDA(cudaMemcpyAsync(next_tok, m->NEXT, 4, cudaMemcpyDeviceToHost, st));
            BN_CUDA(cudaStreamSynchronize(st));
        }
        return BN_OK;
    }
    if (stop_after_block < 0 && getenv("BONSAI_TOKEN_NO_GRAPH") == nullptr) {
        // the whole token is one graph launch; id and position travel as arguments of a one-thread kernel in front of it
        // (no host-to-device copy to wait for), the step counter of the hand-over kernel is cleared on the way
        { const int rc = ensure_token_graph(m); if (rc != BN_OK) return rc; }
        BN_CUDA(cudaMemsetAsync(m->STEP, 0, 4, st));
        k_set_tok_pos<<<1, 32, 0, st>>>(m->TOK, m->POS, tok, pos, nullptr, h.vocab, m->ctx->err_dev);
        BN_COUNT(1);
        BN_CUDA(cudaGraphLaunch(m->token_graph, st));
        BN_COUNT(m->graph_launches);
        if (next_tok) {
            BN_CUDA(cudaMemcpyAsync(next_tok, m->NEXT, 4, cudaMemcpyDeviceToHost, st));
            BN_CUDA(cudaStreamSynchronize(st));
        }
        return BN_OK;
    }
    const int tp[2] = {tok, pos};
    BN_CUDA(cudaMemcpyAsync(m->TOK, &tp[0], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaMemcpyAsync(m->POS, &tp[1], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaStreamSynchronize(st));     // tp lives on this stack frame
    enqueue_token(m, stop_after_block, true);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = m->launch_err;
    m->launch_err = cudaSuccess;
    if (e != cudaSuccess) return bn_cuda_fail(e, "token schedule");
    if (next_tok) {
        BN_CUDA(cudaMemcpyAsync(next_tok, m->NEXT, 4, cudaMemcpyDeviceToHost, st));
        BN_CUDA(cudaStreamSynchronize(st));
    }
    return BN_OK;
}

int bn_model_decode(bn_model *m, int first_tok, int pos0, int n_steps, int *out_tokens) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_decode: model not finalized");
    const bn_hparams &h = m->hp;
    BN_REQUIRE(m->b0 == 0 && m->b1 == h.n_layer, BN_ERR_STATE, "bn_model_decode: this model holds blocks [%d, %d) only; use bn_model_stage", m->b0, m->b1);
    m->cur = 0;
    BN_REQUIRE(first_tok >= 0 && first_tok < h.vocab, BN_ERR_ARG, "bn_model_decode: token %d outside vocab %d", first_tok, h.vocab);
    BN_REQUIRE(n_steps > 0 && pos0 >= 0 && pos0 + n_steps <= h.cap, BN_ERR_BOUNDS,
               "bn_model_decode: positions [%d, %d) do not fit the KV capacity %d", pos0, pos0 + n_steps, h.cap);
    cudaStream_t st = m->ctx->stream;
    if (m->use_token) {
        // all n_steps tokens in ONE launch: the pick of a step is the next step's input inside the kernel
        m->next_pos = pos0 + n_steps;
        int rc = run_token_kernel(m, first_tok, pos0, n_steps, -1);
        if (rc != BN_OK) return rc;
        if (out_tokens) {
            BN_CUDA(cudaMemcpyAsync(out_tokens, m->HIST, size_t(n_steps) * 4, cudaMemcpyDeviceToHost, st));
            BN_CUDA(cudaStreamSynchronize(st));
        }
        return BN_OK;
    }
    { const int rc = ensure_token_graph(m); if (rc != BN_OK) return rc; }
    const int init[3] = {first_tok, pos0, 0};
    BN_CUDA(cudaMemcpyAsync(m->TOK, &init[0], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaMemcpyAsync(m->POS, &init[1], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaMemcpyAsync(m->STEP, &init[2], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaStreamSynchronize(st));
    m->next_pos = pos0 + n_steps;
    for (int i = 0; i < n_steps; ++i) {
        BN_CUDA(cudaGraphLaunch(m->token_graph, st));
        BN_COUNT(m->graph_launches);
    }
    if (out_tokens) {
        BN_CUDA(cudaMemcpyAsync(out_tokens, m->HIST, size_t(n_steps) * 4, cudaMemcpyDeviceToHost, st));
        BN_CUDA(cudaStreamSynchronize(st));
    }
    return BN_OK;
}

int bn_model_stage_prepare(bn_model *m, int stream0, int ncol) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_stage_prepare: model not finalized");
    const bn_hparams &h = m->hp;
    const int S = h.n_streams > 0 ? h.n_streams : 1;
    BN_REQUIRE(ncol >= 0 && stream0 >= 0 && stream0 + (ncol > 0 ? ncol : 1) <= S, BN_ERR_ARG,
               "bn_model_stage_prepare: sequences %d..%d outside [0, %d)", stream0, stream0 + (ncol > 0 ? ncol : 1) - 1, S);
    cudaStream_t st = m->ctx->stream;
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ge = nullptr;
    m->cur = stream0;
    if (ncol == 0) {
        if (m->stage_graphs.empty()) m->stage_graphs.assign(S, nullptr);
        if (m->stage_graphs[stream0]) return BN_OK;
    } else {
        BN_REQUIRE(h.batch_cols > 0 && ncol <= h.batch_cols, BN_ERR_ARG,
                   "bn_model_stage_prepare: %d sequences per pass, the model was created for at most %d (bn_hparams.batch_cols)", ncol, h.batch_cols);
        BN_REQUIRE(m->fused, BN_ERR_STATE, "bn_model_stage_prepare: the multi-sequence pass needs the fused layer kernels");
        if (m->batch_graphs.count(long(stream0) * 64 + ncol)) return BN_OK;
    }
    const unsigned long long before = g_bn_launches;
    BN_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    if (ncol == 0) enqueue_token(m, -1, true); else enqueue_batch(m, ncol);
    cudaError_t e = cudaStreamEndCapture(st, &g);
    if (e == cudaSuccess) e = m->launch_err;
    m->launch_err = cudaSuccess;
    if (e != cudaSuccess) return bn_cuda_fail(e, "cudaStreamEndCapture(stage)");
    (ncol == 0 ? m->graph_launches : m->batch_graph_launches) = int(g_bn_launches - before);
    g_bn_launches = before;               // captured, not launched
    e = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return bn_cuda_fail(e, "cudaGraphInstantiate(stage)");
    if (ncol == 0) m->stage_graphs[stream0] = ge; else m->batch_graphs.emplace(long(stream0) * 64 + ncol, ge);
    return BN_OK;
}

int bn_model_stage(bn_model *m, int stream, int tok, int pos, const bn_buf *in, size_t in_off, bn_buf *out, size_t out_off) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_stage: model not finalized");
    BN_REQUIRE(!m->head_sharded, BN_ERR_STATE, "bn_model_stage: a model with a sharded output head runs through bn_model_stage_batch and bn_model_head_batch");
    const bn_hparams &h = m->hp;
    const int S = h.n_streams > 0 ? h.n_streams : 1;
    BN_REQUIRE(stream >= 0 && stream < S, BN_ERR_ARG, "bn_model_stage: stream %d outside [0, %d)", stream, S);
    BN_REQUIRE(pos >= 0 && pos < h.cap, BN_ERR_BOUNDS, "bn_model_stage: position %d does not fit the KV capacity %d", pos, h.cap);
    const bool first = m->b0 == 0, last = m->b1 == h.n_layer;
    cudaStream_t st = m->ctx->stream;
    if (first) {
        BN_REQUIRE(tok < h.vocab, BN_ERR_ARG, "bn_model_stage: token %d outside vocab %d", tok, h.vocab);
        if (tok < 0) BN_RANGE(in, in_off, 4, 4, "bn_model_stage token input");
    } else BN_RANGE(in, in_off, size_t(h.hidden) * 4, 16, "bn_model_stage hidden input");
    BN_RANGE(out, out_off, last ? 4 : size_t(h.hidden) * 4, 4, "bn_model_stage output");
    m->cur = stream;
    m->next_pos = pos + 1;
    k_set_tok_pos<<<1, 32, 0, st>>>(m->TOK, m->POS, tok, pos, (first && tok < 0) ? bn_ptr<int>(in, in_off) : nullptr, h.vocab, m->ctx->err_dev);
    BN_COUNT(1);
    if (!first) BN_CUDA(cudaMemcpyAsync(m->RES, bn_ptr<char>(in, in_off), size_t(h.hidden) * 4, cudaMemcpyDeviceToDevice, st));
    cudaError_t e = cudaSuccess;
    if (getenv("BONSAI_NO_STAGE_GRAPH")) {
        enqueue_token(m, -1, true);
        e = cudaGetLastError();
    } else {
        // the ~100 launches of a stage are replayed as one graph: the host only feeds copies and NCCL calls. The graph
        // must exist already (bn_model_stage_prepare): building one here could synchronise a device whose stream holds a
        // send/recv kernel that is waiting for its peer
        BN_REQUIRE(stream < int(m->stage_graphs.size()) && m->stage_graphs[stream], BN_ERR_STATE,
                   "bn_model_stage: sequence %d was not prepared; call bn_model_stage_prepare(model, %d, 0) first", stream, stream);
        e = cudaGraphLaunch(m->stage_graphs[stream], st);
        BN_COUNT(m->graph_launches);
    }
    if (e == cudaSuccess) e = m->launch_err;
    m->launch_err = cudaSuccess;
    if (e != cudaSuccess) return bn_cuda_fail(e, "stage schedule");
    if (last) BN_CUDA(cudaMemcpyAsync(bn_ptr<char>(out, out_off), m->NEXT, 4, cudaMemcpyDeviceToDevice, st));
    else BN_CUDA(cudaMemcpyAsync(bn_ptr<char>(out, out_off), m->RES, size_t(h.hidden) * 4, cudaMemcpyDeviceToDevice, st));
    return BN_OK;
}

int bn_model_stage_batch(bn_model *m, int stream0, int ncol, const int *tok, const int *pos, const bn_buf *in, size_t in_off,
                         bn_buf *out, size_t out_off) {
    BN_REQUIRE(m && m->finalized && pos, BN_ERR_STATE, "bn_model_stage_batch: model not finalized or no positions");
    const bn_hparams &h = m->hp;
    const int S = h.n_streams > 0 ? h.n_streams : 1;
    BN_REQUIRE(h.batch_cols > 0 && ncol >= 1 && ncol <= h.batch_cols, BN_ERR_ARG,
               "bn_model_stage_batch: %d sequences per call, the model was created for at most %d (bn_hparams.batch_cols)", ncol, h.batch_cols);
    BN_REQUIRE(stream0 >= 0 && stream0 + ncol <= S, BN_ERR_ARG, "bn_model_stage_batch: sequences %d..%d outside [0, %d)", stream0, stream0 + ncol - 1, S);
    BN_REQUIRE(m->fused, BN_ERR_STATE, "bn_model_stage_batch: needs the fused layer kernels (shapes supported by the streamed projection kernel)");
    const bool first = m->b0 == 0, last = m->b1 == h.n_layer && !m->head_sharded;
    cudaStream_t st = m->ctx->stream;
    ColInit ci = {};
    for (int c = 0; c < ncol; ++c) {
        BN_REQUIRE(pos[c] >= 0 && pos[c] < h.cap, BN_ERR_BOUNDS, "bn_model_stage_batch: position %d does not fit the KV capacity %d", pos[c], h.cap);
        ci.pos[c] = pos[c];
        if (first && tok) {
            BN_REQUIRE(tok[c] >= 0 && tok[c] < h.vocab, BN_ERR_ARG, "bn_model_stage_batch: token %d outside vocab %d", tok[c], h.vocab);
            ci.tok[c] = tok[c];
        }
    }
    if (first) { if (!tok) BN_RANGE(in, in_off, size_t(ncol) * 4, 4, "bn_model_stage_batch token input"); }
    else BN_RANGE(in, in_off, size_t(ncol) * h.hidden * 4, 16, "bn_model_stage_batch hidden input");
    BN_RANGE(out, out_off, last ? size_t(ncol) * 4 : size_t(ncol) * h.hidden * 4, 4, "bn_model_stage_batch output");
    m->cur = stream0;
    m->next_pos = pos[0] + 1;
    k_set_cols<<<1, 32, 0, st>>>(m->TOK, m->POS, m->arena_bytes, ncol, ci, (first && !tok) ? bn_ptr<int>(in, in_off) : nullptr, h.vocab, m->ctx->err_dev);
    BN_COUNT(1);
    if (!first)
        BN_CUDA(cudaMemcpy2DAsync(m->RES, m->arena_bytes, bn_ptr<char>(in, in_off), size_t(h.hidden) * 4, size_t(h.hidden) * 4, ncol,
                                  cudaMemcpyDeviceToDevice, st));
    cudaError_t e = cudaSuccess;
    if (getenv("BONSAI_NO_STAGE_GRAPH")) {
        enqueue_batch(m, ncol);
        e = cudaGetLastError();
    } else {
        auto it = m->batch_graphs.find(long(stream0) * 64 + ncol);
        BN_REQUIRE(it != m->batch_graphs.end(), BN_ERR_STATE,
                   "bn_model_stage_batch: sequences %d..%d were not prepared as one pass; call bn_model_stage_prepare(model, %d, %d) first",
                   stream0, stream0 + ncol - 1, stream0, ncol);
        e = cudaGraphLaunch(it->second, st);
        BN_COUNT(m->batch_graph_launches);
    }
    if (e == cudaSuccess) e = m->launch_err;
    m->launch_err = cudaSuccess;
    if (e != cudaSuccess) return bn_cuda_fail(e, "stage batch schedule");
    if (last) BN_CUDA(cudaMemcpy2DAsync(bn_ptr<char>(out, out_off), 4, m->NEXT, m->arena_bytes, 4, ncol, cudaMemcpyDeviceToDevice, st));
    else BN_CUDA(cudaMemcpy2DAsync(bn_ptr<char>(out, out_off), size_t(h.hidden) * 4, m->RES, m->arena_bytes, size_t(h.hidden) * 4, ncol,
                                   cudaMemcpyDeviceToDevice, st));
    return BN_OK;
}

int bn_model_prefill(bn_model *m, const int *toks, int n, int pos0, int *next_tok) {
    BN_REQUIRE(m && m->finalized && toks, BN_ERR_STATE, "bn_model_prefill: model not finalized or no tokens");
    const bn_hparams &h = m->hp;
    BN_REQUIRE(h.batch_cols > 0 && n >= 1 && n <= h.batch_cols, BN_ERR_ARG,
               "bn_model_prefill: %d tokens per block, the model was created for at most %d (bn_hparams.batch_cols)", n, h.batch_cols);
    BN_REQUIRE(m->fused && m->b0 == 0 && m->b1 == h.n_layer && !m->head_sharded, BN_ERR_STATE,
               "bn_model_prefill: needs the whole model on this device and the fused layer kernels");
    BN_REQUIRE(pos0 >= 0 && pos0 + n <= h.cap, BN_ERR_BOUNDS, "bn_model_prefill: positions %d..%d do not fit the KV capacity %d", pos0, pos0 + n - 1, h.cap);
    ColInit ci = {};
    for (int c = 0; c < n; ++c) {
        BN_REQUIRE(toks[c] >= 0 && toks[c] < h.vocab, BN_ERR_ARG, "bn_model_prefill: token %d outside vocab %d", toks[c], h.vocab);
        ci.tok[c] = toks[c]; ci.pos[c] = pos0 + c;
    }
    cudaStream_t st = m->ctx->stream;
    m->cur = 0;
    m->next_pos = pos0 + n;
    k_set_cols<<<1, 32, 0, st>>>(m->TOK, m->POS, m->arena_bytes, n, ci, nullptr, h.vocab, m->ctx->err_dev);
    BN_COUNT(1);
    enqueue_batch(m, n, true);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = m->launch_err;
    m->launch_err = cudaSuccess;
    if (e != cudaSuccess) return bn_cuda_fail(e, "prefill schedule");
    // the pick after the block: output norm + head + first maximum on the last column's residual, through the
    // single-sequence kernels (whose buffers are column 0's)
    const size_t AS = m->arena_bytes / 4;
    if (n > 1) {
        BN_CUDA(cudaMemcpyAsync(m->RES, m->RES + size_t(n - 1) * AS, size_t(h.hidden) * 4, cudaMemcpyDeviceToDevice, st));
        BN_CUDA(cudaMemcpyAsync(m->POS, m->POS + size_t(n - 1) * AS, 4, cudaMemcpyDeviceToDevice, st));
        BN_CUDA(cudaMemcpyAsync(m->TOK, m->TOK + size_t(n - 1) * AS, 4, cudaMemcpyDeviceToDevice, st));
    }
    bnk::PhaseArgs a = phase_base(m, m->out_w, h.vocab, h.hidden, m->signs);
    a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = m->out_norm; a.out = m->LOGITS;
    launch(m, a);
    bnk::argmax_first(st, m->LOGITS, h.vocab, m->NEXT, m->AMV, m->AMI);
    if (next_tok) {
        BN_CUDA(cudaMemcpyAsync(next_tok, m->NEXT, 4, cudaMemcpyDeviceToHost, st));
        BN_CUDA(cudaStreamSynchronize(st));
    }
    return bn_launch_check(m->ctx, "bn_model_prefill");
}

int bn_model_set_head_rows(bn_model *m, int row_begin, int row_end) {
    BN_REQUIRE(m && !m->finalized, BN_ERR_STATE, "bn_model_set_head_rows: call before bn_model_finalize");
    const bn_hparams &h = m->hp;
    BN_REQUIRE(h.batch_cols > 0, BN_ERR_ARG, "bn_model_set_head_rows: the sharded output head belongs to the multi-sequence pass (bn_hparams.batch_cols > 0)");
    BN_REQUIRE(row_begin >= 0 && row_begin < row_end && row_end <= h.vocab && row_begin % 128 == 0 && (row_end % 128 == 0 || row_end == h.vocab),
               BN_ERR_ARG, "bn_model_set_head_rows: rows [%d, %d) must lie in [0, %d) on 128-row boundaries", row_begin, row_end, h.vocab);
    m->head_r0 = row_begin; m->head_r1 = row_end; m->head_sharded = true;
    return BN_OK;
}

int bn_model_head_batch(bn_model *m, int ncol, const bn_buf *in, size_t in_off, bn_buf *out, size_t out_off) {
    BN_REQUIRE(m && m->finalized && m->head_sharded, BN_ERR_STATE, "bn_model_head_batch: needs a finalized model with bn_model_set_head_rows");
    const bn_hparams &h = m->hp;
    BN_REQUIRE(ncol >= 1 && ncol <= h.batch_cols, BN_ERR_ARG, "bn_model_head_batch: %d sequences, the model was created for at most %d", ncol, h.batch_cols);
    BN_RANGE(in, in_off, size_t(ncol) * h.hidden * 4, 16, "bn_model_head_batch hidden input");
    BN_RANGE(out, out_off, size_t(ncol) * 8, 8, "bn_model_head_batch candidate output");
    cudaStream_t st = m->ctx->stream;
    // Nothing here touches what a stage pass uses (the hidden states are read where they lie, the activation image is the
    // head's own, logits and pick scratch belong to the head alone on a sharded model, no K-split scratch): the caller may
    // run the head on another CUDA stream (bn_use_stream) beside a stage pass of the same model.
    const size_t AS = m->arena_bytes / 4;
    bnk::Cols cols;
    cols.n = ncol; cols.arena = m->arena_bytes; cols.gdn = 0; cols.conv = 0; cols.kv = 0;
    bnk::PrepArgs p = {};
    p.x = bn_ptr<float>(in, in_off); p.x_stride = size_t(h.hidden); p.w = m->out_norm; p.signs = m->signs; p.K = h.hidden; p.hat_block = h.hat_block; p.eps = h.rms_eps; p.ncol = ncol;
    p.image = m->IMG_HD; p.inv_stride = AS; p.mode = bnk::PREP_NORM;
    bnk::prep_cols(st, p);
    const int rows = m->head_r1 - m->head_r0;
    bnk::GemmArgs a = {};
    a.W = m->t_head; a.M = rows; a.K = h.hidden; a.tiled = 1; a.image = m->IMG_HD; a.ncol = ncol; a.out = m->LOGITS; a.out_stride = AS; a.err = m->ctx->err_dev;
    cudaError_t e = bnk::launch_gemm(st, m->ctx->sm_count, a, m->use_pdl);
    if (e != cudaSuccess) return bn_cuda_fail(e, "bn_model_head_batch");
    bnk::argmax_first(st, m->LOGITS, rows, m->NEXT, m->AMV, m->AMI, cols, m->CAND, m->head_r0);
    BN_CUDA(cudaMemcpyAsync(bn_ptr<char>(out, out_off), m->CAND, size_t(ncol) * 8, cudaMemcpyDeviceToDevice, st));
    return bn_launch_check(m->ctx, "bn_model_head_batch");
}

int bn_model_pick_batch(bn_model *m, int ncol, int n_shards, const bn_buf *cands, size_t cands_off, bn_buf *out, size_t out_off) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_pick_batch: model not finalized");
    BN_REQUIRE(ncol >= 1 && ncol <= 32 && n_shards >= 1 && n_shards <= 64, BN_ERR_ARG, "bn_model_pick_batch: %d sequences x %d shards out of range", ncol, n_shards);
    BN_RANGE(cands, cands_off, size_t(n_shards) * ncol * 8, 8, "bn_model_pick_batch candidates");
    BN_RANGE(out, out_off, size_t(ncol) * 4, 4, "bn_model_pick_batch output");
    bnk::pick_shards(m->ctx->stream, bn_ptr<float>(cands, cands_off), n_shards, ncol, bn_ptr<int>(out, out_off));
    return bn_launch_check(m->ctx, "bn_model_pick_batch");
}

int bn_model_fill_kv(bn_model *m, int stream, int n_positions) {
    BN_REQUIRE(m && m->finalized, BN_ERR_STATE, "bn_model_fill_kv: model not finalized");
    const bn_hparams &h = m->hp;
    const int S = h.n_streams > 0 ? h.n_streams : 1;
    BN_REQUIRE(stream >= 0 && stream < S && n_positions >= 0 && n_positions <= h.cap, BN_ERR_ARG, "bn_model_fill_kv: bad stream or count");
    const size_t n = size_t(n_positions) * h.n_kv * h.head_dim;
    m->cur = stream;
    for (int li = 0; li < m->n_attn && n; ++li) {
        const bnk::KvLayer kv = kv_layer(m, li);
        // every stored key / value element = 1.0: codes 127 with scale 1/127 (q8_0) or fp16 1.0
        if (h.k_mode == 0) { BN_CUDA(cudaMemsetAsync(kv.k_data, 127, n, m->ctx->stream)); k_fill_u16<<<256, 256, 0, m->ctx->stream>>>(kv.k_scale, n / 32, 0x2008); }
        else k_fill_u16<<<256, 256, 0, m->ctx->stream>>>(reinterpret_cast<uint16_t *>(kv.k_data), n, 0x3C00);
        if (h.v_mode == 0) { BN_CUDA(cudaMemsetAsync(kv.v_data, 127, n, m->ctx->stream)); k_fill_u16<<<256, 256, 0, m->ctx->stream>>>(kv.v_scale, n / 32, 0x2008); }
        else k_fill_u16<<<256, 256, 0, m->ctx->stream>>>(reinterpret_cast<uint16_t *>(kv.v_data), n, 0x3C00);
        BN_COUNT(2);
    }
    return bn_launch_check(m->ctx, "bn_model_fill_kv");
}

int bn_model_gemv_sweep(bn_model *m, int reps, float *ms_per_sweep) {
    BN_REQUIRE(m && m->finalized && ms_per_sweep && reps > 0, BN_ERR_ARG, "bn_model_gemv_sweep: bad argument");
    BN_REQUIRE(m->b0 == 0 && m->b1 == m->hp.n_layer, BN_ERR_STATE, "bn_model_gemv_sweep: whole model only");
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D, IN = NH * D;
    const int QD = h.n_head * h.head_dim, KD = h.n_kv * h.head_dim;
    cudaStream_t st = m->ctx->stream;
    const int sm = m->ctx->sm_count;
    auto sweep = [&]() {
        if (m->fused) {      // the production launches: every fused projection kernel of one token, nothing else
            m->phases_only = true;
            for (const bn_model::Layer &L : m->layers) { if (L.attn) attn_fused(m, L); else gdn_fused(m, L); ffn_fused(m, L); }
            bnk::PhaseArgs a = phase_base(m, m->out_w, h.vocab, h.hidden, m->signs);
            a.pro = bnk::PRO_NORM; a.x0 = m->RES; a.w = m->out_norm; a.out = m->LOGITS;
            launch(m, a);
            m->phases_only = false;
            return;
        }
        for (const bn_model::Layer &L : m->layers) {
            if (L.attn) {
                bnk::gemv_q81(st, sm, L.q_w, 2 * QD, h.hidden, m->PACK_H, m->QKV, m->GEMV_SCRATCH, nullptr);
                bnk::gemv_q81(st, sm, L.k_w, KD, h.hidden, m->PACK_H, m->KBUF, m->GEMV_SCRATCH, nullptr);
                bnk::gemv_q81(st, sm, L.v_w, KD, h.hidden, m->PACK_H, m->VBUF, m->GEMV_SCRATCH, nullptr);
                bnk::gemv_q81(st, sm, L.o_w, h.hidden, QD, m->PACK_H, m->D, m->GEMV_SCRATCH, nullptr);
            } else {
                bnk::gemv_q81(st, sm, L.qkv, C, h.hidden, m->PACK_H, m->QKV, m->GEMV_SCRATCH, nullptr);
                bnk::gemv_q81(st, sm, L.gate_w, IN, h.hidden, m->PACK_H, m->Z, m->GEMV_SCRATCH, nullptr);
                bnk::gemv_q81(st, sm, L.ssm_out, h.hidden, IN, m->PACK_H, m->D, m->GEMV_SCRATCH, nullptr);
            }
            bnk::gemv_q81(st, sm, L.ffn_gate, h.ffn, h.hidden, m->PACK_H, m->FG, m->GEMV_SCRATCH, nullptr);
            bnk::gemv_q81(st, sm, L.ffn_up, h.ffn, h.hidden, m->PACK_H, m->FU, m->GEMV_SCRATCH, nullptr);
            bnk::gemv_q81(st, sm, L.ffn_down, h.hidden, h.ffn, m->PACK_F, m->D, m->GEMV_SCRATCH, nullptr);
        }
        bnk::gemv_q81(st, sm, m->out_w, h.vocab, h.hidden, m->PACK_H, m->LOGITS, m->GEMV_SCRATCH, nullptr);
    };
    cudaEvent_t e0, e1;
    BN_CUDA(cudaEventCreate(&e0));
    BN_CUDA(cudaEventCreate(&e1));
    sweep();
    BN_CUDA(cudaEventRecord(e0, st));
    for (int r = 0; r < reps; ++r) sweep();
    BN_CUDA(cudaEventRecord(e1, st));
    BN_CUDA(cudaEventSynchronize(e1));
    float ms = 0.0f;
    BN_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_sweep = ms / float(reps);
    return BN_OK;
}

int bn_model_mixer_sweep(bn_model *m, int reps, float *us_per_gdn_layer, float *us_per_attn_layer) {
    BN_REQUIRE(m && m->finalized && reps > 0 && us_per_gdn_layer && us_per_attn_layer, BN_ERR_ARG, "bn_model_mixer_sweep: bad argument");
    BN_REQUIRE(m->fused && m->b0 == 0 && m->b1 == m->hp.n_layer, BN_ERR_STATE, "bn_model_mixer_sweep: whole model with the fused kernels only");
    cudaStream_t st = m->ctx->stream;
    cudaEvent_t e0, e1;
    BN_CUDA(cudaEventCreate(&e0));
    BN_CUDA(cudaEventCreate(&e1));
    m->cur = 0;
    float out[2] = {0.0f, 0.0f};
    for (int kind = 0; kind < 2; ++kind) {         // 0: gated-delta-net cores, 1: attention (insert + decode at POS[0])
        int n = 0;
        for (const bn_model::Layer &L : m->layers) n += (L.attn ? 1 : 0) == kind;
        if (!n) continue;
        auto sweep = [&]() {
            m->mixers_only = true;
            for (const bn_model::Layer &L : m->layers) {
                if (kind == 0 && !L.attn) gdn_fused(m, L);
                if (kind == 1 && L.attn) attn_fused(m, L);
            }
            m->mixers_only = false;
        };
        sweep();
        BN_CUDA(cudaEventRecord(e0, st));
        for (int r = 0; r < reps; ++r) sweep();
        BN_CUDA(cudaEventRecord(e1, st));
        BN_CUDA(cudaEventSynchronize(e1));
        float ms = 0.0f;
        BN_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        out[kind] = ms * 1000.0f / float(reps) / float(n);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *us_per_gdn_layer = out[0];
    *us_per_attn_layer = out[1];
    return bn_launch_check(m->ctx, "bn_model_mixer_sweep");
}

int bn_model_profile_token(bn_model *m, int tok, int pos, unsigned long long *stamps_out, int max_phases, int *n_phases) {
    BN_REQUIRE(m && m->finalized && stamps_out && n_phases, BN_ERR_ARG, "bn_model_profile_token: bad argument");
    BN_REQUIRE(pos >= 0 && pos < m->hp.cap && tok >= 0 && tok < m->hp.vocab, BN_ERR_ARG, "bn_model_profile_token: bad token or position");
    if (!m->stamps) BN_CUDA(cudaMalloc(&m->stamps, 256 * 8 * sizeof(unsigned long long)));
    BN_CUDA(cudaMemset(m->stamps, 0, 256 * 8 * sizeof(unsigned long long)));
    cudaStream_t st = m->ctx->stream;
    const int tp[2] = {tok, pos};
    BN_CUDA(cudaMemcpyAsync(m->TOK, &tp[0], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaMemcpyAsync(m->POS, &tp[1], 4, cudaMemcpyHostToDevice, st));
    BN_CUDA(cudaStreamSynchronize(st));
    m->stamp_idx = 0;
    unsigned long long *keep = m->stamps;
    enqueue_token(m, -1, true);
    const int n = m->stamp_idx;
    m->stamps = nullptr;                 // later tokens run unstamped
    BN_CUDA(cudaStreamSynchronize(st));
    *n_phases = n < max_phases ? n : max_phases;
    BN_CUDA(cudaMemcpy(stamps_out, keep, size_t(*n_phases) * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    m->stamps = keep;
    cudaMemset(keep, 0, 8);
    m->stamps = nullptr;
    cudaFree(keep);
    return BN_OK;
}

int bn_model_read(bn_model *m, int what, int index, void *dst, size_t bytes) {
    BN_REQUIRE(m && m->finalized && dst, BN_ERR_STATE, "bn_model_read: bad state or null destination");
    const bn_hparams &h = m->hp;
    const int NH = h.gdn_heads, NQ = h.gdn_qk_heads, D = h.gdn_dim, C = 2 * NQ * D + NH * D;
    const size_t kvn = size_t(h.cap) * h.n_kv * h.head_dim;
    const void *src = nullptr;
    size_t have = 0;
    switch (what) {
        case BN_READ_LOGITS:
            BN_REQUIRE(index >= 0 && index < m->ncols, BN_ERR_ARG, "bn_model_read: logits of column %d, the model has %d", index, m->ncols);
            src = m->LOGITS + size_t(index) * (m->arena_bytes / 4); have = size_t(h.vocab) * 4; break;
        case BN_READ_RESIDUAL: src = m->RES; have = size_t(h.hidden) * 4; break;
        case BN_READ_GDN_STATE:
            BN_REQUIRE(index >= 0 && index < m->n_gdn, BN_ERR_ARG, "bn_model_read: gdn layer %d out of range", index);
            src = gdn_state_of(m, index); have = size_t(NH) * D * D * 4; break;
        case BN_READ_CONV_HIST:
            BN_REQUIRE(index >= 0 && index < m->n_gdn, BN_ERR_ARG, "bn_model_read: gdn layer %d out of range", index);
            // fused path: the taps the next token will read live in the buffer of its position parity
            src = conv_of(m, (m->fused && (m->next_pos & 1)) ? 1 : 0, index); have = size_t(C) * 3 * 4; break;
        case BN_READ_K_DATA: case BN_READ_K_SCALE: case BN_READ_V_DATA: case BN_READ_V_SCALE: {
            BN_REQUIRE(index >= 0 && index < m->n_attn, BN_ERR_ARG, "bn_model_read: attention layer %d out of range", index);
            const bnk::KvLayer kv = kv_layer(m, index);
            if (what == BN_READ_K_DATA) { src = kv.k_data; have = h.k_mode == 0 ? kvn : kvn * 2; }
            if (what == BN_READ_V_DATA) { src = kv.v_data; have = h.v_mode == 0 ? kvn : kvn * 2; }
            if (what == BN_READ_K_SCALE) { src = kv.k_scale; have = h.k_mode == 0 ? kvn / 32 * 2 : 0; }
            if (what == BN_READ_V_SCALE) { src = kv.v_scale; have = h.v_mode == 0 ? kvn / 32 * 2 : 0; }
            break;
        }
        case 9: src = m->tok_stamps; have = m->tok_stamps ? size_t(bnk::TOKEN_MAX_OPS + 64) * 8 * sizeof(unsigned long long) : 0; break;
        case 8: src = m->graph_stamps; have = m->graph_stamps ? 256 * 8 * sizeof(unsigned long long) : 0; break;
        default: BN_REQUIRE(false, BN_ERR_ARG, "bn_model_read: unknown selector %d", what);
    }
    BN_REQUIRE(src && bytes <= have, BN_ERR_BOUNDS, "bn_model_read: %zu bytes requested, %zu available", bytes, have);
    BN_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, m->ctx->stream));
    BN_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return BN_OK;
}

}  // extern "C"
