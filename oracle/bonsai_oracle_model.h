// bonsai_oracle_model.h - block-level and whole-token CPU restatement of the bonsai-vk forward.
// TEST INFRASTRUCTURE ONLY (see bonsai_oracle.h). Each function cites the reference text it follows
// (paths relative to the reference tree, runtime_vk/ unless stated).
//
// Frozen semantic switches (defaults of the reference's Fwd struct, bonsai_forward.h:225-230):
// gdn_mode 0 (decay before predict), gdn_gmap 0 (q/k head = h % 16), l2 mode 1 with eps 1e-12,
// round_probs 1, softplus threshold 20, swiglu = silu(first operand) * second.
#ifndef BONSAI_ORACLE_MODEL_H
#define BONSAI_ORACLE_MODEL_H

#include "bonsai_oracle.h"

#include <algorithm>
#include <map>
#include <string>
#include <thread>

namespace bo {

enum ActMode { ACT_Q81 = 0, ACT_F32 = 1 };   // activation form of the 201 PTQ1_0 projections
enum KvMode { KV_Q80 = 0, KV_F16 = 1 };

struct HParams {
    int n_layer = 32, hidden = 4096, ffn = 12288, vocab = 248320;
    int n_head = 16, n_kv = 4, head_dim = 256, n_rot = 64, attn_interval = 4;
    int gdn_heads = 32, gdn_qk_heads = 16, gdn_dim = 128, conv_k = 4;
    int hat_block = 4096;
    float rms_eps = 1e-6f, rope_base = 1e7f;
    int act_mode = ACT_Q81, k_mode = KV_Q80, v_mode = KV_Q80;
    int cap = 256;          // KV capacity in positions
    int attn_order = 0;     // 0: the reference's serial order; 1: the CUDA kernels' order (same arithmetic,
    int pv_splits = 1;      //    sums regrouped as stated at attn_core_device_order)
    int threads = 8;        // row-parallel threads for the projections
    unsigned long long attn_mask = 0;   // attn_interval == 0: the resolved explicit layer list, bit b = block b is attention
    bool is_attn(int b) const {         // bonsai_model.h:136-148 (interval rule, or the per-layer list when the file has one)
        return attn_interval > 0 ? (b % attn_interval) == attn_interval - 1 : ((attn_mask >> b) & 1ull) != 0;
    }
    int qkv_dim() const { return 2 * gdn_qk_heads * gdn_dim + gdn_heads * gdn_dim; }  // 8192
    int inner() const { return gdn_heads * gdn_dim; }                                 // 4096
};

struct Model {
    HParams hp;
    std::map<std::string, const void *> t;     // tensor name -> borrowed pointer (GGUF names)
    const int32_t *signs = nullptr;            // prism.hadamard.sign_values: [hidden | ffn]
    // state
    std::vector<std::vector<float>> gdn_state; // per GDN layer [h][j][i]
    std::vector<std::vector<float>> conv_hist; // per GDN layer [c][3]
    // KV per attention layer
    std::vector<std::vector<uint16_t>> k16, v16;         // fp16 modes: [cap][nkv][hd]
    std::vector<std::vector<int8_t>> kq, vq;             // q8_0 codes [cap][nkv][hd]
    std::vector<std::vector<uint16_t>> ks, vs;           // q8_0 scales [cap][nkv][hd/32]
    // taps for block-level tests
    std::vector<float> last_logits;

    const uint8_t *ptq(const std::string &n) const { return static_cast<const uint8_t *>(t.at(n)); }
    const float *f32(const std::string &n) const { return static_cast<const float *>(t.at(n)); }

    void reset() {
        const HParams &h = hp;
        int n_gdn = 0, n_attn = 0;
        for (int b = 0; b < h.n_layer; ++b) (h.is_attn(b) ? n_attn : n_gdn)++;
        gdn_state.assign(n_gdn, std::vector<float>(size_t(h.gdn_heads) * h.gdn_dim * h.gdn_dim, 0.0f));
        conv_hist.assign(n_gdn, std::vector<float>(size_t(h.qkv_dim()) * 3, 0.0f));
        const size_t kvn = size_t(h.cap) * h.n_kv * h.head_dim;
        k16.assign(n_attn, {}); v16.assign(n_attn, {}); kq.assign(n_attn, {}); vq.assign(n_attn, {});
        ks.assign(n_attn, {}); vs.assign(n_attn, {});
        for (int a = 0; a < n_attn; ++a) {
            if (h.k_mode == KV_F16) k16[a].assign(kvn, 0); else { kq[a].assign(kvn, 0); ks[a].assign(kvn / 32, 0); }
            if (h.v_mode == KV_F16) v16[a].assign(kvn, 0); else { vq[a].assign(kvn, 0); vs[a].assign(kvn / 32, 0); }
        }
    }
};

// ---- the PTQ1_0 projection in either activation mode (gemv_ptq, bonsai_forward.h:409-422) --------
static inline int pick_splits(int M, int nblk) {   // bonsai_weights.h:582-588
    int s = 1;
    while (s < 16 && (long(M / 64 + (M % 64 != 0)) * s < 640) && (nblk % (s * 2) == 0)) s *= 2;
    return s;
}
static inline void project(const Model &m, const uint8_t *W, int M, int K, const float *x_rot, float *out) {
    const int threads = m.hp.threads;
    std::vector<uint32_t> xq;
    if (m.hp.act_mode == ACT_Q81) { xq.resize(size_t(K / 128) * Q81_X4_DWORDS); quantize_q8_1_x4(x_rot, K, xq.data()); }
    const size_t rb = size_t(K / 128) * PTQ_BLOCK_BYTES;
    const int S = pick_splits(M, K / 128);
    auto work = [&](int r0, int r1) {
        if (m.hp.act_mode == ACT_Q81) gemv_q81(W + rb * r0, r1 - r0, K, xq.data(), out + r0, nullptr, nullptr);
        else gemv_f32act(W + rb * r0, r1 - r0, K, x_rot, S, out + r0, nullptr);
    };
    if (threads <= 1 || M < 256) { work(0, M); return; }
    std::vector<std::thread> th;
    const int per = (M + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) { const int r0 = t * per, r1 = std::min(M, r0 + per); if (r0 < r1) th.emplace_back(work, r0, r1); }
    for (auto &t : th) t.join();
}
// rotate (signs then H, bonsai_forward.h:471-476) followed by the projection
static inline void rot_project(const Model &m, const std::string &name, int M, int K, const float *x,
                               const int32_t *signs, float *out) {
    std::vector<float> hr(K);
    rotate_fwd(x, signs, K, m.hp.hat_block, hr.data());
    project(m, m.ptq(name), M, K, hr.data(), out);
}

// small fp32 projection (gemv_f32.comp): M rows of K floats. Order fixed here: lane l of 32 takes the
// float4 groups l, l+32, ... ascending with one fmaf per element, then a 32-lane xor tree.
static inline void gemv_f32_small(const float *W, int M, int K, const float *x, float *out) {
    for (int r = 0; r < M; ++r) {
        float part[32];
        for (int l = 0; l < 32; ++l) {
            float a = 0.0f;
            for (int i = l; i < K / 4; i += 32)
                for (int e = 0; e < 4; ++e) a = std::fmaf(W[size_t(r) * K + 4 * i + e], x[4 * i + e], a);
            part[l] = a;
        }
        out[r] = tree_sum(part, 32);
    }
}

// ---- FFN (ffn_block, bonsai_forward.h:489-506) ---------------------------------------------------
static inline void ffn_block(const Model &m, int b, float *res) {
    const HParams &h = m.hp;
    const std::string B = "blk." + std::to_string(b) + ".";
    std::vector<float> an(h.hidden), fg(h.ffn), fu(h.ffn), fs(h.ffn), d(h.hidden);
    rms_norm(res, m.f32(B + "post_attention_norm.weight"), h.hidden, h.rms_eps, an.data());
    std::vector<float> hr(h.hidden);
    rotate_fwd(an.data(), m.signs, h.hidden, h.hat_block, hr.data());
    project(m, m.ptq(B + "ffn_gate.weight"), h.ffn, h.hidden, hr.data(), fg.data());
    project(m, m.ptq(B + "ffn_up.weight"), h.ffn, h.hidden, hr.data(), fu.data());
    for (int i = 0; i < h.ffn; ++i) fs[i] = silu_f(fg[i]) * fu[i];
    rot_project(m, B + "ffn_down.weight", h.hidden, h.ffn, fs.data(), m.signs + h.hidden, d.data());
    for (int i = 0; i < h.hidden; ++i) res[i] = d[i] + res[i];          // add.comp: a + b with a = GDNO
}

// ---- gated delta net block (gdn_block, bonsai_forward.h:509-573) ---------------------------------
static inline float tree128(float *sh) {      // gdn_delta.comp tree_reduce: sh[l] += sh[l+s], s = 64..1
    for (int s = 64; s > 0; s >>= 1) for (int l = 0; l < s; ++l) sh[l] += sh[l + s];
    return sh[0];
}
static inline void gdn_mix(Model &m, int b, int gi, float *res) {
    const HParams &h = m.hp;
    const std::string B = "blk." + std::to_string(b) + ".";
    const int D = h.gdn_dim, NH = h.gdn_heads, NQ = h.gdn_qk_heads, C = h.qkv_dim(), IN = h.inner();
    std::vector<float> an(h.hidden), alpha(NH), beta(NH), gate(NH), hr(h.hidden), qkv(C), z(IN), conv(C), l2(2 * NQ * D);
    rms_norm(res, m.f32(B + "attn_norm.weight"), h.hidden, h.rms_eps, an.data());
    // alpha / beta read the UNROTATED normed vector (bonsai_forward.h:523-525)
    gemv_f32_small(m.f32(B + "ssm_alpha.weight"), NH, h.hidden, an.data(), alpha.data());
    gemv_f32_small(m.f32(B + "ssm_beta.weight"), NH, h.hidden, an.data(), beta.data());
    const float *dtb = m.f32(B + "ssm_dt.bias"), *ssa = m.f32(B + "ssm_a");
    for (int i = 0; i < NH; ++i) {
        gate[i] = softplus_f(alpha[i] + dtb[i], 20.0f) * ssa[i];        // :528-533
        beta[i] = sigmoid_f(beta[i]);                                   // :534
    }
    rotate_fwd(an.data(), m.signs, h.hidden, h.hat_block, hr.data());
    project(m, m.ptq(B + "attn_qkv.weight"), C, h.hidden, hr.data(), qkv.data());
    project(m, m.ptq(B + "attn_gate.weight"), IN, h.hidden, hr.data(), z.data());
    // conv_silu.comp:35-49 - 4-tap causal depthwise conv, silu, 3-deep history shift
    const float *cw = m.f32(B + "ssm_conv1d.weight");
    float *hist = m.conv_hist[gi].data();
    for (int c = 0; c < C; ++c) {
        float *s = hist + 3 * c; const float *w = cw + 4 * c;
        float acc = w[0] * s[0];
        acc = acc + w[1] * s[1]; acc = acc + w[2] * s[2]; acc = acc + w[3] * qkv[c];
        conv[c] = silu_f(acc);
        s[0] = s[1]; s[1] = s[2]; s[2] = qkv[c];
    }
    for (int r = 0; r < 2 * NQ; ++r) l2_norm(conv.data() + r * D, D, 1e-12f, l2.data() + r * D);   // l2_norm.comp mode 1
    const float *q = l2.data(), *k = l2.data() + NQ * D, *v = conv.data() + 2 * NQ * D;
    // gdn_delta.comp:78-102
    std::vector<float> o(IN);
    float *S = m.gdn_state[gi].data();
    const float scale = 1.0f / std::sqrt(float(D));
    float sh[128];
    for (int hh = 0; hh < NH; ++hh) {
        const int hq = hh % NQ;
        const float eg = exp_f(gate[hh]);
        for (int j = 0; j < D; ++j) {
            float *Sj = S + (size_t(hh) * D + j) * D;
            for (int i = 0; i < D; ++i) { Sj[i] = Sj[i] * eg; sh[i] = Sj[i] * k[hq * D + i]; }
            const float pred = tree128(sh);
            const float u = beta[hh] * (v[hh * D + j] - pred);
            for (int i = 0; i < D; ++i) { Sj[i] = std::fmaf(k[hq * D + i], u, Sj[i]); sh[i] = Sj[i] * q[hq * D + i]; }
            o[hh * D + j] = tree128(sh) * scale;
        }
    }
    // per-head RMS (no weight), ssm_norm broadcast, swiglu(z, o), v-grouped permutation (:559-567)
    std::vector<float> on(IN), swg(IN), perm(IN), out(h.hidden);
    const float *sn = m.f32(B + "ssm_norm.weight");
    for (int hh = 0; hh < NH; ++hh) {
        rms_norm(o.data() + hh * D, nullptr, D, h.rms_eps, on.data() + hh * D);
        for (int d = 0; d < D; ++d) on[hh * D + d] = on[hh * D + d] * sn[d];
    }
    for (int i = 0; i < IN; ++i) swg[i] = silu_f(z[i]) * on[i];
    const int sub = NH / NQ;
    for (int hh = 0; hh < NH; ++hh)                                   // permute_vg.comp:32-42
        for (int d = 0; d < D; ++d) perm[hh * D + d] = swg[d + D * (hh / sub + NQ * (hh % sub))];
    rot_project(m, B + "ssm_out.weight", h.hidden, IN, perm.data(), m.signs, out.data());
    for (int i = 0; i < h.hidden; ++i) res[i] = out[i] + res[i];
}

// ---- attention block (attn_block, bonsai_forward.h:581-645; kernels attn_norm_rope2.comp,
//      attn_qk_softmax*.comp, attn_pv_q8v.comp; CPU mirror attn_vk.h:102-311) ----------------------
// norm + NeoX rope on the first n_rot dims of one head row (attn_norm_rope2.comp:137-160)
static inline void head_norm_rope(const HParams &h, const float *x, const float *w, int pos, float *y) {
    const int hd = h.head_dim;
    float ss = 0.0f;                                    // attn_vk.h:102-108: squares summed serially, ascending d
    for (int d = 0; d < hd; ++d) ss = ss + x[d] * x[d];
    const float inv = 1.0f / std::sqrt(ss / float(hd) + h.rms_eps);
    for (int d = 0; d < hd; ++d) y[d] = (x[d] * inv) * w[d];
    const int half = h.n_rot / 2;
    for (int p = 0; p < half; ++p) {
        const float ex = -2.0f * float(p) / float(h.n_rot);
        const float th = float(std::pow(double(h.rope_base), double(ex)));
        const float a = float(pos) * th;
        const float c = float(std::cos(double(a))), s = float(std::sin(double(a)));
        const float lo = (x[p] * inv) * w[p], hi = (x[p + half] * inv) * w[p + half];
        y[p] = lo * c - hi * s;
        y[p + half] = hi * c + lo * s;
    }
}

struct AttnTap { std::vector<float> pregate, gated, prob; };

// Softmax-attention over the layer's cache for one query token at position pos, reference order:
// scores ascending d, max / exp / sum serial ascending j, probabilities rounded to fp16, PV ascending j.
static inline void attn_core(const Model &m, int li, int pos, const float *q16f /*[nh][hd] fp16-rounded*/,
                             const float *gate /*[nh][hd]*/, float *gated, AttnTap *tap) {
    const HParams &h = m.hp;
    const int hd = h.head_dim, nkv = h.n_kv, nfill = pos + 1, gqa = h.n_head / h.n_kv;
    const float scale = 1.0f / std::sqrt(float(hd));
    std::vector<float> sc(nfill), p(nfill), kd(hd);
    if (tap) { tap->pregate.assign(size_t(h.n_head) * hd, 0); tap->gated.assign(size_t(h.n_head) * hd, 0); tap->prob.assign(size_t(h.n_head) * nfill, 0); }
    for (int hh = 0; hh < h.n_head; ++hh) {
        const int kv = hh / gqa;
        const float *q = q16f + size_t(hh) * hd;
        for (int j = 0; j < nfill; ++j) {
            const size_t row = (size_t(j) * nkv + kv) * hd;
            float acc = 0.0f;
            if (h.k_mode == KV_F16) {
                const uint16_t *kr = m.k16[li].data() + row;
                for (int d = 0; d < hd; ++d) acc = acc + q[d] * f16_to_f32(kr[d]);
            } else {     // q8_0 K: element = scale * code in fp32, as the reference dequantises q8_0 V
                const int8_t *kc = m.kq[li].data() + row; const uint16_t *ksc = m.ks[li].data() + row / 32;
                for (int d = 0; d < hd; ++d) acc = acc + q[d] * (f16_to_f32(ksc[d / 32]) * float(kc[d]));
            }
            sc[j] = acc;
        }
        float mx = -INFINITY;
        for (int j = 0; j < nfill; ++j) { const float v = sc[j] * scale + 0.0f; if (v > mx) mx = v; }
        float sum = 0.0f;
        for (int j = 0; j < nfill; ++j) { const float v = sc[j] * scale + 0.0f; p[j] = exp_f(v - mx); sum = sum + p[j]; }
        for (int j = 0; j < nfill; ++j) { p[j] = p[j] / sum; if (tap) tap->prob[size_t(hh) * nfill + j] = p[j]; p[j] = f16_to_f32(f32_to_f16(p[j])); }
        for (int d = 0; d < hd; ++d) {
            float acc = 0.0f;
            for (int j = 0; j < nfill; ++j) {
                const size_t idx = (size_t(j) * nkv + kv) * hd + d;
                const float v = h.v_mode == KV_F16 ? f16_to_f32(m.v16[li][idx])
                                                   : f16_to_f32(m.vs[li][idx / 32]) * float(m.vq[li][idx]);
                acc = acc + p[j] * v;
            }
            const float g = acc * (1.0f / (1.0f + exp_f(-gate[size_t(hh) * hd + d])));
            gated[size_t(hh) * hd + d] = g;
            if (tap) { tap->pregate[size_t(hh) * hd + d] = acc; tap->gated[size_t(hh) * hd + d] = g; }
        }
    }
}

// The same attention with the sums regrouped the way the CUDA kernels group them, so that a whole-token
// run can be compared bit for bit. Differences from attn_core (each within float rounding of it):
//   score: lane l of 32 covers dims 8l..8l+7 with an fmaf chain, lanes combined by the xor tree 16..1;
//   sum of exp: thread t of 1024 adds keys t, t+1024, ... ascending, then the tree 512..1;
//   PV: keys split into pv_splits contiguous runs of ceil(nfill/pv_splits), each run ascending with
//       separate multiply and add, runs added ascending.
static inline void attn_core_device_order(const Model &m, int li, int pos, const float *q16f, const float *gate,
                                          float *gated, AttnTap *tap) {
    const HParams &h = m.hp;
    const int hd = h.head_dim, nkv = h.n_kv, nfill = pos + 1, gqa = h.n_head / h.n_kv;
    const float scale = 1.0f / std::sqrt(float(hd));
    std::vector<float> sc(nfill), p(nfill);
    if (tap) { tap->pregate.assign(size_t(h.n_head) * hd, 0); tap->gated.assign(size_t(h.n_head) * hd, 0); tap->prob.assign(size_t(h.n_head) * nfill, 0); }
    const int splits = h.pv_splits, per = (nfill + splits - 1) / splits;
    for (int hh = 0; hh < h.n_head; ++hh) {
        const int kv = hh / gqa;
        const float *q = q16f + size_t(hh) * hd;
        for (int j = 0; j < nfill; ++j) {
            const size_t row = (size_t(j) * nkv + kv) * hd;
            float part[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.0f;
                for (int e = 0; e < 8; ++e) {
                    const int d = 8 * l + e;
                    const float kvv = h.k_mode == KV_F16 ? f16_to_f32(m.k16[li][row + d])
                                                        : f16_to_f32(m.ks[li][(row + d) / 32]) * float(m.kq[li][row + d]);
                    acc = std::fmaf(q[d], kvv, acc);
                }
                part[l] = acc;
            }
            sc[j] = tree_sum(part, 32);
        }
        float mx = -INFINITY;
        for (int j = 0; j < nfill; ++j) { const float v = sc[j] * scale; if (v > mx) mx = v; }
        std::vector<float> red(1024, 0.0f);
        for (int t = 0; t < 1024; ++t) {
            float sum = 0.0f;
            for (int j = t; j < nfill; j += 1024) { p[j] = exp_f(sc[j] * scale - mx); sum = sum + p[j]; }
            red[t] = sum;
        }
        const float tot = tree_sum(red.data(), 1024);
        for (int j = 0; j < nfill; ++j) { p[j] = p[j] / tot; if (tap) tap->prob[size_t(hh) * nfill + j] = p[j]; p[j] = f16_to_f32(f32_to_f16(p[j])); }
        for (int d = 0; d < hd; ++d) {
            float total = 0.0f;
            for (int s = 0; s < splits; ++s) {
                const int j0 = s * per, j1 = std::min(nfill, j0 + per);
                if (s > 0 && j0 >= nfill) break;
                float acc = 0.0f;
                for (int j = j0; j < j1; ++j) {
                    const size_t idx = (size_t(j) * nkv + kv) * hd + d;
                    const float v = h.v_mode == KV_F16 ? f16_to_f32(m.v16[li][idx])
                                                       : f16_to_f32(m.vs[li][idx / 32]) * float(m.vq[li][idx]);
                    acc = acc + p[j] * v;
                }
                total = s == 0 ? acc : total + acc;
            }
            const float g = total * (1.0f / (1.0f + exp_f(-gate[size_t(hh) * hd + d])));
            gated[size_t(hh) * hd + d] = g;
            if (tap) { tap->pregate[size_t(hh) * hd + d] = total; tap->gated[size_t(hh) * hd + d] = g; }
        }
    }
}

// norm/rope/pack of q, k and the cache insert of k, v at `pos` (attn_norm_rope2.comp:117-218)
static inline void attn_insert(Model &m, int li, int b, int pos, const float *qg /*[nh][2*hd]*/, const float *kin,
                               const float *vin, float *q16f, float *gate) {
    const HParams &h = m.hp;
    const std::string B = "blk." + std::to_string(b) + ".";
    const int hd = h.head_dim;
    std::vector<float> y(hd);
    for (int hh = 0; hh < h.n_head; ++hh) {          // deint_qg.comp: [q(hd) | gate(hd)] per head
        const float *src = qg + size_t(hh) * 2 * hd;
        head_norm_rope(h, src, m.f32(B + "attn_q_norm.weight"), pos, y.data());
        for (int d = 0; d < hd; ++d) { q16f[size_t(hh) * hd + d] = f16_to_f32(f32_to_f16(y[d])); gate[size_t(hh) * hd + d] = src[hd + d]; }
    }
    for (int kv = 0; kv < h.n_kv; ++kv) {
        const size_t row = (size_t(pos) * h.n_kv + kv) * hd;
        head_norm_rope(h, kin + size_t(kv) * hd, m.f32(B + "attn_k_norm.weight"), pos, y.data());
        if (h.k_mode == KV_F16) for (int d = 0; d < hd; ++d) m.k16[li][row + d] = f32_to_f16(y[d]);
        else quantize_q8_0(y.data(), hd, m.kq[li].data() + row, m.ks[li].data() + row / 32);
        const float *v = vin + size_t(kv) * hd;
        if (h.v_mode == KV_F16) for (int d = 0; d < hd; ++d) m.v16[li][row + d] = f32_to_f16(v[d]);
        else quantize_q8_0(v, hd, m.vq[li].data() + row, m.vs[li].data() + row / 32);
    }
}

static inline void attn_mix(Model &m, int b, int li, int pos, float *res, AttnTap *tap = nullptr) {
    const HParams &h = m.hp;
    const std::string B = "blk." + std::to_string(b) + ".";
    const int hd = h.head_dim, QD = h.n_head * hd, KD = h.n_kv * hd;
    std::vector<float> an(h.hidden), hr(h.hidden), qg(2 * QD), k(KD), v(KD), q16f(QD), gate(QD), gout(QD), out(h.hidden);
    rms_norm(res, m.f32(B + "attn_norm.weight"), h.hidden, h.rms_eps, an.data());
    rotate_fwd(an.data(), m.signs, h.hidden, h.hat_block, hr.data());
    project(m, m.ptq(B + "attn_q.weight"), 2 * QD, h.hidden, hr.data(), qg.data());
    project(m, m.ptq(B + "attn_k.weight"), KD, h.hidden, hr.data(), k.data());
    project(m, m.ptq(B + "attn_v.weight"), KD, h.hidden, hr.data(), v.data());
    attn_insert(m, li, b, pos, qg.data(), k.data(), v.data(), q16f.data(), gate.data());
    if (h.attn_order == 1) attn_core_device_order(m, li, pos, q16f.data(), gate.data(), gout.data(), tap);
    else attn_core(m, li, pos, q16f.data(), gate.data(), gout.data(), tap);
    rot_project(m, B + "attn_output.weight", h.hidden, QD, gout.data(), m.signs, out.data());
    for (int i = 0; i < h.hidden; ++i) res[i] = out[i] + res[i];
}

// ---- whole token (fwd_token, bonsai_forward.h:664-758) -------------------------------------------
static inline void embed(const Model &m, int tok, float *res) {
    const HParams &h = m.hp;
    std::vector<float> e(h.hidden);
    const uint8_t *row = m.ptq("token_embd.weight") + size_t(tok) * (h.hidden / 128) * PTQ_BLOCK_BYTES;
    for (int b = 0; b < h.hidden / 128; ++b) ptq_dequant_block(row + b * PTQ_BLOCK_BYTES, e.data() + b * 128);
    rotate_inv(e.data(), m.signs, h.hidden, h.hat_block, res);       // H then signs (:689-691)
}

static inline void forward_token(Model &m, int tok, int pos, float *logits, float *res_out = nullptr, int stop_after = -1) {
    const HParams &h = m.hp;
    std::vector<float> res(h.hidden);
    embed(m, tok, res.data());
    int gi = 0, li = 0;
    for (int b = 0; b < h.n_layer; ++b) {
        if (h.is_attn(b)) attn_mix(m, b, li++, pos, res.data());
        else gdn_mix(m, b, gi++, res.data());
        ffn_block(m, b, res.data());
        if (b == stop_after) break;
    }
    if (res_out) std::copy(res.begin(), res.end(), res_out);
    if (logits && stop_after < 0) {
        std::vector<float> an(h.hidden);
        rms_norm(res.data(), m.f32("output_norm.weight"), h.hidden, h.rms_eps, an.data());
        rot_project(m, "output.weight", h.vocab, h.hidden, an.data(), m.signs, logits);
    }
}

// greedy pick (Sampler::pick with temp <= 0 and penalties off, bonsai_forward.h:2568-2570): first maximum
static inline int argmax_first(const float *lg, int n) {
    int best = 0; float bv = lg[0];
    for (int i = 1; i < n; ++i) if (lg[i] > bv) { bv = lg[i]; best = i; }
    return best;
}

}  // namespace bo
#endif
