// ref_shim.cpp - C entry points over the reference's own CPU headers, compiled from where they
// lie in the reference tree (-I<reference>/runtime_vk). Nothing from the reference is copied into
// this repository; this file only forwards calls. Used by the tests to pin the restatement in
// bonsai_oracle.h against the reference's real code, and by the benchmark's reference leg.
// TEST INFRASTRUCTURE ONLY.
#include "ptq_decode.h"
#include "f16_rne_host.h"
#include "attn_vk.h"

#include <algorithm>
#include <thread>
#include <vector>

extern "C" {

int ref_trit_of_byte(int b, int t) { return trit_of_byte(uint8_t(b), t); }
void ref_elem_to_byte_trit(int e, int *by, int *tr) { elem_to_byte_trit(e, *by, *tr); }
void ref_f16_to_f32(const uint16_t *h, int n, float *out) { for (int i = 0; i < n; ++i) out[i] = f16_to_f32(h[i]); }
void ref_f32_to_f16(const float *f, int n, uint16_t *out) { for (int i = 0; i < n; ++i) out[i] = f32_to_f16_bits(f[i]); }
void ref_ptq_dequant_ours(const uint8_t *W, long nblocks, float *out) {
    for (long b = 0; b < nblocks; ++b) ptq_dequant_ours(W + b * 28, out + b * 128);
}
void ref_ptq_dequant_official(const uint8_t *W, long nblocks, float *out) {
    for (long b = 0; b < nblocks; ++b) ptq_dequant_official_cpu(W + b * 28, out + b * 128);
}

// The reference's GEMV truth: ptq_dequant_ours per block, w*x accumulated in double
// (the loop of runtime_vk/bonsai_weights.h:751-768 around the reference's own dequantiser).
void ref_gemv_dequant_f64(const uint8_t *W, int M, int K, const float *x, double *out, int threads) {
    const int nb = K / 128;
    auto work = [=](int r0, int r1) {
        float w[128];
        for (int r = r0; r < r1; ++r) {
            double acc = 0.0;
            for (int b = 0; b < nb; ++b) {
                ptq_dequant_ours(W + (size_t(r) * nb + b) * 28, w);
                for (int k = 0; k < 128; ++k) acc += double(w[k]) * double(x[b * 128 + k]);
            }
            out[r] = acc;
        }
    };
    if (threads <= 1) { work(0, M); return; }
    std::vector<std::thread> th;
    const int per = (M + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int r0 = t * per, r1 = std::min(M, r0 + per);
        if (r0 < r1) th.emplace_back(work, r0, r1);
    }
    for (auto &t : th) t.join();
}

// attn_vk.h mirror: seq tokens at positions pos[], fp16 K and V arenas, fp16-rounded probabilities.
void ref_attn_forward(int seq, int cap, int nh, int nkv, int hd, int nrot, float eps, float freq_base,
                      const float *q_in, const float *k_in, const float *v_in, const float *gate_in,
                      const float *qn_w, const float *kn_w, const uint32_t *pos, int round_probs,
                      float *pregate, float *gated, float *prob, uint32_t *q16, uint32_t *kc) {
    AttnCfg c; c.hd = hd; c.nh = nh; c.nkv = nkv; c.nrot = nrot; c.seq = seq; c.cap = cap;
    c.eps = eps; c.freq_base = freq_base; c.scale = 1.0f / std::sqrt(float(hd));
    AttnBuffers b; b.alloc(c);
    std::copy(q_in, q_in + size_t(seq) * nh * hd, b.q_in.begin());
    std::copy(k_in, k_in + size_t(seq) * nkv * hd, b.k_in.begin());
    std::copy(v_in, v_in + size_t(seq) * nkv * hd, b.v_in.begin());
    std::copy(gate_in, gate_in + size_t(seq) * nh * hd, b.gate_in.begin());
    std::copy(qn_w, qn_w + hd, b.qn_w.begin());
    std::copy(kn_w, kn_w + hd, b.kn_w.begin());
    std::copy(pos, pos + seq, b.pos.begin());
    if (round_probs) attn_forward<true>(c, b); else attn_forward<false>(c, b);
    std::copy(b.pregate.begin(), b.pregate.end(), pregate);
    std::copy(b.gated.begin(), b.gated.end(), gated);
    if (prob) std::copy(b.prob.begin(), b.prob.end(), prob);
    if (q16) std::copy(b.q16.begin(), b.q16.end(), q16);
    if (kc) std::copy(b.kc.begin(), b.kc.end(), kc);
}

}  // extern "C"
