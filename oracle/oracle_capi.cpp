// oracle_capi.cpp - C entry points over bonsai_oracle.h (and, as they are added, the block and
// whole-token restatements) so the Python tests can drive the CPU oracle through ctypes.
// TEST INFRASTRUCTURE ONLY: nothing in the CUDA library or its host code links this file.
#include "bonsai_oracle.h"
#include "bonsai_oracle_model.h"

#include <thread>

using namespace bo;

template <class F>
static void par_rows(int M, int threads, F f) {
    if (threads <= 1) { f(0, M); return; }
    std::vector<std::thread> th;
    const int per = (M + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int r0 = t * per, r1 = std::min(M, r0 + per);
        if (r0 < r1) th.emplace_back([=] { f(r0, r1); });
    }
    for (auto &t : th) t.join();
}

extern "C" {

int bo_trit_of_byte(int b, int t) { return trit_of_byte(uint32_t(b), t); }
int bo_trit_closed_form(int b, int t) { return trit_closed_form(uint32_t(b), t); }
void bo_elem_to_byte_trit(int e, int *by, int *tr) { elem_to_byte_trit(e, *by, *tr); }

void bo_f16_to_f32(const uint16_t *h, int n, float *out) { for (int i = 0; i < n; ++i) out[i] = f16_to_f32(h[i]); }
void bo_f32_to_f16(const float *f, int n, uint16_t *out) { for (int i = 0; i < n; ++i) out[i] = f32_to_f16(f[i]); }

void bo_ptq_dequant(const uint8_t *W, long nblocks, float *out) {
    for (long b = 0; b < nblocks; ++b) ptq_dequant_block(W + b * 28, out + b * 128);
}
void bo_ptq_trits(const uint8_t *W, long nblocks, int8_t *out) {
    for (long b = 0; b < nblocks; ++b) ptq_trits_block(W + b * 28, out + b * 128);
}
void bo_ptq_encode(const int8_t *sym, const uint16_t *scale_bits, long nblocks, uint8_t *out) {
    for (long b = 0; b < nblocks; ++b) ptq_encode_block(sym + b * 128, scale_bits[b], out + b * 28);
}

void bo_quantize_q8_1(const float *x, int K, uint32_t *out) { quantize_q8_1_x4(x, K, out); }
void bo_quantize_q8_0(const float *x, int n, int8_t *codes, uint16_t *scales) { quantize_q8_0(x, n, codes, scales); }

void bo_block_dots_def(const uint8_t *pb, const uint32_t *xq, int32_t *I) { block_dots_def(pb, xq, I); }
void bo_block_dots_fast(const uint8_t *pb, const uint32_t *xq, int32_t *I) { block_dots_fast(pb, xq, I); }
void bo_block_dots_shader(const uint8_t *pb, const uint32_t *xq, int32_t *I) { block_dots_shader_lanes(pb, xq, I); }

void bo_gemv_q81(const uint8_t *W, int M, int K, const uint32_t *xq, float *out, double *exact,
                 int32_t *dots, int threads) {
    const size_t rb = size_t(K / 128) * 28;
    par_rows(M, threads, [=](int r0, int r1) {
        gemv_q81(W + rb * r0, r1 - r0, K, xq, out + r0, exact ? exact + r0 : nullptr,
                 dots ? dots + size_t(r0) * (K / 128) * 4 : nullptr);
    });
}
void bo_gemv_f32act(const uint8_t *W, int M, int K, const float *x, int n_splits, float *out,
                    double *exact, int threads) {
    const size_t rb = size_t(K / 128) * 28;
    par_rows(M, threads, [=](int r0, int r1) {
        gemv_f32act(W + rb * r0, r1 - r0, K, x, n_splits, out + r0, exact ? exact + r0 : nullptr);
    });
}
void bo_gemv_dequant_f64(const uint8_t *W, int M, int K, const float *x, double *out, int threads) {
    const size_t rb = size_t(K / 128) * 28;
    par_rows(M, threads, [=](int r0, int r1) { gemv_dequant_f64(W + rb * r0, r1 - r0, K, x, out + r0); });
}

void bo_fwht(float *s, int n, int block) {
    const float inv = 1.0f / std::sqrt(float(block));
    for (int b = 0; b < n / block; ++b) fwht_block(s + b * block, block, inv);
}
void bo_rotate_fwd(const float *x, const int32_t *signs, int n, int block, float *y) { rotate_fwd(x, signs, n, block, y); }
void bo_rotate_inv(const float *x, const int32_t *signs, int n, int block, float *y) { rotate_inv(x, signs, n, block, y); }

void bo_rms_norm(const float *x, const float *w, int n, float eps, float *y) { rms_norm(x, w, n, eps, y); }
void bo_l2_norm(const float *x, int n, float eps, float *y) { l2_norm(x, n, eps, y); }
void bo_silu(const float *x, int n, float *y) { for (int i = 0; i < n; ++i) y[i] = silu_f(x[i]); }
void bo_sigmoid(const float *x, int n, float *y) { for (int i = 0; i < n; ++i) y[i] = sigmoid_f(x[i]); }
void bo_softplus(const float *x, int n, float thr, float *y) { for (int i = 0; i < n; ++i) y[i] = softplus_f(x[i], thr); }
void bo_swiglu(const float *a, const float *b, int n, float *y) { for (int i = 0; i < n; ++i) y[i] = silu_f(a[i]) * b[i]; }

}  // extern "C"

#include "oracle_capi_model.inc"
