// ops.cu - the non-GEMV kernels of the decode path: Hadamard rotation, norms, elementwise fusions,
// embedding gather, gated-delta-net update, decode attention over the quantised KV cache, argmax.
//
// Floating-point order is part of the contract with the CPU checker: sums use the fixed trees
// stated next to each kernel, transcendentals are evaluated in double and rounded once, and the
// file is compiled without fused-multiply-add contraction (fmaf is written where one is meant).
#include "ops.cuh"
#include "quant.cuh"

#include <cooperative_groups.h>

namespace {

// ---- block-wide helpers ------------------------------------------------------------------------
// tree over n = blockDim.x partials in shared memory: p[i] += p[i + s], s = n/2 .. 1
__device__ __forceinline__ float block_tree_sum(float *p, int n) {
    for (int s = n >> 1; s > 0; s >>= 1) {
        __syncthreads();
        if (int(threadIdx.x) < s) p[threadIdx.x] = __fadd_rn(p[threadIdx.x], p[threadIdx.x + s]);
    }
    __syncthreads();
    return p[0];
}

// in-place Sylvester-Walsh-Hadamard butterflies over N floats in shared memory, h ascending
// (reference: runtime_vk/shaders/hat4096.comp:41-60), then the 1/sqrt(N) factor.
// N values = N / hb independent transforms of width hb side by side.
__device__ __forceinline__ void fwht_smem(float *s, int N, int hb, float inv) {
    for (int h = 1; h < hb; h <<= 1) {
        __syncthreads();
        for (int i = threadIdx.x; i < (N >> 1); i += blockDim.x) {
            const int j = ((i & ~(h - 1)) << 1) | (i & (h - 1));
            const float a = s[j], c = s[j + h];
            s[j] = __fadd_rn(a, c);
            s[j + h] = __fsub_rn(a, c);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < N; i += blockDim.x) s[i] = __fmul_rn(s[i], inv);
    __syncthreads();
}

// ---- rotation (+ quantisation) -------------------------------------------------------------------
// one CTA of 512 threads per span (a Hadamard block of `hb` values, or 128 values = one quantiser block when the Hadamard
// block is smaller): y = H(s . x); optional q8_1 pack of the span.
__global__ void __launch_bounds__(512) k_rotate_quant(const float *__restrict__ x, const int32_t *__restrict__ signs,
                                                      int block, int hb, float inv, float *__restrict__ y,
                                                      uint32_t *__restrict__ q81, uint32_t *__restrict__ table) {
    bnk::pdl_sync();
    extern __shared__ float s[];                   // block floats + 4 x 128 bytes
    int8_t *qs = reinterpret_cast<int8_t *>(s + block);
    const size_t base = size_t(blockIdx.x) * block;
    for (int i = threadIdx.x; i < block; i += blockDim.x) s[i] = __fmul_rn(x[base + i], float(signs[base + i]));
    fwht_smem(s, block, hb, inv);
    if (y) for (int i = threadIdx.x; i < block; i += blockDim.x) y[base + i] = s[i];
    if (q81) {
        const int grp = threadIdx.x >> 7, i = threadIdx.x & 127;       // 4 groups of 128 threads
        for (int b = grp; b < block / 128; b += 4) {
            const size_t gb = base / 128 + b;
            bnk::quant_block_128(s[b * 128 + i], i, qs + grp * 128, q81 + gb * bnk::Q81_DWORDS,
                                 table + gb * bnk::BF_WORDS, 1 + grp);
        }
    }
}

__global__ void __launch_bounds__(512) k_rotate_inv(const float *__restrict__ x, const int32_t *__restrict__ signs,
                                                    int block, float inv, float *__restrict__ y, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; x = bnk::colp(x, col * cols.arena); y = bnk::colp(y, col * cols.arena); }
    extern __shared__ float s[];
    const size_t base = size_t(blockIdx.x) * block;
    for (int i = threadIdx.x; i < block; i += blockDim.x) s[i] = x[base + i];
    fwht_smem(s, block, block, inv);
    for (int i = threadIdx.x; i < block; i += blockDim.x) y[base + i] = __fmul_rn(s[i], float(signs[base + i]));
}

// ---- embedding gather (reference addressing: runtime_vk/shaders/gather_rows.comp:12-16) ----------
__global__ void k_embed_row(const uint32_t *__restrict__ W, int K, const int *__restrict__ tok_ptr,
                            float *__restrict__ out, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; tok_ptr = bnk::colp(tok_ptr, col * cols.arena); out = bnk::colp(out, col * cols.arena); }
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= K) return;
    const int tok = tok_ptr[0];
    const uint32_t *blk = W + (size_t(tok) * (K / 128) + e / 128) * 7;
    const int el = e & 127;
    int byte, t;
    if (el < 80) { byte = el & 15; t = el >> 4; }
    else if (el < 120) { byte = 16 + ((el - 80) & 7); t = (el - 80) >> 3; }
    else { byte = 24 + ((el - 120) & 1); t = (el - 120) >> 1; }
    uint32_t v = (blk[byte >> 2] >> ((byte & 3) * 8)) & 0xFFu;
    for (int i = 0; i < t; ++i) v = (v * 3u) & 0xFFu;
    const int trit = int((v * 3u) >> 8);
    out[e] = __fmul_rn(float(trit) - 1.0f, half_bits_to_float(blk[6] >> 16));
}

// ---- RMS norm (reference: runtime_vk/shaders/rms_norm.comp:60-103) --------------------------------
// 256 lanes, lane l sums the squares of its `per` consecutive elements ascending, lane partials
// combined by the fixed tree; y = (x * inv) * w.
__global__ void __launch_bounds__(256) k_rms_norm(const float *__restrict__ x, const float *__restrict__ w, int cols,
                                                  float eps, float *__restrict__ y) {
    bnk::pdl_sync();
    __shared__ float part[256];
    const int l = threadIdx.x, per = (cols + 255) / 256;
    const float *xr = x + size_t(blockIdx.x) * cols;
    float s = 0.0f;
    for (int i = 0; i < per; ++i) {
        const int d = l * per + i;
        if (d < cols) { const float v = xr[d]; s = __fadd_rn(s, __fmul_rn(v, v)); }
    }
    part[l] = s;
    const float ss = block_tree_sum(part, 256);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(cols)), eps)));
    float *yr = y + size_t(blockIdx.x) * cols;
    for (int i = 0; i < per; ++i) {
        const int d = l * per + i;
        if (d < cols) { const float v = __fmul_rn(xr[d], inv); yr[d] = w ? __fmul_rn(v, w[d]) : v; }
    }
}

__global__ void k_add_inplace(float *__restrict__ res, const float *__restrict__ d, int n) {
    bnk::pdl_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) res[i] = __fadd_rn(d[i], res[i]);
}

__global__ void k_swiglu(const float *__restrict__ a, const float *__restrict__ b, int n, float *__restrict__ y, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; a = bnk::colp(a, col * cols.arena); b = bnk::colp(b, col * cols.arena); y = bnk::colp(y, col * cols.arena); }
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fmul_rn(silu_f(a[i]), b[i]);
}

// small fp32 projection: one warp per row; lane l takes float4 groups l, l+32, ... with one fmaf per
// element, then a 32-lane xor tree (reference: runtime_vk/shaders/gemv_f32.comp).
__global__ void k_gemv_f32_small(const float *__restrict__ W, int M, int K, const float *__restrict__ x,
                                 float *__restrict__ out) {
    bnk::pdl_sync();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const float4 *wr = reinterpret_cast<const float4 *>(W + size_t(row) * K);
    const float4 *xv = reinterpret_cast<const float4 *>(x);
    float a = 0.0f;
    for (int i = lane; i < K / 4; i += 32) {
        const float4 w = wr[i], v = xv[i];
        a = fmaf(w.x, v.x, a); a = fmaf(w.y, v.y, a); a = fmaf(w.z, v.z, a); a = fmaf(w.w, v.w, a);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, s));
    if (lane == 0) out[row] = a;
}

// ---- gated delta net ------------------------------------------------------------------------------
// gate = ssm_a * softplus(alpha + dt_bias), beta = sigmoid(beta_raw)   (bonsai_forward.h:528-535)
__global__ void k_gdn_gates(const float *alpha, const float *beta_raw, const float *dt_bias, const float *ssm_a, int n,
                            float *gate, float *beta) {
    bnk::pdl_sync();
    const int i = threadIdx.x;
    if (i >= n) return;
    const float a = __fadd_rn(alpha[i], dt_bias[i]);
    const float sp = a > 20.0f ? a : log_f(__fadd_rn(1.0f, exp_f(a)));
    gate[i] = __fmul_rn(sp, ssm_a[i]);
    beta[i] = sigmoid_f(beta_raw[i]);
}

// 4-tap causal depthwise conv + silu + history shift (runtime_vk/shaders/conv_silu.comp:35-49)
__global__ void k_conv_silu(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ hist,
                            int channels, float *__restrict__ y) {
    bnk::pdl_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float *s = hist + 3 * size_t(c);
    const float *wc = w + 4 * size_t(c);
    const float s0 = s[0], s1 = s[1], s2 = s[2], xn = x[c];
    float acc = __fmul_rn(wc[0], s0);
    acc = __fadd_rn(acc, __fmul_rn(wc[1], s1));
    acc = __fadd_rn(acc, __fmul_rn(wc[2], s2));
    acc = __fadd_rn(acc, __fmul_rn(wc[3], xn));
    y[c] = silu_f(acc);
    s[0] = s1; s[1] = s2; s[2] = xn;
}

// sum over 128 values held as 4 per lane (elements l, l+32, l+64, l+96) in the order of the
// reference's shared-memory tree sh[l] += sh[l+s], s = 64..1 (gdn_delta.comp tree_reduce)
__device__ __forceinline__ float warp_tree128(float e0, float e1, float e2, float e3) {
    float a = __fadd_rn(__fadd_rn(e0, e2), __fadd_rn(e1, e3));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, s));
    return a;
}

// L2 norm of 128-wide rows, mode 1 (runtime_vk/shaders/l2_norm.comp:59-78); one warp per row
__global__ void k_l2_norm_rows(const float *__restrict__ x, int rows, float eps, float *__restrict__ y) {
    bnk::pdl_sync();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), l = threadIdx.x & 31;
    if (row >= rows) return;
    const float *xr = x + size_t(row) * 128;
    const float a = xr[l], b = xr[l + 32], c = xr[l + 64], d = xr[l + 96];
    const float ss = warp_tree128(__fmul_rn(a, a), __fmul_rn(b, b), __fmul_rn(c, c), __fmul_rn(d, d));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, eps)));
    float *yr = y + size_t(row) * 128;
    yr[l] = __fmul_rn(a, inv); yr[l + 32] = __fmul_rn(b, inv); yr[l + 64] = __fmul_rn(c, inv); yr[l + 96] = __fmul_rn(d, inv);
}

// delta rule (runtime_vk/shaders/gdn_delta.comp:78-102), one warp per (v-head h, state row j):
// S *= exp(g); pred = sum_i S_i k_i; u = beta (v_j - pred); S_i = fma(k_i, u, S_i); o_j = (sum_i S_i q_i) / sqrt(dim)
__global__ void __launch_bounds__(256) k_gdn_delta(int heads, int qk_heads, const float *__restrict__ q,
                                                   const float *__restrict__ k, const float *__restrict__ v,
                                                   const float *__restrict__ gate, const float *__restrict__ beta,
                                                   float *__restrict__ state, float *__restrict__ o, float scale) {
    bnk::pdl_sync();
    const int h = blockIdx.y, j = blockIdx.x * 8 + (threadIdx.x >> 5), l = threadIdx.x & 31;
    const int hq = h % qk_heads;
    const float eg = exp_f(gate[h]), bt = beta[h];
    const float *kr = k + hq * 128, *qr = q + hq * 128;
    float *S = state + (size_t(h) * 128 + j) * 128;
    float s[4], kk[4], qq[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) { s[e] = __fmul_rn(S[l + 32 * e], eg); kk[e] = kr[l + 32 * e]; qq[e] = qr[l + 32 * e]; }
    const float pred = warp_tree128(__fmul_rn(s[0], kk[0]), __fmul_rn(s[1], kk[1]), __fmul_rn(s[2], kk[2]), __fmul_rn(s[3], kk[3]));
    const float u = __fmul_rn(bt, __fsub_rn(v[h * 128 + j], pred));
#pragma unroll
    for (int e = 0; e < 4; ++e) { s[e] = fmaf(kk[e], u, s[e]); S[l + 32 * e] = s[e]; }
    const float ov = warp_tree128(__fmul_rn(s[0], qq[0]), __fmul_rn(s[1], qq[1]), __fmul_rn(s[2], qq[2]), __fmul_rn(s[3], qq[3]));
    if (l == 0) o[h * 128 + j] = __fmul_rn(ov, scale);
}

// Fused gated-delta-net mixer of one layer, one CTA of 512 threads per v-head: the two small fp32 projections
// of the normed residual and their gate functions (bonsai_forward.h:523-535), conv + silu of the head's q, k
// and v channels, L2 norms, the delta rule on the head's 128 state rows, then the per-head RMS, ssm_norm,
// swiglu(z, .) and the v-grouped permutation (bonsai_forward.h:559-567) straight into the next projection's
// input. The conv history is double-buffered by position parity: the two v-heads that share a q/k head both
// read its taps while one of them writes the shifted taps into the other buffer.
// Arithmetic and its order are those of the stand-alone kernels above.
// MINB = CTAs per SM the register budget is set for: 1 for a single sequence (32 CTAs in all; the loads hoisted above
// the dependency wait keep ~90 registers live, measured 4 % of a token faster than the 64-register build), 2 when many
// sequences fill the GPU with CTAs (measured 3 % of a 32-sequence pass faster than one CTA per SM).
template <int MINB>
__global__ void __launch_bounds__(512, MINB) k_gdn_core(int heads, int qk_heads, int hidden, const float *__restrict__ qkv,
                                                  const float *__restrict__ conv_w, float *__restrict__ hist0,
                                                  float *__restrict__ hist1, const int *__restrict__ pos_ptr,
                                                  const float *__restrict__ x, const float *__restrict__ inv_ptr,
                                                  const float *__restrict__ norm_w, const float *__restrict__ alpha_w,
                                                  const float *__restrict__ beta_w, const float *__restrict__ dt_bias,
                                                  const float *__restrict__ ssm_a, float *__restrict__ state,
                                                  const float *__restrict__ z, const float *__restrict__ ssm_norm, float eps,
                                                  float *__restrict__ y, float scale, bnk::Cols cols) {
    { const size_t col = blockIdx.z; qkv = bnk::colp(qkv, col * cols.arena); hist0 = bnk::colp(hist0, col * cols.conv); hist1 = bnk::colp(hist1, col * cols.conv); pos_ptr = bnk::colp(pos_ptr, col * cols.arena); x = bnk::colp(x, col * cols.arena); inv_ptr = bnk::colp(inv_ptr, col * cols.arena); state = bnk::colp(state, col * cols.gdn); z = bnk::colp(z, col * cols.arena); y = bnk::colp(y, col * cols.arena); }
    __shared__ float sq[128], sk[128], sv[128], so[128], sgb[2];
    extern __shared__ float4 dyn[];                // [3][hidden/4]: normed residual, row h of ssm_alpha, row h of ssm_beta
    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hq = h % qk_heads, n4 = hidden / 4;
    // ---- before the dependency wait: everything that the preceding kernel (the qkv / gate projection) does not write.
    // Constants, this layer's recurrent state and conv taps (last written one token ago) and the position (written at
    // the end of the previous token) are requested while the projection's last CTAs are still running; every kernel of
    // the schedule waits for its predecessor before it releases its successor, so all older kernels are complete here.
    const bool odd = pos_ptr[0] & 1;               // a token at position p reads taps from buffer p & 1, writes the other
    const float *hist_rd = odd ? hist1 : hist0;
    float *hist_wr = odd ? hist0 : hist1;
    float S[8][4];                                 // state rows of this warp (8 of the head's 128)
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const float *Sr = state + (size_t(h) * 128 + warp * 8 + r) * 128;
#pragma unroll
        for (int e = 0; e < 4; ++e) S[r][e] = Sr[lane + 32 * e];
    }
    const int cch = tid < 128 ? hq * 128 + tid : (tid < 256 ? qk_heads * 128 + hq * 128 + (tid - 128) : 2 * qk_heads * 128 + h * 128 + (tid - 256));
    float tap0 = 0.0f, tap1 = 0.0f, tap2 = 0.0f, cw0 = 0.0f, cw1 = 0.0f, cw2 = 0.0f, cw3 = 0.0f;
    if (tid < 384) {
        const float *sr = hist_rd + 3 * size_t(cch);
        const float *wc = conv_w + 4 * size_t(cch);
        tap0 = sr[0]; tap1 = sr[1]; tap2 = sr[2];
        cw0 = wc[0]; cw1 = wc[1]; cw2 = wc[2]; cw3 = wc[3];
    }
    {
        const float4 *ra = reinterpret_cast<const float4 *>(alpha_w + size_t(h) * hidden), *rb = reinterpret_cast<const float4 *>(beta_w + size_t(h) * hidden);
        for (int i = tid; i < n4; i += 512) { dyn[n4 + i] = ra[i]; dyn[2 * n4 + i] = rb[i]; }
    }
    bnk::pdl_sync();
    {   // the normed residual goes to shared memory for the two dependent dot-product chains
        const float inv = inv_ptr[0];
        const float4 *xv = reinterpret_cast<const float4 *>(x), *nw = reinterpret_cast<const float4 *>(norm_w);
        for (int i = tid; i < n4; i += 512) {
            const float4 a4 = xv[i], w4 = nw[i];
            dyn[i] = make_float4(__fmul_rn(__fmul_rn(a4.x, inv), w4.x), __fmul_rn(__fmul_rn(a4.y, inv), w4.y),
                                 __fmul_rn(__fmul_rn(a4.z, inv), w4.z), __fmul_rn(__fmul_rn(a4.w, inv), w4.w));
        }
    }
    const bool own_qk = h < qk_heads;              // the first of the v-heads sharing q/k head hq writes its taps
    if (tid < 384) {
        const float xn = qkv[cch];
        float acc = __fmul_rn(cw0, tap0);
        acc = __fadd_rn(acc, __fmul_rn(cw1, tap1));
        acc = __fadd_rn(acc, __fmul_rn(cw2, tap2));
        acc = __fadd_rn(acc, __fmul_rn(cw3, xn));
        if (tid >= 256 || own_qk) { float *sw = hist_wr + 3 * size_t(cch); sw[0] = tap1; sw[1] = tap2; sw[2] = xn; }
        const float cv = silu_f(acc);
        if (tid < 128) sq[tid] = cv; else if (tid < 256) sk[tid - 128] = cv; else sv[tid - 256] = cv;
    }
    __syncthreads();
    if (warp >= 14) {
        // row h of ssm_alpha (warp 14) or ssm_beta (warp 15) times the normed residual: lane l takes float4 groups
        // l, l+32, ... with one fmaf per element, then a 32-lane xor tree (k_gemv_f32_small)
        const float4 *wr = dyn + (warp == 14 ? n4 : 2 * n4);
        float acc = 0.0f;
        for (int i = lane; i < n4; i += 32) {
            const float4 w4 = wr[i], a4 = dyn[i];
            acc = fmaf(w4.x, a4.x, acc); acc = fmaf(w4.y, a4.y, acc); acc = fmaf(w4.z, a4.z, acc); acc = fmaf(w4.w, a4.w, acc);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, s));
        if (lane == 0) {
            if (warp == 14) {
                const float al = __fadd_rn(acc, dt_bias[h]);
                const float sp = al > 20.0f ? al : log_f(__fadd_rn(1.0f, exp_f(al)));
                sgb[0] = __fmul_rn(sp, ssm_a[h]);
            } else sgb[1] = sigmoid_f(acc);
        }
    }
    float qq[4], kk[4];
    {
        const float a0 = sq[lane], a1 = sq[lane + 32], a2 = sq[lane + 64], a3 = sq[lane + 96];
        const float iq = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(warp_tree128(__fmul_rn(a0, a0), __fmul_rn(a1, a1), __fmul_rn(a2, a2), __fmul_rn(a3, a3)), 1e-12f)));
        qq[0] = __fmul_rn(a0, iq); qq[1] = __fmul_rn(a1, iq); qq[2] = __fmul_rn(a2, iq); qq[3] = __fmul_rn(a3, iq);
        const float b0 = sk[lane], b1 = sk[lane + 32], b2 = sk[lane + 64], b3 = sk[lane + 96];
        const float ik = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(warp_tree128(__fmul_rn(b0, b0), __fmul_rn(b1, b1), __fmul_rn(b2, b2), __fmul_rn(b3, b3)), 1e-12f)));
        kk[0] = __fmul_rn(b0, ik); kk[1] = __fmul_rn(b1, ik); kk[2] = __fmul_rn(b2, ik); kk[3] = __fmul_rn(b3, ik);
    }
    __syncthreads();
    const float eg = exp_f(sgb[0]), bt = sgb[1];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int j = warp * 8 + r;
        float *Sr = state + (size_t(h) * 128 + j) * 128;
        float s[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] = __fmul_rn(S[r][e], eg);
        const float pred = warp_tree128(__fmul_rn(s[0], kk[0]), __fmul_rn(s[1], kk[1]), __fmul_rn(s[2], kk[2]), __fmul_rn(s[3], kk[3]));
        const float u = __fmul_rn(bt, __fsub_rn(sv[j], pred));
#pragma unroll
        for (int e = 0; e < 4; ++e) { s[e] = fmaf(kk[e], u, s[e]); Sr[lane + 32 * e] = s[e]; }
        const float ov = warp_tree128(__fmul_rn(s[0], qq[0]), __fmul_rn(s[1], qq[1]), __fmul_rn(s[2], qq[2]), __fmul_rn(s[3], qq[3]));
        if (lane == 0) so[j] = __fmul_rn(ov, scale);
    }
    __syncthreads();
    if (warp == 0) {
        // per-head RMS (no weight), * ssm_norm, swiglu(z, .), destination head of the v-grouped permutation
        float e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) e[i] = so[lane + 32 * i];
        const float ss = warp_tree128(__fmul_rn(e[0], e[0]), __fmul_rn(e[1], e[1]), __fmul_rn(e[2], e[2]), __fmul_rn(e[3], e[3]));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), eps)));
        const int sub = heads / qk_heads, hd = sub * (h % qk_heads) + h / qk_heads;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = lane + 32 * i;
            const float nrm = __fmul_rn(__fmul_rn(e[i], inv), ssm_norm[d]);
            y[hd * 128 + d] = __fmul_rn(silu_f(z[h * 128 + d]), nrm);
        }
    }
}

// The same mixer core for one sequence, split four ways per value head so that a 148-SM GPU is filled (heads x 4 CTAs,
// 128 at 32 heads): the 4 CTAs of a head form a thread-block cluster, each owns 32 of the head's 128 state rows, two per
// warp. Everything that does not depend on the preceding projection is requested before the dependency wait: state rows,
// conv taps and weights, the two small projections' weight rows (staged in shared memory by all threads). After the wait:
// normed residual, the two dot products (warps 14 / 15), conv + silu, L2 norms, delta rule. The per-head output norm needs
// all 128 outputs of the head: every CTA reads the other three quarters from their shared memory (distributed shared
// memory) and evaluates the same 128-value tree as k_gdn_core, then finishes its own 32 values (ssm_norm, swiglu(z, .),
// v-grouped permutation). Arithmetic and its order are those of k_gdn_core.
__global__ void __cluster_dims__(4, 1, 1) __launch_bounds__(512, 1)
k_gdn_split(int heads, int qk_heads, int hidden, const float *__restrict__ qkv, const float *__restrict__ conv_w,
            float *__restrict__ hist0, float *__restrict__ hist1, const int *__restrict__ pos_ptr, const float *__restrict__ x,
            const float *__restrict__ inv_ptr, const float *__restrict__ norm_w, const float *__restrict__ alpha_w,
            const float *__restrict__ beta_w, const float *__restrict__ dt_bias, const float *__restrict__ ssm_a,
            float *__restrict__ state, const float *__restrict__ z, const float *__restrict__ ssm_norm, float eps,
            float *__restrict__ y, float scale) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float sq[128], sk[128], sv[32], so[128], sgb[2];   // so: the head's 128 outputs, every quarter pushed here by its CTA
    extern __shared__ float4 dyn[];                // [3][hidden/4]: normed residual, row h of ssm_alpha, row h of ssm_beta
    const int unit = blockIdx.x, h = unit >> 2, q4 = unit & 3, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hq = h % qk_heads, n4 = hidden / 4;
    // "I am running": the matching wait sits in front of the first store into a neighbour's shared memory, which must
    // not happen before that neighbour has started (by then everybody has long arrived - nobody waits here)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const bool odd = pos_ptr[0] & 1;               // a token at position p reads taps from buffer p & 1, writes the other
    const float *hist_rd = odd ? hist1 : hist0;
    float *hist_wr = odd ? hist0 : hist1;
    float S[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float *Sr = state + (size_t(h) * 128 + q4 * 32 + warp * 2 + r) * 128;
#pragma unroll
        for (int e = 0; e < 4; ++e) S[r][e] = Sr[lane + 32 * e];
    }
    const int cch = tid < 128 ? hq * 128 + tid : (tid < 256 ? qk_heads * 128 + hq * 128 + (tid - 128) : 2 * qk_heads * 128 + h * 128 + q4 * 32 + (tid - 256));
    float tap0 = 0.0f, tap1 = 0.0f, tap2 = 0.0f, cw0 = 0.0f, cw1 = 0.0f, cw2 = 0.0f, cw3 = 0.0f;
    if (tid < 288) {
        const float *sr = hist_rd + 3 * size_t(cch);
        const float *wc = conv_w + 4 * size_t(cch);
        tap0 = sr[0]; tap1 = sr[1]; tap2 = sr[2];
        cw0 = wc[0]; cw1 = wc[1]; cw2 = wc[2]; cw3 = wc[3];
    }
    {
        const float4 *ra = reinterpret_cast<const float4 *>(alpha_w + size_t(h) * hidden), *rb = reinterpret_cast<const float4 *>(beta_w + size_t(h) * hidden);
        for (int i = tid; i < n4; i += 512) { dyn[n4 + i] = ra[i]; dyn[2 * n4 + i] = rb[i]; }
    }
    bnk::pdl_sync();
    {
        const float inv = inv_ptr[0];
        const float4 *xv = reinterpret_cast<const float4 *>(x), *nw = reinterpret_cast<const float4 *>(norm_w);
        for (int i = tid; i < n4; i += 512) {
            const float4 a4 = xv[i], w4 = nw[i];
            dyn[i] = make_float4(__fmul_rn(__fmul_rn(a4.x, inv), w4.x), __fmul_rn(__fmul_rn(a4.y, inv), w4.y),
                                 __fmul_rn(__fmul_rn(a4.z, inv), w4.z), __fmul_rn(__fmul_rn(a4.w, inv), w4.w));
        }
    }
    if (tid < 288) {
        const float xn = qkv[cch];
        float acc = __fmul_rn(cw0, tap0);
        acc = __fadd_rn(acc, __fmul_rn(cw1, tap1));
        acc = __fadd_rn(acc, __fmul_rn(cw2, tap2));
        acc = __fadd_rn(acc, __fmul_rn(cw3, xn));
        // one writer per channel: this CTA's own 32 value channels; the q / k channels by the first quarter of the first of
        // the value heads that share them
        if (tid >= 256 || (h < qk_heads && q4 == 0)) { float *sw = hist_wr + 3 * size_t(cch); sw[0] = tap1; sw[1] = tap2; sw[2] = xn; }
        const float cv = silu_f(acc);
        if (tid < 128) sq[tid] = cv; else if (tid < 256) sk[tid - 128] = cv; else sv[tid - 256] = cv;
    }
    __syncthreads();
    if (warp >= 14) {
        const float4 *wr = dyn + (warp == 14 ? n4 : 2 * n4);
        float acc = 0.0f;
        for (int i = lane; i < n4; i += 32) {
            const float4 w4 = wr[i], a4 = dyn[i];
            acc = fmaf(w4.x, a4.x, acc); acc = fmaf(w4.y, a4.y, acc); acc = fmaf(w4.z, a4.z, acc); acc = fmaf(w4.w, a4.w, acc);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, s));
        if (lane == 0) {
            if (warp == 14) {
                const float al = __fadd_rn(acc, dt_bias[h]);
                const float sp = al > 20.0f ? al : log_f(__fadd_rn(1.0f, exp_f(al)));
                sgb[0] = __fmul_rn(sp, ssm_a[h]);
            } else sgb[1] = sigmoid_f(acc);
        }
    }
    float qq[4], kk[4];
    {
        const float a0 = sq[lane], a1 = sq[lane + 32], a2 = sq[lane + 64], a3 = sq[lane + 96];
        const float iq = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(warp_tree128(__fmul_rn(a0, a0), __fmul_rn(a1, a1), __fmul_rn(a2, a2), __fmul_rn(a3, a3)), 1e-12f)));
        qq[0] = __fmul_rn(a0, iq); qq[1] = __fmul_rn(a1, iq); qq[2] = __fmul_rn(a2, iq); qq[3] = __fmul_rn(a3, iq);
        const float b0 = sk[lane], b1 = sk[lane + 32], b2 = sk[lane + 64], b3 = sk[lane + 96];
        const float ik = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(warp_tree128(__fmul_rn(b0, b0), __fmul_rn(b1, b1), __fmul_rn(b2, b2), __fmul_rn(b3, b3)), 1e-12f)));
        kk[0] = __fmul_rn(b0, ik); kk[1] = __fmul_rn(b1, ik); kk[2] = __fmul_rn(b2, ik); kk[3] = __fmul_rn(b3, ik);
    }
    __syncthreads();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");      // all four CTAs of the head are running
    const float eg = exp_f(sgb[0]), bt = sgb[1];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int jl = warp * 2 + r, j = q4 * 32 + jl;
        float *Sr = state + (size_t(h) * 128 + j) * 128;
        float s[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] = __fmul_rn(S[r][e], eg);
        const float pred = warp_tree128(__fmul_rn(s[0], kk[0]), __fmul_rn(s[1], kk[1]), __fmul_rn(s[2], kk[2]), __fmul_rn(s[3], kk[3]));
        const float u = __fmul_rn(bt, __fsub_rn(sv[jl], pred));
#pragma unroll
        for (int e = 0; e < 4; ++e) { s[e] = fmaf(kk[e], u, s[e]); Sr[lane + 32 * e] = s[e]; }
        const float ov = warp_tree128(__fmul_rn(s[0], qq[0]), __fmul_rn(s[1], qq[1]), __fmul_rn(s[2], qq[2]), __fmul_rn(s[3], qq[3]));
        // lanes 0..3 push the value into the so[] of the cluster's four CTAs (distributed shared memory): after the one
        // cluster barrier below everybody reads its own shared memory only, so nobody has to wait for a neighbour to leave
        if (lane < 4) cluster.map_shared_rank(so, lane)[j] = __fmul_rn(ov, scale);
    }
    // this CTA's share of the gate, off the tail (a double-precision exp): lane l of warp 0 finishes output q4 * 32 + l
    float gz = 0.0f, nw = 0.0f;
    if (warp == 0) { gz = silu_f(z[h * 128 + q4 * 32 + lane]); nw = ssm_norm[q4 * 32 + lane]; }
    cluster.sync();                                 // the head's 128 outputs are in every CTA's so[]
    if (warp == 0) {
        // per-head RMS over all 128 outputs: lane l holds elements l, l+32, l+64, l+96
        float e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) e[i] = so[i * 32 + lane];
        const float ss = warp_tree128(__fmul_rn(e[0], e[0]), __fmul_rn(e[1], e[1]), __fmul_rn(e[2], e[2]), __fmul_rn(e[3], e[3]));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), eps)));
        const int sub = heads / qk_heads, hd = sub * (h % qk_heads) + h / qk_heads;
        const int d = q4 * 32 + lane;               // this CTA finishes its own quarter
        const float nrm = __fmul_rn(__fmul_rn(so[d], inv), nw);
        y[hd * 128 + d] = __fmul_rn(gz, nrm);
    }
}

// per-head RMS (no weight; 128 squares, tree), * ssm_norm, swiglu(z, .), v-grouped permutation
// (bonsai_forward.h:559-567, permute_vg.comp:32-42). One warp per SOURCE head.
__global__ void k_gdn_out(int heads, int qk_heads, const float *__restrict__ o, const float *__restrict__ z,
                          const float *__restrict__ ssm_norm, float eps, float *__restrict__ y) {
    bnk::pdl_sync();
    const int hs = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), l = threadIdx.x & 31;
    if (hs >= heads) return;
    const float *orow = o + hs * 128;
    float e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = orow[l + 32 * i];
    const float ss = warp_tree128(__fmul_rn(e[0], e[0]), __fmul_rn(e[1], e[1]), __fmul_rn(e[2], e[2]), __fmul_rn(e[3], e[3]));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), eps)));
    // destination head hd reads source head hd/sub + nq*(hd%sub)  =>  source hs feeds hd = sub*(hs%nq) + hs/nq
    const int sub = heads / qk_heads;
    const int hd = sub * (hs % qk_heads) + hs / qk_heads;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int d = l + 32 * i;
        const float n = __fmul_rn(__fmul_rn(e[i], inv), ssm_norm[d]);
        y[hd * 128 + d] = __fmul_rn(silu_f(z[hs * 128 + d]), n);
    }
}

// ---- attention ------------------------------------------------------------------------------------
// q8_0 of one 32-element block held one value per lane (recipe: attn_norm_rope2.comp:39-49,184-217)
__device__ __forceinline__ void q80_store(float v, int lane, int8_t *codes, uint16_t *scale) {
    float amax = fabsf(v);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, s));
    const float d = amax > 1e-35f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    float r = roundf(__fmul_rn(v, id));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    codes[lane] = int8_t(int(r));
    if (lane == 0) *scale = (uint16_t)float_to_half_bits(d);
}

// one CTA per head row (n_head query rows, then n_kv key rows); blockDim = head_dim = 256.
// Query rows: RMS norm * weight, NeoX rope on the first n_rot dims, fp16 rounding, gate split.
// Key rows: the same norm/rope, then cache insert (fp16 or q8_0) of K and of the raw V row.
__global__ void __launch_bounds__(256) k_attn_prep(bnk::AttnDims a, const float *__restrict__ qg,
                                                   const float *__restrict__ kin, const float *__restrict__ vin,
                                                   const float *__restrict__ qn_w, const float *__restrict__ kn_w,
                                                   const int *__restrict__ pos_ptr, bnk::KvLayer kv,
                                                   float *__restrict__ q16f, float *__restrict__ gate, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; qg = bnk::colp(qg, col * cols.arena); kin = bnk::colp(kin, col * cols.arena); vin = bnk::colp(vin, col * cols.arena); pos_ptr = bnk::colp(pos_ptr, col * cols.arena); kv.k_data = bnk::colp(kv.k_data, col * cols.kv); kv.k_scale = bnk::colp(kv.k_scale, col * cols.kv); kv.v_data = bnk::colp(kv.v_data, col * cols.kv); kv.v_scale = bnk::colp(kv.v_scale, col * cols.kv); q16f = bnk::colp(q16f, col * cols.arena); gate = bnk::colp(gate, col * cols.arena); }
    __shared__ __align__(16) float part[256];
    __shared__ float sx[256];
    const int d = threadIdx.x, hd = a.head_dim, w = blockIdx.x;
    const bool is_q = w < a.n_head;
    const int h = is_q ? w : w - a.n_head;
    const int pos = pos_ptr[0];
    const float *src = is_q ? qg + size_t(h) * 2 * hd : kin + size_t(h) * hd;
    const float *nw = is_q ? qn_w : kn_w;
    const float x = src[d];
    sx[d] = x;
    part[d] = __fmul_rn(x, x);
    __syncthreads();
    // the 256 squares are added serially in ascending order, as the reference's CPU mirror adds them
    // (attn_vk.h:102-108), so that the fp16 operands below are the mirror's bit for bit
    __shared__ float ssum;
    if (d == 0) {
        float acc = 0.0f;
        const float4 *p4 = reinterpret_cast<const float4 *>(part);
#pragma unroll 8
        for (int i = 0; i < 64; ++i) {
            const float4 v = p4[i];
            acc = __fadd_rn(acc, v.x); acc = __fadd_rn(acc, v.y); acc = __fadd_rn(acc, v.z); acc = __fadd_rn(acc, v.w);
        }
        ssum = acc;
    }
    __syncthreads();
    const float ss = ssum;
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(hd)), a.eps)));
    float y = __fmul_rn(__fmul_rn(x, inv), nw[d]);
    if (d < a.n_rot) {
        const int half = a.n_rot >> 1;
        const bool low = d < half;
        const int p = low ? d : d - half, pd = low ? d + half : d - half;
        const float ex = __fdiv_rn(__fmul_rn(-2.0f, float(p)), float(a.n_rot));
        const float th = float(pow(double(a.rope_base), double(ex)));
        const float ang = __fmul_rn(float(pos), th);
        const float c = float(cos(double(ang))), s = float(sin(double(ang)));
        const float xp = __fmul_rn(__fmul_rn(sx[pd], inv), nw[pd]);
        y = low ? __fsub_rn(__fmul_rn(y, c), __fmul_rn(xp, s)) : __fadd_rn(__fmul_rn(y, c), __fmul_rn(xp, s));
    }
    if (is_q) {
        q16f[size_t(h) * hd + d] = __half2float(__float2half_rn(y));
        gate[size_t(h) * hd + d] = src[hd + d];
        return;
    }
    const size_t row = (size_t(pos) * a.n_kv + h) * hd;
    const int lane = d & 31, blk = d >> 5;
    if (a.k_mode == 1) reinterpret_cast<__half *>(kv.k_data)[row + d] = __float2half_rn(y);
    else q80_store(y, lane, reinterpret_cast<int8_t *>(kv.k_data) + row + blk * 32, kv.k_scale + row / 32 + blk);
    const float v = vin[size_t(h) * hd + d];
    if (a.v_mode == 1) reinterpret_cast<__half *>(kv.v_data)[row + d] = __float2half_rn(v);
    else q80_store(v, lane, reinterpret_cast<int8_t *>(kv.v_data) + row + blk * 32, kv.v_scale + row / 32 + blk);
}

// ---- packed fp32 pairs: two IEEE single operations per instruction, each half rounded as the scalar instruction ----
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float a, float b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void unpk2(f32x2 v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
// int8 code -> float without the conversion unit: the word's bytes are biased by 128 (one xor for four codes), a byte
// is dropped into the mantissa of 2^23 and 2^23 + 128 is subtracted: exact for every code
constexpr float CODE_MAGIC = 8388736.0f;       // 2^23 + 128
__device__ __forceinline__ float code_f(uint32_t biased_word, int byte) {
    const uint32_t sel = byte == 0 ? 0x7440u : (byte == 1 ? 0x7441u : (byte == 2 ? 0x7442u : 0x7443u));
    return __uint_as_float(__byte_perm(biased_word, 0x4B000000u, sel));   // 2^23 + (code + 128), magic still to subtract
}

// scores: each warp takes 8 consecutive keys of one kv head; the gqa query heads of that kv head share every K row
// (merge idea: attn_qk_softmax_gqa.glslh:15-24). Per key and head: lane l covers dims 8l..8l+7 with an fmaf chain,
// then the 32 lane sums meet in the xor-butterfly tree (16, 8, 4, 2, 1). Two keys travel in the halves of packed
// registers (the duplicated query values are loop constants), and the 32 trees of a warp (8 keys x 4 heads) run as
// one transposed butterfly - every lane ends up with one total - which forms the same pair sums in the same order.
template <int GQA, int KMODE>
__global__ void __launch_bounds__(256) k_attn_scores(bnk::AttnDims a, const float *__restrict__ q16f,
                                                     const int *__restrict__ pos_ptr, bnk::KvLayer kv,
                                                     float *__restrict__ score, unsigned *__restrict__ counters, bnk::Cols cols) {
    static_assert(GQA == 4, "the transposed reduction is laid out for 8 keys x 4 heads");
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; q16f = bnk::colp(q16f, col * cols.arena); pos_ptr = bnk::colp(pos_ptr, col * cols.arena); kv.k_data = bnk::colp(kv.k_data, col * cols.kv); kv.k_scale = bnk::colp(kv.k_scale, col * cols.kv); score = bnk::colp(score, col * cols.arena); counters = bnk::colp(counters, col * cols.arena); }
    const int kvh = blockIdx.y, lane = threadIdx.x & 31, hd = a.head_dim;
    // arrival counters of the softmax-sum kernel that follows: zero before it starts
    if (blockIdx.x == 0 && kvh == 0 && int(threadIdx.x) < a.n_head) counters[threadIdx.x] = 0u;
    const int nfill = pos_ptr[0] + 1;
    const int jb = (blockIdx.x * 8 + (threadIdx.x >> 5)) * 8;
    if (jb >= nfill) return;
    f32x2 qd[GQA][8];                            // (q, q): both keys of a pair meet the same query value
#pragma unroll
    for (int g = 0; g < GQA; ++g) {
        const float4 *qv = reinterpret_cast<const float4 *>(q16f + size_t(kvh * GQA + g) * hd + lane * 8);
        const float4 q0 = qv[0], q1 = qv[1];
        const float qe[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) qd[g][e] = pk2(qe[e], qe[e]);
    }
    uint4 raw16[KMODE == 1 ? 8 : 1];
    uint2 raw8[KMODE == 1 ? 1 : 8];
    float sc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int j = min(jb + u, nfill - 1);
        const size_t row = (size_t(j) * a.n_kv + kvh) * hd;
        if (KMODE == 1) raw16[u] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(kv.k_data) + row + lane * 8);
        else {
            raw8[u] = *reinterpret_cast<const uint2 *>(reinterpret_cast<const int8_t *>(kv.k_data) + row + lane * 8);
            sc[u] = half_bits_to_float(kv.k_scale[row / 32 + (lane >> 2)]);
        }
    }
    float v[32];                                 // v[4u + g]: this lane's part of (key jb+u, head g)
    const f32x2 magic2 = pk2(CODE_MAGIC, CODE_MAGIC);
#pragma unroll
    for (int up = 0; up < 4; ++up) {             // keys jb+2up, jb+2up+1
        f32x2 kf[8];
        if (KMODE == 1) {
            const __half2 *ha = reinterpret_cast<const __half2 *>(&raw16[2 * up]), *hb = reinterpret_cast<const __half2 *>(&raw16[2 * up + 1]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 fa = __half22float2(ha[e]), fb = __half22float2(hb[e]);
                kf[2 * e] = pk2(fa.x, fb.x); kf[2 * e + 1] = pk2(fa.y, fb.y);
            }
        } else {
            const uint32_t a0 = raw8[2 * up].x ^ 0x80808080u, a1 = raw8[2 * up].y ^ 0x80808080u;
            const uint32_t b0 = raw8[2 * up + 1].x ^ 0x80808080u, b1 = raw8[2 * up + 1].y ^ 0x80808080u;
            const f32x2 sc2 = pk2(sc[2 * up], sc[2 * up + 1]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const f32x2 c = sub2(pk2(code_f(e < 4 ? a0 : a1, e & 3), code_f(e < 4 ? b0 : b1, e & 3)), magic2);
                kf[e] = mul2(sc2, c);
            }
        }
#pragma unroll
        for (int g = 0; g < GQA; ++g) {
            f32x2 acc = 0ull;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fma2(qd[g][e], kf[e], acc);
            unpk2(acc, v[8 * up + g], v[8 * up + 4 + g]);
        }
    }
    // transposed butterfly: at distance `off` a lane keeps the half of its values that its bit selects and adds the
    // partner's copy of the same values; lane l ends with the total of value l
#pragma unroll
    for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
        const bool upper = lane & off;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? v[i] : v[i + n / 2];
            const float keep = upper ? v[i + n / 2] : v[i];
            v[i] = __fadd_rn(keep, __shfl_xor_sync(0xFFFFFFFFu, send, off));
        }
    }
    const int u = lane >> 2, g = lane & 3, j = jb + u;
    if (j < nfill) score[size_t(kvh * GQA + g) * a.cap + j] = v[0];
}

// The same scores for any number of query heads per kv head (the kernel above is laid out for four): a warp takes 8
// consecutive keys of one kv head and walks the query heads one after the other - per (key, head) the same fmaf chain over
// the lane's 8 dims and the same xor-butterfly tree, so the same floats.
template <int KMODE>
__global__ void __launch_bounds__(256) k_attn_scores_any(bnk::AttnDims a, int gqa, const float *__restrict__ q16f,
                                                         const int *__restrict__ pos_ptr, bnk::KvLayer kv,
                                                         float *__restrict__ score, unsigned *__restrict__ counters, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; q16f = bnk::colp(q16f, col * cols.arena); pos_ptr = bnk::colp(pos_ptr, col * cols.arena); kv.k_data = bnk::colp(kv.k_data, col * cols.kv); kv.k_scale = bnk::colp(kv.k_scale, col * cols.kv); score = bnk::colp(score, col * cols.arena); counters = bnk::colp(counters, col * cols.arena); }
    const int kvh = blockIdx.y, lane = threadIdx.x & 31, hd = a.head_dim;
    if (blockIdx.x == 0 && kvh == 0) for (int i = threadIdx.x; i < a.n_head; i += 256) counters[i] = 0u;
    const int nfill = pos_ptr[0] + 1;
    const int jb = (blockIdx.x * 8 + (threadIdx.x >> 5)) * 8;
    if (jb >= nfill) return;
    float kf[8][8];                              // this lane's 8 dims of the 8 keys
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int j = min(jb + u, nfill - 1);
        const size_t row = (size_t(j) * a.n_kv + kvh) * hd;
        if (KMODE == 1) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(kv.k_data) + row + lane * 8);
            const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h2[e]); kf[u][2 * e] = f.x; kf[u][2 * e + 1] = f.y; }
        } else {
            const uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const int8_t *>(kv.k_data) + row + lane * 8);
            const float sc = half_bits_to_float(kv.k_scale[row / 32 + (lane >> 2)]);
            const int8_t *c8 = reinterpret_cast<const int8_t *>(&raw);
#pragma unroll
            for (int e = 0; e < 8; ++e) kf[u][e] = __fmul_rn(sc, float(int(c8[e])));
        }
    }
    for (int g = 0; g < gqa; ++g) {
        const float4 *qv = reinterpret_cast<const float4 *>(q16f + size_t(kvh * gqa + g) * hd + lane * 8);
        const float4 q0 = qv[0], q1 = qv[1];
        const float qe[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float acc = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(qe[e], kf[u][e], acc);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, off));
            if (lane == u && jb + u < nfill) score[size_t(kvh * gqa + g) * a.cap + jb + u] = acc;
        }
    }
}

// Softmax numerators and their sum, spread over EXPSUM_PARTS CTAs per head with the summation order of one
// 1024-thread CTA: "virtual thread" vt adds the keys vt, vt+1024, ... ascending, and the 1024 partial sums are
// then combined by the fixed tree (attn_qk_softmax.comp / attn_vk.h:175-190 in the regrouped order the CPU
// checker also carries). Every CTA recomputes the row maximum (a maximum does not depend on order); the
// exponentials of one virtual thread are evaluated by 8 real threads, then its owner adds them in order. The CTA of
// a head that finishes last (arrival counter, no waiting) runs the tree and leaves the head's total.
constexpr int EXPSUM_PARTS = 8;
__global__ void __launch_bounds__(1024) k_attn_expsum(bnk::AttnDims a, const int *__restrict__ pos_ptr,
                                                      const float *__restrict__ score, float scale,
                                                      float *__restrict__ pe, float *__restrict__ partial, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; pos_ptr = bnk::colp(pos_ptr, col * cols.arena); score = bnk::colp(score, col * cols.arena); pe = bnk::colp(pe, col * cols.arena); partial = bnk::colp(partial, col * cols.arena); }
    __shared__ float red[1024];
    __shared__ unsigned arrived;
    const int h = blockIdx.x, c = blockIdx.y, t = threadIdx.x, nfill = pos_ptr[0] + 1;
    float *total = partial + size_t(a.n_head) * 1024;
    unsigned *counters = reinterpret_cast<unsigned *>(total + a.n_head);
    const float *sr = score + size_t(h) * a.cap;
    float mx = -INFINITY;
    for (int j = t; j < nfill; j += 1024) mx = fmaxf(mx, __fmul_rn(sr[j], scale));
    red[t] = mx;
    for (int s = 512; s > 0; s >>= 1) { __syncthreads(); if (t < s) red[t] = fmaxf(red[t], red[t + s]); }
    __syncthreads();
    mx = red[0];
    float *pr = pe + size_t(h) * a.cap;
    const int vt = c * 128 + (t & 127), sub = t >> 7;
    for (int j = vt + 1024 * sub; j < nfill; j += 1024 * 8) pr[j] = exp_f(__fsub_rn(__fmul_rn(sr[j], scale), mx));
    __syncthreads();
    if (sub == 0) {
        float sum = 0.0f;
        for (int j = vt; j < nfill; j += 1024) sum = __fadd_rn(sum, pr[j]);
        partial[size_t(h) * 1024 + vt] = sum;
        __threadfence();
    }
    __syncthreads();
    if (t == 0) arrived = atomicAdd(counters + h, 1u);
    __syncthreads();
    if (arrived != EXPSUM_PARTS - 1) return;
    __threadfence();
    red[t] = __ldcg(partial + size_t(h) * 1024 + t);
    const float tot = block_tree_sum(red, 1024);
    if (t == 0) total[h] = tot;
}

// PV: grid (n_kv, splits); thread d = output dim; keys of the split ascending; acc = acc + p*v with p = fp16(e / total)
// formed while the split's numerators are staged in shared memory
// (no fused multiply-add, runtime_vk/shaders/attn_pv_q8v.comp:85-112). The split's probabilities are staged in
// shared memory and the V bytes of 8 keys are requested before the 8 dependent adds run.
template <int GQA>
__global__ void __launch_bounds__(256) k_attn_pv(bnk::AttnDims a, const float *__restrict__ p16f, const float *__restrict__ total,
                                                 const int *__restrict__ pos_ptr, bnk::KvLayer kv, int splits,
                                                 float *__restrict__ part, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; p16f = bnk::colp(p16f, col * cols.arena); total = bnk::colp(total, col * cols.arena); pos_ptr = bnk::colp(pos_ptr, col * cols.arena); kv.k_data = bnk::colp(kv.k_data, col * cols.kv); kv.k_scale = bnk::colp(kv.k_scale, col * cols.kv); kv.v_data = bnk::colp(kv.v_data, col * cols.kv); kv.v_scale = bnk::colp(kv.v_scale, col * cols.kv); part = bnk::colp(part, col * cols.arena); }
    extern __shared__ float ps[];                     // [GQA][per]
    const int kvh = blockIdx.x, sp = blockIdx.y, d = threadIdx.x, hd = a.head_dim;
    const int nfill = pos_ptr[0] + 1;
    const int per = (nfill + splits - 1) / splits;
    const int j0 = sp * per, j1 = min(nfill, j0 + per);
    const int n = max(0, j1 - j0);
    for (int i = d; i < GQA * n; i += 256) {
        const int g = i / n, jj = i - g * n;
        ps[g * per + jj] = __half2float(__float2half_rn(__fdiv_rn(p16f[size_t(kvh * GQA + g) * a.cap + j0 + jj], total[kvh * GQA + g])));
    }
    __syncthreads();
    float acc[GQA];
#pragma unroll
    for (int g = 0; g < GQA; ++g) acc[g] = 0.0f;
    if (a.v_mode == 0) {
        // q8_0 V: tiles of 32 keys x 256 bytes come in with 16-byte loads (the next tile is in flight while this one
        // is consumed) and are walked from shared memory, key by key in ascending order as before
        __shared__ uint4 vt[2][32 * 16];
        __shared__ uint16_t vsc[2][32 * 8];
        const int8_t *vd = reinterpret_cast<const int8_t *>(kv.v_data);
        uint4 r0, r1;
        uint16_t rs;
        auto fetch = [&](int jb) {
            const int k0 = min(jb + (d >> 4), n - 1), k1 = min(jb + 16 + (d >> 4), n - 1), ks = min(jb + (d >> 3), n - 1);
            r0 = *reinterpret_cast<const uint4 *>(vd + (size_t(j0 + k0) * a.n_kv + kvh) * hd + (d & 15) * 16);
            r1 = *reinterpret_cast<const uint4 *>(vd + (size_t(j0 + k1) * a.n_kv + kvh) * hd + (d & 15) * 16);
            rs = kv.v_scale[(size_t(j0 + ks) * a.n_kv + kvh) * (hd / 32) + (d & 7)];
        };
        if (n > 0) fetch(0);
        int buf = 0;
        for (int jb = 0; jb < n; jb += 32, buf ^= 1) {
            vt[buf][d] = r0; vt[buf][256 + d] = r1; vsc[buf][d] = rs;
            __syncthreads();
            if (jb + 32 < n) fetch(jb + 32);
            const int8_t *tile = reinterpret_cast<const int8_t *>(vt[buf]);
            const int lim = min(32, n - jb);
            for (int u = 0; u < lim; ++u) {
                const float v = __fmul_rn(half_bits_to_float(vsc[buf][u * 8 + (d >> 5)]), float(tile[u * 256 + d]));
#pragma unroll
                for (int g = 0; g < GQA; ++g) acc[g] = __fadd_rn(acc[g], __fmul_rn(ps[g * per + jb + u], v));
            }
        }
    } else
    for (int jb = 0; jb < n; jb += 8) {            // fp16 V
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int jj = min(jb + u, n - 1);
            const size_t idx = (size_t(j0 + jj) * a.n_kv + kvh) * hd + d;
            v[u] = __half2float(reinterpret_cast<const __half *>(kv.v_data)[idx]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (jb + u < n) {
#pragma unroll
                for (int g = 0; g < GQA; ++g) acc[g] = __fadd_rn(acc[g], __fmul_rn(ps[g * per + jb + u], v[u]));
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GQA; ++g) part[(size_t(sp) * a.n_head + kvh * GQA + g) * hd + d] = acc[g];
}

// combine the splits ascending, then the sigmoid gate
__global__ void k_attn_combine(bnk::AttnDims a, const float *__restrict__ part, int splits, const int *pos_ptr,
                               const float *__restrict__ gate, float *__restrict__ pregate, float *__restrict__ gated, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; part = bnk::colp(part, col * cols.arena); pos_ptr = bnk::colp(pos_ptr, col * cols.arena); gate = bnk::colp(gate, col * cols.arena); pregate = bnk::colp(pregate, col * cols.arena); gated = bnk::colp(gated, col * cols.arena); }
    const int i = blockIdx.x * blockDim.x + threadIdx.x, n = a.n_head * a.head_dim;
    if (i >= n) return;
    const int nfill = pos_ptr[0] + 1;
    const int per = (nfill + splits - 1) / splits;
    float acc = part[i];
    for (int sb = 1; sb < splits; sb += 64) {          // 64 partials in flight, added in ascending order
        float v[64];
#pragma unroll
        for (int u = 0; u < 64; ++u) v[u] = (sb + u < splits && (sb + u) * per < nfill) ? part[size_t(sb + u) * n + i] : 0.0f;
#pragma unroll
        for (int u = 0; u < 64; ++u) if (sb + u < splits && (sb + u) * per < nfill) acc = __fadd_rn(acc, v[u]);
    }
    if (pregate) pregate[i] = acc;
    gated[i] = __fmul_rn(acc, __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(-gate[i]))));
}

// ---- greedy pick: first maximum (Sampler::pick, runtime_vk/bonsai_forward.h:2568-2570) ----------
__global__ void __launch_bounds__(1024) k_argmax_part(const float *__restrict__ x, int n, float *__restrict__ bv,
                                                      int *__restrict__ bi, bnk::Cols cols) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; x = bnk::colp(x, col * cols.arena); bv = bnk::colp(bv, col * cols.arena); bi = bnk::colp(bi, col * cols.arena); }
    __shared__ float sv[1024];
    __shared__ int si[1024];
    const int t = threadIdx.x;
    float best = -INFINITY; int idx = 0x7FFFFFFF;
    for (int i = blockIdx.x * 1024 + t; i < n; i += gridDim.x * 1024) {
        const float v = x[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    sv[t] = best; si[t] = idx;
    for (int s = 512; s > 0; s >>= 1) {
        __syncthreads();
        if (t < s) {
            const float v = sv[t + s]; const int i = si[t + s];
            if (v > sv[t] || (v == sv[t] && i < si[t])) { sv[t] = v; si[t] = i; }
        }
    }
    if (t == 0) { bv[blockIdx.x] = sv[0]; bi[blockIdx.x] = si[0]; }
}
// cand != null (the rows are one shard of the output head, starting at row0): the column's candidate (value, global
// row or 0x7FFFFFFF when no row qualified) also goes to cand[2 * column], for the pick over all shards
__global__ void k_argmax_final(const float *__restrict__ bv, const int *__restrict__ bi, int nparts, int *out, bnk::Cols cols,
                               float *__restrict__ cand, int row0) {
    bnk::pdl_sync();
    { const size_t col = blockIdx.z; bv = bnk::colp(bv, col * cols.arena); bi = bnk::colp(bi, col * cols.arena); out = bnk::colp(out, col * cols.arena); }
    if (threadIdx.x != 0) return;
    float best = bv[0]; int idx = bi[0];
    for (int p = 1; p < nparts; ++p) if (bv[p] > best || (bv[p] == best && bi[p] < idx)) { best = bv[p]; idx = bi[p]; }
    // a row of NaN or -inf never satisfies v > best: fall back to index 0 as the scalar loop does
    out[0] = idx == 0x7FFFFFFF ? 0 : idx;
    if (cand) {
        cand[2 * blockIdx.z] = best;
        reinterpret_cast<int *>(cand)[2 * blockIdx.z + 1] = idx == 0x7FFFFFFF ? idx : idx + row0;
    }
}
// the pick over the shards' candidates: first maximum, shards in ascending row order. One thread per column.
__global__ void k_pick_shards(const float *__restrict__ cands, int n_shards, int ncol, int *__restrict__ out) {
    bnk::pdl_sync();
    const int c = threadIdx.x;
    if (c >= ncol) return;
    float best = -INFINITY; int idx = 0x7FFFFFFF;
    for (int s = 0; s < n_shards; ++s) {
        const float v = cands[(size_t(s) * ncol + c) * 2];
        const int i = reinterpret_cast<const int *>(cands)[(size_t(s) * ncol + c) * 2 + 1];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    out[c] = idx == 0x7FFFFFFF ? 0 : idx;
}

}  // namespace

namespace bnk {

bool g_pdl = true;

void rotate_quant(cudaStream_t st, const float *x, const int32_t *signs, int n, int block, float *y, uint32_t *pack) {
    const float inv = 1.0f / sqrtf(float(block));
    uint32_t *q81 = pack, *table = pack ? pack + size_t(n / 128) * Q81_DWORDS : nullptr;
    const int span = block < 128 ? 128 : block;
    launch(k_rotate_quant, dim3(n / span), dim3(512), size_t(span) * 4 + 512, st, x, signs, span, block, inv, y, q81, table);
}
void rotate_inv(cudaStream_t st, const float *x, const int32_t *signs, int n, int block, float *y, Cols cols) {
    launch(k_rotate_inv, dim3(n / block, 1, cols.z()), dim3(512), size_t(block) * 4, st, x, signs, block, 1.0f / sqrtf(float(block)), y, cols); 
}
void embed_row(cudaStream_t st, const uint32_t *W, int K, const int *tok_ptr, float *out, Cols cols) {
    launch(k_embed_row, dim3((K + 255) / 256, 1, cols.z()), dim3(256), 0, st, W, K, tok_ptr, out, cols); 
}
void rms_norm(cudaStream_t st, const float *x, const float *w, int rows, int cols, float eps, float *y) {
    launch(k_rms_norm, dim3(rows), dim3(256), 0, st, x, w, cols, eps, y); 
}
void add_inplace(cudaStream_t st, float *res, const float *d, int n) { launch(k_add_inplace, dim3((n + 255) / 256), dim3(256), 0, st, res, d, n);  }
void swiglu(cudaStream_t st, const float *a, const float *b, int n, float *y, Cols cols) {
    launch(k_swiglu, dim3((n + 255) / 256, 1, cols.z()), dim3(256), 0, st, a, b, n, y, cols);
}
void gemv_f32_small(cudaStream_t st, const float *W, int M, int K, const float *x, float *out) {
    launch(k_gemv_f32_small, dim3((M + 7) / 8), dim3(256), 0, st, W, M, K, x, out); 
}
void gdn_gates(cudaStream_t st, const float *alpha, const float *beta_raw, const float *dt_bias, const float *ssm_a, int n,
               float *gate, float *beta) {
    launch(k_gdn_gates, dim3(1), dim3(64), 0, st, alpha, beta_raw, dt_bias, ssm_a, n, gate, beta); 
}
void conv_silu(cudaStream_t st, const float *x, const float *w, float *hist, int channels, float *y) {
    launch(k_conv_silu, dim3((channels + 255) / 256), dim3(256), 0, st, x, w, hist, channels, y); 
}
void l2_norm_rows(cudaStream_t st, const float *x, int rows, float eps, float *y) {
    launch(k_l2_norm_rows, dim3((rows + 7) / 8), dim3(256), 0, st, x, rows, eps, y); 
}
void gdn_delta(cudaStream_t st, GdnDims d, const float *q, const float *k, const float *v, const float *gate,
               const float *beta, float *state, float *o) {
    launch(k_gdn_delta, dim3(dim3(d.dim / 8, d.heads)), dim3(256), 0, st, d.heads, d.qk_heads, q, k, v, gate, beta, state, o,
                                                          1.0f / sqrtf(float(d.dim))); 
}
void gdn_core_fused(cudaStream_t st, GdnDims d, int hidden, const float *qkv, const float *conv_w, float *hist0,
                    float *hist1, const int *pos_ptr, const float *x, const float *inv_ptr, const float *norm_w, const float *alpha_w,
                    const float *beta_w, const float *dt_bias, const float *ssm_a, float *state, const float *z,
                    const float *ssm_norm, float eps, float *y, Cols cols) {
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(k_gdn_core<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384 * 4);
        cudaFuncSetAttribute(k_gdn_core<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384 * 4);
        attr = true;
    }
    if (cols.z() > 1) launch(k_gdn_core<2>, dim3(d.heads, 1, cols.z()), dim3(512), size_t(hidden) * 12, st, d.heads, d.qk_heads, hidden, qkv, conv_w, hist0, hist1, pos_ptr, x, inv_ptr,
                                                         norm_w, alpha_w, beta_w, dt_bias, ssm_a, state, z, ssm_norm, eps, y,
                                                         1.0f / sqrtf(float(d.dim)), cols);
    else launch(k_gdn_core<1>, dim3(d.heads, 1, cols.z()), dim3(512), size_t(hidden) * 12, st, d.heads, d.qk_heads, hidden, qkv, conv_w, hist0, hist1, pos_ptr, x, inv_ptr,
                                                         norm_w, alpha_w, beta_w, dt_bias, ssm_a, state, z, ssm_norm, eps, y,
                                                         1.0f / sqrtf(float(d.dim)), cols); 
}
void gdn_core_split(cudaStream_t st, GdnDims d, int hidden, const float *qkv, const float *conv_w, float *hist0, float *hist1,
                    const int *pos_ptr, const float *x, const float *inv_ptr, const float *norm_w, const float *alpha_w,
                    const float *beta_w, const float *dt_bias, const float *ssm_a, float *state, const float *z,
                    const float *ssm_norm, float eps, float *y) {
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(k_gdn_split, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384 * 4); attr = true; }
    launch(k_gdn_split, dim3(d.heads * 4), dim3(512), size_t(hidden) * 12, st, d.heads, d.qk_heads, hidden, qkv, conv_w, hist0, hist1, pos_ptr, x,
           inv_ptr, norm_w, alpha_w, beta_w, dt_bias, ssm_a, state, z, ssm_norm, eps, y, 1.0f / sqrtf(float(d.dim)));
}
void gdn_out(cudaStream_t st, GdnDims d, const float *o, const float *z, const float *ssm_norm, float eps, float *y) {
    launch(k_gdn_out, dim3((d.heads + 7) / 8), dim3(256), 0, st, d.heads, d.qk_heads, o, z, ssm_norm, eps, y); 
}
void attn_prep(cudaStream_t st, AttnDims a, const float *qg, const float *kin, const float *vin, const float *qn_w,
               const float *kn_w, const int *pos_ptr, KvLayer kv, float *q16f, float *gate, Cols cols) {
    launch(k_attn_prep, dim3(a.n_head + a.n_kv, 1, cols.z()), dim3(256), 0, st, a, qg, kin, vin, qn_w, kn_w, pos_ptr, kv, q16f, gate, cols); 
}
void attn_decode(cudaStream_t st, AttnDims a, const float *q16f, const float *gate, const int *pos_ptr, KvLayer kv,
                 float *score, float *p16f, float *esum, float *pv_part, int splits, float *pregate, float *gated, bool combine,
                 Cols cols) {
    // grids are sized for the cache capacity; warps beyond the filled prefix return at once.
    // esum: [n_head][1024] partial sums, then n_head totals, then n_head arrival counters
    float *total = esum + size_t(a.n_head) * 1024;
    unsigned *counters = reinterpret_cast<unsigned *>(total + a.n_head);
    const dim3 sg((a.cap + 63) / 64, a.n_kv, cols.z());
    const int gqa = a.n_head / a.n_kv;            // 1, 2, 4 or 8 (checked where the dimensions enter: bn_model_create, the attention ABI)
    if (gqa == 4) {
        if (a.k_mode == 1) launch(k_attn_scores<4, 1>, sg, dim3(256), 0, st, a, q16f, pos_ptr, kv, score, counters, cols);
        else launch(k_attn_scores<4, 0>, sg, dim3(256), 0, st, a, q16f, pos_ptr, kv, score, counters, cols);
    } else {
        if (a.k_mode == 1) launch(k_attn_scores_any<1>, sg, dim3(256), 0, st, a, gqa, q16f, pos_ptr, kv, score, counters, cols);
        else launch(k_attn_scores_any<0>, sg, dim3(256), 0, st, a, gqa, q16f, pos_ptr, kv, score, counters, cols);
    }
    launch(k_attn_expsum, dim3(a.n_head, EXPSUM_PARTS, cols.z()), dim3(1024), 0, st, a, pos_ptr, score, 1.0f / sqrtf(float(a.head_dim)), p16f, esum, cols);
    const dim3 pg(a.n_kv, splits, cols.z());
    const size_t ps_bytes = size_t(gqa) * ((a.cap + splits - 1) / splits) * 4;
    const float *pe = static_cast<const float *>(p16f), *tot = static_cast<const float *>(total);
    if (gqa == 4) launch(k_attn_pv<4>, pg, dim3(256), ps_bytes, st, a, pe, tot, pos_ptr, kv, splits, pv_part, cols);
    else if (gqa == 1) launch(k_attn_pv<1>, pg, dim3(256), ps_bytes, st, a, pe, tot, pos_ptr, kv, splits, pv_part, cols);
    else if (gqa == 2) launch(k_attn_pv<2>, pg, dim3(256), ps_bytes, st, a, pe, tot, pos_ptr, kv, splits, pv_part, cols);
    else {
        static bool attr = false;
        if (!attr) { cudaFuncSetAttribute(k_attn_pv<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); attr = true; }
        launch(k_attn_pv<8>, pg, dim3(256), ps_bytes, st, a, pe, tot, pos_ptr, kv, splits, pv_part, cols);
    }
    if (!combine) return;
    const int n = a.n_head * a.head_dim;
    launch(k_attn_combine, dim3((n + 255) / 256, 1, cols.z()), dim3(256), 0, st, a, pv_part, splits, pos_ptr, gate, pregate, gated, cols); 
}
void argmax_first(cudaStream_t st, const float *x, int n, int *out_idx, float *scratch_val, int *scratch_idx, Cols cols, float *cand, int row0) {
    const int parts = 64;
    launch(k_argmax_part, dim3(parts, 1, cols.z()), dim3(1024), 0, st, x, n, scratch_val, scratch_idx, cols); 
    launch(k_argmax_final, dim3(1, 1, cols.z()), dim3(32), 0, st, scratch_val, scratch_idx, parts, out_idx, cols, cand, row0);
}
void pick_shards(cudaStream_t st, const float *cands, int n_shards, int ncol, int *out) {
    launch(k_pick_shards, dim3(1), dim3(32), 0, st, cands, n_shards, ncol, out);
}

}  // namespace bnk
