// token_kernel.cu - see token_kernel.cuh. One cooperative launch of one CTA (16 warps) per SM runs a whole decode token (or
// n greedy tokens back to back): the phase list lives in the constant bank, every CTA walks it in the same order, and a
// grid-wide barrier (one atomic counter, bounded spin) separates consecutive phases.
//
// Weights. The projections' 16-row tile slices flow through the same 8-stage bulk-copy ring as in the per-projection
// kernel, but no warp is set aside to feed it: ring items carry one running number over all projections of all tokens of
// the launch, and at the iteration of item g the warp g % 16 refills the stage of item g - 2 with item g + 6 - whatever
// projection that is (a per-CTA table maps running numbers to projection and tile). The ring therefore always holds the
// next 6 to 8 items (about 100 KB per SM, 15 MB over the GPU - more than most projections have), also across barriers,
// prologues and the non-projection phases: weights depend on nothing. (A 17th copy-only warp would cap the kernel at 96
// registers per thread - 5 warps on one of the 4 schedulers - and the main loop then spills.)
//
// Arithmetic and its order are those of the stand-alone kernels in ops.cu (same CPU checker). Values that another CTA of
// the same launch wrote are always read through L2 (ld.global.cg): an SM's L1 is not coherent with other SMs' stores.
//
// No wait is unbounded: a grid barrier or ring wait that gives up sets the error word (code 4 / 1), raises the CTA's
// abort flag, every later wait of the CTA returns at once, the other CTAs see the error word in their own spins, and the
// kernel runs to its end with invalid results; the host reports BN_ERR_TIMEOUT.
#include "token_kernel.cuh"
#include "phase_body.cuh"

namespace {
using namespace bnk;
using namespace bnk::phase;

__constant__ TokOp c_ops[TOKEN_MAX_OPS];

// ---- grid barrier --------------------------------------------------------------------------------------------------
// The kernel's loop state lives in shared memory, not in registers: a phase function is a real call, and every register
// the caller keeps alive across the call is one the callee cannot use (the projection's main loop needs all 96).
struct OpShared { PhaseArgs a; Work w; };
static_assert(sizeof(OpShared) <= 300, "phase record does not fit its shared-memory slot");

struct LoopState {
    unsigned git;                 // running ring item number
    unsigned done;                // phases this CTA has arrived at
    int tok;                      // current token id
    int step, i;                  // token of the launch, phase of the token
    unsigned total, limit;        // ring items per token / in the whole launch (this CTA)
    unsigned fbase[16];           // per warp: running number of the first item of the token its last refill was in
    int fhint[16];                // per warp: table position of its last refill
};
static_assert(sizeof(LoopState) <= 192, "loop state does not fit its slot");
__device__ __forceinline__ LoopState *loop_state() { return reinterpret_cast<LoopState *>(dyn_smem() + SL::op + 320); }

struct GridBar {
    unsigned *ctr;
    unsigned ncta;
    int *err;
};
// thread 0 publishes this CTA's arrival; `items` = ring items the finished phase consumed
__device__ __forceinline__ void grid_arrive(const GridBar &b, unsigned items) {
    csync();                                          // every compute thread's stores are ordered before thread 0's release
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(b.ctr, 1u);
        LoopState *ls = loop_state();
        ls->git += items;
        ls->done += 1;
        ls->i += 1;
    }
    csync();
}
__device__ __forceinline__ void grid_wait(const GridBar &b) {
    if (threadIdx.x == 0) {
        volatile int *abort = carve(dyn_smem()).abort;
        const unsigned target = loop_state()->done * b.ncta;
        for (int it = 0;; ++it) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(b.ctr) : "memory");
            if (int(v - target) >= 0) break;
            if (*abort) break;
            if (it > 64) {
                __nanosleep(40);
                if ((it & 255) == 0 && *reinterpret_cast<volatile int *>(b.err) != 0) { *abort = 1; break; }   // another CTA gave up
                if (it > (1 << 22)) { atomicExch(b.err, 4); *abort = 1; break; }
            }
        }
        __threadfence();
    }
    csync();
}

// ---- embedding: row `tok` dequantised, H then signs, into the residual stream (every CTA writes the same values) -----
__device__ __forceinline__ void embed_phase(const TokenArgs &ta, const Smem &s, int tok) {
    const int tid = threadIdx.x, HB = ta.hat_block, K = ta.hidden;
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(float(HB)));
    float *xs = s.xs;
    for (int hb = 0; hb < K / HB; ++hb) {
        const int base = hb * HB;
        csync();
        for (int i = tid; i < HB; i += NT) {
            const int e = base + i;
            const uint32_t *blk = ta.embd + (size_t(tok) * (K / 128) + e / 128) * 7;
            const int el = e & 127;
            int byte, t;
            if (el < 80) { byte = el & 15; t = el >> 4; }
            else if (el < 120) { byte = 16 + ((el - 80) & 7); t = (el - 80) >> 3; }
            else { byte = 24 + ((el - 120) & 1); t = (el - 120) >> 1; }
            uint32_t v = (blk[byte >> 2] >> ((byte & 3) * 8)) & 0xFFu;
            for (int k = 0; k < t; ++k) v = (v * 3u) & 0xFFu;
            const int trit = int((v * 3u) >> 8);
            xs[i] = __fmul_rn(float(trit) - 1.0f, half_bits_to_float(blk[6] >> 16));
        }
        fwht_smem(xs, HB, HB, inv);
        for (int i = tid; i < HB; i += NT) ta.res[base + i] = __fmul_rn(xs[i], float(ta.signs[base + i]));
    }
    csync();
}

// ---- gated-delta-net core of one layer (ops.cu k_gdn_core, split four ways per value head) ----------------------------
// unit = (value head h, quarter q4): 32 of the head's 128 state rows, two per warp. Everything that does not depend on
// the preceding projection (state rows, conv taps and weights, the two small projections of the normed residual and their
// gate functions) is done before the grid wait. The per-head output norm, ssm_norm, swiglu and the v-grouped permutation
// are the consuming projection's prologue (PRO_GDN_OUT_SZ).
__device__ __forceinline__ void gdn_phase(const GdnOp &o, const Smem &s, const GridBar &bar, bool wait, int cta, int ncta, int pos) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = o.qk_heads, hidden = o.hidden, n4 = hidden / 4;
    float4 *xn = reinterpret_cast<float4 *>(s.scratch);             // normed residual
    float *sq = reinterpret_cast<float *>(xn + n4), *sk = sq + 128, *svv = sk + 128, *sgb = svv + 32;
    const bool odd = pos & 1;                        // a token at position p reads taps from buffer p & 1, writes the other
    const float *hist_rd = odd ? o.hist1 : o.hist0;
    float *hist_wr = odd ? o.hist0 : o.hist1;
    bool waited = !wait;
    for (int unit = cta; unit < o.heads * 4; unit += ncta) {
        const int h = unit >> 2, q4 = unit & 3, hq = h % nq;
        float S[2][4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float *Sr = o.state + (size_t(h) * 128 + q4 * 32 + warp * 2 + r) * 128;
#pragma unroll
            for (int e = 0; e < 4; ++e) S[r][e] = __ldcg(Sr + lane + 32 * e);
        }
        const int cch = tid < 128 ? hq * 128 + tid : (tid < 256 ? nq * 128 + hq * 128 + (tid - 128) : 2 * nq * 128 + h * 128 + q4 * 32 + (tid - 256));
        float tap0 = 0.0f, tap1 = 0.0f, tap2 = 0.0f, cw0 = 0.0f, cw1 = 0.0f, cw2 = 0.0f, cw3 = 0.0f;
        if (tid < 288) {
            const float *sr = hist_rd + 3 * size_t(cch);
            const float *wc = o.conv_w + 4 * size_t(cch);
            tap0 = __ldcg(sr); tap1 = __ldcg(sr + 1); tap2 = __ldcg(sr + 2);
            cw0 = wc[0]; cw1 = wc[1]; cw2 = wc[2]; cw3 = wc[3];
        }
        {   // the normed residual (norm factor: this CTA's own, kept from the preceding projection's prologue)
            const float inv = s.hinv[0];
            const float4 *nw = reinterpret_cast<const float4 *>(o.norm_w);
            for (int i = tid; i < n4; i += NT) {
                const float4 a4 = __ldcg(reinterpret_cast<const float4 *>(o.x) + i), w4 = nw[i];
                xn[i] = make_float4(__fmul_rn(__fmul_rn(a4.x, inv), w4.x), __fmul_rn(__fmul_rn(a4.y, inv), w4.y),
                                    __fmul_rn(__fmul_rn(a4.z, inv), w4.z), __fmul_rn(__fmul_rn(a4.w, inv), w4.w));
            }
        }
        csync();
        if (warp >= 14) {
            // row h of ssm_alpha (warp 14) or ssm_beta (warp 15) times the normed residual: lane l takes float4 groups
            // l, l+32, ... with one fmaf per element, then a 32-lane xor tree (k_gemv_f32_small)
            const float4 *wr = reinterpret_cast<const float4 *>((warp == 14 ? o.alpha_w : o.beta_w) + size_t(h) * hidden);
            float acc = 0.0f;
#pragma unroll 8
            for (int i = lane; i < n4; i += 32) {
                const float4 w4 = wr[i], a4 = xn[i];
                acc = fmaf(w4.x, a4.x, acc); acc = fmaf(w4.y, a4.y, acc); acc = fmaf(w4.z, a4.z, acc); acc = fmaf(w4.w, a4.w, acc);
            }
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, sft));
            if (lane == 0) {
                if (warp == 14) {
                    const float al = __fadd_rn(acc, o.dt_bias[h]);
                    const float sp = al > 20.0f ? al : log_f(__fadd_rn(1.0f, exp_f(al)));
                    sgb[0] = __fmul_rn(sp, o.ssm_a[h]);
                } else sgb[1] = sigmoid_f(acc);
            }
        }
        if (!waited) { grid_wait(bar); waited = true; }
        if (tid < 288) {
            const float xv = __ldcg(o.qkv + cch);
            float acc = __fmul_rn(cw0, tap0);
            acc = __fadd_rn(acc, __fmul_rn(cw1, tap1));
            acc = __fadd_rn(acc, __fmul_rn(cw2, tap2));
            acc = __fadd_rn(acc, __fmul_rn(cw3, xv));
            // one writer per channel: the unit's own 32 value channels; the q / k channels by the first quarter of the first
            // of the value heads that share them
            if (tid >= 256 || (h < nq && q4 == 0)) { float *sw = hist_wr + 3 * size_t(cch); sw[0] = tap1; sw[1] = tap2; sw[2] = xv; }
            const float cv = silu_f(acc);
            if (tid < 128) sq[tid] = cv; else if (tid < 256) sk[tid - 128] = cv; else svv[tid - 256] = cv;
        }
        csync();
        float qq[4], kk[4];
        {
            const float a0 = sq[lane], a1 = sq[lane + 32], a2 = sq[lane + 64], a3 = sq[lane + 96];
            const float iq = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(warp_tree128(__fmul_rn(a0, a0), __fmul_rn(a1, a1), __fmul_rn(a2, a2), __fmul_rn(a3, a3)), 1e-12f)));
            qq[0] = __fmul_rn(a0, iq); qq[1] = __fmul_rn(a1, iq); qq[2] = __fmul_rn(a2, iq); qq[3] = __fmul_rn(a3, iq);
            const float b0 = sk[lane], b1 = sk[lane + 32], b2 = sk[lane + 64], b3 = sk[lane + 96];
            const float ik = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(warp_tree128(__fmul_rn(b0, b0), __fmul_rn(b1, b1), __fmul_rn(b2, b2), __fmul_rn(b3, b3)), 1e-12f)));
            kk[0] = __fmul_rn(b0, ik); kk[1] = __fmul_rn(b1, ik); kk[2] = __fmul_rn(b2, ik); kk[3] = __fmul_rn(b3, ik);
        }
        const float eg = exp_f(sgb[0]), bt = sgb[1];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int jl = warp * 2 + r, j = q4 * 32 + jl;
            float *Sr = o.state + (size_t(h) * 128 + j) * 128;
            float st[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) st[e] = __fmul_rn(S[r][e], eg);
            const float pred = warp_tree128(__fmul_rn(st[0], kk[0]), __fmul_rn(st[1], kk[1]), __fmul_rn(st[2], kk[2]), __fmul_rn(st[3], kk[3]));
            const float u = __fmul_rn(bt, __fsub_rn(svv[jl], pred));
#pragma unroll
            for (int e = 0; e < 4; ++e) { st[e] = fmaf(kk[e], u, st[e]); Sr[lane + 32 * e] = st[e]; }
            const float ov = warp_tree128(__fmul_rn(st[0], qq[0]), __fmul_rn(st[1], qq[1]), __fmul_rn(st[2], qq[2]), __fmul_rn(st[3], qq[3]));
            if (lane == 0) o.o[h * 128 + j] = __fmul_rn(ov, o.scale);
        }
        csync();                                     // shared memory is reused by the next unit
    }
    if (!waited) grid_wait(bar);
}

// ---- attention: head norm + rope + fp16 Q, K / V cache insert (ops.cu k_attn_prep) -----------------------------------
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
__device__ __forceinline__ void attn_prep_phase(const AttnOp &o, const Smem &s, int cta, int ncta, int pos) {
    const AttnDims &a = o.d;
    const int d = threadIdx.x, hd = a.head_dim;
    float *part = reinterpret_cast<float *>(s.scratch), *sx = part + 256, *ssum = sx + 256;
    for (int w = cta; w < a.n_head + a.n_kv; w += ncta) {
        const bool is_q = w < a.n_head;
        const int h = is_q ? w : w - a.n_head;
        const float *src = is_q ? o.qg + size_t(h) * 2 * hd : o.kin + size_t(h) * hd;
        const float *nw = is_q ? o.qn_w : o.kn_w;
        float x = 0.0f;
        if (d < 256) { x = __ldcg(src + d); sx[d] = x; part[d] = __fmul_rn(x, x); }
        csync();
        if (d == 0) {   // the 256 squares added serially in ascending order (attn_vk.h:102-108)
            float acc = 0.0f;
            const float4 *p4 = reinterpret_cast<const float4 *>(part);
#pragma unroll 8
            for (int i = 0; i < 64; ++i) {
                const float4 v = p4[i];
                acc = __fadd_rn(acc, v.x); acc = __fadd_rn(acc, v.y); acc = __fadd_rn(acc, v.z); acc = __fadd_rn(acc, v.w);
            }
            ssum[0] = acc;
        }
        csync();
        if (d < 256) {
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssum[0], float(hd)), a.eps)));
            float y = __fmul_rn(__fmul_rn(x, inv), nw[d]);
            if (d < a.n_rot) {
                const int half = a.n_rot >> 1;
                const bool low = d < half;
                const int p = low ? d : d - half, pd = low ? d + half : d - half;
                const float ex = __fdiv_rn(__fmul_rn(-2.0f, float(p)), float(a.n_rot));
                const float th = float(pow(double(a.rope_base), double(ex)));
                const float ang = __fmul_rn(float(pos), th);
                const float c = float(cos(double(ang))), sn = float(sin(double(ang)));
                const float xp = __fmul_rn(__fmul_rn(sx[pd], inv), nw[pd]);
                y = low ? __fsub_rn(__fmul_rn(y, c), __fmul_rn(xp, sn)) : __fadd_rn(__fmul_rn(y, c), __fmul_rn(xp, sn));
            }
            if (is_q) {
                o.q16f[size_t(h) * hd + d] = __half2float(__float2half_rn(y));
                o.gate[size_t(h) * hd + d] = __ldcg(src + hd + d);
            } else {
                const size_t row = (size_t(pos) * a.n_kv + h) * hd;
                const int lane = d & 31, blk = d >> 5;
                if (a.k_mode == 1) reinterpret_cast<__half *>(o.kv.k_data)[row + d] = __float2half_rn(y);
                else q80_store(y, lane, reinterpret_cast<int8_t *>(o.kv.k_data) + row + blk * 32, o.kv.k_scale + row / 32 + blk);
                const float v = __ldcg(o.vin + size_t(h) * hd + d);
                if (a.v_mode == 1) reinterpret_cast<__half *>(o.kv.v_data)[row + d] = __float2half_rn(v);
                else q80_store(v, lane, reinterpret_cast<int8_t *>(o.kv.v_data) + row + blk * 32, o.kv.v_scale + row / 32 + blk);
            }
        }
        csync();
    }
}

// ---- attention scores (ops.cu k_attn_scores): each warp takes 8 consecutive keys of one kv head ------------------------
__device__ __forceinline__ void attn_scores_phase(const AttnOp &o, int cta, int ncta, int pos) {
    constexpr int GQA = 4;
    const AttnDims &a = o.d;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, hd = a.head_dim;
    const int nfill = pos + 1;
    const int nkb = (nfill + 127) / 128;
    for (int unit = cta; unit < nkb * a.n_kv; unit += ncta) {
        const int kb = unit / a.n_kv, kvh = unit - kb * a.n_kv;
        const int jb = (kb * 16 + warp) * 8;
        if (jb >= nfill) continue;
        float q[GQA][8];
#pragma unroll
        for (int g = 0; g < GQA; ++g) {
            const float4 *qv = reinterpret_cast<const float4 *>(o.q16f + size_t(kvh * GQA + g) * hd + lane * 8);
            const float4 q0 = __ldcg(qv), q1 = __ldcg(qv + 1);
            q[g][0] = q0.x; q[g][1] = q0.y; q[g][2] = q0.z; q[g][3] = q0.w; q[g][4] = q1.x; q[g][5] = q1.y; q[g][6] = q1.z; q[g][7] = q1.w;
        }
        // two rounds of 4 keys: the 4 K rows of a round are requested before any of them is used
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
            uint4 raw16[4];
            uint2 raw8[4];
            float sc[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = min(jb + half * 4 + u, nfill - 1);
                const size_t row = (size_t(j) * a.n_kv + kvh) * hd;
                if (a.k_mode == 1) raw16[u] = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(o.kv.k_data) + row + lane * 8));
                else {
                    raw8[u] = __ldcg(reinterpret_cast<const uint2 *>(reinterpret_cast<const int8_t *>(o.kv.k_data) + row + lane * 8));
                    sc[u] = half_bits_to_float(__ldcg(o.kv.k_scale + row / 32 + (lane >> 2)));
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = jb + half * 4 + u;
                float kf[8];
                if (a.k_mode == 1) {
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw16[u]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h2[e]); kf[2 * e] = f.x; kf[2 * e + 1] = f.y; }
                } else {
                    const int8_t *c = reinterpret_cast<const int8_t *>(&raw8[u]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) kf[e] = __fmul_rn(sc[u], float(c[e]));
                }
#pragma unroll
                for (int g = 0; g < GQA; ++g) {
                    float acc = 0.0f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc = fmaf(q[g][e], kf[e], acc);
#pragma unroll
                    for (int sft = 16; sft > 0; sft >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, sft));
                    if (lane == 0 && j < nfill) o.score[size_t(kvh * GQA + g) * a.cap + j] = acc;
                }
            }
        }
    }
}

// ---- softmax numerators and their partial sums (ops.cu k_attn_expsum, 8 parts per head) ---------------------------------
__device__ __forceinline__ void attn_expsum_phase(const AttnOp &o, const Smem &s, int cta, int ncta, int pos) {
    const AttnDims &a = o.d;
    const int t = threadIdx.x, nfill = pos + 1;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(float(a.head_dim)));
    float *red = reinterpret_cast<float *>(s.scratch);
    for (int unit = cta; unit < a.n_head * 8; unit += ncta) {
        const int h = unit >> 3, c = unit & 7;
        const float *sr = o.score + size_t(h) * a.cap;
        float mx = -INFINITY;
        for (int j = t; j < nfill; j += NT) mx = fmaxf(mx, __fmul_rn(__ldcg(sr + j), scale));
        red[t] = mx;
        for (int sft = NT / 2; sft > 0; sft >>= 1) { csync(); if (t < sft) red[t] = fmaxf(red[t], red[t + sft]); }
        csync();
        mx = red[0];
        float *pr = o.pe + size_t(h) * a.cap;
        const int vt = c * 128 + (t & 127), sub = t >> 7;
        for (int j = vt + 1024 * sub; j < nfill; j += 1024 * 4) pr[j] = exp_f(__fsub_rn(__fmul_rn(__ldcg(sr + j), scale), mx));
        csync();
        if (sub == 0) {   // "virtual thread" vt of 1024 adds the keys vt, vt + 1024, ... in ascending order
            float sum = 0.0f;
            for (int j = vt; j < nfill; j += 1024) sum = __fadd_rn(sum, __ldcg(pr + j));
            o.esum[size_t(h) * 1024 + vt] = sum;
        }
        csync();
    }
}

// ---- probabilities (fp16-rounded) x V over one split of the keys (ops.cu k_attn_normalise + k_attn_pv) ------------------
__device__ __forceinline__ void attn_pv_phase(const AttnOp &o, const Smem &s, int cta, int ncta, int pos) {
    constexpr int GQA = 4;
    const AttnDims &a = o.d;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, hd = a.head_dim, nfill = pos + 1;
    const int splits = o.splits, per = (nfill + splits - 1) / splits;
    float *red4 = reinterpret_cast<float *>(s.scratch);            // [4][512]
    float *tot = red4 + 4 * 512;                                    // [4]
    uint4 *vt = reinterpret_cast<uint4 *>(tot + 4);                 // [2][32 * 16]
    uint16_t *vsc = reinterpret_cast<uint16_t *>(vt + 2 * 32 * 16); // [2][32 * 8]
    float *ps = reinterpret_cast<float *>(vsc + 2 * 32 * 8);        // [GQA][per]
    for (int unit = cta; unit < a.n_kv * splits; unit += ncta) {
        const int kvh = unit / splits, sp = unit - kvh * splits;
        const int j0 = sp * per, j1 = min(nfill, j0 + per);
        const int n = max(0, j1 - j0);
        if (n == 0 && sp > 0) continue;          // nothing reads this split (the combine skips splits that start beyond the prefix)
        // softmax denominators of the 4 query heads: the fixed tree p[i] += p[i + s], s = 512 .. 1, over the 1024 partial sums
#pragma unroll
        for (int g = 0; g < GQA; ++g) {
            const float *pp = o.esum + size_t(kvh * GQA + g) * 1024;
            red4[g * 512 + t] = __fadd_rn(__ldcg(pp + t), __ldcg(pp + t + 512));
        }
        for (int sft = 256; sft >= 32; sft >>= 1) {
            csync();
            if (t < sft) {
#pragma unroll
                for (int g = 0; g < GQA; ++g) red4[g * 512 + t] = __fadd_rn(red4[g * 512 + t], red4[g * 512 + t + sft]);
            }
        }
        csync();
        if (warp < GQA) {
            float v = red4[warp * 512 + lane];
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, sft));
            if (lane == 0) tot[warp] = v;
        }
        csync();
        for (int i = t; i < GQA * n; i += NT) {
            const int g = i / n, jj = i - g * n;
            const float e = __ldcg(o.pe + size_t(kvh * GQA + g) * a.cap + j0 + jj);
            ps[g * per + jj] = __half2float(__float2half_rn(__fdiv_rn(e, tot[g])));
        }
        csync();
        const int d = t;
        float acc[GQA];
#pragma unroll
        for (int g = 0; g < GQA; ++g) acc[g] = 0.0f;
        if (a.v_mode == 0) {
            const int8_t *vd = reinterpret_cast<const int8_t *>(o.kv.v_data);
            uint4 r0 = make_uint4(0, 0, 0, 0), r1 = r0;
            uint16_t rs = 0;
            auto fetch = [&](int jb) {
                const int k0 = min(jb + (d >> 4), n - 1), k1 = min(jb + 16 + (d >> 4), n - 1), ks = min(jb + (d >> 3), n - 1);
                r0 = __ldcg(reinterpret_cast<const uint4 *>(vd + (size_t(j0 + k0) * a.n_kv + kvh) * hd + (d & 15) * 16));
                r1 = __ldcg(reinterpret_cast<const uint4 *>(vd + (size_t(j0 + k1) * a.n_kv + kvh) * hd + (d & 15) * 16));
                rs = __ldcg(o.kv.v_scale + (size_t(j0 + ks) * a.n_kv + kvh) * (hd / 32) + (d & 7));
            };
            if (n > 0 && d < 256) fetch(0);
            int buf = 0;
            for (int jb = 0; jb < n; jb += 32, buf ^= 1) {
                if (d < 256) { vt[buf * 512 + d] = r0; vt[buf * 512 + 256 + d] = r1; vsc[buf * 256 + d] = rs; }
                csync();
                if (d < 256) {
                    if (jb + 32 < n) fetch(jb + 32);
                    const int8_t *tile = reinterpret_cast<const int8_t *>(vt + buf * 512);
                    const int lim = min(32, n - jb);
                    for (int u = 0; u < lim; ++u) {
                        const float v = __fmul_rn(half_bits_to_float(vsc[buf * 256 + u * 8 + (d >> 5)]), float(tile[u * 256 + d]));
#pragma unroll
                        for (int g = 0; g < GQA; ++g) acc[g] = __fadd_rn(acc[g], __fmul_rn(ps[g * per + jb + u], v));
                    }
                }
            }
        } else if (d < 256) {
            for (int jb = 0; jb < n; jb += 8) {            // fp16 V
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int jj = min(jb + u, n - 1);
                    const size_t idx = (size_t(j0 + jj) * a.n_kv + kvh) * hd + d;
                    v[u] = __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short *>(o.kv.v_data) + idx)));
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (jb + u < n) {
#pragma unroll
                        for (int g = 0; g < GQA; ++g) acc[g] = __fadd_rn(acc[g], __fmul_rn(ps[g * per + jb + u], v[u]));
                    }
                }
            }
        }
        if (d < 256) {
#pragma unroll
            for (int g = 0; g < GQA; ++g) o.pv_part[(size_t(sp) * a.n_head + kvh * GQA + g) * hd + d] = acc[g];
        }
        csync();
    }
}

// ---- splits added in ascending order, then the sigmoid gate (ops.cu k_attn_combine) -------------------------------------
__device__ __forceinline__ void attn_combine_phase(const AttnOp &o, int cta, int ncta, int pos) {
    const AttnDims &a = o.d;
    const int n = a.n_head * a.head_dim, nfill = pos + 1, splits = o.splits;
    const int per = (nfill + splits - 1) / splits;
    for (int i = cta * NT + int(threadIdx.x); i < n; i += ncta * NT) {
        float acc = __ldcg(o.pv_part + i);
        for (int sb = 1; sb < splits; sb += 16) {          // 16 partials in flight, added in ascending order
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = (sb + u < splits && (sb + u) * per < nfill) ? __ldcg(o.pv_part + size_t(sb + u) * n + i) : 0.0f;
#pragma unroll
            for (int u = 0; u < 16; ++u) if (sb + u < splits && (sb + u) * per < nfill) acc = __fadd_rn(acc, v[u]);
        }
        o.gated[i] = __fmul_rn(acc, __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(-__ldcg(o.gate + i)))));
    }
}

// ---- the ring's feed: running item number -> (projection, chunk, tile) -------------------------------------------------
// One 32-byte record per projection of the token in shared memory holds all that a refill needs, so that the warp on
// feed duty spends a few dozen instructions on it (no division, no constant-bank walk).
struct FeedEnt {
    int cum;                  // items of this CTA in the token's earlier projections
    int t0, nt;               // this CTA's run of (virtual) tiles
    int M, nb;                // rows, blocks per row
    int half_tiles;           // >= 0: gate / up row pairs (EPI_SWIGLU), virtual tile v -> tile v/2 of the first or second half
    const uint8_t *W;
};
static_assert(sizeof(FeedEnt) == 32, "feed record");
constexpr int FEED_MAX = 215;
struct TokFeed {
    static constexpr bool on = true;
    __device__ __forceinline__ void operator()(uint32_t G) const {
        unsigned char *smem = dyn_smem();
        LoopState *ls = loop_state();
        if (G >= ls->limit) return;
        const Smem s = carve(smem);
        const FeedEnt *tab = reinterpret_cast<const FeedEnt *>(smem + SL::feed);
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const uint32_t total = ls->total;
        uint32_t base = ls->fbase[warp], r = G - base;
        int j = ls->fhint[warp];
        while (r >= total) { r -= total; base += total; j = 0; }
        while (int(r) >= tab[j + 1].cum) ++j;
        __syncwarp();
        if (lane == 0) { ls->fbase[warp] = base; ls->fhint[warp] = j; }
        const FeedEnt e = tab[j];
        int it = int(r) - e.cum, chunk = 0;
        while (it >= e.nt) { it -= e.nt; ++chunk; }
        const int v = e.t0 + it;
        const int tile = e.half_tiles >= 0 ? ((v & 1) ? e.half_tiles + (v >> 1) : (v >> 1)) : v;
        const int CH = e.nb <= MAXCH ? e.nb : MAXCH, rowb = CH * 28, stage = int(G % STAGES);
        if (lane == 0) mbar_expect_tx(s.full + stage, 16u * uint32_t(rowb));
        __syncwarp();
        if (lane < 16) {
            const int row = min(tile * 16 + lane, e.M - 1);
            bulk_copy(s.ring + stage * STAGE_BYTES + lane * (rowb + 16), e.W + (size_t(row) * e.nb + size_t(chunk) * CH) * 28, uint32_t(rowb), s.full + stage);
        }
    }
};

// every CTA reduces the per-CTA candidates of the output head to the first maximum: the next token id
__device__ __forceinline__ void pick_phase(const TokenArgs &ta, const GridBar &bar, int step, int cta, int ncta) {
    grid_wait(bar);
    const Smem s = carve(dyn_smem());
    const int tid = threadIdx.x;
    float *cv = s.red;
    int *ci = reinterpret_cast<int *>(s.red + 256);          // the s.sv region follows s.red: free between projections
    if (tid < 256) {
        float bv = -INFINITY; int bi = 0x7FFFFFFF;
        for (int c = tid; c < ncta; c += 256) {
            const float v = __ldcg(ta.cand_val + c); const int ix = __ldcg(ta.cand_idx + c);
            if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
        }
        cv[tid] = bv; ci[tid] = bi;
    }
    csync();
    if (tid < 32) {
        float bv = cv[tid]; int bi = ci[tid];
        for (int c = tid + 32; c < 256; c += 32) if (cv[c] > bv || (cv[c] == bv && ci[c] < bi)) { bv = cv[c]; bi = ci[c]; }
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, sft); const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, sft);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (tid == 0) {
            const int tok = bi == 0x7FFFFFFF ? 0 : bi;       // a row of NaN or -inf: index 0, as the scalar loop does
            loop_state()->tok = tok;
            if (cta == 0) { ta.hist[step] = tok; ta.next[0] = tok; }
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------------------------------
// The loop counters live in shared memory and are re-read after every phase: nothing but the running phase's own values
// occupies registers while a projection's main loop runs (a spilled value costs an L2 round trip here - the L1 is almost
// entirely carved out as shared memory).
__global__ void __launch_bounds__(NT, 1) k_token(const TokenArgs ta) {
    {
        unsigned char *smem = dyn_smem();
        const Smem s = carve(smem);
        const int tid = threadIdx.x, cta = blockIdx.x, ncta = gridDim.x;
        FeedEnt *tab = reinterpret_cast<FeedEnt *>(smem + SL::feed);
        // this CTA's share of every projection of the token (the two 64-bit divisions per projection are spread over threads)
        int *tmp = reinterpret_cast<int *>(s.scratch);
        for (int i = tid; i < ta.n_ops; i += NT) {
            int t0 = 0, nt = 0, items = -1;
            if (c_ops[i].kind == TOP_GEMV) { const Work w = phase_work(c_ops[i].ph, cta, ncta); t0 = w.t0; nt = w.nt; items = w.items; }
            tmp[3 * i] = t0; tmp[3 * i + 1] = nt; tmp[3 * i + 2] = items;
        }
        if (tid == 0) {
            init_barriers(s);
        }
        build_btab(s.btab, tid);
        __syncthreads();
        if (tid == 0) {
            int n = 0, cum = 0;
            for (int i = 0; i < ta.n_ops; ++i) {
                if (tmp[3 * i + 2] < 0) continue;
                const PhaseArgs &a = c_ops[i].ph;
                tab[n].cum = cum; tab[n].t0 = tmp[3 * i]; tab[n].nt = tmp[3 * i + 1];
                tab[n].M = a.M; tab[n].nb = a.K >> 7; tab[n].half_tiles = a.epi == EPI_SWIGLU ? (((a.M + 15) >> 4) >> 1) : -1; tab[n].W = a.W;
                cum += tmp[3 * i + 2]; ++n;
            }
            tab[n].cum = cum;                                                    // sentinel: items per token
            LoopState *ls = loop_state();
            ls->git = 0; ls->done = 0; ls->tok = ta.first_tok; ls->step = 0; ls->i = 0;
            ls->total = unsigned(cum); ls->limit = unsigned(cum) * unsigned(ta.n_steps);
            for (int w = 0; w < 16; ++w) { ls->fbase[w] = 0; ls->fhint[w] = 0; }
        }
        __syncthreads();
        if (tid < 32) { TokFeed feed; for (uint32_t G = 0; G < uint32_t(STAGES); ++G) feed(G); }      // prime the ring
    }
    for (;;) {
        unsigned char *smem = dyn_smem();
        const Smem s = carve(smem);
        LoopState *ls = loop_state();
        const int step = ls->step;
        if (step >= ta.n_steps) break;
        const int cta = blockIdx.x, ncta = gridDim.x, tid = threadIdx.x;
        const GridBar bar{ta.bar, unsigned(ncta), ta.err};
        const int i = ls->i, pos = ta.pos0 + step;
        if (i == 0 && ta.embd) embed_phase(ta, s, min(max(ls->tok, 0), ta.vocab - 1));
        unsigned long long *stamps = (ta.stamps && step == 0 && cta == 0 && tid == 0) ? ta.stamps : nullptr;
        if (stamps) stamps[i * 8 + 0] = gtime();
        const int kind = c_ops[i].kind;
        unsigned items = 0;
        if (kind == TOP_GEMV) {
            // the phase's record and its tile assignment go to shared memory at a fixed address: the main loop re-reads what
            // it needs where it needs it with one immediate-address load instead of holding it in registers
            OpShared *os = reinterpret_cast<OpShared *>(smem + SL::op);
            if (tid < int(sizeof(PhaseArgs) / 4)) reinterpret_cast<uint32_t *>(&os->a)[tid] = reinterpret_cast<const uint32_t *>(&c_ops[i].ph)[tid];
            if (tid == 32) os->w = phase_work(c_ops[i].ph, cta, ncta);
            csync();
            const PhaseArgs &a = os->a;
            const Work &w = os->w;
            {
                Preload pl;
                preload(a, tid, pl);
                if (c_ops[i].wait) grid_wait(bar);
                if (stamps) stamps[i * 8 + 1] = gtime();
                prologue<true>(a, s, pl, cta);
                if (stamps) { stamps[i * 8 + 2] = gtime(); stamps[i * 8 + 6] = stamps[i * 8 + 2]; }
            }
            TokFeed feed;
            main_loop<-1>(a, w, s, ls->git, cta, feed);
            items = unsigned(w.items);
        } else if (kind == TOP_GDN) {
            gdn_phase(c_ops[i].gdn, s, bar, c_ops[i].wait != 0, cta, ncta, pos);
        } else {
            if (c_ops[i].wait) grid_wait(bar);
            if (kind == TOP_ATTN_PREP) attn_prep_phase(c_ops[i].at, s, cta, ncta, pos);
            else if (kind == TOP_ATTN_SCORES) attn_scores_phase(c_ops[i].at, cta, ncta, pos);
            else if (kind == TOP_ATTN_EXPSUM) attn_expsum_phase(c_ops[i].at, s, cta, ncta, pos);
            else if (kind == TOP_ATTN_PV) attn_pv_phase(c_ops[i].at, s, cta, ncta, pos);
            else attn_combine_phase(c_ops[i].at, cta, ncta, pos);
        }
        if (ta.stamps && step == 0 && cta == 0 && tid == 0) ta.stamps[i * 8 + 7] = gtime();
        grid_arrive(bar, items);                      // also advances the phase counter
        if (ta.stamps && step == 0 && cta == 0 && tid == 0) ta.stamps[i * 8 + 5] = gtime();
        if (ls->i == ta.n_ops) {                      // end of the token
            if (ta.pick) pick_phase(ta, bar, step, cta, ncta);
            if (tid == 0) {
                ls->i = 0; ls->step = step + 1;
                if (cta == 0 && ta.pos_out) ta.pos_out[0] = pos;
            }
            csync();
        }
    }
}

const void *g_ops_owner = nullptr;

}  // namespace

namespace bnk {

size_t token_smem_bytes(int hat_block) { return size_t(phase::smem_bytes(hat_block)); }

bool token_supported(int sm_count, int hat_block, int hidden) {
    (void)sm_count;
    // non-projection phases carve their working set out of the projection's operand area
    const size_t scratch = token_smem_bytes(hat_block) - size_t(phase::SL::scratch) - 128;
    const size_t gdn = size_t(hidden) * 4 + (128 + 128 + 32 + 8) * 4;
    const size_t pv = (4 * 512 + 4) * 4 + 2 * 32 * 16 * 16 + 2 * 32 * 8 * 2 + 4 * 512 * 4;
    return gdn <= scratch && pv <= scratch && hat_block <= 4096;
}

cudaError_t token_upload_ops(cudaStream_t st, const TokOp *ops, int n_ops, const void *owner) {
    if (g_ops_owner == owner) return cudaSuccess;
    if (n_ops > TOKEN_MAX_OPS) return cudaErrorInvalidValue;
    cudaError_t e = cudaMemcpyToSymbolAsync(c_ops, ops, size_t(n_ops) * sizeof(TokOp), 0, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) g_ops_owner = owner;
    return e;
}

cudaError_t launch_token(cudaStream_t st, int sm_count, const TokenArgs &a) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(k_token, cudaFuncAttributeMaxDynamicSharedMemorySize, int(token_smem_bytes(4096)));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count);
    cfg.blockDim = dim3(phase::NT);
    cfg.dynamicSmemBytes = token_smem_bytes(a.hat_block);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once (or the launch is refused): the barriers need it
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    BN_COUNT(1);
    return cudaLaunchKernelEx(&cfg, k_token, a);
}

}  // namespace bnk
