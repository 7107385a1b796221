// bonsai_oracle.h - CPU restatement of the bonsai-vk decode hot path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test-suite, the smoke check and the
// benchmark's cpu_baseline / reference legs may compile, link or call anything in this directory.
// The CUDA library never includes this header and has no CPU fallback.
//
// Every function names the reference file:line whose arithmetic it restates (paths relative to the
// reference tree). The file is written from the reference's documented behaviour; no reference
// source text is reproduced. Where the reference leaves an order of floating-point operations to a
// work-group size or to a GLSL built-in of unspecified precision, the choice made here is stated
// next to the function, and the CUDA kernels follow the same choice so that both sides round alike:
//   * transcendentals (exp, log, sin, cos, pow) are evaluated in double and rounded once to float;
//   * sums over "256 lane partials" use a fixed pairwise tree instead of a serial walk;
//   * no fused multiply-add unless written as fmaf() (build with -ffp-contract=off).
//
// Parity status of the pieces:
//   PTQ1_0 decode, element map, fp16 conversions ..... pinned (reference CPU code + synth matrix)
//   q8_0 / q8_1 quantiser rounding .................... parity unpinned (the llama.cpp-fork
//       quantize_q8_1 shader is not in the reference tree; the recipe is the one the reference
//       documents for its own q8_0 V cache, runtime_vk/shaders/attn_norm_rope2.comp:39-49)
//   integer block dots ................................ pinned against the definition sum(trit*q)
//       and against a lane-level restatement of _mul_mat_vecq_ptq1_0.comp
//   FWHT, norms, GDN, attention ....................... restated from shader text (GLSL is not
//       compilable here); attention cross-checked against the reference's attn_vk.h CPU mirror.
#ifndef BONSAI_ORACLE_H
#define BONSAI_ORACLE_H

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace bo {

// ---------------------------------------------------------------------------------------------
// PTQ1_0 block format (runtime_vk/ptq_decode.h:8-19): 28 bytes = 128 ternary weights + fp16 scale.
static const int PTQ_BLOCK_BYTES = 28;
static const int PTQ_BLOCK_ELEMS = 128;

// runtime_vk/ptq_decode.h:34-38 - trit t of byte b by the *3 mod 256 recurrence, value in {0,1,2}.
static inline int trit_of_byte(uint32_t b, int t) {
    uint32_t v = b & 0xFFu;
    for (int i = 0; i < t; ++i) v = (v * 3u) & 0xFFu;
    return int((v * 3u) >> 8);
}

// runtime_vk/align_27b.cpp:56-75 - closed form of the same digit: floor(b*3^(t+1)/256) mod 3.
static inline int trit_closed_form(uint32_t b, int t) {
    uint32_t p = 3u;
    for (int i = 0; i < t; ++i) p *= 3u;
    return int(((b & 0xFFu) * p >> 8) % 3u);
}

// runtime_vk/ptq_decode.h:41-45 - element index -> (byte within the block, trit level).
static inline void elem_to_byte_trit(int e, int &byte, int &trit) {
    if (e < 80)       { byte = e & 15;              trit = e >> 4; }
    else if (e < 120) { byte = 16 + ((e - 80) & 7); trit = (e - 80) >> 3; }
    else              { byte = 24 + ((e - 120) & 1); trit = (e - 120) >> 1; }
}

// runtime_vk/ptq_decode.h:47-76 - binary16 -> binary32. Subnormals are man * 2^-24 exactly, NaN
// keeps its payload (mantissa shifted left by 13, not replaced by a canonical NaN).
static inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    const uint32_t ex = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (ex == 0) {
        if (man == 0) bits = sign;
        else {
            // man * 2^-24: normalise into a binary32 normal number, exactly.
            int sh = 0; uint32_t m = man;
            while (!(m & 0x400u)) { m <<= 1; ++sh; }
            bits = sign | (uint32_t(113 - sh) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (ex == 0x1F) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((ex + 112u) << 23) | (man << 13);
    float f; std::memcpy(&f, &bits, 4); return f;
}

// runtime_vk/f16_rne_host.h:27-55 - binary32 -> binary16, round to nearest even, overflow to Inf,
// binary32 subnormals flush to signed zero, NaN -> quiet NaN 0x7E00|sign.
static inline uint16_t f32_to_f16(float f) {
    uint32_t x; std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int e = int((x >> 23) & 0xFFu);
    const uint32_t m = x & 0x7FFFFFu;
    if (e == 0xFF) return uint16_t(sign | 0x7C00u | (m ? 0x0200u : 0u));
    if (e > 142) return uint16_t(sign | 0x7C00u);
    if (e >= 113) {
        uint32_t h = sign | (uint32_t(e - 112) << 10) | (m >> 13);
        const uint32_t rest = m & 0x1FFFu;
        if (rest > 0x1000u || (rest == 0x1000u && (h & 1u))) ++h;
        return uint16_t(h);
    }
    if (e == 0) return uint16_t(sign);
    const uint32_t shift = uint32_t(126 - e);
    if (shift >= 25) return uint16_t(sign);
    const uint32_t mant = m | 0x800000u;
    const uint32_t half = 1u << (shift - 1), rest = mant & ((1u << shift) - 1u);
    uint32_t k = mant >> shift;
    if (rest > half || (rest == half && (k & 1u))) ++k;
    return uint16_t(sign | k);
}

static inline float ptq_scale(const uint8_t *pb) {   // runtime_vk/ptq_decode.h:79-81
    return f16_to_f32(uint16_t(pb[26] | (uint16_t(pb[27]) << 8)));
}

// runtime_vk/ptq_decode.h:86-92 - w[e] = (trit - 1) * d for the 128 elements of one block.
static inline void ptq_dequant_block(const uint8_t *pb, float *w) {
    const float d = ptq_scale(pb);
    for (int e = 0; e < PTQ_BLOCK_ELEMS; ++e) {
        int by, tr; elem_to_byte_trit(e, by, tr);
        w[e] = (float(trit_of_byte(pb[by], tr)) - 1.0f) * d;
    }
}

// raw symbols {0,1,2} of a block in element order
static inline void ptq_trits_block(const uint8_t *pb, int8_t *t) {
    for (int e = 0; e < PTQ_BLOCK_ELEMS; ++e) {
        int by, tr; elem_to_byte_trit(e, by, tr);
        t[e] = int8_t(trit_of_byte(pb[by], tr));
    }
}

// Encoder. The reference ships no encoder (weights arrive packed in the GGUF); this is the inverse
// of trit_of_byte: n = sum_t trit_t * 3^(T-1-t), byte = ceil(n * 256 / 3^T), T = 5 for the 24 qs
// bytes and 4 for the 2 qh bytes. Checked exhaustively against trit_of_byte by the tests.
static inline void ptq_encode_block(const int8_t *sym /*128 values in {0,1,2}*/, uint16_t scale_bits,
                                    uint8_t *pb) {
    for (int by = 0; by < 26; ++by) {
        const int T = by < 24 ? 5 : 4;
        uint32_t n = 0, p = 1;
        for (int t = 0; t < T; ++t) {
            int e;
            if (by < 16)      e = 16 * t + by;
            else if (by < 24) e = 80 + 8 * t + (by - 16);
            else              e = 120 + 2 * t + (by - 24);
            n = n * 3u + uint32_t(sym[e]);
            p *= 3u;
        }
        pb[by] = uint8_t((n * 256u + p - 1u) / p);
    }
    pb[26] = uint8_t(scale_bits & 0xFF);
    pb[27] = uint8_t(scale_bits >> 8);
}

// ---------------------------------------------------------------------------------------------
// q8_0 / q8_1 quantiser. Recipe (runtime_vk/shaders/attn_norm_rope2.comp:39-49,184-217):
//   amax over the 32-element block; d = amax > 1e-35 ? amax / 127 : 0; id = d != 0 ? 1/d : 0;
//   q = clamp(round(x * id), -127, 127) with round() = half away from zero; d stored as fp16 RNE.
// q8_1 adds s = fp16_rne(d * sum(q)) with the fp32 d (_mul_mat_vecq_ptq1_0.comp:8).
static inline float q8_scale(float amax) { return amax > 1e-35f ? amax / 127.0f : 0.0f; }
static inline int q8_code(float x, float id) {
    float r = std::round(x * id);
    if (r > 127.0f) r = 127.0f;
    if (r < -127.0f) r = -127.0f;
    return int(r);
}

// block_q8_1_x4 (_mul_mat_vecq_ptq1_0.comp:27-28): 36 dwords per 128 activations; dwords 0..3 hold
// (fp16 d | fp16 s << 16) of sub-blocks 0..3, dwords 4..35 the 128 int8 codes in element order.
static const int Q81_X4_DWORDS = 36;
static inline void quantize_q8_1_x4(const float *x, int K, uint32_t *out) {
    for (int b = 0; b < K / 128; ++b) {
        uint32_t *o = out + size_t(b) * Q81_X4_DWORDS;
        int8_t *q = reinterpret_cast<int8_t *>(o + 4);
        for (int sb = 0; sb < 4; ++sb) {
            const float *xs = x + b * 128 + sb * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) { const float a = std::fabs(xs[i]); if (a > amax) amax = a; }
            const float d = q8_scale(amax);
            const float id = d != 0.0f ? 1.0f / d : 0.0f;
            int sum = 0;
            for (int i = 0; i < 32; ++i) { const int c = q8_code(xs[i], id); q[sb * 32 + i] = int8_t(c); sum += c; }
            o[sb] = uint32_t(f32_to_f16(d)) | (uint32_t(f32_to_f16(d * float(sum))) << 16);
        }
    }
}

// q8_0 row quantiser (32-element blocks): codes[n] int8 and scales[n/32] fp16 bits.
static inline void quantize_q8_0(const float *x, int n, int8_t *codes, uint16_t *scales) {
    for (int b = 0; b < n / 32; ++b) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) { const float a = std::fabs(x[b * 32 + i]); if (a > amax) amax = a; }
        const float d = q8_scale(amax);
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        for (int i = 0; i < 32; ++i) codes[b * 32 + i] = int8_t(q8_code(x[b * 32 + i], id));
        scales[b] = f32_to_f16(d);
    }
}

// ---------------------------------------------------------------------------------------------
// Integer block dots I_sb = sum_{e in sub-block sb} trit_e * q_e  (trit in {0,1,2}, q int8):
// the lane-independent quantity of _mul_mat_vecq_ptq1_0.comp:92-202 (its accA/accB registers are
// lane-partial sums of exactly these four numbers).
static inline void block_dots_def(const uint8_t *pb, const uint32_t *xq, int32_t I[4]) {
    const int8_t *q = reinterpret_cast<const int8_t *>(xq + 4);
    I[0] = I[1] = I[2] = I[3] = 0;
    for (int e = 0; e < 128; ++e) {
        int by, tr; elem_to_byte_trit(e, by, tr);
        I[e >> 5] += trit_of_byte(pb[by], tr) * int(q[e]);
    }
}

// The same four numbers through a 256-entry table of each byte's five trits (built once from trit_of_byte):
// the whole-token checker at the 9B shape evaluates 62 million row-blocks per token, which the per-element
// walk above is too slow for. Integer arithmetic, so equality with block_dots_def is exact; the tests compare
// the two on random and on edge-case blocks.
struct TritTable {
    int8_t t[256][8];
    TritTable() { for (int b = 0; b < 256; ++b) for (int l = 0; l < 8; ++l) t[b][l] = l < 5 ? int8_t(trit_of_byte(uint32_t(b), l)) : 0; }
};
static inline const TritTable &trit_table() { static const TritTable tt; return tt; }
static inline void block_trits_fast(const uint8_t *pb, int8_t *sym /*128, element order*/) {
    const TritTable &tt = trit_table();
    for (int by = 0; by < 16; ++by) { const int8_t *r = tt.t[pb[by]]; for (int l = 0; l < 5; ++l) sym[16 * l + by] = r[l]; }
    for (int by = 16; by < 24; ++by) { const int8_t *r = tt.t[pb[by]]; for (int l = 0; l < 5; ++l) sym[80 + 8 * l + (by - 16)] = r[l]; }
    for (int by = 24; by < 26; ++by) { const int8_t *r = tt.t[pb[by]]; for (int l = 0; l < 4; ++l) sym[120 + 2 * l + (by - 24)] = r[l]; }
}
static inline void block_dots_fast(const uint8_t *pb, const uint32_t *xq, int32_t I[4]) {
    const int8_t *q = reinterpret_cast<const int8_t *>(xq + 4);
    int8_t sym[128];
    block_trits_fast(pb, sym);
    for (int sb = 0; sb < 4; ++sb) {
        int32_t acc = 0;
        for (int i = 0; i < 32; ++i) acc += int32_t(sym[sb * 32 + i]) * int32_t(q[sb * 32 + i]);
        I[sb] = acc;
    }
}

// The same four numbers computed the way the shader's two lanes do (16-bit-lane multiply by 3,
// residue left in place and cancelled by pre-masked activations, packed 4x8 dot products):
// _mul_mat_vecq_ptq1_0.comp:66-82 (TRIT_LEVEL), :99-186 (single-column path). Returned per lane
// as (accA0..2, accB0..2); the caller folds them into sub-block sums.
static inline int32_t dot4(uint32_t a, uint32_t b, int32_t acc) {
    for (int i = 0; i < 4; ++i) acc += int32_t(int8_t(a >> (8 * i))) * int32_t(int8_t(b >> (8 * i)));
    return acc;
}
static inline void block_dots_shader_lanes(const uint8_t *pb, const uint32_t *xq, int32_t I[4]) {
    uint32_t w[7];
    std::memcpy(w, pb, 28);
    const uint32_t *y = xq + 4;   // 32 dwords of int8x4
    I[0] = I[1] = I[2] = I[3] = 0;
    for (uint32_t sub = 0; sub < 2; ++sub) {
        int32_t accA[3] = {0, 0, 0}, accB[3] = {0, 0, 0};
        uint32_t vl[3], vh[3];
        for (int k = 0; k < 3; ++k) {
            const uint32_t wk = w[3 * sub + k];
            vl[k] = wk & 0x00FF00FFu;
            vh[k] = (wk >> 8) & 0x00FF00FFu;
        }
        for (uint32_t t = 0; t < 5; ++t) {
            uint32_t yk[3];
            // lane 0: dwords 4t..4t+2 ; lane 1: dword 4t+3 and dwords 20+2t, 21+2t
            yk[0] = y[4 * t + 3 * sub];
            yk[1] = sub ? y[20 + 2 * t] : y[4 * t + 1];
            yk[2] = sub ? y[21 + 2 * t] : y[4 * t + 2];
            for (int k = 0; k < 3; ++k) {
                const uint32_t yh = yk[k] & 0xFF00FF00u, yl = (yk[k] << 8) & 0xFF00FF00u;
                const uint32_t wl = vl[k] * 3u, wh = vh[k] * 3u;
                vl[k] = wl & 0x00FF00FFu; vh[k] = wh & 0x00FF00FFu;
                int32_t &acc = (k == 0) ? accA[t >> 1] : accB[t >> 1];
                acc = dot4(wl, yl, acc);
                acc = dot4(wh, yh, acc);
            }
        }
        if (sub) {   // qh: elements 120..127, trit levels 0..3 of bytes 24, 25
            uint32_t vq = (w[6] & 0xFFu) | ((w[6] & 0xFF00u) << 8);
            uint32_t q01 = 0, q23 = 0, wq;
            wq = vq * 3u; vq = wq & 0x00FF00FFu; q01 = ((wq >> 8) & 0x3u) | ((wq >> 16) & 0x300u);
            wq = vq * 3u; vq = wq & 0x00FF00FFu; q01 |= ((wq << 8) & 0x30000u) | (wq & 0x03000000u);
            wq = vq * 3u; vq = wq & 0x00FF00FFu; q23 = ((wq >> 8) & 0x3u) | ((wq >> 16) & 0x300u);
            wq = vq * 3u;                         q23 |= ((wq << 8) & 0x30000u) | (wq & 0x03000000u);
            accB[2] = dot4(q01, y[30], accB[2]);
            accB[2] = dot4(q23, y[31], accB[2]);
        }
        // accA[i] is sub-block i on both lanes; accB[i] is sub-block i on lane 0 and 2,3,3 on lane 1
        static const int mapB[2][3] = {{0, 1, 2}, {2, 3, 3}};
        for (int i = 0; i < 3; ++i) { I[i] += accA[i]; I[mapB[sub][i]] += accB[i]; }
    }
}

// ---------------------------------------------------------------------------------------------
// q8_1 GEMV, fp32 result. Per 128-block the shader evaluates d_w * (sum_sb d_sb*I_sb - sum_sb s_sb)
// (_mul_mat_vecq_ptq1_0.comp:188-196); the order in which blocks are added is a property of its
// work-group size. The order fixed here (and used by the CUDA kernels):
//   t_sb  = fmaf(d_sb, float(I_sb), -s_sb)                       sb = 0..3
//   v_b   = d_w[b] * ((t_0 + t_1) + (t_2 + t_3))                 per 128-block b
//   p_g   = (v_{4g} + v_{4g+1}) + (v_{4g+2} + v_{4g+3})          per group of 4 blocks (512 weights)
//   out   = p_0 + p_1 + ... ascending (left to right)
// When K/128 is not a multiple of 4 the last group is padded with v = +0.
// exact[] (optional) receives the same formula evaluated in double: the reference value for the
// "within 1e-5 relative" check.
#if defined(__x86_64__) && defined(__GNUC__)
__attribute__((target_clones("avx2", "default")))     // same C code, vectorised where the host has AVX2 (integer work: exact)
#endif
static void gemv_q81(const uint8_t *W, int M, int K, const uint32_t *xq, float *out,
                            double *exact, int32_t *dots /* [M][K/128][4] or null */) {
    const int nb = K / 128;
    std::vector<float> dsb(size_t(nb) * 4), ssb(size_t(nb) * 4);
    for (int b = 0; b < nb; ++b)
        for (int sb = 0; sb < 4; ++sb) {
            const uint32_t ds = xq[size_t(b) * Q81_X4_DWORDS + sb];
            dsb[b * 4 + sb] = f16_to_f32(uint16_t(ds & 0xFFFF));
            ssb[b * 4 + sb] = f16_to_f32(uint16_t(ds >> 16));
        }
    for (int r = 0; r < M; ++r) {
        float acc = 0.0f, v4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        double ex = 0.0;
        for (int b = 0; b < nb; ++b) {
            const uint8_t *pb = W + (size_t(r) * nb + b) * PTQ_BLOCK_BYTES;
            int32_t I[4];
            block_dots_fast(pb, xq + size_t(b) * Q81_X4_DWORDS, I);     // == block_dots_def (tested)
            if (dots) std::memcpy(dots + (size_t(r) * nb + b) * 4, I, 16);
            float t[4]; double te = 0.0;
            for (int sb = 0; sb < 4; ++sb) {
                t[sb] = std::fmaf(dsb[b * 4 + sb], float(I[sb]), -ssb[b * 4 + sb]);
                te += double(dsb[b * 4 + sb]) * double(I[sb]) - double(ssb[b * 4 + sb]);
            }
            const float dw = ptq_scale(pb);
            v4[b & 3] = dw * ((t[0] + t[1]) + (t[2] + t[3]));
            ex += double(dw) * te;
            if ((b & 3) == 3 || b == nb - 1) {
                const float p = (v4[0] + v4[1]) + (v4[2] + v4[3]);
                acc = (b < 4) ? p : acc + p;
                v4[0] = v4[1] = v4[2] = v4[3] = 0.0f;
            }
        }
        out[r] = acc;
        if (exact) exact[r] = ex;
    }
}

// fp32-activation GEMV, the engine's own arithmetic (runtime_vk/shaders/gemv_ternary.comp:74-118,
// xsum.comp, reduce.comp): out = sum_b d_b * (sum_k c_k x_k - xsum_b), c in {0,1,2}; within a
// 64-code half block four strided accumulators combined as (s0+s1)+(s2+s3); blocks ascending inside
// a split, split partials added ascending. The reference walks a repacked 2-bit layout whose code
// order inside a 64-code word is the element order, so element order is used here.
static inline void gemv_f32act(const uint8_t *W, int M, int K, const float *x, int n_splits,
                               float *out, double *exact) {
    const int nb = K / 128;
    std::vector<float> xsum(nb);
    for (int b = 0; b < nb; ++b) {   // xsum.comp: per lane (v.x+v.y)+(v.z+v.w), then a 32-lane tree
        float part[32];
        for (int l = 0; l < 32; ++l) {
            const float *v = x + b * 128 + l * 4;
            part[l] = (v[0] + v[1]) + (v[2] + v[3]);
        }
        for (int s = 16; s > 0; s >>= 1) for (int l = 0; l < s; ++l) part[l] += part[l + s];
        xsum[b] = part[0];
    }
    const int per = nb / n_splits;
    int8_t sym[128];
    for (int r = 0; r < M; ++r) {
        float total = 0.0f; double ex = 0.0;
        for (int s = 0; s < n_splits; ++s) {
            float acc = 0.0f;
            for (int b = s * per; b < (s + 1) * per; ++b) {
                const uint8_t *pb = W + (size_t(r) * nb + b) * PTQ_BLOCK_BYTES;
                ptq_trits_block(pb, sym);
                float cp = 0.0f; double cs = 0.0, xs = 0.0;
                for (int h = 0; h < 2; ++h) {
                    float a[4] = {0, 0, 0, 0};
                    for (int i = 0; i < 64; ++i) {
                        const int e = h * 64 + i;
                        a[i & 3] = std::fmaf(float(sym[e]), x[b * 128 + e], a[i & 3]);
                    }
                    const float hp = (a[0] + a[1]) + (a[2] + a[3]);
                    cp = h == 0 ? hp : cp + hp;
                }
                for (int e = 0; e < 128; ++e) { cs += double(sym[e]) * double(x[b * 128 + e]); xs += double(x[b * 128 + e]); }
                const float d = ptq_scale(pb);
                acc = std::fmaf(d, cp - xsum[b], acc);
                ex += double(d) * (cs - xs);
            }
            total = s == 0 ? acc : total + acc;
        }
        out[r] = total;
        if (exact) exact[r] = ex;
    }
}

// The reference's GEMV truth (runtime_vk/bonsai_weights.h:751-768, bonsai_vk.cpp:752-772):
// dequantise each block, accumulate w*x in double. This is the timed CPU baseline as well.
static inline void gemv_dequant_f64(const uint8_t *W, int M, int K, const float *x, double *out) {
    const int nb = K / 128;
    float w[128];
    for (int r = 0; r < M; ++r) {
        double acc = 0.0;
        for (int b = 0; b < nb; ++b) {
            ptq_dequant_block(W + (size_t(r) * nb + b) * PTQ_BLOCK_BYTES, w);
            for (int k = 0; k < 128; ++k) acc += double(w[k]) * double(x[b * 128 + k]);
        }
        out[r] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Hadamard rotation. runtime_vk/shaders/hat4096.comp:41-60: radix-2 butterflies, h = 1,2,...,N/2
// ascending, pair (j, j+h) -> (a+c, a-c), then every element times 1/sqrt(N) (exactly 1/64 at
// N = 4096). hadamard_fwht.comp is the same network for N = 16..4096 with a host-supplied factor.
static inline void fwht_block(float *s, int N, float inv_sqrt_n) {
    for (int h = 1; h < N; h <<= 1)
        for (int i = 0; i < N / 2; ++i) {
            const int j = ((i & ~(h - 1)) << 1) | (i & (h - 1));
            const float a = s[j], c = s[j + h];
            s[j] = a + c; s[j + h] = a - c;
        }
    for (int i = 0; i < N; ++i) s[i] *= inv_sqrt_n;
}
// forward rotation before a projection: y = H (s . x)  (bonsai_forward.h:471-476, signs_mul.comp)
static inline void rotate_fwd(const float *x, const int32_t *signs, int n, int block, float *y) {
    for (int i = 0; i < n; ++i) y[i] = x[i] * float(signs[i]);
    const float inv = 1.0f / std::sqrt(float(block));
    for (int b = 0; b < n / block; ++b) fwht_block(y + b * block, block, inv);
}
// embedding side: y = s . (H x)  (bonsai_forward.h:689-691)
static inline void rotate_inv(const float *x, const int32_t *signs, int n, int block, float *y) {
    for (int i = 0; i < n; ++i) y[i] = x[i];
    const float inv = 1.0f / std::sqrt(float(block));
    for (int b = 0; b < n / block; ++b) fwht_block(y + b * block, block, inv);
    for (int i = 0; i < n; ++i) y[i] = y[i] * float(signs[i]);
}

// ---------------------------------------------------------------------------------------------
// transcendental policy: double evaluation, one rounding to float.
static inline float exp_f(float x)  { return float(std::exp(double(x))); }
static inline float log_f(float x)  { return float(std::log(double(x))); }
static inline float sigmoid_f(float x) { return 1.0f / (1.0f + exp_f(-x)); }     // sigmoid.comp
static inline float silu_f(float x)    { return x / (1.0f + exp_f(-x)); }        // swiglu.comp silu1
static inline float softplus_f(float x, float thr) {                            // softplus.comp mode 0
    return x > thr ? x : log_f(1.0f + exp_f(x));
}

// pairwise tree over n = 2^k partials: p[i] += p[i + s] for s = n/2 .. 1 (fixed order).
static inline float tree_sum(float *p, int n) {
    for (int s = n / 2; s > 0; s >>= 1) for (int i = 0; i < s; ++i) p[i] += p[i + s];
    return p[0];
}

// RMS norm (runtime_vk/shaders/rms_norm.comp:60-103): squares materialised (no FMA into the sum),
// 256 lane slices of per = ceil(n/256) consecutive elements summed ascending, slices combined
// (reference: serially; here: the fixed tree above), inv = 1/sqrt(ss/n + eps), y = (x*inv)*w.
static inline void rms_norm(const float *x, const float *w, int n, float eps, float *y) {
    float part[256];
    const int per = (n + 255) / 256;
    for (int l = 0; l < 256; ++l) {
        float s = 0.0f;
        for (int i = 0; i < per; ++i) { const int d = l * per + i; if (d < n) { const float q = x[d] * x[d]; s = s + q; } }
        part[l] = s;
    }
    const float ss = tree_sum(part, 256);
    const float inv = 1.0f / std::sqrt(ss / float(n) + eps);
    for (int d = 0; d < n; ++d) { const float v = x[d] * inv; y[d] = w ? v * w[d] : v; }
}

// L2 norm, mode 1 (runtime_vk/shaders/l2_norm.comp:59-78): y = x * (1/sqrt(ss + eps)); the
// reference sums the 128 squares serially, here the fixed tree.
static inline void l2_norm(const float *x, int n, float eps, float *y) {
    float sq[256] = {0};
    for (int i = 0; i < n; ++i) sq[i] = x[i] * x[i];
    const float ss = tree_sum(sq, n);
    const float inv = 1.0f / std::sqrt(ss + eps);
    for (int i = 0; i < n; ++i) y[i] = x[i] * inv;
}

}  // namespace bo
#endif
