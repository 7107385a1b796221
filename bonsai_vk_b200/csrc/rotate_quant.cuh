// rotate_quant.cuh - the pieces of "rotate, then quantise" that the single-sequence prologue (phase_body.cuh), the
// packed swiglu kernel (phase_gemv.cu) and the multi-column activation image (gemm_tc.cu) share, so that all three
// produce the same bits: the mean of a power-of-two count, the sign flip, the register / shuffle butterflies of the
// Sylvester-Walsh-Hadamard transform (reference network: runtime_vk/shaders/hat4096.comp:41-60) and the q8_1 quantiser
// of eight values (recipe: runtime_vk/shaders/attn_norm_rope2.comp:39-49).
#pragma once
#include "common.cuh"

namespace bnk {

// t / K rounded to nearest: for a power of two the product with 1/K is the same float (an exact scaling, rounded once
// when the result is subnormal, as the quotient is) and skips the division sequence. 1 / x below is __frcp_rn, the
// correctly rounded reciprocal, which is what the division 1.0f / x returns.
__device__ __forceinline__ float mean_of(float t, int K) {
    return (K & (K - 1)) == 0 ? __fmul_rn(t, __frcp_rn(float(K))) : __fdiv_rn(t, float(K));
}
// x * sign for sign = +1 / -1 (bn_model_set_signs refuses anything else): flipping the sign bit is the same float as the
// product, zeros and NaNs included, and needs no int -> float conversion
__device__ __forceinline__ float apply_sign(float x, int sg) { return __uint_as_float(__float_as_uint(x) ^ (uint32_t(sg) & 0x80000000u)); }
// butterflies h = 1, 2, 4 inside a thread's 8 consecutive elements, h = 8..128 across the lanes of a warp
__device__ __forceinline__ void fwht_regs_lanes(float (&v)[8], int lane) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (!(r & h)) { const float x = v[r], y = v[r + h]; v[r] = __fadd_rn(x, y); v[r + h] = __fsub_rn(x, y); }
    // the upper lane of a pair takes partner - own, the lower one own + partner: one fused multiply-add with +-1 (the
    // product is exact, so the result is the rounded difference / sum, bit for bit what fsub / fadd give)
#pragma unroll
    for (int m2 = 1; m2 < 32; m2 <<= 1) {
        const float sgn = (lane & m2) ? -1.0f : 1.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float pr = __shfl_xor_sync(0xFFFFFFFFu, v[r], m2);
            v[r] = __fmaf_rn(v[r], sgn, pr);
        }
    }
}
// butterflies h = 256, 512, 1024 inside a thread (elements 256 apart), h = 2048 between lanes l and l^16, then the scale;
// each thread rewrites only what it read
__device__ __forceinline__ void fwht_4096_tail(float *xs, int warp, int lane, float hat_inv) {
    const int i0 = (lane & 15) + 16 * warp + 2048 * (lane >> 4);
    float u[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) u[r] = xs[i0 + 256 * r];
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (!(r & h)) { const float x = u[r], y = u[r + h]; u[r] = __fadd_rn(x, y); u[r + h] = __fsub_rn(x, y); }
    const float sgn = (lane & 16) ? -1.0f : 1.0f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const float pr = __shfl_xor_sync(0xFFFFFFFFu, u[r], 16);
        u[r] = __fmaf_rn(u[r], sgn, pr);
        xs[i0 + 256 * r] = __fmul_rn(u[r], hat_inv);
    }
}
// q8_1 of a 32-value sub-block held by four neighbouring lanes (4k .. 4k+3), eight consecutive values each; all 32 lanes
// of the warp call it (lanes without a sub-block pass zeros). d = amax / 127 (0 below 1e-35), codes = round half away of
// x / d clamped to +-127, sum = the sub-block's code sum. The low byte of (code + 1.5 * 2^23) read as an integer is the
// code in two's complement (no float -> int conversion); four bytes are gathered with byte permutes and the sum of the
// eight codes is two byte dot products with ones.
struct Q8x8 { uint32_t w0, w1; float d; int sum; };
__device__ __forceinline__ Q8x8 quant8_of32(const float (&e)[8]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(e[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    Q8x8 r;
    r.d = amax > 1e-35f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    const float id = r.d != 0.0f ? __frcp_rn(r.d) : 0.0f;
    uint32_t q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float c = roundf(__fmul_rn(e[i], id));
        c = fminf(fmaxf(c, -127.0f), 127.0f);
        q[i] = __float_as_uint(__fadd_rn(c, 12582912.0f));
    }
    r.w0 = __byte_perm(__byte_perm(q[0], q[1], 0x0040u), __byte_perm(q[2], q[3], 0x0040u), 0x5410u);
    r.w1 = __byte_perm(__byte_perm(q[4], q[5], 0x0040u), __byte_perm(q[6], q[7], 0x0040u), 0x5410u);
    int sum = __dp4a(int(r.w0), 0x01010101, __dp4a(int(r.w1), 0x01010101, 0));
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    r.sum = sum;
    return r;
}

}  // namespace bnk
