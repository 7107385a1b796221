// quant.cuh - q8_1 quantisation of 128 activations and the tensor-core operand table built from it.
#pragma once
#include "ops.cuh"

namespace bnk {

__device__ __forceinline__ int elem_of(int byte, int t) {
    return byte < 16 ? 16 * t + byte : (byte < 24 ? 80 + 8 * t + (byte - 16) : 120 + 2 * t + (byte - 24));
}

// Which two weight bytes feed A-register L (0..15) of a lane with thread-in-group `tig`, and at
// which trit level. Registers 0..14 are three byte pairs x five levels; register 15 is the qh pair
// at level tig. Byte pairs: (first dword low/high byte lanes, one half of a shared second dword).
__device__ __forceinline__ void areg_bytes(int tig, int L, int &byteA, int &byteB, int &t) {
    const int first = (tig == 0) ? 0 : (tig == 1) ? 2 : (tig == 2) ? 3 : 5;
    const int second = tig < 2 ? 1 : 4;
    if (L == 15) { byteA = 24; byteB = 25; t = tig; return; }
    const int hd = L / 5;
    t = L - 5 * hd;
    if (hd == 0)      { byteA = 4 * first;     byteB = 4 * first + 2; }
    else if (hd == 1) { byteA = 4 * first + 1; byteB = 4 * first + 3; }
    else              { byteA = 4 * second + (tig & 1); byteB = 4 * second + 2 + (tig & 1); }
}

// Column pair of sub-block sb: I_sb = D[2sb] - 3*D[2sb+1]. T(byte, t) enters D[2sb] with the activation
// of its own element (level t) and D[2sb+1] with the activation of the next level's element, each only
// when that element lies in sub-block sb: sum_t trit_t*y_t = sum_t T_t*y_t - 3*sum_t T_t*y_(t+1).
__device__ __forceinline__ int coef(const int8_t *q, int byte, int t, int sb, int part) {
    const int tmax = byte < 24 ? 4 : 3;
    const int tt = t + part;
    if (tt > tmax) return 0;
    const int e = elem_of(byte, tt);
    return ((e >> 5) == sb) ? int(q[e]) : 0;
}

// 128 threads cooperate on one 128-activation block: thread i owns value v (element i). q8_1
// quantisation (recipe of runtime_vk/shaders/attn_norm_rope2.comp:39-49 per 32-element block,
// s = d*sum(q) as in _mul_mat_vecq_ptq1_0.comp:8) into blk[36], then the operand table into table[512].
// qs: 128 bytes of shared memory private to this group of 128 threads. `bar_id`: named barrier (1..15)
// shared by exactly these 128 threads.
__device__ __forceinline__ void quant_block_128(float v, int i, int8_t *qs, uint32_t *__restrict__ blk,
                                                uint32_t *__restrict__ table, int bar_id) {
    const int lane = i & 31, sb = i >> 5;
    float amax = fabsf(v);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, s));
    const float d = amax > 1e-35f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    float r = roundf(__fmul_rn(v, id));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    const int qi = int(r);
    int sum = qi;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, s);
    qs[i] = int8_t(qi);
    if (lane == 0) blk[sb] = float_to_half_bits(d) | (float_to_half_bits(__fmul_rn(d, float(sum))) << 16);
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (i < 32) blk[4 + i] = reinterpret_cast<const uint32_t *>(qs)[i];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int w = i + 128 * k;                 // word index: ((m*32 + lane)*2 + j)
        const int j = w & 1, ln = (w >> 1) & 31, m = w >> 6;
        const int g = ln >> 2, tig = ln & 3;
        int byteA, byteB, t;
        areg_bytes(tig, 2 * m + j, byteA, byteB, t);
        const int csb = g >> 1, part = g & 1;
        const uint32_t zA = uint32_t(coef(qs, byteA, t, csb, part)) & 0xFFu;
        const uint32_t zB = uint32_t(coef(qs, byteB, t, csb, part)) & 0xFFu;
        table[w] = (zA << 8) | (zB << 24);
    }
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");   // qs may be reused by the caller
}

}  // namespace bnk
