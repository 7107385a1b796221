// gemv_f32act.cu - PTQ1_0 projection of an fp32 activation vector, the reference engine's own arithmetic
// (gemv_ptq, runtime_vk/bonsai_forward.h:409-422 -> xsum.comp, gemv_ternary.comp:74-118, reduce.comp):
//   out[r] = sum_b d[r,b] * (sum_{k in b} c_k x_k - xsum_b),  c = trit + 1 in {0, 1, 2}
// with the reference's summation shape: inside each 64-code half of a block four strided fma chains
// a[i & 3] += c_i * x_i combined as (a0 + a1) + (a2 + a3), the two halves added, blocks ascending through
// acc = fma(d, cp - xsum_b, acc), split-K partials added ascending; xsum_b = per lane (v.x + v.y) + (v.z + v.w) of
// its four values, then a 32-lane tree. This mode is multiply-bound (one fp32 fma per weight) and exists for
// parity with engines that run it; the q8_1 integer-dot kernels are the fast path.
//
// One warp per (row, split). A lane owns one of the 8 chains (half h, accumulator j) of one of 4 blocks handled
// per step; lanes 0, 8, 16, 24 end up with the blocks' cp values and lane 0 applies them in block order.
#include "ops.cuh"

namespace {

__global__ void __launch_bounds__(256) k_xsum(const float *__restrict__ x, int nb, float *__restrict__ xsum) {
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (b >= nb) return;
    const float4 v = *reinterpret_cast<const float4 *>(x + size_t(b) * 128 + lane * 4);
    float p = __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float o = __shfl_down_sync(0xFFFFFFFFu, p, s);
        if (lane < s) p = __fadd_rn(p, o);
    }
    if (lane == 0) xsum[b] = p;
}

// trit + 1 of element e of a 28-byte block (5 trits per byte, v = (v*3) & 0xFF; code = (v*3) >> 8)
__device__ __forceinline__ float code_of(const uint8_t *blk, int e) {
    int byte, t;
    if (e < 80) { byte = e & 15; t = e >> 4; }
    else if (e < 120) { byte = 16 + ((e - 80) & 7); t = (e - 80) >> 3; }
    else { byte = 24 + ((e - 120) & 1); t = (e - 120) >> 1; }
    uint32_t v = blk[byte];
    for (int i = 0; i < t; ++i) v = (v * 3u) & 0xFFu;
    return float(int((v * 3u) >> 8));
}

__global__ void __launch_bounds__(256) k_gemv_f32act(const uint8_t *__restrict__ W, int M, int nb, int per,
                                                     const float *__restrict__ x, const float *__restrict__ xsum,
                                                     float *__restrict__ part) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31, split = blockIdx.y;
    if (row >= M) return;
    const int sub = lane >> 3, chain = lane & 7, h = chain >> 2, j = chain & 3;
    const uint8_t *wr = W + size_t(row) * nb * 28;
    float acc = 0.0f;
    for (int b0 = split * per; b0 < (split + 1) * per; b0 += 4) {
        const int b = b0 + sub;
        float a = 0.0f;
        if (b < (split + 1) * per) {
            const uint8_t *blk = wr + size_t(b) * 28;
            const float *xb = x + size_t(b) * 128 + h * 64;
#pragma unroll 4
            for (int k = 0; k < 16; ++k) a = fmaf(code_of(blk, h * 64 + j + 4 * k), xb[j + 4 * k], a);
        }
        // (a0 + a1) + (a2 + a3) inside each group of four lanes, then the two halves
        const float a1 = __shfl_xor_sync(0xFFFFFFFFu, a, 1);
        const float s01 = (j & 1) ? __fadd_rn(a1, a) : __fadd_rn(a, a1);
        const float s23 = __shfl_xor_sync(0xFFFFFFFFu, s01, 2);
        const float hp = (j & 2) ? __fadd_rn(s23, s01) : __fadd_rn(s01, s23);
        const float hq = __shfl_xor_sync(0xFFFFFFFFu, hp, 4);
        const float cp = h ? __fadd_rn(hq, hp) : __fadd_rn(hp, hq);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float c = __shfl_sync(0xFFFFFFFFu, cp, i * 8);
            const int bb = b0 + i;
            if (lane == 0 && bb < (split + 1) * per) {
                const uint32_t sc = uint32_t(wr[size_t(bb) * 28 + 26]) | (uint32_t(wr[size_t(bb) * 28 + 27]) << 8);
                acc = fmaf(half_bits_to_float(sc), __fsub_rn(c, xsum[bb]), acc);
            }
        }
    }
    if (lane == 0) part[size_t(split) * M + row] = acc;
}

__global__ void k_reduce_splits(const float *__restrict__ part, int M, int n_splits, float *__restrict__ out) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    float s = part[row];
    for (int g = 1; g < n_splits; ++g) s = __fadd_rn(s, part[size_t(g) * M + row]);
    out[row] = s;
}

}  // namespace

namespace bnk {
size_t gemv_f32act_scratch_floats(int M, int K, int n_splits) { return ((size_t(K / 128) + 63) & ~size_t(63)) + size_t(n_splits) * M; }
// block sums of x, the split partial dot products, then the splits added in order (the reference's two dispatches)
void gemv_f32act(cudaStream_t st, const uint8_t *W, int M, int K, const float *x, int n_splits, float *out, float *scratch) {
    const int nb = K / 128;
    const size_t xs_floats = (size_t(nb) + 63) & ~size_t(63);
    float *xsum = scratch, *part = scratch + xs_floats;
    k_xsum<<<(nb + 7) / 8, 256, 0, st>>>(x, nb, xsum);
    k_gemv_f32act<<<dim3((M + 7) / 8, n_splits), 256, 0, st>>>(W, M, nb, nb / n_splits, x, xsum, part);
    k_reduce_splits<<<(M + 255) / 256, 256, 0, st>>>(part, M, n_splits, out);
    BN_COUNT(3);
}
}  // namespace bnk

extern "C" {

// the reference's split rule (pick_splits, runtime_vk/bonsai_weights.h:581-588)
int bn_gemv_f32act_splits(int M, int K) {
    if (M <= 0 || K <= 0 || K % 128) return 0;
    const unsigned nblk = unsigned(K / 128);
    unsigned s = 1;
    while (s < 16u && (unsigned long long)(M / 64 + (M % 64 != 0)) * s < 640ull && (nblk % (s * 2u) == 0)) s *= 2u;
    return int(s);
}

int bn_gemv_f32act(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, const bn_buf *x, size_t x_off, int n_splits,
                   bn_buf *out, size_t out_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_gemv_f32act: null context");
    BN_REQUIRE(M > 0 && K > 0 && K % 128 == 0, BN_ERR_ARG, "bn_gemv_f32act: bad shape M=%d K=%d (K %% 128 != 0)", M, K);
    const int nb = K / 128;
    if (n_splits == 0) n_splits = bn_gemv_f32act_splits(M, K);
    BN_REQUIRE(n_splits >= 1 && n_splits <= 16 && nb % n_splits == 0, BN_ERR_ARG,
               "bn_gemv_f32act: %d splits must divide the %d blocks of a row (1..16)", n_splits, nb);
    BN_RANGE(w, w_off, size_t(M) * nb * 28, 4, "bn_gemv_f32act W");
    BN_RANGE(x, x_off, size_t(K) * 4, 16, "bn_gemv_f32act x");
    BN_RANGE(out, out_off, size_t(M) * 4, 4, "bn_gemv_f32act out");
    int rc = bn_scratch_reserve(ctx, bnk::gemv_f32act_scratch_floats(M, K, n_splits) * 4);
    if (rc != BN_OK) return rc;
    bnk::gemv_f32act(ctx->stream, bn_ptr<uint8_t>(w, w_off), M, K, bn_ptr<float>(x, x_off), n_splits, bn_ptr<float>(out, out_off), ctx->scratch);
    return bn_launch_check(ctx, "k_gemv_f32act");
}

}  // extern "C"
