// ptq_gemv.cu - PTQ1_0 x q8_1 matrix-vector product on tensor cores (sm_100a).
//
// Arithmetic contract (reference: _mul_mat_vecq_ptq1_0.comp:92-202): for every row and every
// 128-weight block, the four integer dots I_sb = sum_{e in sub-block sb} trit_e * q_e (trit in
// {0,1,2}, q int8) are formed exactly; then
//     t_sb = fmaf(d_sb, float(I_sb), -s_sb);  v_b = d_w[b] * ((t_0 + t_1) + (t_2 + t_3))
//     p_g  = (v_4g + v_4g+1) + (v_4g+2 + v_4g+3);  out = p_0 + p_1 + ...   (ascending)
//
// How the trits reach the tensor cores without being unpacked one by one. A weight byte b stores
// five base-3 digits as a fixed-point fraction: T_t = (b * 3^(t+1)) >> 8 is the number formed by
// digits 0..t, so trit_t = T_t - 3*T_(t-1). A dot product with the trits is therefore LINEAR in
// the T_t:  sum_t trit_t*y_t = sum_t T_t*(y_t - 3*y_(t+1)).  Two weight bytes sit in the 16-bit
// halves of a register; ONE integer multiply by 3^(t+1) (no carry between the halves, 255*243 <
// 65536) yields a register whose bytes are [r, T, r', T'] - exactly an int8 tensor-core operand
// in which the residue bytes r are multiplied by zero. The two sums sum_t T_t*y_t and
// sum_t T_t*y_(t+1), each restricted to one q8_1 sub-block, are the 8 columns of the B operand:
// column 2*sb pairs T_t with the activation of its own element, column 2*sb+1 with the activation of
// the next level's element, so I_sb = D[2sb] - 3*D[2sb+1] exactly and every B byte is a plain int8
// activation code (or zero). That table depends only on the activations and is built once per
// activation vector by k_act_quant_q81.
//
// One warp owns one 128-weight block column and walks 16-row tiles: 32 integer multiplies, 8
// byte-permutes and 8 mma.sync.m16n8k32.u8.s8 per 2048 weights.
#include "ops.cuh"
#include "phase_gemv.cuh"
#include "quant.cuh"

namespace {
using bnk::Q81_DWORDS;
using bnk::BF_WORDS;

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// the three byte-pair registers and the qh pair of one row's block, from its three dwords
struct RowRegs { uint32_t h0, h1, h2, hq; };
__device__ __forceinline__ RowRegs split_row(uint32_t first, uint32_t second, uint32_t w6, int tig) {
    RowRegs r;
    r.h0 = __byte_perm(first, 0, 0x4240);                       // bytes 0,2 -> 16-bit lanes
    r.h1 = __byte_perm(first, 0, 0x4341);                       // bytes 1,3
    r.h2 = __byte_perm(second, 0, (tig & 1) ? 0x4341 : 0x4240);
    r.hq = __byte_perm(w6, 0, 0x4140);                          // qh bytes 24, 25
    return r;
}

// 16 rows x 1 block: accumulate the 8 tensor-core steps into c (rows g and g+8 of the tile)
__device__ __forceinline__ void tile_mma(int (&c)[4], const RowRegs &ra, const RowRegs &rb, const uint2 (&B)[8],
                                         uint32_t cq) {
    mma_u8s8(c, ra.h0 * 3u,   rb.h0 * 3u,   ra.h0 * 9u,   rb.h0 * 9u,   B[0].x, B[0].y);
    mma_u8s8(c, ra.h0 * 27u,  rb.h0 * 27u,  ra.h0 * 81u,  rb.h0 * 81u,  B[1].x, B[1].y);
    mma_u8s8(c, ra.h0 * 243u, rb.h0 * 243u, ra.h1 * 3u,   rb.h1 * 3u,   B[2].x, B[2].y);
    mma_u8s8(c, ra.h1 * 9u,   rb.h1 * 9u,   ra.h1 * 27u,  rb.h1 * 27u,  B[3].x, B[3].y);
    mma_u8s8(c, ra.h1 * 81u,  rb.h1 * 81u,  ra.h1 * 243u, rb.h1 * 243u, B[4].x, B[4].y);
    mma_u8s8(c, ra.h2 * 3u,   rb.h2 * 3u,   ra.h2 * 9u,   rb.h2 * 9u,   B[5].x, B[5].y);
    mma_u8s8(c, ra.h2 * 27u,  rb.h2 * 27u,  ra.h2 * 81u,  rb.h2 * 81u,  B[6].x, B[6].y);
    mma_u8s8(c, ra.h2 * 243u, rb.h2 * 243u, ra.hq * cq,   rb.hq * cq,   B[7].x, B[7].y);
}

// First-generation kernel: CTA = 4 warps = one group of 4 blocks (512 weights) x a run of 16-row
// tiles; weights read with plain global loads. part[g][row] receives p_g.
template <bool DUMP>
__global__ void __launch_bounds__(128) k_gemv_q81_direct(const uint32_t *__restrict__ W, int M, int nb,
                                                         const uint32_t *__restrict__ q81,
                                                         const uint2 *__restrict__ bf, float *__restrict__ part,
                                                         int tiles_per_cta, int32_t *__restrict__ dots) {
    __shared__ float sv[4][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int kg = blockIdx.y, b = kg * 4 + warp;
    const bool active = b < nb;
    uint2 B[8];
    float dsb = 0.0f, ssb = 0.0f;
    if (active) {
#pragma unroll
        for (int m = 0; m < 8; ++m) B[m] = bf[(size_t(b) * 8 + m) * 32 + lane];
        const uint32_t ds = q81[size_t(b) * Q81_DWORDS + tig];
        dsb = half_bits_to_float(ds);
        ssb = half_bits_to_float(ds >> 16);
    }
    const int first = (tig == 0) ? 0 : (tig == 1) ? 2 : (tig == 2) ? 3 : 5;
    const int second = tig < 2 ? 1 : 4;
    const uint32_t cq = (tig == 0) ? 3u : (tig == 1) ? 9u : (tig == 2) ? 27u : 81u;
    const int ntiles = (M + 15) >> 4;
    const int t0 = blockIdx.x * tiles_per_cta;
    const int t1 = min(ntiles, t0 + tiles_per_cta);
    for (int tile = t0; tile < t1; ++tile) {
        float v0 = 0.0f, v1 = 0.0f;
        if (active) {
            const int row0 = tile * 16 + g, row1 = row0 + 8;
            const uint32_t *p0 = W + (size_t(min(row0, M - 1)) * nb + b) * 7;
            const uint32_t *p1 = W + (size_t(min(row1, M - 1)) * nb + b) * 7;
            const uint32_t a_first = __ldg(p0 + first), a_second = __ldg(p0 + second), a6 = __ldg(p0 + 6);
            const uint32_t b_first = __ldg(p1 + first), b_second = __ldg(p1 + second), b6 = __ldg(p1 + 6);
            const RowRegs ra = split_row(a_first, a_second, a6, tig);
            const RowRegs rb = split_row(b_first, b_second, b6, tig);
            int c[4] = {0, 0, 0, 0};
            tile_mma(c, ra, rb, B, cq);
            const int I0 = c[0] - 3 * c[1], I1 = c[2] - 3 * c[3];
            if (DUMP) {
                if (row0 < M) dots[(size_t(row0) * nb + b) * 4 + tig] = I0;
                if (row1 < M) dots[(size_t(row1) * nb + b) * 4 + tig] = I1;
            }
            float s0 = fmaf(dsb, float(I0), -ssb), s1 = fmaf(dsb, float(I1), -ssb);
            s0 = __fadd_rn(s0, __shfl_xor_sync(0xFFFFFFFFu, s0, 1));
            s1 = __fadd_rn(s1, __shfl_xor_sync(0xFFFFFFFFu, s1, 1));
            s0 = __fadd_rn(s0, __shfl_xor_sync(0xFFFFFFFFu, s0, 2));
            s1 = __fadd_rn(s1, __shfl_xor_sync(0xFFFFFFFFu, s1, 2));
            v0 = __fmul_rn(half_bits_to_float(a6 >> 16), s0);
            v1 = __fmul_rn(half_bits_to_float(b6 >> 16), s1);
        }
        if (tig == 0) { sv[warp][g] = v0; sv[warp][g + 8] = v1; }
        __syncthreads();
        if (threadIdx.x < 16) {
            const int row = tile * 16 + threadIdx.x;
            if (row < M) {
                const int i = threadIdx.x;
                part[size_t(kg) * M + row] = __fadd_rn(__fadd_rn(sv[0][i], sv[1][i]), __fadd_rn(sv[2][i], sv[3][i]));
            }
        }
        __syncthreads();
    }
}

// out[row] = part[0][row] + part[1][row] + ... ascending (reference: reduce.comp)
__global__ void k_sum_groups(const float *__restrict__ part, int M, int ngroups, float *__restrict__ out) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    float s = part[row];
    for (int g = 1; g < ngroups; ++g) s = __fadd_rn(s, part[size_t(g) * M + row]);
    out[row] = s;
}

// One CTA (128 threads) per 128 activations.
__global__ void __launch_bounds__(128) k_act_quant_q81(const float *__restrict__ x, uint32_t *__restrict__ q81,
                                                       uint32_t *__restrict__ bf) {
    __shared__ int8_t qs[128];
    const int b = blockIdx.x, i = threadIdx.x;
    bnk::quant_block_128(x[size_t(b) * 128 + i], i, qs, q81 + size_t(b) * Q81_DWORDS, bf + size_t(b) * BF_WORDS, 1);
}

}  // namespace

namespace bnk {

void act_quant_q81(cudaStream_t st, const float *x, int K, uint32_t *pack) {
    const int nb = K / 128;
    k_act_quant_q81<<<nb, 128, 0, st>>>(x, pack, pack + size_t(nb) * Q81_DWORDS);
    BN_COUNT(1);
}

void gemv_q81(cudaStream_t st, int sm_count, const uint32_t *W, int M, int K, const uint32_t *pack, float *out,
              float *scratch, int32_t *dots) {
    const int nb = K / 128, ngroups = (nb + 3) / 4;
    const uint2 *bf = reinterpret_cast<const uint2 *>(pack + size_t(nb) * Q81_DWORDS);
    const int ntiles = (M + 15) / 16;
    // enough CTAs to cover the machine a few times over, but runs of tiles long enough to
    // amortise the operand-table load
    int want_x = (sm_count * 8 + ngroups - 1) / ngroups;
    if (want_x < 1) want_x = 1;
    int tiles_per_cta = (ntiles + want_x - 1) / want_x;
    if (tiles_per_cta < 1) tiles_per_cta = 1;
    dim3 grid((ntiles + tiles_per_cta - 1) / tiles_per_cta, ngroups);
    if (dots) k_gemv_q81_direct<true><<<grid, 128, 0, st>>>(W, M, nb, pack, bf, scratch, tiles_per_cta, dots);
    else k_gemv_q81_direct<false><<<grid, 128, 0, st>>>(W, M, nb, pack, bf, scratch, tiles_per_cta, nullptr);
    k_sum_groups<<<(M + 255) / 256, 256, 0, st>>>(scratch, M, ngroups, out);
    BN_COUNT(2);
}

}  // namespace bnk

extern "C" {

size_t bn_act_pack_bytes(int K) {
    if (K <= 0 || K % 128) return 0;
    return bnk::act_pack_bytes(K);
}

int bn_act_quant_q81(bn_ctx *ctx, const bn_buf *x, size_t x_off, int K, bn_buf *pack, size_t pack_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_act_quant_q81: null context");
    BN_REQUIRE(K > 0 && K % 128 == 0, BN_ERR_ARG, "bn_act_quant_q81: K=%d must be a positive multiple of 128", K);
    BN_RANGE(x, x_off, size_t(K) * 4, 4, "bn_act_quant_q81 x");
    BN_RANGE(pack, pack_off, bn_act_pack_bytes(K), 16, "bn_act_quant_q81 pack");
    bnk::act_quant_q81(ctx->stream, bn_ptr<float>(x, x_off), K, bn_ptr<uint32_t>(pack, pack_off));
    return bn_launch_check(ctx, "k_act_quant_q81");
}

int bn_gemv_q81(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, const bn_buf *pack, size_t pack_off,
                bn_buf *out, size_t out_off, bn_buf *dots, size_t dots_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_gemv_q81: null context");
    BN_REQUIRE(M > 0 && K > 0 && K % 128 == 0, BN_ERR_ARG, "bn_gemv_q81: bad shape M=%d K=%d (K %% 128 != 0)", M, K);
    const int nb = K / 128, ngroups = (nb + 3) / 4;
    BN_RANGE(w, w_off, size_t(M) * nb * 28, 4, "bn_gemv_q81 W");
    BN_RANGE(pack, pack_off, bn_act_pack_bytes(K), 16, "bn_gemv_q81 pack");
    BN_RANGE(out, out_off, size_t(M) * 4, 4, "bn_gemv_q81 out");
    if (dots) BN_RANGE(dots, dots_off, size_t(M) * nb * 16, 4, "bn_gemv_q81 dots");
    int rc = bn_scratch_reserve(ctx, size_t(ngroups) * M * 4);
    if (rc != BN_OK) return rc;
    // the streamed kernel moves rows with bulk copies, which need a 16-byte aligned source; any other 4-byte aligned
    // placement goes through the kernel that reads with plain 4-byte loads (same results)
    const bool w16 = (reinterpret_cast<uintptr_t>(bn_ptr<uint8_t>(w, w_off)) & 15u) == 0;
    if (!dots && w16 && bnk::phase_supported(M, K, 512) && (M + 15) / 16 <= BN_MAX_TILES) {
        // streamed kernel; the op-level call hands it a ready-made activation pack
        bnk::PhaseArgs a = {};
        a.W = bn_ptr<uint8_t>(w, w_off); a.M = M; a.K = K;
        a.out = bn_ptr<float>(out, out_off);
        a.part = ctx->scratch; a.counters = ctx->counters;
        a.pro = bnk::PRO_PACKED; a.pack = bn_ptr<uint32_t>(pack, pack_off);
        a.hat_block = 512; a.err = ctx->err_dev;
        cudaError_t e = bnk::launch_phase(ctx->stream, ctx->sm_count, a, false);
        if (e != cudaSuccess) return bn_cuda_fail(e, "k_phase_gemv");
        return bn_launch_check(ctx, "k_phase_gemv");
    }
    bnk::gemv_q81(ctx->stream, ctx->sm_count, bn_ptr<uint32_t>(w, w_off), M, K, bn_ptr<uint32_t>(pack, pack_off),
                  bn_ptr<float>(out, out_off), ctx->scratch, dots ? bn_ptr<int32_t>(dots, dots_off) : nullptr);
    return bn_launch_check(ctx, "gemv_q81");
}

// ---- projection without any allocation ----------------------------------------------------------------
// Some hosts may not allocate device memory once they are running: a server that sized every device buffer
// when it loaded the model and promised the rest of the card to other tenants, an engine that (like the
// reference, which refuses at start-up rather than grow later) treats a mid-generation allocation as a bug,
// or code that is inside a stream capture, where cudaMalloc is not allowed. bn_gemv_q81 keeps its split-K
// partial sums in a library buffer that it grows with cudaMalloc on demand; this variant keeps them in a
// fixed array that is part of the library image instead, so it never allocates.
//
// The array lives on every GPU that loads the library, for the life of the process: 8 MiB.
// Its name is only a stand-in on the host; the address a kernel needs comes from cudaGetSymbolAddress, asked
// once per device with that device current. That happens inside the first call on a device, so make that
// first call before any stream capture begins. All calls share the one array and it keeps whatever the
// last call left: nothing in it has to start at zero (each call writes every partial sum before reading
// it), but two calls that overlap on the GPU - different streams or contexts on the same device - would
// overwrite each other's partial sums. Run them one after another.
constexpr size_t BN_STATIC_PARTIAL_FLOATS = size_t(2) << 20;       // (K / 512) * M must not exceed this
static __device__ __align__(256) float g_static_partials[BN_STATIC_PARTIAL_FLOATS];
static float *g_static_partials_ptr[64] = {};                       // per device, filled on first use

int bn_gemv_q81_static(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, const bn_buf *pack, size_t pack_off,
                       bn_buf *out, size_t out_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_gemv_q81_static: null context");
    BN_REQUIRE(M > 0 && K > 0 && K % 128 == 0, BN_ERR_ARG, "bn_gemv_q81_static: bad shape M=%d K=%d (K %% 128 != 0)", M, K);
    const int nb = K / 128, ngroups = (nb + 3) / 4;
    BN_REQUIRE(size_t(ngroups) * size_t(M) <= BN_STATIC_PARTIAL_FLOATS, BN_ERR_ARG,
               "bn_gemv_q81_static: ceil(K/512) * M = %zu partial sums exceed the built-in scratch of %zu floats; "
               "use bn_gemv_q81 (which allocates) for this shape", size_t(ngroups) * size_t(M), BN_STATIC_PARTIAL_FLOATS);
    BN_REQUIRE(ctx->device >= 0 && ctx->device < 64, BN_ERR_ARG, "bn_gemv_q81_static: device index %d out of range", ctx->device);
    BN_RANGE(w, w_off, size_t(M) * nb * 28, 4, "bn_gemv_q81_static W");
    BN_RANGE(pack, pack_off, bn_act_pack_bytes(K), 16, "bn_gemv_q81_static pack");
    BN_RANGE(out, out_off, size_t(M) * 4, 4, "bn_gemv_q81_static out");
    if (!g_static_partials_ptr[ctx->device]) {
        // first call on this device: the address lookup below is not allowed while the stream is recording a capture
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        BN_CUDA(cudaStreamIsCapturing(ctx->stream, &cs));
        BN_REQUIRE(cs == cudaStreamCaptureStatusNone, BN_ERR_STATE,
                   "bn_gemv_q81_static: the first call on a device looks up the built-in scratch array and must come before any stream capture");
        BN_CUDA(cudaSetDevice(ctx->device));
        float *p = nullptr;
        BN_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_partials));
        g_static_partials_ptr[ctx->device] = p;
    }
    bnk::gemv_q81(ctx->stream, ctx->sm_count, bn_ptr<uint32_t>(w, w_off), M, K, bn_ptr<uint32_t>(pack, pack_off),
                  bn_ptr<float>(out, out_off), g_static_partials_ptr[ctx->device], nullptr);
    return bn_launch_check(ctx, "gemv_q81 (static scratch)");
}

}  // extern "C"
