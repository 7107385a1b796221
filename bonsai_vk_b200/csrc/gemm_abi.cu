// gemm_abi.cu - C entry points of the multi-column tensor-core projection (declared in include/bonsai_cuda.h).
#include "gemm_tc.cuh"
#include "phase_gemv.cuh"

#include <cstdio>
#include <cstdlib>

extern "C" {

size_t bn_gemm_image_bytes(int K, int ncol) {
    if (K <= 0 || K % 128 || ncol < 1 || ncol > bnk::GEMM_MAX_COLS) return 0;
    return bnk::gemm_image_bytes(K, ncol);
}

int bn_gemm_act_quant(bn_ctx *ctx, const bn_buf *x, size_t x_off, size_t x_stride, int K, int ncol, const bn_buf *signs,
                      size_t signs_off, int hat_block, bn_buf *image, size_t image_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_gemm_act_quant: null context");
    BN_REQUIRE(K > 0 && K % 1024 == 0, BN_ERR_ARG, "bn_gemm_act_quant: K=%d must be a multiple of 1024", K);
    BN_REQUIRE(ncol >= 1 && ncol <= bnk::GEMM_MAX_COLS, BN_ERR_ARG, "bn_gemm_act_quant: %d columns (1..%d)", ncol, bnk::GEMM_MAX_COLS);
    BN_REQUIRE(x_stride >= size_t(K), BN_ERR_ARG, "bn_gemm_act_quant: column stride %zu is shorter than K", x_stride);
    BN_RANGE(x, x_off, (size_t(ncol - 1) * x_stride + K) * 4, 4, "bn_gemm_act_quant x");
    BN_RANGE(image, image_off, bnk::gemm_image_bytes(K, ncol), 128, "bn_gemm_act_quant image");
    if (signs) {
        BN_REQUIRE(hat_block >= 16 && hat_block <= 4096 && (hat_block & (hat_block - 1)) == 0 && K % hat_block == 0, BN_ERR_ARG,
                   "bn_gemm_act_quant: hadamard block %d must be a power of two in [16, 4096] dividing K", hat_block);
        BN_RANGE(signs, signs_off, size_t(K) * 4, 4, "bn_gemm_act_quant signs");
    }
    bnk::PrepArgs a = {};
    a.x = bn_ptr<float>(x, x_off); a.x_stride = x_stride;
    a.signs = signs ? bn_ptr<int32_t>(signs, signs_off) : nullptr;
    a.K = K; a.hat_block = hat_block; a.ncol = ncol; a.image = bn_ptr<uint8_t>(image, image_off); a.mode = bnk::PREP_PLAIN;
    bnk::prep_cols(ctx->stream, a);
    return bn_launch_check(ctx, "k_prep_cols");
}

size_t bn_gemm_tiled_bytes(int M, int K) {
    if (M <= 0 || K <= 0 || K % 1024) return 0;
    return bnk::gemm_tiled_bytes(M, K);
}

int bn_gemm_repack(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, bn_buf *tiled, size_t tiled_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_gemm_repack: null context");
    BN_REQUIRE(M > 0 && K > 0 && K % 1024 == 0, BN_ERR_ARG, "bn_gemm_repack: bad shape M=%d K=%d (K %% 1024 != 0)", M, K);
    BN_RANGE(w, w_off, size_t(M) * (K / 128) * 28, 4, "bn_gemm_repack W");
    BN_RANGE(tiled, tiled_off, bnk::gemm_tiled_bytes(M, K), 128, "bn_gemm_repack out");
    bnk::repack_tiles(ctx->stream, bn_ptr<uint32_t>(w, w_off), M, K, bn_ptr<uint32_t>(tiled, tiled_off));
    return bn_launch_check(ctx, "k_repack_tiles");
}

int bn_gemm_q81(bn_ctx *ctx, const bn_buf *w, size_t w_off, int w_tiled, int M, int K, const bn_buf *image, size_t image_off, int ncol,
                bn_buf *out, size_t out_off, size_t out_stride) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_gemm_q81: null context");
    BN_REQUIRE(bnk::gemm_supported(M, K, ncol), BN_ERR_ARG, "bn_gemm_q81: unsupported shape M=%d K=%d columns=%d (K %% 1024 == 0, 1..%d columns)",
               M, K, ncol, bnk::GEMM_MAX_COLS);
    BN_REQUIRE(out_stride >= size_t(M), BN_ERR_ARG, "bn_gemm_q81: column stride %zu is shorter than M", out_stride);
    if (w_tiled) BN_RANGE(w, w_off, bnk::gemm_tiled_bytes(M, K), 128, "bn_gemm_q81 W (tiled)");
    else BN_RANGE(w, w_off, size_t(M) * (K / 128) * 28, 16, "bn_gemm_q81 W");
    BN_RANGE(image, image_off, bnk::gemm_image_bytes(K, ncol), 128, "bn_gemm_q81 image");
    BN_RANGE(out, out_off, (size_t(ncol - 1) * out_stride + M) * 4, 4, "bn_gemm_q81 out");
    bnk::GemmArgs a = {};
    a.W = bn_ptr<uint8_t>(w, w_off); a.M = M; a.K = K; a.tiled = w_tiled ? 1 : 0;
    a.image = bn_ptr<uint8_t>(image, image_off); a.ncol = ncol;
    a.out = bn_ptr<float>(out, out_off); a.out_stride = out_stride;
    a.err = ctx->err_dev;
    if (bnk::gemm_wants_split(ctx->sm_count, M, K, ncol)) {
        int rc = bn_scratch_reserve(ctx, bnk::gemm_group_floats(M, K, ncol) * 4);
        if (rc != BN_OK) return rc;
        a.groups = ctx->scratch;
    }
    // profiling aid (library built with -DGEMM_PROF): BONSAI_GEMM_PROF=1 prints where the roles of CTA 0 spent their
    // cycles (waiting vs working); without that build flag the counters stay zero
    static const bool want_prof = getenv("BONSAI_GEMM_PROF") != nullptr;
    long long *prof = nullptr;
    if (want_prof) {
        BN_CUDA(cudaMalloc(&prof, 128 * sizeof(long long)));
        BN_CUDA(cudaMemsetAsync(prof, 0, 128 * sizeof(long long), ctx->stream));
        a.prof = prof;
    }
    cudaError_t e = bnk::launch_gemm(ctx->stream, ctx->sm_count, a, false);
    if (e != cudaSuccess) return bn_cuda_fail(e, "k_ptq_gemm_tc");
    // timing aid: BONSAI_GEMM_REPS=n repeats the launch n-1 more times (same result) so that a host loop in an
    // interpreted language does not become the bottleneck when small shapes are timed
    static const int reps = getenv("BONSAI_GEMM_REPS") ? atoi(getenv("BONSAI_GEMM_REPS")) : 1;
    for (int r = 1; r < reps; ++r) bnk::launch_gemm(ctx->stream, ctx->sm_count, a, false);
    if (want_prof) {
        long long h[128];
        BN_CUDA(cudaStreamSynchronize(ctx->stream));
        BN_CUDA(cudaMemcpy(h, prof, sizeof h, cudaMemcpyDeviceToHost));
        cudaFree(prof);
        fprintf(stderr, "gemm prof (cycles, CTA 0): decode[wait full %lld, unpack %lld, publish %lld, wait slot %lld] "
                        "mma[wait full %lld, wait A %lld, wait D %lld] epilogue[wait D %lld, wait ld %lld, combine %lld]; CTA 0 set-up %lld ns, "
                        "whole CTA %lld ns; last CTA after set-up %lld ns\n",
                h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[8], h[9], h[10], h[12], h[14], h[13]);
        if (getenv("BONSAI_GEMM_PROF_EVENTS")) {
            static const char *names[7] = {"decode start", "decode stored", "mma has A", "mma has D", "mma committed", "epilogue has D", "epilogue done"};
            long long t0 = h[16];
            for (int ev = 0; ev < 7; ++ev) {
                fprintf(stderr, "%-16s", names[ev]);
                for (int g = 0; g < 16; ++g) fprintf(stderr, " %6lld", h[16 + ev * 16 + g] - t0);
                fprintf(stderr, "\n");
            }
        }
    }
    return bn_launch_check(ctx, "k_ptq_gemm_tc");
}

int bn_selftest_wait(bn_ctx *ctx, int which) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_selftest_wait: null context");
    BN_REQUIRE(which == 0 || which == 1, BN_ERR_ARG, "bn_selftest_wait: which=%d (0 = copy-ring wait, 1 = tensor-core pipeline wait)", which);
    cudaError_t e = which == 0 ? bnk::launch_wait_selftest_ring(ctx->stream, ctx->err_dev)
                               : bnk::launch_wait_selftest_tc(ctx->stream, ctx->err_dev);
    if (e != cudaSuccess) return bn_cuda_fail(e, "bn_selftest_wait");
    return BN_OK;
}

}  // extern "C"
