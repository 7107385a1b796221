// gemm_tc.cuh - PTQ1_0 x q8_1 projection of several activation columns at once (prefill tokens or concurrent
// sequences) on the 5th-generation tensor cores: tcgen05.mma kind::i8, the weight operand decoded into tensor
// memory, int32 accumulators in tensor memory, fp32 combination in the GEMV's operation order.
#pragma once
#include "ops.cuh"

namespace bnk {

constexpr int GEMM_MAX_COLS = 32;
// columns are padded to 8, 16 or 32 (the N of the tensor-core instruction)
inline int gemm_padded_cols(int ncol) { return ncol <= 8 ? 8 : (ncol <= 16 ? 16 : 32); }
// The "activation image" the kernel consumes, per 128 activations (one PTQ1_0 block) of ncp = 8, 16 or 32 columns:
//   codes: column n, sub-block sb (32 activations), k-half kh (16 of them): int8 codes at
//          (n/8) * 1024 + (sb*2 + kh) * 128 + (n%8) * 16   - per group of 8 columns the shared-memory operand layout
//          of the instruction (8 x 16-byte core matrices, K-major, no swizzle), so a stage is one contiguous bulk copy
//   scales: per group of 8 columns 256 bytes at ncp*128 + (n/8)*256: entry (sb, column pair p) at (sb*4 + p) * 16 holds
//           fp32 (d[2p], d[2p+1], -s[2p], -s[2p+1]) - the fp16 values of the q8_1 record, widened, s negated - so that the
//           epilogue's packed two-column arithmetic reads its operands with one 16-byte load
inline size_t gemm_image_block_bytes(int ncp) { return size_t(ncp) * 160; }
inline size_t gemm_image_bytes(int K, int ncol) { return size_t(K / 128) * gemm_image_block_bytes(gemm_padded_cols(ncol)); }

enum PrepMode { PREP_PLAIN = 0, PREP_NORM = 1 };
struct PrepArgs {
    const float *x; size_t x_stride;      // column c reads x + c * x_stride (floats)
    const float *w;                       // PREP_NORM: x <- rms_norm(x) * w over all K values
    const int32_t *signs;                 // K sign values; null = no rotation (quantise x as it is)
    int K, hat_block;
    float eps;
    int ncol;
    uint8_t *image;
    float *inv_out; size_t inv_stride;    // PREP_NORM, optional: the norm factor of column c at inv_out + c * inv_stride
    int mode;
};
void prep_cols(cudaStream_t st, const PrepArgs &a);

struct GemmArgs {
    const uint8_t *W; int M, K;           // M rows of K/128 PTQ1_0 blocks; K % 1024 == 0
    int tiled;                            // 0: W is the native row-major matrix; 1: W is its repacked copy (repack_tiles)
    const uint8_t *image; int ncol;
    float *out; size_t out_stride;        // column c writes out + c * out_stride (floats)
    const float *resid; size_t resid_stride;   // optional: out = acc + resid (may alias out)
    int *err;                             // device error word (bounded waits)
    // split over K for matrices with few row tiles (M = 4096 has 32 tiles of 128 rows - a fifth of the GPU): every ring stage
    // (8 blocks of K = two groups of 4 blocks) becomes a work item of its own and the kernel writes the two group sums
    // p_g of every (row, column) to groups[(g * padded columns + column) * M + row]; gemm_sum_groups then adds the
    // groups in ascending order (+ residual), which is the order the unsplit kernel and the single-column kernel use
    float *groups;                        // null = no split
    long long *prof;                      // optional: 12 cycle counters of CTA 0 (decode 0-3, MMA thread 4-7, epilogue 8-11)
};
bool gemm_supported(int M, int K, int ncol);
// Repacked weights: per tile of 128 rows and 8 blocks of K one contiguous 28 672-byte piece, [block][dword 0..6][row],
// so that a pipeline stage is a single bulk copy and the decode warps read consecutive dwords. Rows beyond M are zero.
size_t gemm_tiled_bytes(int M, int K);
void repack_tiles(cudaStream_t st, const uint32_t *W, int M, int K, uint32_t *out);
cudaError_t launch_gemm(cudaStream_t st, int sm_count, const GemmArgs &a, bool pdl);
// whether launch_gemm would like to split this shape over K, and the scratch floats it then needs (a.groups)
bool gemm_wants_split(int sm_count, int M, int K, int ncol);
size_t gemm_group_floats(int M, int K, int ncol);
// one tiny kernel whose only wait can never complete and gives up after one round of tries: sets *err = 2 and returns
cudaError_t launch_wait_selftest_tc(cudaStream_t st, int *err);

}  // namespace bnk
