// phase_gemv.cuh - the fused "phase" kernel: [prologue that rebuilds the rotated, quantised input of a
// projection from the previous phase's outputs] + [PTQ1_0 x q8_1 GEMV streamed through a bulk-copy ring]
// + [split-K finalisation and residual add by the last CTA to touch a row tile].
#pragma once
#include "ops.cuh"

namespace bnk {

enum Prologue {
    PRO_PACKED = 0,   // activation pack already in global memory (op-level entry point)
    PRO_PLAIN = 1,    // x0 is the plain fp32 input: rotate + quantise
    PRO_NORM = 2,     // x = rms_norm(x0) * w                                   (pre_norm, bonsai_forward.h:480)
    PRO_SWIGLU = 3,   // x = silu(x0) * x1                                       (ffn_block :498)
    PRO_GDN_OUT = 4,  // x = permute(silu(z = x1) * (rms_head(o = x0) * w))      (gdn_block :559-567)
    PRO_ATTN_OUT = 5, // x = (sum_s pv[s]) * sigmoid(gate = x1)                  (attn_pv_q8v.comp tail)
    PRO_GDN_OUT_SZ = 6 // as PRO_GDN_OUT with x1 = silu(z) already applied by the producing phase's epilogue
};

enum Epilogue {
    EPI_PLAIN = 0,     // out[row] = sum; optional resid_out = sum + resid_in
    EPI_SWIGLU = 1,    // rows [0, M/2) are gate rows, [M/2, M) up rows: out2[r] = silu(gate_r) * up_r   (ffn_block :498);
                       // needs K <= 4096 (one chunk) and M/2 a multiple of 16
    EPI_SILU_FROM = 2, // out[row] = row >= epi_arg ? silu(sum) : sum   (the z rows of a gated-delta-net block, gdn_block :563)
    EPI_ARGMAX = 3     // EPI_PLAIN + the CTA's first-maximum candidate (cand_val / cand_idx [cta])   (Sampler::pick, temp <= 0)
};

struct PhaseArgs {
    // projection
    const uint8_t *W;        // M rows of K/128 PTQ1_0 blocks
    int M, K;                // K % 512 == 0
    float *out;              // [M] final sums (may be null when resid_out is set)
    const float *resid_in;   // optional [M]
    float *resid_out;        // optional [M]: resid_out = out + resid_in
    float *part;             // unused by the streamed kernel (kept for the op-level callers)
    unsigned *counters;
    int epi, epi_arg;        // Epilogue
    float *out2;             // EPI_SWIGLU: [M/2]
    float *cand_val;         // EPI_ARGMAX: per-CTA candidate
    int *cand_idx;
    // prologue
    int pro;
    const float *x0, *x1, *w;
    const uint32_t *pack;    // PRO_PACKED
    const int32_t *signs;    // K sign values
    int hat_block;
    float hat_inv, eps;
    int gdn_heads, gdn_qk_heads;   // PRO_GDN_OUT
    int pv_splits;                 // PRO_ATTN_OUT: x0 = pv partials [splits][K]
    const int *pos_ptr;            // PRO_ATTN_OUT: number of filled keys = pos + 1
    float *inv_out;                // PRO_NORM: optional, receives 1/sqrt(mean(x0^2) + eps) for a later consumer
    int *err;                      // device error word (bounded waits)
    unsigned long long *stamps;    // optional: 8 nanosecond time stamps of CTA 0 (start, copies issued, previous grid
                                   // done, norm, input built, quantised, operands built, end) for profiling
};

constexpr int PHASE_THREADS = 512;
size_t phase_smem_bytes(int hat_block);
// y = silu(gate) * up (n floats, y may be null) and the activation pack of the down projection's rotated, quantised input
// (signs of n entries; y is written always); the projection then runs with PRO_PACKED.
bool swiglu_pack_supported(int n, int hat_block);
// count: one zeroed int per Hadamard block (the kernel leaves it zero).
void swiglu_pack(cudaStream_t st, const float *gate, const float *up, int n, const int32_t *signs, float hat_inv, float *y, uint32_t *pack, int *count);
// launches with programmatic dependent launch when pdl is true
cudaError_t launch_phase(cudaStream_t st, int sm_count, const PhaseArgs &a, bool pdl);
bool phase_supported(int M, int K, int hat_block);
// one tiny kernel whose only wait can never complete and gives up after ~1000 tries: sets *err = 1 and returns
cudaError_t launch_wait_selftest_ring(cudaStream_t st, int *err);

}  // namespace bnk
