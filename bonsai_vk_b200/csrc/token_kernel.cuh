// token_kernel.cuh - the whole-token kernel: ONE launch runs every phase of one decode token (or of a run of greedy
// tokens) on all SMs, with grid-wide barriers between phases (reference: one command-buffer submit per token,
// fwd_token, runtime_vk/bonsai_forward.h:664-722). The host describes a token as a list of phase records.
#pragma once
#include "phase_gemv.cuh"

namespace bnk {

enum TokOpKind {
    TOP_GEMV = 0,          // fused projection phase (phase_body.cuh)
    TOP_GDN = 1,           // gated-delta-net mixer core of one layer: gates, conv + silu, L2 norms, delta rule
    TOP_ATTN_PREP = 2,     // head norm + rope + fp16 Q, K / V cache insert
    TOP_ATTN_SCORES = 3,   // q . k over the filled prefix
    TOP_ATTN_EXPSUM = 4,   // softmax numerators and their partial sums
    TOP_ATTN_PV = 5,       // fp16-rounded probabilities x V, split over keys
    TOP_ATTN_COMBINE = 6   // splits added ascending, sigmoid gate
};

struct GdnOp {
    int heads, qk_heads, hidden;
    const float *qkv, *conv_w;           // projection output [q | k | v] and the 4-tap conv weights
    float *hist0, *hist1;                // conv taps, double-buffered by position parity
    const float *x, *norm_w;             // residual and the block's norm weight (input of the two small projections)
    const float *alpha_w, *beta_w, *dt_bias, *ssm_a;
    float *state;                        // [heads][128][128]
    float *o;                            // [heads][128]: delta-rule output * 1/sqrt(128), before the per-head norm
    float scale;
};

struct AttnOp {
    AttnDims d;
    KvLayer kv;
    const float *qg, *kin, *vin, *qn_w, *kn_w;
    float *q16f, *gate, *score, *pe, *esum, *pv_part, *gated;
    int splits;
};

struct TokOp {
    int kind;
    int wait;                            // 1: the phase reads what the previous phase wrote (wait for the grid first)
    union {
        PhaseArgs ph;                    // TOP_GEMV
        GdnOp gdn;                       // TOP_GDN
        AttnOp at;                       // TOP_ATTN_*
    };
};

constexpr int TOKEN_MAX_OPS = 208;       // fits the 64 KB constant bank together with the rest of the module

struct TokenArgs {
    int n_ops;
    int first_tok, pos0, n_steps;
    int pick;                            // 1: the list ends with the output head; pick the first maximum and feed it back
    // embedding (first phase of a token): row `tok` of token_embd dequantised, H then signs (fwd_token :685-691)
    const uint32_t *embd;
    const int32_t *signs;
    int hidden, hat_block, vocab;
    float *res;                          // residual stream [hidden]
    float *cand_val; int *cand_idx;      // per-CTA first-maximum candidates of the output head
    int *hist;                           // [n_steps] picked ids
    int *next;                           // [1] last pick
    int *pos_out;                        // [1] position of the last token run (for later readers)
    unsigned *bar;                       // grid barrier counter, zero at launch
    int *err;                            // device error word
    unsigned long long *stamps;          // optional: 8 time stamps per phase of CTA 0 in ns, first token of the launch only
};

// uploads the phase list of a model to the constant bank (queued on `st`); `owner` identifies the list so that repeated
// launches of the same model skip the copy
cudaError_t token_upload_ops(cudaStream_t st, const TokOp *ops, int n_ops, const void *owner);
// cooperative launch on all SMs
cudaError_t launch_token(cudaStream_t st, int sm_count, const TokenArgs &a);
size_t token_smem_bytes(int hat_block);
bool token_supported(int sm_count, int hat_block, int hidden);

}  // namespace bnk
