// ops.cuh - internal launch helpers shared between the op-level entry points and the token schedule.
#pragma once
#include "common.cuh"

#include <type_traits>

// All helpers enqueue on `st` and return cudaGetLastError() state through bn_launch_check by the caller.
namespace bnk {

// Programmatic dependent launch for every kernel of the token schedule: a kernel may be scheduled while its
// predecessor drains; it blocks in pdl_sync() (first statement of every kernel) until the predecessor's
// memory is visible. Hides the launch latency between the ~230 small kernels of a token.
extern bool g_pdl;
template <class... KArgs, class... Args>
inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    BN_COUNT(1);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

// Several sequences ("columns") in one launch: blockIdx.z is the column; its activations live at the column-0
// pointer + col * arena bytes, its recurrent state, conv taps and KV cache at + col * the respective stream strides.
// The default (no columns) leaves every pointer as it is.
struct Cols {
    int n = 0;
    size_t arena = 0, gdn = 0, conv = 0, kv = 0;
    unsigned z() const { return n > 0 ? unsigned(n) : 1u; }
};
#ifdef __CUDACC__
template <class T> __device__ __forceinline__ T *colp(T *p, size_t bytes) {
    return p ? reinterpret_cast<T *>(reinterpret_cast<char *>(const_cast<typename std::remove_const<T>::type *>(p)) + bytes) : p;
}
#endif

constexpr int Q81_DWORDS = 36;
constexpr int BF_WORDS = 512;
inline size_t act_pack_bytes(int K) { return size_t(K / 128) * (Q81_DWORDS + BF_WORDS) * 4; }

// PTQ1_0 x q8_1 GEMV. out[M] final fp32. scratch: >= ceil(K/512) * M floats.
void gemv_q81(cudaStream_t st, int sm_count, const uint32_t *W, int M, int K, const uint32_t *pack, float *out,
              float *scratch, int32_t *dots);
void act_quant_q81(cudaStream_t st, const float *x, int K, uint32_t *pack);

// y = H(s . x) per `block`-wide chunk, then q8_1 + operand table into pack (pack may be null: rotate only,
// y may be null when only the pack is wanted). n % block == 0, block = power of two in [128, 4096].
void rotate_quant(cudaStream_t st, const float *x, const int32_t *signs, int n, int block, float *y, uint32_t *pack);
// embedding side: y = s . H(x)
void rotate_inv(cudaStream_t st, const float *x, const int32_t *signs, int n, int block, float *y, Cols cols = {});
// PTQ1_0 row gather: out[K] = dequantised row `tok` (tok read from tok_ptr[0])
void embed_row(cudaStream_t st, const uint32_t *W, int K, const int *tok_ptr, float *out, Cols cols = {});

void rms_norm(cudaStream_t st, const float *x, const float *w, int rows, int cols, float eps, float *y);
void add_inplace(cudaStream_t st, float *res, const float *d, int n);       // res = d + res
void swiglu(cudaStream_t st, const float *a, const float *b, int n, float *y, Cols cols = {});
void gemv_f32_small(cudaStream_t st, const float *W, int M, int K, const float *x, float *out);

struct GdnDims { int heads, qk_heads, dim; };
void gdn_gates(cudaStream_t st, const float *alpha, const float *beta_raw, const float *dt_bias, const float *ssm_a,
               int n, float *gate, float *beta);
void conv_silu(cudaStream_t st, const float *x, const float *w, float *hist, int channels, float *y);
void l2_norm_rows(cudaStream_t st, const float *x, int rows, float eps, float *y);   // 128-wide rows
void gdn_delta(cudaStream_t st, GdnDims d, const float *q, const float *k, const float *v, const float *gate,
               const float *beta, float *state, float *o);
// fused layer mixer: alpha/beta projections of the normed residual + gates, conv + silu, L2 norms, delta rule,
// per-head RMS * ssm_norm, swiglu(z, .), v-grouped permutation -> y. hist0 / hist1: the two conv-history
// buffers; position parity picks which is read and which is written. hidden <= 16384.
void gdn_core_fused(cudaStream_t st, GdnDims d, int hidden, const float *qkv, const float *conv_w, float *hist0,
                    float *hist1, const int *pos_ptr, const float *x, const float *inv_ptr, const float *norm_w, const float *alpha_w,
                    const float *beta_w, const float *dt_bias, const float *ssm_a, float *state, const float *z,
                    const float *ssm_norm, float eps, float *y, Cols cols = {});
// the same fused mixer for one sequence on heads x 4 CTAs (clusters of 4, 32 state rows per CTA, the head norm through
// distributed shared memory): same arguments and results as gdn_core_fused
void gdn_core_split(cudaStream_t st, GdnDims d, int hidden, const float *qkv, const float *conv_w, float *hist0, float *hist1,
                    const int *pos_ptr, const float *x, const float *inv_ptr, const float *norm_w, const float *alpha_w,
                    const float *beta_w, const float *dt_bias, const float *ssm_a, float *state, const float *z,
                    const float *ssm_norm, float eps, float *y);
// per-head RMS (no weight) * ssm_norm, swiglu(z, .), v-grouped permutation -> y[heads*dim]
void gdn_out(cudaStream_t st, GdnDims d, const float *o, const float *z, const float *ssm_norm, float eps, float *y);

struct AttnDims { int n_head, n_kv, head_dim, n_rot, cap; float eps, rope_base; int k_mode, v_mode; };
struct KvLayer { void *k_data; uint16_t *k_scale; void *v_data; uint16_t *v_scale; };   // scales null in fp16 mode
// norm + rope + fp16 rounding of q, gate split, K/V quantise + insert at *pos_ptr
void attn_prep(cudaStream_t st, AttnDims a, const float *qg, const float *kin, const float *vin, const float *qn_w,
               const float *kn_w, const int *pos_ptr, KvLayer kv, float *q16f, float *gate, Cols cols = {});
// scores -> softmax (fp16-rounded probabilities) -> PV -> sigmoid gate. Scratch buffers sized by cap.
void attn_decode(cudaStream_t st, AttnDims a, const float *q16f, const float *gate, const int *pos_ptr, KvLayer kv,
                 float *score /*[nh][cap]*/, float *p16f /*[nh][cap]*/, float *esum /*[nh][1024] partial sums + [nh] totals + [nh] counters*/,
                 float *pv_part /*[splits][nh][hd]*/, int splits,
                 float *pregate /*[nh][hd] or null*/, float *gated, bool combine /*false: leave the split partials*/, Cols cols = {});
// cand (optional): per column (value, row0 + index) of the maximum, for an output head whose rows are sharded
void argmax_first(cudaStream_t st, const float *x, int n, int *out_idx, float *scratch_val, int *scratch_idx, Cols cols = {},
                  float *cand = nullptr, int row0 = 0);
// first maximum over n_shards x ncol candidates (value, row), shards in ascending row order
void pick_shards(cudaStream_t st, const float *cands, int n_shards, int ncol, int *out);

// fp32-activation projection (the reference engine's own arithmetic, gemv_ternary.comp): scratch holds
// gemv_f32act_scratch_floats(M, K, n_splits) floats
size_t gemv_f32act_scratch_floats(int M, int K, int n_splits);
void gemv_f32act(cudaStream_t st, const uint8_t *W, int M, int K, const float *x, int n_splits, float *out, float *scratch);

}  // namespace bnk
