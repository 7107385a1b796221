/* bonsai_cuda.h - C ABI of libbonsai_cuda.so: the device layer of the bonsai decode path on B200.
 *
 * What this replaces. The reference engine has no plugin interface; its device layer is a set of
 * Vulkan helpers that the forward pass calls directly. Each entry point below names the reference
 * helper (file:line, relative to the reference tree) whose role it takes over:
 *
 *   vk_ctx_init                      runtime_vk/bonsai_weights.h:45     -> bn_init
 *   Arena::reserve/commit/create_at  runtime_vk/bonsai_weights.h:126    -> bn_alloc / bn_free
 *   flush_batch (staging upload)     runtime_vk/bonsai_weights.h:446    -> bn_upload
 *   act_store / act_rd               runtime_vk/bonsai_forward.h:1294   -> bn_upload / bn_download
 *   dsp(pipeline, push constants)    runtime_vk/bonsai_forward.h:352    -> one bn_<op>() per kernel
 *   begin_cmd / submit_wait_sig      runtime_vk/bonsai_weights.h:263,287-> bn_sync (ops are queued on
 *                                                                          the context's stream)
 *   timestamp query pool             runtime_vk/bonsai_forward.h:676    -> bn_event_*
 *
 * Conventions. Plain C types only. Device memory is owned by the library and named by opaque
 * bn_buf handles plus byte offsets; every op checks offsets and sizes against the buffer before it
 * launches anything and refuses (negative return, message in bn_last_error) instead of faulting.
 * Every call returns 0 on success or a negative bn_err. Calls on one context must be serialised by
 * the caller (the reference engine is single-threaded, runtime_vk/bonsai_http.h:458). One process drives
 * one GPU: bn_init refuses a second device index in the same process (a multi-GPU host runs one process
 * per pipeline stage). There is no CPU fallback: without a CUDA device bn_init fails.
 */
#ifndef BONSAI_CUDA_H
#define BONSAI_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct bn_ctx bn_ctx;
typedef struct bn_buf bn_buf;
typedef struct bn_event bn_event;

enum bn_err {
    BN_OK = 0,
    BN_ERR_CUDA = -1,      /* a CUDA runtime call failed                       */
    BN_ERR_ARG = -2,       /* bad argument: shape, alignment, range            */
    BN_ERR_BOUNDS = -3,    /* offset + size exceeds the buffer                 */
    BN_ERR_NOMEM = -4,     /* device allocation failed                         */
    BN_ERR_TIMEOUT = -5,   /* a bounded device-side wait gave up               */
    BN_ERR_STATE = -6      /* call not valid in the current state              */
};

/* last error message of the calling thread ("" if none) */
const char *bn_last_error(void);

/* ---- context and memory -------------------------------------------------------------------- */
int bn_init(int device, bn_ctx **out);
void bn_destroy(bn_ctx *ctx);
int bn_device_info(bn_ctx *ctx, int *sm_count, size_t *free_bytes, size_t *total_bytes);
int bn_alloc(bn_ctx *ctx, size_t bytes, bn_buf **out);
int bn_free(bn_ctx *ctx, bn_buf *buf);
size_t bn_buf_size(const bn_buf *buf);
int bn_upload(bn_ctx *ctx, bn_buf *dst, size_t off, const void *src, size_t n);
/* queued copy from page-locked memory (bn_host_alloc): returns at once; src must stay untouched until the next bn_sync.
 * The loader overlaps reading the next piece of the file with this copy (reference: the staged upload loop of
 * bonsai_weights.h:440-529, which waits for every batch). */
int bn_upload_async(bn_ctx *ctx, bn_buf *dst, size_t off, const void *src, size_t n);
int bn_download(bn_ctx *ctx, const bn_buf *src, size_t off, void *dst, size_t n);
int bn_memset(bn_ctx *ctx, bn_buf *dst, size_t off, int byte, size_t n);
int bn_sync(bn_ctx *ctx);
/* Failure detection without a fault: queues one tiny kernel whose only wait can never complete, with the wait's limit
 * cut to a few milliseconds (which = 0: the copy-ring wait of the single-column projection; 1: the pipeline wait of the
 * tensor-core projection). The kernel gives up, sets the context's error word and returns; the next bn_sync reports
 * BN_ERR_TIMEOUT and clears the word, and the context stays usable. (The reference has no counterpart: its waits are
 * Vulkan fences with an unbounded timeout, bonsai_weights.h:287.) */
int bn_selftest_wait(bn_ctx *ctx, int which);

/* page-locked host staging memory (reference: the mapped host_buf, bonsai_weights.h:199) */
int bn_host_alloc(size_t bytes, void **out);
int bn_host_free(void *p);

/* CUDA events on the context's stream (reference: VkQueryPool timestamps) */
int bn_event_create(bn_ctx *ctx, bn_event **out);
int bn_event_record(bn_ctx *ctx, bn_event *ev);
int bn_event_elapsed_ms(bn_ctx *ctx, bn_event *start, bn_event *stop, float *ms);
int bn_event_destroy(bn_ctx *ctx, bn_event *ev);

/* number of kernels this library has launched on ctx since bn_init (for launch accounting) */
uint64_t bn_launch_count(const bn_ctx *ctx);

/* ---- PTQ1_0 x q8_1 GEMV (reference arithmetic: _mul_mat_vecq_ptq1_0.comp:92-202;
 *      reference call site: gemv_ptq, runtime_vk/bonsai_forward.h:409-422) ------------------------
 * An "activation pack" is what a GEMV consumes: for every 128 activations the block_q8_1_x4 record
 * (36 dwords: 4 x (fp16 d | fp16 s << 16), then 128 int8) followed, after all records, by the
 * tensor-core operand table derived from it (2048 bytes per 128 activations). */
size_t bn_act_pack_bytes(int K);
/* x: K fp32 values at (x, x_off). Writes the pack at (pack, pack_off). K % 128 == 0. */
int bn_act_quant_q81(bn_ctx *ctx, const bn_buf *x, size_t x_off, int K, bn_buf *pack, size_t pack_off);
/* W: M rows of K/128 PTQ1_0 blocks (28 bytes each, row-major) at (w, w_off); out: M fp32.
 * dots (may be NULL): receives the int32 block dots [M][K/128][4] for bit-exact checking. */
int bn_gemv_q81(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, const bn_buf *pack,
                size_t pack_off, bn_buf *out, size_t out_off, bn_buf *dots, size_t dots_off);

/* The same projection for callers that must not allocate device memory while running (a host that fixed its
 * device budget at load time, or one inside a stream capture). No counterpart in the reference: its engine
 * sizes everything in fwd_init and has no such call. The split-K partial sums live in an 8 MiB array built
 * into the library (present on every GPU that loads it), so ceil(K/512) * M must be <= 2 097 152; larger
 * shapes are refused. The first call on a device looks the array's address up - make it before any stream
 * capture. Calls share the array: do not let two of them overlap on one GPU. Same results as bn_gemv_q81. */
int bn_gemv_q81_static(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, const bn_buf *pack,
                       size_t pack_off, bn_buf *out, size_t out_off);

/* ---- PTQ1_0 x fp32 activations, the reference engine's own projection arithmetic (gemv_ptq,
 *      runtime_vk/bonsai_forward.h:409-422 -> xsum.comp, gemv_ternary.comp:74-118, reduce.comp): out[r] =
 *      sum_b d[r,b] * (sum c*x - xsum_b), c in {0,1,2}, four strided fma chains per 64-code half combined as
 *      (a0+a1)+(a2+a3), blocks ascending, split-K partials added ascending. One fp32 fma per weight: a parity mode,
 *      not the fast path. x: K fp32 (already rotated by the caller). n_splits: 1..16 dividing K/128, or 0 = the
 *      reference's rule (pick_splits, bonsai_weights.h:581-588), which bn_gemv_f32act_splits also returns. ------------ */
int bn_gemv_f32act_splits(int M, int K);
int bn_gemv_f32act(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, const bn_buf *x, size_t x_off, int n_splits,
                   bn_buf *out, size_t out_off);

/* ---- the same projection for several activation columns at once (prefill tokens, concurrent sequences) on the
 *      tcgen05 tensor cores. Reference: the multi-column path of _mul_mat_vecq_ptq1_0.comp:204-347 (<= 8 columns;
 *      beyond that the reference falls back to dequantise + f16 matmul, _ggml-vulkan.cpp:2195-2197, which has no
 *      integer block dots). Every column of the result is bit-identical to bn_gemv_q81 on that column's vector. -----
 * The activations are handed over as one "image" for all columns: int8 codes in the tensor-core operand layout plus
 * the (d, s) scale pairs per 32 activations. bn_gemm_act_quant builds it from ncol fp32 vectors of K values
 * (column c at x + c * x_stride floats): optional rotation y = H(s . x) per hat_block (signs NULL = none), then the
 * q8_1 quantiser. K % 1024 == 0, 1 <= ncol <= 32. */
size_t bn_gemm_image_bytes(int K, int ncol);
int bn_gemm_act_quant(bn_ctx *ctx, const bn_buf *x, size_t x_off, size_t x_stride, int K, int ncol, const bn_buf *signs,
                      size_t signs_off, int hat_block, bn_buf *image, size_t image_off);
/* Optional second copy of a weight matrix for this kernel (reference: the engine also repacks its weights once at load,
 * bonsai_weights.h:502-558): per tile of 128 rows and 8 blocks of K one contiguous piece, so that a pipeline stage is a
 * single bulk copy. Same bytes, other order; rows beyond M are zero. */
size_t bn_gemm_tiled_bytes(int M, int K);
int bn_gemm_repack(bn_ctx *ctx, const bn_buf *w, size_t w_off, int M, int K, bn_buf *tiled, size_t tiled_off);
/* w_tiled = 0: w is the native row-major matrix; 1: w is the copy made by bn_gemm_repack.
 * out: column c at out + c * out_stride floats, M values each */
int bn_gemm_q81(bn_ctx *ctx, const bn_buf *w, size_t w_off, int w_tiled, int M, int K, const bn_buf *image, size_t image_off,
                int ncol, bn_buf *out, size_t out_off, size_t out_stride);

/* ---- decode attention as stand-alone ops (reference: attn_block, runtime_vk/bonsai_forward.h:581-645; kernels
 *      attn_norm_rope2.comp, attn_qk_softmax*.comp, attn_pv_q8v*.comp; test harness align_attn.cpp) ------------
 * One layer's cache lives in a caller buffer of bn_attn_kv_bytes(); working memory of bn_attn_scratch_bytes(). */
typedef struct bn_attn_dims {
    int32_t n_head, n_kv, head_dim, n_rot, cap;   /* cap = cache capacity in positions */
    int32_t k_mode, v_mode;                        /* 0 = q8_0, 1 = fp16 */
    float rms_eps, rope_base;
} bn_attn_dims;
size_t bn_attn_kv_bytes(const bn_attn_dims *d);
size_t bn_attn_scratch_bytes(const bn_attn_dims *d);
/* n consecutive tokens at positions pos0.. : per token the K row gets head norm * k_norm, rope, then (like the raw
 * V row) is quantised / rounded into the cache; the q|gate row [n_head][2*head_dim] (layout of attn_q's output,
 * deint_qg.comp) is normed, roped at the LAST position and kept in scratch for bn_attn_attend. */
int bn_attn_insert(bn_ctx *ctx, const bn_attn_dims *d, bn_buf *kv, size_t kv_off, const bn_buf *k_rows, size_t k_off,
                   const bn_buf *v_rows, size_t v_off, int n, int pos0, const bn_buf *qg, size_t qg_off,
                   const bn_buf *q_norm, size_t qn_off, const bn_buf *k_norm, size_t kn_off, bn_buf *scratch, size_t scratch_off);
/* softmax attention of the kept query over positions 0..pos; pregate (may be NULL) and gated: [n_head][head_dim] */
int bn_attn_attend(bn_ctx *ctx, const bn_attn_dims *d, const bn_buf *kv, size_t kv_off, int pos, bn_buf *scratch,
                   size_t scratch_off, bn_buf *pregate, size_t pg_off, bn_buf *gated, size_t g_off);

/* ---- whole-token decode (reference: fwd_token, runtime_vk/bonsai_forward.h:664-758) ---------------
 * The host registers every tensor of the GGUF by its GGUF name (PTQ1_0 tensors as the file's native
 * 28-byte blocks, row-major, d0 = K; f32 tensors as they are) plus the prism.hadamard sign values,
 * then finalises. Hyper-parameters mirror the GGUF keys the reference reads (bonsai_model.h:642-760). */
typedef struct bn_model bn_model;
typedef struct bn_hparams {
    int32_t n_layer, hidden, ffn, vocab;
    int32_t n_head, n_kv, head_dim, n_rot;    /* attention.head_count(_kv), key_length, rope.dimension_count */
    int32_t attn_interval;                    /* full_attention_interval: block b is attention iff b % i == i-1;
                                                 0 = the explicit per-layer list in attn_mask_lo/hi is used instead */
    int32_t gdn_heads, gdn_qk_heads, gdn_dim; /* ssm.time_step_rank, ssm.group_count, ssm.state_size */
    int32_t hat_block;                        /* prism.hadamard.block_size */
    int32_t act_mode;                         /* 0 = q8_1 activations + integer dots */
    int32_t k_mode, v_mode;                   /* KV cache: 0 = q8_0, 1 = fp16 */
    int32_t cap;                              /* KV capacity in positions (reference: BONSAI_CAP, even) */
    float rms_eps, rope_base;
    /* multi-stream / pipeline-stage extensions (0 = one stream, whole model) */
    int32_t n_streams;                        /* independent sequences, each with its own KV cache and recurrent state */
    int32_t block_begin, block_end;           /* this device holds blocks [begin, end); end 0 = n_layer. The embedding
                                                 belongs to the stage with block 0, the output head to the last one */
    int32_t batch_cols;                       /* > 0: bn_model_stage_batch may run up to this many sequences per call
                                                 (<= 32); costs one more activation arena per column and a tile-major
                                                 copy of the local projection weights for the tensor-core kernel */
    /* explicit layer typing (reference: the resolved 64-bit mask of bonsai_model.h:470-472), read only when
     * attn_interval == 0: block b (n_layer <= 64) is an attention block iff bit b is set, else a gated-delta-net block */
    uint32_t attn_mask_lo, attn_mask_hi;
} bn_hparams;

enum bn_read_what {
    BN_READ_LOGITS = 0, BN_READ_RESIDUAL = 1, BN_READ_GDN_STATE = 2, BN_READ_CONV_HIST = 3,
    BN_READ_K_DATA = 4, BN_READ_K_SCALE = 5, BN_READ_V_DATA = 6, BN_READ_V_SCALE = 7
};

int bn_model_create(bn_ctx *ctx, const bn_hparams *hp, bn_model **out);
int bn_model_set_tensor(bn_model *m, const char *name, const bn_buf *buf, size_t off, size_t bytes);
int bn_model_set_signs(bn_model *m, const bn_buf *buf, size_t off, int count);
/* resolves every tensor the architecture needs (refuses with the missing name), allocates the
 * activation arena, the KV cache and the recurrent state (reference: fwd_init, bonsai_forward.h:1490) */
int bn_model_finalize(bn_model *m);
/* zero KV, recurrent state and scratch (reference: fwd_reset_state, bonsai_forward.h:2624-2643) */
int bn_model_reset(bn_model *m);
/* the same for ONE sequence of a multi-sequence model: its recurrent state, conv taps and KV cache (the reference resets
 * per request, runtime_vk/bonsai_http.h:592-623; with several conversations in flight only the slot that takes the new
 * request is cleared). Enqueues only. */
int bn_model_reset_stream(bn_model *m, int stream);
void bn_model_destroy(bn_model *m);
/* one token at absolute position pos. stop_after_block < 0 runs the whole network and the greedy pick
 * (first maximum, as Sampler::pick with temp <= 0); >= 0 stops after that block (alignment harness,
 * reference: BONSAI_LADDER / stop_at_block). next_tok may be NULL (nothing is copied back then). The whole-network
 * form is one launch of the token's CUDA graph (captured by the first call) behind a small kernel that carries tok and
 * pos as arguments; the host waits once per call, for the pick, and only when next_tok is given. */
int bn_model_token(bn_model *m, int tok, int pos, int stop_after_block, int *next_tok);
/* Batched prefill: n consecutive tokens of the sequence at positions pos0 .. pos0+n-1 as ONE pass (the reference feeds
 * its prompt token by token, runtime_vk/bonsai_forward.h:2752-2757; this reads every projection's weights once per
 * block of n tokens through the tensor-core kernel). The recurrent mixer walks the n positions in order on the one
 * state, attention inserts all n K/V rows and lets each position attend causally. Every position's result - cache
 * rows, recurrent state, the logits of the last one - is bit-identical to n calls of bn_model_token. Needs
 * bn_hparams.batch_cols >= n and the whole model on this device. next_tok (may be NULL) receives the greedy pick after
 * the last position. */
int bn_model_prefill(bn_model *m, const int *toks, int n, int pos0, int *next_tok);
/* Builds the replayable schedule of a pipeline stage before any traffic flows (reference: the engine records its command
 * buffers and refuses bad plans before the first dispatch, runtime_vk/bonsai_weights.h:349-353): ncol = 0 prepares
 * bn_model_stage for sequence stream0, ncol >= 1 prepares bn_model_stage_batch for the pass over sequences
 * stream0 .. stream0+ncol-1. This call may synchronise the device, so make it while no kernel that waits for a peer (an
 * NCCL send/recv) is queued - in practice right after bn_model_finalize, once for every (stream0, ncol) the host will use.
 * bn_model_stage and bn_model_stage_batch never build a schedule themselves: a pair that was not prepared is refused
 * with BN_ERR_STATE. */
int bn_model_stage_prepare(bn_model *m, int stream0, int ncol);
/* One pipeline stage (reference: the contiguous layer ranges of fleet_split_schedule, runtime_vk/gpu_fleet.h:990,
 * and the per-hop 16 KiB hidden-state hand-off, gpu_fleet.h:97): run this device's blocks for one token of
 * sequence `stream` at position pos. First stage: tok >= 0 is the token id, tok < 0 reads it from the int at
 * (in, in_off). Other stages: (in, in_off) holds the `hidden` fp32 values from the previous stage. Output: the
 * hidden state at (out, out_off), or on the last stage the greedy pick as one int. Enqueues only - no host wait.
 * Needs bn_model_stage_prepare(m, stream, 0). A token id read from device memory that lies outside the vocabulary is
 * replaced by 0 and reported by the next bn_sync (BN_ERR_ARG). */
int bn_model_stage(bn_model *m, int stream, int tok, int pos, const bn_buf *in, size_t in_off, bn_buf *out, size_t out_off);
/* The same stage for ncol consecutive sequences stream0 .. stream0+ncol-1 in one pass (the micro-batch of the layer
 * pipeline): every projection reads its weights once for all of them (tcgen05 kernel, bn_gemm_q81), the other
 * kernels run one grid slice per sequence. pos[c] is the position of sequence stream0+c. First stage: tok != NULL gives
 * the token ids, tok == NULL reads ncol ints from (in, in_off). Other stages: (in, in_off) holds ncol x hidden fp32,
 * sequence-major. Output: ncol x hidden fp32, or ncol ints (the greedy picks) on the last stage. Each sequence's result
 * is bit-identical to what bn_model_stage gives for it alone. Needs bn_hparams.batch_cols >= ncol and
 * bn_model_stage_prepare(m, stream0, ncol). Enqueues only. */
int bn_model_stage_batch(bn_model *m, int stream0, int ncol, const int *tok, const int *pos, const bn_buf *in, size_t in_off,
                         bn_buf *out, size_t out_off);

/* Output head sharded by rows over the stages of a pipeline (the reference charges the head's bytes to the last GPU of
 * its byte-balanced split, runtime_vk/gpu_fleet.h:1013-1020; here every stage takes an equal slice of the rows instead,
 * so the last stage is no longer the long one). Call before bn_model_finalize: this model keeps rows
 * [row_begin, row_end) of output.weight (128-row boundaries; row_end may be the vocabulary size) for the multi-sequence
 * pass and needs output.weight and output_norm.weight whatever its block range. Its last stage then returns the
 * hidden state from bn_model_stage_batch like every other stage, and bn_model_stage refuses. */
int bn_model_set_head_rows(bn_model *m, int row_begin, int row_end);
/* One shard of the head for ncol sequences: (in, in_off) holds the final hidden state, ncol x hidden fp32; output norm,
 * rotation, this model's rows of the head and the first maximum over them. Writes ncol candidates to (out, out_off):
 * 8 bytes each, fp32 value then int32 row in the whole vocabulary (0x7FFFFFFF when no row of the shard qualified).
 * Enqueues only. It reads the hidden states where they lie and uses no scratch that a stage pass uses, so it may be
 * enqueued on another stream (bn_use_stream around the call) while a stage pass of the same model runs; two head calls
 * must not overlap each other. */
int bn_model_head_batch(bn_model *m, int ncol, const bn_buf *in, size_t in_off, bn_buf *out, size_t out_off);
/* The pick over all shards: (cands, cands_off) holds n_shards x ncol candidates, shards in ascending row order; the
 * first maximum of every sequence (Sampler::pick's rule, runtime_vk/bonsai_forward.h:2568-2570: greater value, then
 * lower row) goes to (out, out_off) as ncol int32 token ids - the same ids the unsharded head gives. Enqueues only. */
int bn_model_pick_batch(bn_model *m, int ncol, int n_shards, const bn_buf *cands, size_t cands_off, bn_buf *out, size_t out_off);
/* timing fixture (reference: BONSAI_KVFILL, bonsai_forward.h:1338-1378): mark the first n_positions of a
 * stream's KV caches as filled with 1.0 so long-context steps can be timed without a long prefill */
int bn_model_fill_kv(bn_model *m, int stream, int n_positions);
/* wrap device memory owned by the caller (the benchmark's NCCL buffers) as a bn_buf; bn_free releases only the handle */
int bn_wrap(bn_ctx *ctx, void *device_ptr, size_t bytes, bn_buf **out);
/* run this context's work on a stream owned by the caller (so it orders with the caller's NCCL calls) */
int bn_use_stream(bn_ctx *ctx, void *cuda_stream);

/* n_steps greedy tokens chained on the device: the pick of step i is the input of step i+1 with no
 * host round trip (the reference reads 248 320 logits back and picks on the host every token,
 * bonsai_forward.h:712,749,2890-2997). out_tokens (may be NULL) receives the n_steps picks; when it
 * is NULL the call only enqueues and returns. The first call captures the token schedule into a CUDA
 * graph. */
int bn_model_decode(bn_model *m, int first_tok, int pos0, int n_steps, int *out_tokens);
/* measurement aid (reference: the BONSAI_PIPE probe that brackets all 201 projections,
 * runtime_vk/bonsai_vk.cpp:1452): launch every PTQ1_0 projection of one token back to back on the
 * model's own weights, `reps` times after one untimed pass, and return the CUDA-event time of one sweep */
int bn_model_gemv_sweep(bn_model *m, int reps, float *ms_per_sweep);
/* lab: device time of what runs between a block's projections, per layer, averaged over `reps` sweeps of all layers of
 * the kind: the gated-delta-net core (reads and writes the layer's recurrent state once) and the attention chain (K/V
 * insert + decode over the prefix that ends at the current position). Advances the recurrent state and rewrites the
 * cache row of the current position: for measurement on a model that is reset or discarded afterwards. */
int bn_model_mixer_sweep(bn_model *m, int reps, float *us_per_gdn_layer, float *us_per_attn_layer);
/* profiling aid (reference: BONSAI_PROFILE per-token ledger, bonsai_forward.h:650-662): run one token with
 * every fused projection kernel recording 8 device time stamps in ns (CTA 0: start, first copies issued,
 * previous kernel done, norm done, rotated input built, quantised, first weights awaited, end).
 * stamps_out receives [n_phases][8]. */
int bn_model_profile_token(bn_model *m, int tok, int pos, unsigned long long *stamps_out, int max_phases, int *n_phases);
/* copy a device-side result or state region to the host (reference: act_rd / kv_dump). index = the recurrent or
 * attention layer for the state / cache selectors; for BN_READ_LOGITS the column of the last multi-sequence pass (0 for
 * a single sequence) - what a host-side sampler reads (reference: Sampler::pick over the logits, bonsai_forward.h:2544) */
int bn_model_read(bn_model *m, int what, int index, void *dst, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif
