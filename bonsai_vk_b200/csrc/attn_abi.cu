// attn_abi.cu - op-level entry points of the decode-attention layer (reference harness: align_attn.cpp legs A-F
// drive the same three stages - norm/rope/pack + cache insert, QK + softmax, PV + gate - on caller-supplied rows).
#include "ops.cuh"

namespace {

struct Lay { size_t k_scale, v_data, v_scale, bytes; };
Lay kv_layout(const bn_attn_dims &d) {
    const size_t n = size_t(d.cap) * d.n_kv * d.head_dim;
    size_t o = 0;
    auto al = [&](size_t b) { size_t r = o; o += (b + 255) & ~size_t(255); return r; };
    Lay L;
    al(d.k_mode == 0 ? n : n * 2);
    L.k_scale = al(d.k_mode == 0 ? n / 32 * 2 : 0);
    L.v_data = al(d.v_mode == 0 ? n : n * 2);
    L.v_scale = al(d.v_mode == 0 ? n / 32 * 2 : 0);
    L.bytes = o;
    return L;
}
int splits_for(int cap) { return cap >= 16384 ? 256 : (cap >= 4096 ? 64 : (cap >= 512 ? 8 : 1)); }

struct Scr { size_t pos, q16f, gate, score, pe, esum, pv, bytes; };
Scr scratch_layout(const bn_attn_dims &d) {
    const size_t QD = size_t(d.n_head) * d.head_dim;
    size_t o = 0;
    auto al = [&](size_t b) { size_t r = o; o += (b + 255) & ~size_t(255); return r; };
    Scr s;
    s.pos = al(size_t(d.cap) * 4); s.q16f = al(QD * 4); s.gate = al(QD * 4);
    s.score = al(size_t(d.n_head) * d.cap * 4); s.pe = al(size_t(d.n_head) * d.cap * 4);
    s.esum = al(size_t(d.n_head) * 1026 * 4); s.pv = al(size_t(splits_for(d.cap)) * QD * 4);
    s.bytes = o;
    return s;
}
int check_dims(const bn_attn_dims *d, const char *who) {
    BN_REQUIRE(d, BN_ERR_ARG, "%s: null dims", who);
    BN_REQUIRE(d->head_dim == 256 && d->n_kv > 0 && d->n_head % d->n_kv == 0, BN_ERR_ARG, "%s: head_dim must be 256 and n_head a multiple of n_kv", who);
    { const int g = d->n_head / d->n_kv; BN_REQUIRE((g == 1 || g == 2 || g == 4 || g == 8) && d->n_head <= 256, BN_ERR_ARG, "%s: %d query heads per kv head (1, 2, 4 or 8 are built)", who, g); }
    BN_REQUIRE(d->cap > 0 && d->cap % 2 == 0 && d->n_rot > 0 && d->n_rot <= 256 && d->n_rot % 2 == 0, BN_ERR_ARG, "%s: bad cap or rope dims", who);
    BN_REQUIRE((d->k_mode | 1) == 1 && (d->v_mode | 1) == 1, BN_ERR_ARG, "%s: kv modes are 0 (q8_0) or 1 (fp16)", who);
    return BN_OK;
}
bnk::AttnDims to_dims(const bn_attn_dims &d) {
    return bnk::AttnDims{d.n_head, d.n_kv, d.head_dim, d.n_rot, d.cap, d.rms_eps, d.rope_base, d.k_mode, d.v_mode};
}
bnk::KvLayer kv_of(const bn_attn_dims &d, const bn_buf *kv, size_t off) {
    const Lay L = kv_layout(d);
    char *base = bn_ptr<char>(kv, off);
    bnk::KvLayer k;
    k.k_data = base;
    k.k_scale = d.k_mode == 0 ? reinterpret_cast<uint16_t *>(base + L.k_scale) : nullptr;
    k.v_data = base + L.v_data;
    k.v_scale = d.v_mode == 0 ? reinterpret_cast<uint16_t *>(base + L.v_scale) : nullptr;
    return k;
}
__global__ void k_iota(int *p, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = i;
}

}  // namespace

extern "C" {

size_t bn_attn_kv_bytes(const bn_attn_dims *d) { return d ? kv_layout(*d).bytes : 0; }
size_t bn_attn_scratch_bytes(const bn_attn_dims *d) { return d ? scratch_layout(*d).bytes : 0; }

int bn_attn_insert(bn_ctx *ctx, const bn_attn_dims *d, bn_buf *kv, size_t kv_off, const bn_buf *k_rows, size_t k_off,
                   const bn_buf *v_rows, size_t v_off, int n, int pos0, const bn_buf *qg, size_t qg_off, const bn_buf *q_norm,
                   size_t qn_off, const bn_buf *k_norm, size_t kn_off, bn_buf *scratch, size_t scratch_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_attn_insert: null context");
    int rc = check_dims(d, "bn_attn_insert");
    if (rc) return rc;
    const size_t QD = size_t(d->n_head) * d->head_dim, KD = size_t(d->n_kv) * d->head_dim;
    BN_REQUIRE(n > 0 && pos0 >= 0 && pos0 + n <= d->cap, BN_ERR_BOUNDS, "bn_attn_insert: positions [%d, %d) outside capacity %d", pos0, pos0 + n, d->cap);
    BN_RANGE(kv, kv_off, kv_layout(*d).bytes, 256, "bn_attn_insert kv");
    BN_RANGE(k_rows, k_off, size_t(n) * KD * 4, 16, "bn_attn_insert k rows");
    BN_RANGE(v_rows, v_off, size_t(n) * KD * 4, 16, "bn_attn_insert v rows");
    BN_RANGE(qg, qg_off, 2 * QD * 4, 16, "bn_attn_insert q|gate row");
    BN_RANGE(q_norm, qn_off, size_t(d->head_dim) * 4, 4, "bn_attn_insert q norm");
    BN_RANGE(k_norm, kn_off, size_t(d->head_dim) * 4, 4, "bn_attn_insert k norm");
    const Scr S = scratch_layout(*d);
    BN_RANGE(scratch, scratch_off, S.bytes, 256, "bn_attn_insert scratch");
    char *sb = bn_ptr<char>(scratch, scratch_off);
    int *pos = reinterpret_cast<int *>(sb + S.pos);
    k_iota<<<(d->cap + 255) / 256, 256, 0, ctx->stream>>>(pos, d->cap);
    BN_COUNT(1);
    const bnk::AttnDims a = to_dims(*d);
    const bnk::KvLayer K = kv_of(*d, kv, kv_off);
    for (int t = 0; t < n; ++t)
        bnk::attn_prep(ctx->stream, a, bn_ptr<float>(qg, qg_off), bn_ptr<float>(k_rows, k_off) + size_t(t) * KD,
                       bn_ptr<float>(v_rows, v_off) + size_t(t) * KD, bn_ptr<float>(q_norm, qn_off), bn_ptr<float>(k_norm, kn_off),
                       pos + pos0 + t, K, reinterpret_cast<float *>(sb + S.q16f), reinterpret_cast<float *>(sb + S.gate));
    return bn_launch_check(ctx, "bn_attn_insert");
}

int bn_attn_attend(bn_ctx *ctx, const bn_attn_dims *d, const bn_buf *kv, size_t kv_off, int pos, bn_buf *scratch,
                   size_t scratch_off, bn_buf *pregate, size_t pg_off, bn_buf *gated, size_t g_off) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_attn_attend: null context");
    int rc = check_dims(d, "bn_attn_attend");
    if (rc) return rc;
    const size_t QD = size_t(d->n_head) * d->head_dim;
    BN_REQUIRE(pos >= 0 && pos < d->cap, BN_ERR_BOUNDS, "bn_attn_attend: position %d outside capacity %d", pos, d->cap);
    BN_RANGE(kv, kv_off, kv_layout(*d).bytes, 256, "bn_attn_attend kv");
    const Scr S = scratch_layout(*d);
    BN_RANGE(scratch, scratch_off, S.bytes, 256, "bn_attn_attend scratch");
    if (pregate) BN_RANGE(pregate, pg_off, QD * 4, 4, "bn_attn_attend pregate");
    BN_RANGE(gated, g_off, QD * 4, 4, "bn_attn_attend gated");
    char *sb = bn_ptr<char>(scratch, scratch_off);
    bnk::attn_decode(ctx->stream, to_dims(*d), reinterpret_cast<float *>(sb + S.q16f), reinterpret_cast<float *>(sb + S.gate),
                     reinterpret_cast<int *>(sb + S.pos) + pos, kv_of(*d, kv, kv_off), reinterpret_cast<float *>(sb + S.score),
                     reinterpret_cast<float *>(sb + S.pe), reinterpret_cast<float *>(sb + S.esum), reinterpret_cast<float *>(sb + S.pv),
                     splits_for(d->cap), pregate ? bn_ptr<float>(pregate, pg_off) : nullptr, bn_ptr<float>(gated, g_off), true);
    return bn_launch_check(ctx, "bn_attn_attend");
}

}  // extern "C"
