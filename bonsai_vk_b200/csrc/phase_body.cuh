// phase_body.cuh - device-side body of the fused projection "phase": [prologue that rebuilds the rotated, q8_1-quantised
// input of a projection from the previous phase's outputs] + [PTQ1_0 x q8_1 GEMV streamed through a bulk-copy ring] +
// [epilogue: residual add, swiglu of a gate/up row pair, silu of a row range, or a first-maximum pick]. Two kernels are
// built from it: k_phase_gemv (one launch per projection, phase_gemv.cu) and k_token (one launch per token or per run of
// tokens, token_kernel.cu), which walks a list of phases with grid-wide barriers between them.
//
// Work split. A CTA (16 compute warps + 1 copy warp) owns a contiguous run of 16-row tiles and computes those rows over
// ALL of K, so no partial sums ever leave the CTA (no atomics, no fences). K is walked in chunks of up to 32 blocks (4096
// weights); inside a chunk warp w owns blocks 2w and 2w+1 and keeps the tensor-core operand registers of those two blocks
// for the whole chunk. The canonical summation order of the projection,
//     v_b = d_w * ((t0 + t1) + (t2 + t3)),  p_g = (v_4g + v_4g+1) + (v_4g+2 + v_4g+3),  out = p_0 + p_1 + ...
// falls out of that ownership: a warp adds its two blocks, a pair of warps forms p_g, and 16 threads add the p_g in
// ascending order.
//
// Data movement. Per item = (chunk, tile) the 16 row slices (28 bytes x blocks-per-chunk each, contiguous in global
// memory) are fetched by 16 cp.async.bulk copies into a ring stage with a padded row pitch (bank-conflict-free register
// loads); 8 stages (117 KB in flight per SM). The copy warp refills a stage when all 16 compute warps have arrived on the
// stage's "empty" mbarrier, which they do as soon as the rows are in registers. Items are numbered by a counter that
// keeps running across phases (`git`), so in the whole-token kernel the copy warp streams the next projection's weights
// while the compute warps are still in a barrier, a prologue or a non-projection phase: weights depend on nothing.
//
// Every wait on an mbarrier is bounded; a wait that gives up records it in the error word, raises the CTA's abort flag
// (every later wait returns at once) and the kernel runs to its end (results are then invalid; the host reports
// BN_ERR_TIMEOUT).
#pragma once
#include "phase_gemv.cuh"
#include "quant.cuh"
#include "rotate_quant.cuh"

namespace bnk {
namespace phase {

constexpr int NT = PHASE_THREADS, NWARP = NT / 32, STAGES = 8, MAXCH = 32, MAXK = 12288 + 4096;
constexpr int NTHREADS = NT + 32;      // 16 compute warps + 1 copy-issuing warp
constexpr int RB = 8;                  // tiles per cross-warp reduction batch (2 batches of slots)
constexpr int STAGE_BYTES = 16 * (MAXCH * 28 + 16);     // 14592

struct SL {   // shared-memory layout, byte offsets from a 128-byte aligned base
    static constexpr int ring = 0;
    static constexpr int bars = ring + STAGES * STAGE_BYTES;               // full[STAGES], empty[STAGES], abort flag
    static constexpr int op = bars + (2 * STAGES + 16) * 8 + 64;                  // the running phase's record (whole-token kernel)
    static constexpr int feed = op + 512;                                  // whole-token kernel: this CTA's item table of the token's projections
    static constexpr int btab = feed + 32 * 216;                           // operand-build table, [4][32] x 16 bytes (build_btab)
    static constexpr int hinv = btab + 2048;                               // norm factors (survive until the next norm)
    static constexpr int codes = hinv + 128 * 4;                           // int8 codes of the whole input (K bytes)
    static constexpr int ds = codes + MAXK;                                // (fp16 d | fp16 s) per sub-block
    static constexpr int red = ds + (MAXK / 128) * 16;
    static constexpr int sv = red + 256 * 4;                               // [2 * RB][NWARP][16] floats
    static constexpr int acc = sv + 2 * RB * NWARP * 16 * 4;               // [<=64][16] running sums across chunks
    static constexpr int xs = acc + 64 * 16 * 4;                           // hat_block floats follow
    // everything from `codes` on is free for the other phases of the whole-token kernel while no projection runs
    static constexpr int scratch = codes;
};
__host__ __device__ constexpr int smem_bytes(int hat_block) { return SL::xs + (hat_block < 32 ? 32 : hat_block) * 4 + 128; }

// the kernel's dynamic shared memory, named here so that every function can form its addresses from the symbol itself
// (a pointer passed through a function argument would turn shared-memory accesses into generic ones)
__device__ __forceinline__ unsigned char *dyn_smem() {
    extern __shared__ __align__(128) unsigned char bn_dyn_smem[];
    return bn_dyn_smem;
}

struct Smem {
    unsigned char *ring;
    int8_t *codes;
    uint32_t *dsw;
    float *red, *sv, *accs, *hinv, *xs;
    uint4 *btab;
    uint64_t *full, *empty, *done;
    volatile int *abort;
    volatile uint32_t *red_seq;
    unsigned char *scratch;
};
__device__ __forceinline__ Smem carve(unsigned char *smem) {
    Smem s;
    s.ring = smem + SL::ring;
    s.full = reinterpret_cast<uint64_t *>(smem + SL::bars);
    s.empty = s.full + STAGES;
    s.done = s.empty + STAGES;
    s.abort = reinterpret_cast<volatile int *>(s.done + 16);
    s.red_seq = reinterpret_cast<volatile uint32_t *>(s.abort + 1);
    s.hinv = reinterpret_cast<float *>(smem + SL::hinv);
    s.btab = reinterpret_cast<uint4 *>(smem + SL::btab);
    s.codes = reinterpret_cast<int8_t *>(smem + SL::codes);
    s.dsw = reinterpret_cast<uint32_t *>(smem + SL::ds);
    s.red = reinterpret_cast<float *>(smem + SL::red);
    s.sv = reinterpret_cast<float *>(smem + SL::sv);
    s.accs = reinterpret_cast<float *>(smem + SL::acc);
    s.xs = reinterpret_cast<float *>(smem + SL::xs);
    s.scratch = smem + SL::scratch;
    return s;
}

__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t *b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
// bounded wait; on giving up records the fact, raises the CTA's abort flag and returns (no trap, no endless loop)
__device__ __forceinline__ void mbar_wait(uint64_t *b, uint32_t parity, int *err, volatile int *abort, int limit = 1 << 22) {
    const uint32_t addr = smem_u32(b);
    {   // the common case: the phase is complete when the wait is reached (one try, no loop bookkeeping)
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (__builtin_expect(ok != 0u, 1)) return;
    }
    for (int it = 0; it < limit; ++it) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return;
        if (it > 256) { __nanosleep(20); if (abort && *abort) return; }
    }
    if (err) atomicExch(err, 1);
    if (abort) *abort = 1;
}
__device__ __forceinline__ void init_barriers(const Smem &s) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(s.full + i, 1); mbar_init(s.empty + i, NWARP); }
    *s.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bulk_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// barrier over the 16 compute warps (the copy warp never joins it)
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); }

// loads of values another CTA of the same launch may have written: through L2, never from this SM's L1
template <bool CG> __device__ __forceinline__ float ldf(const float *p) { return CG ? __ldcg(p) : *p; }
template <bool CG> __device__ __forceinline__ float4 ldf4(const float *p) {
    return CG ? __ldcg(reinterpret_cast<const float4 *>(p)) : *reinterpret_cast<const float4 *>(p);
}

__device__ __forceinline__ float warp_tree128(float e0, float e1, float e2, float e3) {
    float a = __fadd_rn(__fadd_rn(e0, e2), __fadd_rn(e1, e3));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, s));
    return a;
}

// Sylvester-Walsh-Hadamard butterflies, h ascending (hat4096.comp:41-60), any thread mapping gives the
// same floats because every stage is a set of independent (a+c, a-c) pairs.
// N values = N / hb independent transforms of width hb side by side (a butterfly of distance h < hb never leaves its
// hb-aligned block).
__device__ __forceinline__ void fwht_smem(float *s, int N, int hb, float inv) {
    for (int h = 1; h < hb; h <<= 1) {
        csync();
        for (int i = threadIdx.x; i < (N >> 1); i += NT) {
            const int j = ((i & ~(h - 1)) << 1) | (i & (h - 1));
            const float a = s[j], c = s[j + h];
            s[j] = __fadd_rn(a, c);
            s[j + h] = __fsub_rn(a, c);
        }
    }
    csync();
    for (int i = threadIdx.x; i < N; i += NT) s[i] = __fmul_rn(s[i], inv);
    csync();
}

// Operand registers of one block for a lane, straight from the block's int8 codes (32 dwords in element order). Word L
// pairs with A-register L (quant.cuh: three byte pairs x five levels, then the qh pair): bytes 1 and 3 hold the
// activation codes of the two weight bytes' elements at level t (even column) or t+1 (odd column), zero when that element
// lies outside this lane's sub-block column; bytes 0 and 2 are zero (they face the residue bytes of the product
// registers). Same table as quant.cuh coef().
// Which code dword a word comes from and which two of its bytes it takes depends on the lane only, so it is worked out
// once per kernel (build_btab, before the kernel waits for its input) and kept in shared memory as one entry per (lane,
// word): byte offset of the dword << 16 | byte-permute selector (0x4444 = all zero). Building a block's 16 words is then
// a load and a permute per word.
__device__ __forceinline__ void build_btab(uint4 *btab, int tid) {          // the first 512 threads, one entry each
    const int lane = tid >> 4, i = tid & 15, g = lane >> 2, tig = lane & 3, csb = g >> 1, odd = g & 1;
    uint32_t off = 0u, sel = 0x4444u;
    if (i < 15) {
        const int hd = i / 5, t = i - hd * 5;
        const int dwf = (tig == 0) ? 0 : (tig == 1) ? 2 : (tig == 2) ? 3 : 5;
        const int dws = tig < 2 ? 1 : 4;
        const int dw = hd < 2 ? dwf : dws;
        const int h = hd == 0 ? 0 : (hd == 1 ? 1 : (tig & 1));
        const bool cls_a = dw < 4;                            // bytes 0..15 vs bytes 16..23
        const int base = cls_a ? dw : 16 + dw, stride = cls_a ? 4 : 2;
        const int ts = t + odd;                               // odd columns pair level t with the element of level t + 1
        if (ts <= 4) {
            const int sb = cls_a ? (ts >> 1) : (ts < 2 ? 2 : 3);
            if (sb == csb) { off = uint32_t(base + stride * ts); sel = h ? 0x3414u : 0x2404u; }     // [0, b_h, 0, b_(h+2)]
        }
    } else {
        const int t = tig + odd;                              // qh pair: level tig, elements 120+2t, 121+2t
        if (csb == 3 && t <= 3) { off = uint32_t(30 + (t >> 1)); sel = (t & 1) ? 0x3424u : 0x1404u; }
    }
    reinterpret_cast<uint32_t *>(btab)[((i >> 2) * 32 + lane) * 4 + (i & 3)] = ((off * 4u) << 16) | sel;
}
struct BTab { uint4 e[4]; };
__device__ __forceinline__ BTab load_btab(const uint4 *btab, int lane) {
    BTab t;
#pragma unroll
    for (int k = 0; k < 4; ++k) t.e[k] = btab[k * 32 + lane];
    return t;
}
__device__ __forceinline__ uint32_t breg_word(const unsigned char *cb, uint32_t e) {
    return __byte_perm(*reinterpret_cast<const uint32_t *>(cb + (e >> 16)), 0u, e & 0xFFFFu);
}
__device__ __forceinline__ void build_breg(const uint32_t *c32, const BTab &t, uint2 (&B)[8]) {
    const unsigned char *cb = reinterpret_cast<const unsigned char *>(c32);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        B[2 * k] = make_uint2(breg_word(cb, t.e[k].x), breg_word(cb, t.e[k].y));
        B[2 * k + 1] = make_uint2(breg_word(cb, t.e[k].z), breg_word(cb, t.e[k].w));
    }
}

struct RowRegs { uint32_t h0, h1, h2, hq; };
// The five products v*3^(t+1) of one byte-pair register. x3 and x9 are written as shift-adds so they go to
// the integer ALU while x27, x81, x243 use the multiplier: the two pipes share the decode work evenly.
struct Pow5 { uint32_t p1, p2, p3, p4, p5; };
__device__ __forceinline__ Pow5 pow5(uint32_t v) {
    Pow5 r;
    r.p1 = (v << 1) + v;
    r.p2 = (v << 3) + v;
    r.p3 = v * 27u; r.p4 = v * 81u; r.p5 = v * 243u;
    return r;
}
// two blocks of the same 16 rows: two independent accumulator chains of eight tensor-core steps each
// (integer adds are exact, so the order of the steps changes nothing)
__device__ __forceinline__ void tile_mma2(int (&c)[4], int (&d)[4], const RowRegs &ra, const RowRegs &rb, const uint2 (&B)[8],
                                          const RowRegs &sa, const RowRegs &sb, const uint2 (&C)[8], uint32_t cq) {
    // one accumulator chain per block (8 dependent steps each). Two chains per block, added at the end, were measured
    // slower: the other three warps of the scheduler hide the chain's latency, the extra adds and zero registers cost.
    int (&c2)[4] = c, (&d2)[4] = d;
    Pow5 a = pow5(ra.h0), b = pow5(rb.h0), e = pow5(sa.h0), f = pow5(sb.h0);
    mma_u8s8(c, a.p1, b.p1, a.p2, b.p2, B[0].x, B[0].y);
    mma_u8s8(d, e.p1, f.p1, e.p2, f.p2, C[0].x, C[0].y);
    mma_u8s8(c2, a.p3, b.p3, a.p4, b.p4, B[1].x, B[1].y);
    mma_u8s8(d2, e.p3, f.p3, e.p4, f.p4, C[1].x, C[1].y);
    Pow5 a1 = pow5(ra.h1), b1 = pow5(rb.h1), e1 = pow5(sa.h1), f1 = pow5(sb.h1);
    mma_u8s8(c, a.p5, b.p5, a1.p1, b1.p1, B[2].x, B[2].y);
    mma_u8s8(d, e.p5, f.p5, e1.p1, f1.p1, C[2].x, C[2].y);
    mma_u8s8(c2, a1.p2, b1.p2, a1.p3, b1.p3, B[3].x, B[3].y);
    mma_u8s8(d2, e1.p2, f1.p2, e1.p3, f1.p3, C[3].x, C[3].y);
    mma_u8s8(c, a1.p4, b1.p4, a1.p5, b1.p5, B[4].x, B[4].y);
    mma_u8s8(d, e1.p4, f1.p4, e1.p5, f1.p5, C[4].x, C[4].y);
    a = pow5(ra.h2); b = pow5(rb.h2); e = pow5(sa.h2); f = pow5(sb.h2);
    mma_u8s8(c2, a.p1, b.p1, a.p2, b.p2, B[5].x, B[5].y);
    mma_u8s8(d2, e.p1, f.p1, e.p2, f.p2, C[5].x, C[5].y);
    mma_u8s8(c, a.p3, b.p3, a.p4, b.p4, B[6].x, B[6].y);
    mma_u8s8(d, e.p3, f.p3, e.p4, f.p4, C[6].x, C[6].y);
    mma_u8s8(c2, a.p5, b.p5, ra.hq * cq, rb.hq * cq, B[7].x, B[7].y);
    mma_u8s8(d2, e.p5, f.p5, sa.hq * cq, sb.hq * cq, C[7].x, C[7].y);
}
// exact int -> float for |i| < 2^22 without the conversion unit
__device__ __forceinline__ float small_int_to_float(int i) { return __fsub_rn(__int_as_float(0x4B400000 + i), 12582912.0f); }
__device__ __forceinline__ RowRegs split_row(uint32_t f, uint32_t s2, uint32_t w6, uint32_t sel2) {
    RowRegs r;
    r.h0 = __byte_perm(f, 0u, 0x4240u); r.h1 = __byte_perm(f, 0u, 0x4341u);
    r.h2 = __byte_perm(s2, 0u, sel2);   r.hq = __byte_perm(w6, 0u, 0x4140u);
    return r;
}

// ---- which tiles a CTA owns ------------------------------------------------------------------------------------------
struct Work {
    int nb, ntiles, CH, nchunks, rowb, gpitch;
    int t0, nt, items;          // run of (virtual) tiles [t0, t0 + nt), items = nt * nchunks, chunk-major
    int pair, half_tiles;       // EPI_SWIGLU: virtual tile v = 2p / 2p+1 is tile p of the first / second half of the rows
};
__device__ __forceinline__ Work phase_work(const PhaseArgs &a, int cta, int ncta) {
    Work w;
    w.nb = a.K >> 7;
    w.ntiles = (a.M + 15) >> 4;
    w.CH = w.nb <= MAXCH ? w.nb : MAXCH;
    w.nchunks = w.nb / w.CH;
    w.rowb = w.CH * 28;
    w.gpitch = w.rowb + 16;
    w.pair = a.epi == EPI_SWIGLU;
    w.half_tiles = w.ntiles >> 1;
    if (w.pair) {   // whole pairs per CTA
        const int np = w.half_tiles;
        const int p0 = int((long long)cta * np / ncta), p1 = int((long long)(cta + 1) * np / ncta);
        w.t0 = 2 * p0; w.nt = 2 * (p1 - p0);
    } else {
        w.t0 = int((long long)cta * w.ntiles / ncta);
        w.nt = int((long long)(cta + 1) * w.ntiles / ncta) - w.t0;
    }
    w.items = w.nt * w.nchunks;
    return w;
}
__device__ __forceinline__ int tile_of(const Work &w, int v) { return w.pair ? ((v & 1) ? w.half_tiles + (v >> 1) : (v >> 1)) : v; }

// copy warp: request item `it` of this phase into ring stage git % STAGES (git = running item number of the launch)
__device__ __forceinline__ void issue_item(const PhaseArgs &a, const Work &w, const Smem &s, int it, uint32_t git, int lane) {
    const int chunk = it / w.nt, tile = tile_of(w, w.t0 + (it - chunk * w.nt)), stage = int(git % STAGES);
    if (lane == 0) mbar_expect_tx(s.full + stage, 16u * uint32_t(w.CH) * 28u);
    __syncwarp();
    if (lane < 16) {
        // the last tile of the matrix may be short: clamp so the copy stays inside the matrix
        const int row = min(tile * 16 + lane, a.M - 1);
        bulk_copy(s.ring + stage * STAGE_BYTES + lane * w.gpitch, a.W + (size_t(row) * w.nb + size_t(chunk) * w.CH) * 28,
                  uint32_t(w.rowb), s.full + stage);
    }
}

// constants of the prologue (norm weights, sign vector) that do not depend on the previous phase: load them early
struct Preload { bool on; int sg[8]; float w[8]; };
__device__ __forceinline__ void preload(const PhaseArgs &a, int tid, Preload &p) {
    p.on = (a.pro == PRO_NORM || a.pro == PRO_PLAIN) && a.hat_block >= 256 && tid < a.hat_block / 8;
    if (!p.on) return;
    const int4 s0 = *reinterpret_cast<const int4 *>(a.signs + tid * 8), s1 = *reinterpret_cast<const int4 *>(a.signs + tid * 8 + 4);
    p.sg[0] = s0.x; p.sg[1] = s0.y; p.sg[2] = s0.z; p.sg[3] = s0.w; p.sg[4] = s1.x; p.sg[5] = s1.y; p.sg[6] = s1.z; p.sg[7] = s1.w;
    if (a.pro == PRO_NORM) {
        const float4 n0 = *reinterpret_cast<const float4 *>(a.w + tid * 8), n1 = *reinterpret_cast<const float4 *>(a.w + tid * 8 + 4);
        p.w[0] = n0.x; p.w[1] = n0.y; p.w[2] = n0.z; p.w[3] = n0.w; p.w[4] = n1.x; p.w[5] = n1.y; p.w[6] = n1.z; p.w[7] = n1.w;
    }
}

// q8_1 of nsub 32-element sub-blocks of xs: 4 threads per sub-block, 8 consecutive elements each. codes / dsw point at
// the first sub-block's codes and (d | s) word.
__device__ __forceinline__ void q81_pass(const float *xs, int8_t *codes, uint32_t *dsw, int nsub, int tid) {
    for (int sbk0 = 0; sbk0 < nsub; sbk0 += NT / 4) {
        const int sbk = sbk0 + (tid >> 2), q4 = tid & 3;
        const bool live = sbk < nsub;
        float e[8];
        if (live) {
            const float4 *src = reinterpret_cast<const float4 *>(xs + sbk * 32 + q4 * 8);
            const float4 v0 = src[0], v1 = src[1];
            e[0] = v0.x; e[1] = v0.y; e[2] = v0.z; e[3] = v0.w; e[4] = v1.x; e[5] = v1.y; e[6] = v1.z; e[7] = v1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = 0.0f;
        }
        const Q8x8 q = quant8_of32(e);
        if (live) {
            uint32_t *cw = reinterpret_cast<uint32_t *>(codes + sbk * 32 + q4 * 8);
            cw[0] = q.w0; cw[1] = q.w1;
            if (q4 == 0) dsw[sbk] = float_to_half_bits(q.d) | (float_to_half_bits(__fmul_rn(q.d, float(q.sum))) << 16);
        }
    }
}

#define BN_STAMP(i) do { if (a.stamps && cta == 0 && threadIdx.x == 0) a.stamps[i] = gtime(); } while (0)

// ---- prologue: int8 codes and (d, s) of the whole rotated input, in shared memory (compute warps only) -----------------
// CG: the inputs may have been written by other CTAs of this launch (whole-token kernel): read them through L2.
template <bool CG>
__device__ __forceinline__ void prologue(const PhaseArgs &a, const Smem &s, const Preload &pl, int cta) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = a.K, nb = K >> 7;
    int8_t *codes = s.codes;
    uint32_t *dsw = s.dsw;
    float *red = s.red, *hinv = s.hinv, *xs = s.xs;
    if (a.pro == PRO_PACKED) {
        BN_STAMP(3); BN_STAMP(4);
        for (int i = tid; i < nb * 32; i += NT) reinterpret_cast<uint32_t *>(codes)[i] = a.pack[size_t(i >> 5) * Q81_DWORDS + 4 + (i & 31)];
        for (int i = tid; i < nb * 4; i += NT) dsw[i] = a.pack[size_t(i >> 2) * Q81_DWORDS + (i & 3)];
        csync();
        return;
    }
    float inv = 1.0f;
    float xe[8];
    const bool merged = a.pro == PRO_NORM && K == 4096 && a.hat_block == 4096;   // one pass over x0: norm and input
    if (merged) {
        const float4 x0 = ldf4<CG>(a.x0 + tid * 8), x1 = ldf4<CG>(a.x0 + tid * 8 + 4);
        xe[0] = x0.x; xe[1] = x0.y; xe[2] = x0.z; xe[3] = x0.w; xe[4] = x1.x; xe[5] = x1.y; xe[6] = x1.z; xe[7] = x1.w;
        // lane slice l = elements 16l .. 16l+15 summed ascending: the even thread sums its 8 squares, hands the
        // running sum to its odd neighbour, which continues the same chain
        float sq = 0.0f;
        if (!(tid & 1)) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sq = __fadd_rn(sq, __fmul_rn(xe[i], xe[i]));
        }
        const float up = __shfl_up_sync(0xFFFFFFFFu, sq, 1);
        if (tid & 1) {
            sq = up;
#pragma unroll
            for (int i = 0; i < 8; ++i) sq = __fadd_rn(sq, __fmul_rn(xe[i], xe[i]));
            red[tid >> 1] = sq;
        }
        csync();
        {
            // every warp runs the same tree over the 256 partial sums (the same adds in the same order give the same
            // float in every warp): no second barrier, no trip through shared memory for the factor
            float v[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) v[w] = red[32 * w + lane];
            float t = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[4]), __fadd_rn(v[2], v[6])),
                                __fadd_rn(__fadd_rn(v[1], v[5]), __fadd_rn(v[3], v[7])));
#pragma unroll
            for (int s2 = 16; s2 > 0; s2 >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xFFFFFFFFu, t, s2));
            inv = __frcp_rn(__fsqrt_rn(__fadd_rn(mean_of(t, K), a.eps)));
            if (tid == 0) {
                hinv[0] = inv;
                if (a.inv_out && cta == 0) a.inv_out[0] = inv;
            }
        }
    } else if (a.pro == PRO_NORM) {
        // rms_norm.comp order: 256 lane slices of `per` consecutive elements summed ascending, then the
        // fixed tree p[i] += p[i+s], s = 128..1 (steps 128, 64, 32 across warps, 16..1 inside warp 0)
        const int per = (K + 255) / 256;
        if (tid < 256) {
            float sq = 0.0f;
            if (per == 16 && K == 4096) {
                const float4 v0 = ldf4<CG>(a.x0 + tid * 16), v1 = ldf4<CG>(a.x0 + tid * 16 + 4), v2 = ldf4<CG>(a.x0 + tid * 16 + 8), v3 = ldf4<CG>(a.x0 + tid * 16 + 12);
                const float e[16] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w};
#pragma unroll
                for (int i = 0; i < 16; ++i) sq = __fadd_rn(sq, __fmul_rn(e[i], e[i]));
            } else {
                for (int i = 0; i < per; ++i) {
                    const int d = tid * per + i;
                    if (d < K) { const float v = ldf<CG>(a.x0 + d); sq = __fadd_rn(sq, __fmul_rn(v, v)); }
                }
            }
            red[tid] = sq;
        }
        csync();
        if (warp == 0) {
            float v[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) v[w] = red[32 * w + lane];
            float t = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[4]), __fadd_rn(v[2], v[6])),
                                __fadd_rn(__fadd_rn(v[1], v[5]), __fadd_rn(v[3], v[7])));
#pragma unroll
            for (int s2 = 16; s2 > 0; s2 >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xFFFFFFFFu, t, s2));
            if (lane == 0) {
                const float r = __frcp_rn(__fsqrt_rn(__fadd_rn(mean_of(t, K), a.eps)));
                hinv[0] = r;
                if (a.inv_out && cta == 0) a.inv_out[0] = r;
            }
        }
        csync();
        inv = hinv[0];
    }
    BN_STAMP(3);
    if (a.pro == PRO_GDN_OUT || a.pro == PRO_GDN_OUT_SZ) {
        // per-head RMS factor of the delta-rule output (no weight; 128 squares, tree)
        for (int h = warp; h < a.gdn_heads; h += NWARP) {
            const float *o = a.x0 + h * 128;
            const float e0 = ldf<CG>(o + lane), e1 = ldf<CG>(o + lane + 32), e2 = ldf<CG>(o + lane + 64), e3 = ldf<CG>(o + lane + 96);
            const float ss = warp_tree128(__fmul_rn(e0, e0), __fmul_rn(e1, e1), __fmul_rn(e2, e2), __fmul_rn(e3, e3));
            if (lane == 0) hinv[1 + h] = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(ss, 0.0078125f), a.eps)));
        }
        csync();
    }
    const int HB = a.hat_block;
    const bool fast = HB >= 256;                 // register/shuffle butterflies need 8 elements x >= 32 threads
    // a span = one Hadamard block, or the 32 values of a q8_1 sub-block when the Hadamard block is smaller than that
    const int SP = HB < 32 ? 32 : HB;
    for (int hb = 0; hb < K / SP; ++hb) {
        const int base = hb * SP;
        csync();
        // the input value at absolute index t, before the sign
        auto input = [&](int t) -> float {
            if (a.pro == PRO_PLAIN) return ldf<CG>(a.x0 + t);
            if (a.pro == PRO_NORM) return __fmul_rn(__fmul_rn(ldf<CG>(a.x0 + t), inv), a.w[t]);
            if (a.pro == PRO_SWIGLU) return __fmul_rn(silu_f(ldf<CG>(a.x0 + t)), ldf<CG>(a.x1 + t));
            if (a.pro == PRO_GDN_OUT || a.pro == PRO_GDN_OUT_SZ) {
                const int hd = t >> 7, d = t & 127, sub = a.gdn_heads / a.gdn_qk_heads;
                const int hs = hd / sub + a.gdn_qk_heads * (hd % sub);
                const float nrm = __fmul_rn(__fmul_rn(ldf<CG>(a.x0 + hs * 128 + d), hinv[1 + hs]), a.w[d]);
                const float z = ldf<CG>(a.x1 + hs * 128 + d);          // PRO_GDN_OUT_SZ: silu already applied by the producer
                return __fmul_rn(a.pro == PRO_GDN_OUT ? silu_f(z) : z, nrm);
            }
            const int nfill = a.pos_ptr[0] + 1, per = (nfill + a.pv_splits - 1) / a.pv_splits;   // PRO_ATTN_OUT
            float acc = ldf<CG>(a.x0 + t);
            for (int s2 = 1; s2 < a.pv_splits; ++s2) if (s2 * per < nfill) acc = __fadd_rn(acc, ldf<CG>(a.x0 + size_t(s2) * K + t));
            return __fmul_rn(acc, __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(-ldf<CG>(a.x1 + t)))));
        };
        if (fast) {
            // butterflies h = 1, 2, 4 inside a thread's 8 consecutive elements, h = 8..128 across lanes
            const bool on = tid < HB / 8;
            float v[8];
            if (on) {
                const int tb = base + tid * 8;
                int sg[8];
                if (pl.on && hb == 0) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) sg[r] = pl.sg[r];
                } else {
                    const int4 sg0 = *reinterpret_cast<const int4 *>(a.signs + tb), sg1 = *reinterpret_cast<const int4 *>(a.signs + tb + 4);
                    sg[0] = sg0.x; sg[1] = sg0.y; sg[2] = sg0.z; sg[3] = sg0.w; sg[4] = sg1.x; sg[5] = sg1.y; sg[6] = sg1.z; sg[7] = sg1.w;
                }
                if (merged) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) v[r] = apply_sign(__fmul_rn(__fmul_rn(xe[r], inv), pl.w[r]), sg[r]);
                } else if (a.pro == PRO_PLAIN || a.pro == PRO_NORM) {
                    const float4 x0 = ldf4<CG>(a.x0 + tb), x1 = ldf4<CG>(a.x0 + tb + 4);
                    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                    if (a.pro == PRO_NORM) {
                        const float4 n0 = *reinterpret_cast<const float4 *>(a.w + tb), n1 = *reinterpret_cast<const float4 *>(a.w + tb + 4);
                        const float ne[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                        for (int r = 0; r < 8; ++r) v[r] = apply_sign(__fmul_rn(__fmul_rn(xv[r], inv), ne[r]), sg[r]);
                    } else {
#pragma unroll
                        for (int r = 0; r < 8; ++r) v[r] = apply_sign(xv[r], sg[r]);
                    }
                } else if (a.pro == PRO_GDN_OUT || a.pro == PRO_GDN_OUT_SZ) {
                    // 8 consecutive values lie in one destination head: one source head, three 32-byte loads
                    const int hd = tb >> 7, d0 = tb & 127, sub = a.gdn_heads / a.gdn_qk_heads;
                    const int hs = hd / sub + a.gdn_qk_heads * (hd % sub);
                    const float hi = hinv[1 + hs];
                    const float4 o0 = ldf4<CG>(a.x0 + hs * 128 + d0), o1 = ldf4<CG>(a.x0 + hs * 128 + d0 + 4);
                    const float4 z0 = ldf4<CG>(a.x1 + hs * 128 + d0), z1 = ldf4<CG>(a.x1 + hs * 128 + d0 + 4);
                    const float4 n0 = *reinterpret_cast<const float4 *>(a.w + d0), n1 = *reinterpret_cast<const float4 *>(a.w + d0 + 4);
                    const float ov[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
                    const float zv[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
                    const float nv[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const float nrm = __fmul_rn(__fmul_rn(ov[r], hi), nv[r]);
                        const float zz = a.pro == PRO_GDN_OUT ? silu_f(zv[r]) : zv[r];
                        v[r] = apply_sign(__fmul_rn(zz, nrm), sg[r]);
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < 8; ++r) v[r] = apply_sign(input(tb + r), sg[r]);
                }
                fwht_regs_lanes(v, lane);
                float4 *dst = reinterpret_cast<float4 *>(xs + tid * 8);
                dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            }
            csync();
            if (HB == 4096) {
                fwht_4096_tail(xs, warp, lane, a.hat_inv);
            } else {
                for (int h = 256; h < HB; h <<= 1) {
                    for (int i = tid; i < (HB >> 1); i += NT) {
                        const int j = ((i & ~(h - 1)) << 1) | (i & (h - 1));
                        const float x = xs[j], y = xs[j + h];
                        xs[j] = __fadd_rn(x, y);
                        xs[j + h] = __fsub_rn(x, y);
                    }
                    csync();
                }
                for (int i = tid; i < HB; i += NT) xs[i] = __fmul_rn(xs[i], a.hat_inv);
            }
            csync();
        } else {
            for (int i = tid; i < SP; i += NT) { const int t = base + i; xs[i] = apply_sign(input(t), a.signs[t]); }
            fwht_smem(xs, SP, HB, a.hat_inv);
        }
        BN_STAMP(4);
        q81_pass(xs, codes + base, dsw + (base >> 5), SP / 32, tid);
    }
    csync();
}

// ---- main loop: consume this phase's items from the ring, starting at running item number git0 (compute warps only) ----
// Who refills the ring. The per-projection kernel has a 17th warp that only issues copies (NoFeed here). The whole-token
// kernel has no such warp: at the iteration of running item g the compute warp g % 16 refills the stage of item g - FEED_LAG
// (every warp has taken that item's rows into registers by then, or will within a few hundred cycles) with item
// g - FEED_LAG + STAGES, whatever projection of whatever token that item belongs to.
constexpr int FEED_LAG = 2;
struct NoFeed {
    static constexpr bool on = false;
    __device__ __forceinline__ void operator()(uint32_t) const {}
};
// EPI >= 0: the epilogue is fixed at compile time (the per-projection kernel only ever needs EPI_PLAIN and keeps its lean
// loop); EPI < 0: taken from the phase record at run time (whole-token kernel: one copy of the loop for all phases).
template <int EPI, class Feed>
__device__ __forceinline__ void main_loop(const PhaseArgs &a, const Work &w, const Smem &s, uint32_t git0, int cta, Feed &feed) {
    const int epi = EPI >= 0 ? EPI : a.epi;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int CH = w.CH, nt = w.nt, items = w.items, gpitch = w.gpitch;
    float *sv = s.sv, *accs = s.accs;
    const int first = (tig == 0) ? 0 : (tig == 1) ? 2 : (tig == 2) ? 3 : 5;
    const int second = tig < 2 ? 1 : 4;
    const uint32_t cq = (tig == 0) ? 3u : (tig == 1) ? 9u : (tig == 2) ? 27u : 81u;
    const uint32_t sel2 = (tig & 1) ? 0x4341u : 0x4240u;
    const bool active = 2 * warp < CH;
    const int nactive = CH / 2;                       // warps that own blocks
    uint2 B0[8], B1[8];
    float d0 = 0.0f, s0w = 0.0f, d1 = 0.0f, s1w = 0.0f;
    int chunk = 0, tl = 0;
    bool fresh = true;
    // EPI_ARGMAX: the first maximum over the rows a finishing thread has seen so far lives in shared memory (s.red is free
    // during the main loop), not in registers that would have to survive the whole loop
    float *cand_v = s.red;
    int *cand_i = reinterpret_cast<int *>(s.red + 128);
    if (epi == EPI_ARGMAX && tid < 128) { cand_v[tid] = -INFINITY; cand_i[tid] = 0x7FFFFFFF; }

    // cross-warp sums of a batch of tiles: thread (row, group) walks the batch in order and takes the tiles
    // whose index within the CTA's run is congruent to its group, so the running sum of one tile over the
    // chunks of K always passes through the same thread, in ascending chunk order
    auto reduce_batch = [&](int it_begin, int it_end) {
        if (tid >= 16 * RB) return;
        const int row16 = tid & 15, grp = tid >> 4;
        int c = it_begin / nt, t = it_begin - c * nt;
        for (int it = it_begin; it < it_end; ++it, ++t) {
            if (t == nt) { t = 0; ++c; }
            if ((t & (RB - 1)) != grp) continue;
            const float *bufv = sv + (it & (2 * RB - 1)) * (NWARP * 16);
            float acc = c == 0 ? 0.0f : accs[t * 16 + row16];   // running sum over earlier chunks
            for (int p = 0; p < nactive; p += 2) {
                const float pg = __fadd_rn(bufv[p * 16 + row16], bufv[(p + 1) * 16 + row16]);
                acc = (c == 0 && p == 0) ? pg : __fadd_rn(acc, pg);
            }
            if (c + 1 < w.nchunks) accs[t * 16 + row16] = acc;
            else if (epi == EPI_SWIGLU) accs[t * 16 + row16] = acc;          // gate and up sums meet after the loop
            else {
                const int row = tile_of(w, w.t0 + t) * 16 + row16;
                if (row < a.M) {
                    if (epi == EPI_SILU_FROM && row >= a.epi_arg) accs[t * 16 + row16] = acc;      // silu after the loop
                    else {
                        if (a.out) a.out[row] = acc;
                        if (a.resid_out) a.resid_out[row] = __fadd_rn(acc, ldf<Feed::on>(a.resid_in + row));
                        if (epi == EPI_ARGMAX && (acc > cand_v[tid] || (acc == cand_v[tid] && row < cand_i[tid]))) { cand_v[tid] = acc; cand_i[tid] = row; }
                    }
                }
            }
        }
    };

    int batch_begin = 0;
    for (int it = 0; it < items; ++it, ++tl) {
        if (tl == nt) { tl = 0; ++chunk; fresh = true; }
        const uint32_t git = git0 + uint32_t(it);
        const int stage = int(git % STAGES);
        if (fresh) {
            fresh = false;
            if (active) {
                const int b0 = chunk * CH + 2 * warp;
                const BTab bt = load_btab(s.btab, lane);
                build_breg(reinterpret_cast<const uint32_t *>(s.codes) + b0 * 32, bt, B0);
                build_breg(reinterpret_cast<const uint32_t *>(s.codes) + b0 * 32 + 32, bt, B1);
                const uint32_t w0 = s.dsw[b0 * 4 + tig], w1 = s.dsw[b0 * 4 + 4 + tig];
                d0 = half_bits_to_float(w0); s0w = half_bits_to_float(w0 >> 16);
                d1 = half_bits_to_float(w1); s1w = half_bits_to_float(w1 >> 16);
            }
        }
        if (it == 0) BN_STAMP(6);
        mbar_wait(s.full + stage, (git / STAGES) & 1, a.err, s.abort);
        float va = 0.0f, vb = 0.0f;      // rows g and g+8: v_(2w) + v_(2w+1)
        if (active) {
            const uint32_t *r0 = reinterpret_cast<const uint32_t *>(s.ring + stage * STAGE_BYTES + g * gpitch + warp * 56);
            const uint32_t *r1 = reinterpret_cast<const uint32_t *>(s.ring + stage * STAGE_BYTES + (g + 8) * gpitch + warp * 56);
            const uint32_t a6 = r0[6], b6 = r1[6], e6 = r0[13], f6 = r1[13];
            const uint32_t af = r0[first], as = r0[second], bf = r1[first], bs = r1[second];
            const uint32_t ef = r0[7 + first], es = r0[7 + second], ff = r1[7 + first], fs = r1[7 + second];
            __syncwarp();
            if (lane == 0) mbar_arrive(s.empty + stage);          // rows are in registers: the stage may be refilled
            if (Feed::on && warp == int(git & (NWARP - 1)) && git >= uint32_t(FEED_LAG)) {
                const uint32_t gr = git - FEED_LAG;
                mbar_wait(s.empty + gr % STAGES, (gr / STAGES) & 1, a.err, s.abort);
                feed(gr + STAGES);
            }
            const RowRegs ra = split_row(af, as, a6, sel2), rb = split_row(bf, bs, b6, sel2);
            const RowRegs sa = split_row(ef, es, e6, sel2), sb = split_row(ff, fs, f6, sel2);
            int c[4] = {0, 0, 0, 0}, d[4] = {0, 0, 0, 0};
            tile_mma2(c, d, ra, rb, B0, sa, sb, B1, cq);
            float x0 = fmaf(d0, small_int_to_float(c[0] - 3 * c[1]), -s0w), x1 = fmaf(d0, small_int_to_float(c[2] - 3 * c[3]), -s0w);
            float y0 = fmaf(d1, small_int_to_float(d[0] - 3 * d[1]), -s1w), y1 = fmaf(d1, small_int_to_float(d[2] - 3 * d[3]), -s1w);
            x0 = __fadd_rn(x0, __shfl_xor_sync(0xFFFFFFFFu, x0, 1)); x1 = __fadd_rn(x1, __shfl_xor_sync(0xFFFFFFFFu, x1, 1));
            y0 = __fadd_rn(y0, __shfl_xor_sync(0xFFFFFFFFu, y0, 1)); y1 = __fadd_rn(y1, __shfl_xor_sync(0xFFFFFFFFu, y1, 1));
            x0 = __fadd_rn(x0, __shfl_xor_sync(0xFFFFFFFFu, x0, 2)); x1 = __fadd_rn(x1, __shfl_xor_sync(0xFFFFFFFFu, x1, 2));
            y0 = __fadd_rn(y0, __shfl_xor_sync(0xFFFFFFFFu, y0, 2)); y1 = __fadd_rn(y1, __shfl_xor_sync(0xFFFFFFFFu, y1, 2));
            va = __fadd_rn(__fmul_rn(half_bits_to_float(a6 >> 16), x0), __fmul_rn(half_bits_to_float(e6 >> 16), y0));
            vb = __fadd_rn(__fmul_rn(half_bits_to_float(b6 >> 16), x1), __fmul_rn(half_bits_to_float(f6 >> 16), y1));
            float *bufv = sv + (it & (2 * RB - 1)) * (NWARP * 16);
            if (tig == 0) { bufv[warp * 16 + g] = va; bufv[warp * 16 + g + 8] = vb; }
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(s.empty + stage);
            if (Feed::on && warp == int(git & (NWARP - 1)) && git >= uint32_t(FEED_LAG)) {
                const uint32_t gr = git - FEED_LAG;
                mbar_wait(s.empty + gr % STAGES, (gr / STAGES) & 1, a.err, s.abort);
                feed(gr + STAGES);
            }
        }
        if (it + 1 - batch_begin == RB || it + 1 == items) {
            csync();                                  // every warp has published the tiles of this batch
            reduce_batch(batch_begin, it + 1);
            batch_begin = it + 1;
        }
    }
    if (epi == EPI_SWIGLU) {
        csync();
        for (int idx = tid; idx < (nt >> 1) * 16; idx += NT) {
            const int p = idx >> 4, r16 = idx & 15;
            const int row = ((w.t0 >> 1) + p) * 16 + r16;
            if (row < (a.M >> 1)) a.out2[row] = __fmul_rn(silu_f(accs[(2 * p) * 16 + r16]), accs[(2 * p + 1) * 16 + r16]);
        }
    } else if (epi == EPI_SILU_FROM) {
        csync();
        for (int idx = tid; idx < nt * 16; idx += NT) {
            const int row = (w.t0 + (idx >> 4)) * 16 + (idx & 15);
            if (row < a.M && row >= a.epi_arg) a.out[row] = silu_f(accs[idx]);
        }
    }
    if (epi == EPI_ARGMAX) {
        // the CTA's candidate: first maximum over its rows (128 finishing threads), for the pick over all CTAs
        csync();
        if (tid == 0) {
            float bv = cand_v[0]; int bi = cand_i[0];
            for (int i = 1; i < 128; ++i) if (cand_v[i] > bv || (cand_v[i] == bv && cand_i[i] < bi)) { bv = cand_v[i]; bi = cand_i[i]; }
            a.cand_val[cta] = bv; a.cand_idx[cta] = bi;
        }
    }
    BN_STAMP(7);
}

}  // namespace phase
}  // namespace bnk
