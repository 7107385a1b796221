// phase_gemv.cu - see phase_gemv.cuh. One CTA of 512 threads per SM.
//
// Work split. A CTA owns a contiguous run of 16-row tiles and computes those rows over ALL of K, so no
// partial sums ever leave the CTA (no atomics, no fences). K is walked in chunks of up to 32 blocks
// (4096 weights); inside a chunk warp w owns blocks 2w and 2w+1 and keeps the tensor-core operand
// registers of those two blocks for the whole chunk. The canonical summation order of the projection,
//     v_b = d_w * ((t0 + t1) + (t2 + t3)),  p_g = (v_4g + v_4g+1) + (v_4g+2 + v_4g+3),  out = p_0 + p_1 + ...
// falls out of that ownership: a warp adds its two blocks, a pair of warps forms p_g, and 16 threads
// add the p_g in ascending order.
//
// Data movement. Per (chunk, tile) the 16 row slices (28 bytes x blocks-per-chunk each, contiguous in
// global memory) are fetched by 16 cp.async.bulk copies into a shared-memory stage with a padded row
// pitch (bank-conflict-free register loads); 8 stages (117 KB in flight per SM). A 17th warp only issues copies: it refills a
// stage when all 16 compute warps have arrived on the stage's "empty" mbarrier, which they do as soon as
// the rows are in registers, so warps drift apart by up to 4 tiles and their multiply, tensor-core and
// epilogue phases overlap instead of running in lock-step. The cross-warp sum of a tile is deferred:
// warps park their 16 row values in one of 16 slots and the CTA meets once per 8 tiles.
// The copies of the first stages are issued before the kernel waits for the previous grid
// (programmatic dependent launch) - weights do not depend on it.
//
// Prologue. Every CTA rebuilds the rotated, q8_1-quantised input vector from the previous phase's
// outputs in shared memory (norm / swiglu / gated-delta-net output transform / attention combine, then
// signs, Hadamard butterflies, quantiser), bit-identically to the stand-alone kernels in ops.cu.
//
// Every wait on an mbarrier is bounded; a wait that gives up records it in the error word and the
// kernel carries on to its end (results are then invalid and the host reports BN_ERR_TIMEOUT).
#include "phase_gemv.cuh"
#include "quant.cuh"

namespace {
using namespace bnk;

constexpr int NT = PHASE_THREADS, NWARP = NT / 32, STAGES = 8, MAXCH = 32, MAXK = 12288 + 4096;
constexpr int NTHREADS = NT + 32;      // 16 compute warps + 1 copy-issuing warp
constexpr int RB = 8;                  // tiles per cross-warp reduction batch (2 batches of slots)
constexpr int RPC = 1;                 // matrix rows per bulk copy (rows are contiguous in global memory)
constexpr int STAGE_BYTES = 16 * (MAXCH * 28 + 16);     // 14592 (upper bound for every RPC)

struct SL {   // shared-memory layout, byte offsets from a 128-byte aligned base
    static constexpr int ring = 0;
    static constexpr int codes = ring + STAGES * STAGE_BYTES;          // int8 codes of the whole input (K bytes)
    static constexpr int ds = codes + MAXK;                            // (fp16 d | fp16 s) per sub-block
    static constexpr int red = ds + (MAXK / 128) * 16;
    static constexpr int sv = red + 256 * 4;                           // [2 * RB][NWARP][16] floats
    static constexpr int acc = sv + 2 * RB * NWARP * 16 * 4;                // [<=2][16] running sums across chunks
    static constexpr int hinv = acc + 64 * 16 * 4;
    static constexpr int bars = hinv + 64 * 4;
    static constexpr int xs = bars + 2 * STAGES * 8 + 64;                  // hat_block floats follow
};

__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define STAMP(i) do { if (a.stamps && blockIdx.x == 0 && threadIdx.x == 0) a.stamps[i] = gtime(); } while (0)
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
// bounded wait; on giving up records the fact and returns (no trap, no endless loop)
__device__ __forceinline__ void mbar_wait(uint64_t *b, uint32_t parity, int *err, int limit = 1 << 22) {
    const uint32_t addr = smem_u32(b);
    for (int it = 0; it < limit; ++it) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return;
        if (it > 256) __nanosleep(20);
    }
    if (err) atomicExch(err, 1);
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

__device__ __forceinline__ float warp_tree128(float e0, float e1, float e2, float e3) {
    float a = __fadd_rn(__fadd_rn(e0, e2), __fadd_rn(e1, e3));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, s));
    return a;
}

// Sylvester-Walsh-Hadamard butterflies, h ascending (hat4096.comp:41-60), any thread mapping gives the
// same floats because every stage is a set of independent (a+c, a-c) pairs.
__device__ __forceinline__ void fwht_smem(float *s, int N, float inv) {
    for (int h = 1; h < N; h <<= 1) {
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

// Operand registers of one block for this lane, straight from the block's int8 codes (32 dwords in element
// order). Word L pairs with A-register L (quant.cuh: three byte pairs x five levels, then the qh pair):
// bytes 1 and 3 hold the activation codes of the two weight bytes' elements at level t (even column) or
// t+1 (odd column), zero when that element lies outside this lane's sub-block column; bytes 0 and 2 are
// zero (they face the residue bytes of the product registers). Same table as quant.cuh coef().
__device__ __forceinline__ void build_breg(const uint32_t *c32, int g, int tig, uint2 (&B)[8]) {
    const int csb = g >> 1;
    const bool odd = g & 1;
    const int dwf = (tig == 0) ? 0 : (tig == 1) ? 2 : (tig == 2) ? 3 : 5;
    const int dws = tig < 2 ? 1 : 4;
    uint32_t w[16];
#pragma unroll
    for (int hd = 0; hd < 3; ++hd) {
        const int dw = hd < 2 ? dwf : dws;
        const int h = hd == 0 ? 0 : (hd == 1 ? 1 : (tig & 1));
        const uint32_t sel = h ? 0x3414u : 0x2404u;          // [0, b_h, 0, b_(h+2)]
        const bool cls_a = dw < 4;                            // bytes 0..15 vs bytes 16..23
        const int base = cls_a ? dw : 16 + dw, stride = cls_a ? 4 : 2;
        uint32_t P[6];
#pragma unroll
        for (int t = 0; t < 5; ++t) {
            const int sb = cls_a ? (t >> 1) : (t < 2 ? 2 : 3);
            const uint32_t x = c32[base + stride * t];
            P[t] = (sb == csb) ? __byte_perm(x, 0u, sel) : 0u;
        }
        P[5] = 0u;
#pragma unroll
        for (int t = 0; t < 5; ++t) w[hd * 5 + t] = odd ? P[t + 1] : P[t];
    }
    {
        const int t = tig + (odd ? 1 : 0);                    // qh pair: level tig, elements 120+2t, 121+2t
        uint32_t v = 0u;
        if (csb == 3 && t <= 3) v = __byte_perm(c32[30 + (t >> 1)], 0u, (t & 1) ? 0x3424u : 0x1404u);
        w[15] = v;
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) B[m] = make_uint2(w[2 * m], w[2 * m + 1]);
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
// two blocks of the same 16 rows: four independent accumulator chains of four tensor-core steps each
// (a dependent mma.sync costs tens of cycles; integer adds are exact, so splitting the sum changes nothing)
__device__ __forceinline__ void tile_mma2(int (&c)[4], int (&d)[4], const RowRegs &ra, const RowRegs &rb, const uint2 (&B)[8],
                                          const RowRegs &sa, const RowRegs &sb, const uint2 (&C)[8], uint32_t cq) {
    int c2[4] = {0, 0, 0, 0}, d2[4] = {0, 0, 0, 0};
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
#pragma unroll
    for (int i = 0; i < 4; ++i) { c[i] += c2[i]; d[i] += d2[i]; }
}
// exact int -> float for |i| < 2^22 without the conversion unit
__device__ __forceinline__ float small_int_to_float(int i) { return __fsub_rn(__int_as_float(0x4B400000 + i), 12582912.0f); }
__device__ __forceinline__ RowRegs split_row(uint32_t f, uint32_t s2, uint32_t w6, uint32_t sel2) {
    RowRegs r;
    r.h0 = __byte_perm(f, 0u, 0x4240u); r.h1 = __byte_perm(f, 0u, 0x4341u);
    r.h2 = __byte_perm(s2, 0u, sel2);   r.hq = __byte_perm(w6, 0u, 0x4140u);
    return r;
}

__global__ void __launch_bounds__(NTHREADS, 1) k_phase_gemv(const PhaseArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *ring = smem + SL::ring;
    int8_t *codes = reinterpret_cast<int8_t *>(smem + SL::codes);
    uint32_t *dsw = reinterpret_cast<uint32_t *>(smem + SL::ds);
    float *red = reinterpret_cast<float *>(smem + SL::red);
    float *sv = reinterpret_cast<float *>(smem + SL::sv);
    float *accs = reinterpret_cast<float *>(smem + SL::acc);
    float *hinv = reinterpret_cast<float *>(smem + SL::hinv);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + SL::bars);
    uint64_t *empty = full + STAGES;
    float *xs = reinterpret_cast<float *>(smem + SL::xs);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int M = a.M, K = a.K, nb = K >> 7, ntiles = (M + 15) >> 4;
    const int CH = nb <= MAXCH ? nb : MAXCH, nchunks = nb / CH;      // blocks per chunk, chunks
    // a copy brings RPC consecutive rows when the chunk spans whole rows (they are contiguous in memory)
    const int rpc = (nchunks == 1 && M % RPC == 0) ? RPC : 1;
    const int rowb = CH * 28;                       // bytes of one row slice
    const int gpitch = rpc * rowb + 16;             // pitch of a group of rpc rows
    const int t0 = int((long long)blockIdx.x * ntiles / gridDim.x), t1 = int((long long)(blockIdx.x + 1) * ntiles / gridDim.x);
    const int nt = t1 - t0, items = nt * nchunks;                     // item = (chunk, tile), chunk-major

    STAMP(0);
    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, NWARP); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto issue = [&](int it) {       // called by the copy warp
        const int chunk = it / nt, tile = t0 + (it - chunk * nt), stage = it % STAGES;
        if (lane == 0) mbar_expect_tx(full + stage, 16u * uint32_t(CH) * 28u);
        __syncwarp();
        if (lane < 16 / rpc) {
            // the last tile of the matrix may be short: clamp the group so it stays inside the matrix
            const int row = min(tile * 16 + lane * rpc, M - rpc);
            bulk_copy(ring + stage * STAGE_BYTES + lane * gpitch, a.W + (size_t(row) * nb + size_t(chunk) * CH) * 28,
                      uint32_t(rpc * rowb), full + stage);
        }
    };
    const bool copy_warp = warp == NWARP;
    if (copy_warp) for (int it = 0; it < min(items, STAGES); ++it) issue(it);

    // constants of the prologue (norm weights, sign vector) do not depend on the previous grid either
    const bool pre = (a.pro == PRO_NORM || a.pro == PRO_PLAIN) && a.hat_block >= 256 && tid < a.hat_block / 8;
    int pre_sg[8];
    float pre_w[8];
    if (pre) {
        const int4 s0 = *reinterpret_cast<const int4 *>(a.signs + tid * 8), s1 = *reinterpret_cast<const int4 *>(a.signs + tid * 8 + 4);
        pre_sg[0] = s0.x; pre_sg[1] = s0.y; pre_sg[2] = s0.z; pre_sg[3] = s0.w; pre_sg[4] = s1.x; pre_sg[5] = s1.y; pre_sg[6] = s1.z; pre_sg[7] = s1.w;
        if (a.pro == PRO_NORM) {
            const float4 n0 = *reinterpret_cast<const float4 *>(a.w + tid * 8), n1 = *reinterpret_cast<const float4 *>(a.w + tid * 8 + 4);
            pre_w[0] = n0.x; pre_w[1] = n0.y; pre_w[2] = n0.z; pre_w[3] = n0.w; pre_w[4] = n1.x; pre_w[5] = n1.y; pre_w[6] = n1.z; pre_w[7] = n1.w;
        }
    }
    STAMP(1);
    // everything above touched only constant weights; from here on we read the previous grid's output
    asm volatile("griddepcontrol.wait;" ::: "memory");
    STAMP(2);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (copy_warp) {
        // refill a stage as soon as all 16 compute warps have taken its rows into registers
        for (int it = STAGES; it < items; ++it) {
            mbar_wait(empty + it % STAGES, ((it / STAGES) - 1) & 1, a.err);
            issue(it);
        }
        return;
    }

    // ---- prologue: int8 codes and (d, s) of the whole rotated input, in shared memory ------------------
    if (a.pro == PRO_PACKED) {
        for (int i = tid; i < nb * 32; i += NT) reinterpret_cast<uint32_t *>(codes)[i] = a.pack[size_t(i >> 5) * Q81_DWORDS + 4 + (i & 31)];
        for (int i = tid; i < nb * 4; i += NT) dsw[i] = a.pack[size_t(i >> 2) * Q81_DWORDS + (i & 3)];
    } else {
        float inv = 1.0f;
        float xe[8];
        const bool merged = a.pro == PRO_NORM && K == 4096 && a.hat_block == 4096;   // one pass over x0: norm and input
        if (merged) {
            const float4 x0 = *reinterpret_cast<const float4 *>(a.x0 + tid * 8), x1 = *reinterpret_cast<const float4 *>(a.x0 + tid * 8 + 4);
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
            if (warp == 0) {
                float v[8];
#pragma unroll
                for (int w = 0; w < 8; ++w) v[w] = red[32 * w + lane];
                float t = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[4]), __fadd_rn(v[2], v[6])),
                                    __fadd_rn(__fadd_rn(v[1], v[5]), __fadd_rn(v[3], v[7])));
#pragma unroll
                for (int s2 = 16; s2 > 0; s2 >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xFFFFFFFFu, t, s2));
                if (lane == 0) {
                    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, float(K)), a.eps)));
                    hinv[0] = r;
                    if (a.inv_out && blockIdx.x == 0) a.inv_out[0] = r;
                }
            }
            csync();
            inv = hinv[0];
        } else if (a.pro == PRO_NORM) {
            // rms_norm.comp order: 256 lane slices of `per` consecutive elements summed ascending, then the
            // fixed tree p[i] += p[i+s], s = 128..1 (steps 128, 64, 32 across warps, 16..1 inside warp 0)
            const int per = (K + 255) / 256;
            if (tid < 256) {
                float sq = 0.0f;
                if (per == 16 && K == 4096) {
                    const float4 *xv = reinterpret_cast<const float4 *>(a.x0) + tid * 4;
                    const float4 v0 = xv[0], v1 = xv[1], v2 = xv[2], v3 = xv[3];
                    const float e[16] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w};
#pragma unroll
                    for (int i = 0; i < 16; ++i) sq = __fadd_rn(sq, __fmul_rn(e[i], e[i]));
                } else {
                    for (int i = 0; i < per; ++i) {
                        const int d = tid * per + i;
                        if (d < K) { const float v = a.x0[d]; sq = __fadd_rn(sq, __fmul_rn(v, v)); }
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
                    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, float(K)), a.eps)));
                    hinv[0] = r;
                    if (a.inv_out && blockIdx.x == 0) a.inv_out[0] = r;
                }
            }
            csync();
            inv = hinv[0];
        }
        STAMP(3);
        if (a.pro == PRO_GDN_OUT) {
            for (int h = warp; h < a.gdn_heads; h += NWARP) {
                const float *o = a.x0 + h * 128;
                const float e0 = o[lane], e1 = o[lane + 32], e2 = o[lane + 64], e3 = o[lane + 96];
                const float ss = warp_tree128(__fmul_rn(e0, e0), __fmul_rn(e1, e1), __fmul_rn(e2, e2), __fmul_rn(e3, e3));
                if (lane == 0) hinv[h] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), a.eps)));
            }
            csync();
        }
        const int HB = a.hat_block;
        const bool fast = HB >= 256;                 // register/shuffle butterflies need 8 elements x >= 32 threads
        for (int hb = 0; hb < K / HB; ++hb) {
            const int base = hb * HB;
            csync();
            // the input value at absolute index t, before the sign
            auto input = [&](int t) -> float {
                if (a.pro == PRO_PLAIN) return a.x0[t];
                if (a.pro == PRO_NORM) return __fmul_rn(__fmul_rn(a.x0[t], inv), a.w[t]);
                if (a.pro == PRO_SWIGLU) return __fmul_rn(silu_f(a.x0[t]), a.x1[t]);
                if (a.pro == PRO_GDN_OUT) {
                    const int hd = t >> 7, d = t & 127, sub = a.gdn_heads / a.gdn_qk_heads;
                    const int hs = hd / sub + a.gdn_qk_heads * (hd % sub);
                    const float nrm = __fmul_rn(__fmul_rn(a.x0[hs * 128 + d], hinv[hs]), a.w[d]);
                    return __fmul_rn(silu_f(a.x1[hs * 128 + d]), nrm);
                }
                const int nfill = a.pos_ptr[0] + 1, per = (nfill + a.pv_splits - 1) / a.pv_splits;   // PRO_ATTN_OUT
                float acc = a.x0[t];
                for (int s2 = 1; s2 < a.pv_splits; ++s2) if (s2 * per < nfill) acc = __fadd_rn(acc, a.x0[size_t(s2) * K + t]);
                return __fmul_rn(acc, __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(-a.x1[t]))));
            };
            if (fast) {
                // butterflies h = 1, 2, 4 inside a thread's 8 consecutive elements, h = 8..128 across lanes
                const bool on = tid < HB / 8;
                float v[8];
                if (on) {
                    const int tb = base + tid * 8;
                    int sg[8];
                    if (pre && hb == 0) {
#pragma unroll
                        for (int r = 0; r < 8; ++r) sg[r] = pre_sg[r];
                    } else {
                        const int4 sg0 = *reinterpret_cast<const int4 *>(a.signs + tb), sg1 = *reinterpret_cast<const int4 *>(a.signs + tb + 4);
                        sg[0] = sg0.x; sg[1] = sg0.y; sg[2] = sg0.z; sg[3] = sg0.w; sg[4] = sg1.x; sg[5] = sg1.y; sg[6] = sg1.z; sg[7] = sg1.w;
                    }
                    if (merged) {
#pragma unroll
                        for (int r = 0; r < 8; ++r) v[r] = __fmul_rn(__fmul_rn(__fmul_rn(xe[r], inv), pre_w[r]), float(sg[r]));
                    } else if (a.pro == PRO_PLAIN || a.pro == PRO_NORM) {
                        const float4 x0 = *reinterpret_cast<const float4 *>(a.x0 + tb), x1 = *reinterpret_cast<const float4 *>(a.x0 + tb + 4);
                        const float xe[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        if (a.pro == PRO_NORM) {
                            const float4 n0 = *reinterpret_cast<const float4 *>(a.w + tb), n1 = *reinterpret_cast<const float4 *>(a.w + tb + 4);
                            const float ne[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                            for (int r = 0; r < 8; ++r) v[r] = __fmul_rn(__fmul_rn(__fmul_rn(xe[r], inv), ne[r]), float(sg[r]));
                        } else {
#pragma unroll
                            for (int r = 0; r < 8; ++r) v[r] = __fmul_rn(xe[r], float(sg[r]));
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < 8; ++r) v[r] = __fmul_rn(input(tb + r), float(sg[r]));
                    }
#pragma unroll
                    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
                        for (int r = 0; r < 8; ++r)
                            if (!(r & h)) { const float x = v[r], y = v[r + h]; v[r] = __fadd_rn(x, y); v[r + h] = __fsub_rn(x, y); }
#pragma unroll
                    for (int m2 = 1; m2 < 32; m2 <<= 1)
#pragma unroll
                        for (int r = 0; r < 8; ++r) {
                            const float pr = __shfl_xor_sync(0xFFFFFFFFu, v[r], m2);
                            v[r] = (lane & m2) ? __fsub_rn(pr, v[r]) : __fadd_rn(v[r], pr);
                        }
                    float4 *dst = reinterpret_cast<float4 *>(xs + tid * 8);
                    dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                    dst[1] = make_float4(v[4], v[5], v[6], v[7]);
                }
                csync();
                if (HB == 4096) {
                    // h = 256, 512, 1024 inside a thread (elements 256 apart), h = 2048 between lanes l and l^16
                    const int i0 = (lane & 15) + 16 * warp + 2048 * (lane >> 4);
                    float u[8];
#pragma unroll
                    for (int r = 0; r < 8; ++r) u[r] = xs[i0 + 256 * r];
#pragma unroll
                    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
                        for (int r = 0; r < 8; ++r)
                            if (!(r & h)) { const float x = u[r], y = u[r + h]; u[r] = __fadd_rn(x, y); u[r + h] = __fsub_rn(x, y); }
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const float pr = __shfl_xor_sync(0xFFFFFFFFu, u[r], 16);
                        u[r] = (lane & 16) ? __fsub_rn(pr, u[r]) : __fadd_rn(u[r], pr);
                        xs[i0 + 256 * r] = __fmul_rn(u[r], a.hat_inv);     // each thread rewrites only what it read
                    }
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
                for (int i = tid; i < HB; i += NT) { const int t = base + i; xs[i] = __fmul_rn(input(t), float(a.signs[t])); }
                fwht_smem(xs, HB, a.hat_inv);
            }
            STAMP(4);
            // q8_1: 4 threads per 32-element sub-block, 8 consecutive elements each
            for (int sbk0 = 0; sbk0 < HB / 32; sbk0 += NT / 4) {
                const int sbk = sbk0 + (tid >> 2), q4 = tid & 3;
                const bool live = sbk < HB / 32;
                float e[8];
                if (live) {
                    const float4 *src = reinterpret_cast<const float4 *>(xs + sbk * 32 + q4 * 8);
                    const float4 v0 = src[0], v1 = src[1];
                    e[0] = v0.x; e[1] = v0.y; e[2] = v0.z; e[3] = v0.w; e[4] = v1.x; e[5] = v1.y; e[6] = v1.z; e[7] = v1.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) e[i] = 0.0f;
                }
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(e[i]));
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
                const float d = amax > 1e-35f ? __fdiv_rn(amax, 127.0f) : 0.0f;
                const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                int sum = 0;
                uint32_t w0 = 0, w1 = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float r = roundf(__fmul_rn(e[i], id));
                    r = fminf(fmaxf(r, -127.0f), 127.0f);
                    const int qi = int(r);
                    sum += qi;
                    if (i < 4) w0 |= (uint32_t(qi) & 0xFFu) << (8 * i); else w1 |= (uint32_t(qi) & 0xFFu) << (8 * (i - 4));
                }
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                if (live) {
                    uint32_t *cw = reinterpret_cast<uint32_t *>(codes + base + sbk * 32 + q4 * 8);
                    cw[0] = w0; cw[1] = w1;
                    if (q4 == 0) dsw[(base >> 5) + sbk] = float_to_half_bits(d) | (float_to_half_bits(__fmul_rn(d, float(sum))) << 16);
                }
            }
        }
    }
    csync();

    STAMP(5);
    // ---- main loop ----------------------------------------------------------------------------------------
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
            if (c + 1 < nchunks) accs[t * 16 + row16] = acc;
            else {
                const int row = (t0 + t) * 16 + row16;
                if (row < M) {
                    if (a.out) a.out[row] = acc;
                    if (a.resid_out) a.resid_out[row] = __fadd_rn(acc, a.resid_in[row]);
                }
            }
        }
    };

    int batch_begin = 0;
    for (int it = 0; it < items; ++it, ++tl) {
        if (tl == nt) { tl = 0; ++chunk; fresh = true; }
        const int stage = it % STAGES;
        if (fresh) {
            fresh = false;
            if (active) {
                const int b0 = chunk * CH + 2 * warp;
                build_breg(reinterpret_cast<const uint32_t *>(codes) + b0 * 32, g, tig, B0);
                build_breg(reinterpret_cast<const uint32_t *>(codes) + b0 * 32 + 32, g, tig, B1);
                const uint32_t w0 = dsw[b0 * 4 + tig], w1 = dsw[b0 * 4 + 4 + tig];
                d0 = half_bits_to_float(w0); s0w = half_bits_to_float(w0 >> 16);
                d1 = half_bits_to_float(w1); s1w = half_bits_to_float(w1 >> 16);
            }
        }
        if (it == 0) STAMP(6);
        mbar_wait(full + stage, (it / STAGES) & 1, a.err);
        float va = 0.0f, vb = 0.0f;      // rows g and g+8: v_(2w) + v_(2w+1)
        if (active) {
            const int ga = g, gb = g + 8;
            const uint32_t *r0 = reinterpret_cast<const uint32_t *>(ring + stage * STAGE_BYTES + (ga / rpc) * gpitch + (ga % rpc) * rowb + warp * 56);
            const uint32_t *r1 = reinterpret_cast<const uint32_t *>(ring + stage * STAGE_BYTES + (gb / rpc) * gpitch + (gb % rpc) * rowb + warp * 56);
            const uint32_t a6 = r0[6], b6 = r1[6], e6 = r0[13], f6 = r1[13];
            const uint32_t af = r0[first], as = r0[second], bf = r1[first], bs = r1[second];
            const uint32_t ef = r0[7 + first], es = r0[7 + second], ff = r1[7 + first], fs = r1[7 + second];
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + stage);          // rows are in registers: the stage may be refilled
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
            if (lane == 0) mbar_arrive(empty + stage);
        }
        if (it + 1 - batch_begin == RB || it + 1 == items) {
            csync();                                  // every warp has published the tiles of this batch
            reduce_batch(batch_begin, it + 1);
            batch_begin = it + 1;
        }
    }
    STAMP(7);
}

// A wait that nothing will ever satisfy, with a short limit: the give-up path of mbar_wait (error word set, kernel
// returns, context stays usable) can be exercised without hanging anything.
__global__ void k_wait_selftest(int *err, int limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(&bar, 0, err, limit);
}

}  // namespace

namespace bnk {

size_t phase_smem_bytes(int hat_block) { return size_t(SL::xs) + size_t(hat_block) * 4 + 128; }

bool phase_supported(int M, int K, int hat_block) {
    const int nb = K / 128;
    if (K % 512 || K > MAXK || M < 1) return false;
    if (nb > MAXCH && nb % MAXCH) return false;
    if (hat_block < 32 || hat_block > 4096 || K % hat_block || (hat_block & (hat_block - 1))) return false;
    return true;
}

cudaError_t launch_phase(cudaStream_t st, int sm_count, const PhaseArgs &a, bool pdl) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(k_phase_gemv, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             int(phase_smem_bytes(4096)));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const int ntiles = (a.M + 15) / 16, nchunks = (a.K / 128 + MAXCH - 1) / MAXCH;
    int grid = ntiles < sm_count ? ntiles : sm_count;
    // multi-chunk projections keep per-tile running sums in shared memory: at most 64 tiles per CTA
    while (nchunks > 1 && (ntiles + grid - 1) / grid > 64) ++grid;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = phase_smem_bytes(a.hat_block);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    BN_COUNT(1);
    return cudaLaunchKernelEx(&cfg, k_phase_gemv, a);
}

cudaError_t launch_wait_selftest_ring(cudaStream_t st, int *err) {
    BN_COUNT(1);
    k_wait_selftest<<<1, 32, 0, st>>>(err, 1 << 10);
    return cudaGetLastError();
}

}  // namespace bnk
