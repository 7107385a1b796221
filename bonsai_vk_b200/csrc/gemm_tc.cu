// gemm_tc.cu - multi-column PTQ1_0 x q8_1 projection on tcgen05 (see gemm_tc.cuh).
//
// Arithmetic (reference: _mul_mat_vecq_ptq1_0.comp:92-202 per column; multi-column shader :204-347): for every
// row, column and 128-weight block the four integer sub-block dots I_sb = sum code * q (code = trit + 1 in
// {0,1,2}, q = int8 activation code) are exact; they are combined exactly as the single-column kernel does:
// t_sb = fma(d_sb, float(I_sb), -s_sb); v = d_w * ((t0 + t1) + (t2 + t3)); blocks are added in groups of four,
// (v0 + v1) + (v2 + v3), groups in ascending order. A column of this kernel is therefore bit-identical to the
// single-column projection of the same activation vector.
//
// One CTA owns tiles of 128 rows over all of K. Per 128-weight block of the tile:
//   producer warp   bulk-copies the rows' PTQ1_0 bytes and the activation image of 8 blocks into a ring stage
//   4 decode warps  (lane = row) unpack 5 trits per byte with the multiply-by-3 chain on byte pairs held in the
//                   16-bit halves of a register, and store the 128 codes as the A operand into tensor memory
//   2 MMA threads   issue the tcgen05.mma.kind::i8 of two sub-blocks each (M=128, N=8, K=32 per sub-block and group of 8 columns), A from tensor
//                   memory, B = the int8 codes in shared memory, D = int32 in tensor memory
//   8 epilogue warps read D with tcgen05.ld and do the fp32 combination for their row and half of the columns
// Every wait is bounded: on giving up the kernel records it in the error word and drains.
#include "gemm_tc.cuh"
#include "rotate_quant.cuh"

#include <algorithm>
#include <cstdlib>

#include <cuda_fp16.h>

namespace {

using namespace bnk;

#ifndef GEMM_BK
#define GEMM_BK 8
#endif
constexpr int BK = GEMM_BK;                 // blocks per ring stage
constexpr int ROWP = BK * 28 + 16;         // shared-memory pitch of a row's BK*28 bytes
constexpr int WBYTES = 128 * ROWP;
constexpr int TBYTES = BK * 7 * 128 * 4;     // one stage of repacked weights: [block][word][row] dwords
constexpr int A_COL = 0;                   // tensor-memory columns: NA operand slots x 32, then ND accumulator slots x 4*NCP
constexpr int IMG_COL = 160;               // image bytes per column and block: 128 int8 codes + 4 x (fp32 d, fp32 -s)
constexpr int DWS = 16;                    // ring of per-row block scales handed from the decode warps to the epilogue
constexpr uint32_t MAGIC = 0x4B400000u;    // float 12582912.0: adding an int |i| < 2^22 to its bits gives the float 12582912 + i

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
// Bounded wait. try_wait suspends the thread until the phase completes or its time hint (ns) runs out; the retry loop
// is four instructions, so a waiting warp takes few issue slots from the warps that are working. After 2^20 tries
// (well over a second) it gives up: the error word is set and the abort flag drains every role of the CTA.
__device__ __forceinline__ bool mbar_wait(uint64_t *b, uint32_t parity, int *err, volatile int *abort_flag, int rounds = 1024) {
    const uint32_t addr = smem_u32(b);
    for (int round = 0; round < rounds; ++round) {
        uint32_t ok;
        asm volatile("{\n"
                     ".reg .pred p, q;\n"
                     ".reg .u32 n;\n"
                     "mov.u32 n, 0;\n"
                     "WAIT_LOOP:\n"
                                          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
                     "@p bra WAIT_DONE;\n"
                     "add.u32 n, n, 1;\n"
                     "setp.lt.u32 q, n, 1024;\n"
                     "@q bra WAIT_LOOP;\n"
                     "WAIT_DONE:\n"
                     "selp.u32 %0, 1, 0, p;\n"
                     "}\n"
                     : "=r"(ok) : "r"(addr), "r"(parity), "r"(2000u) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
    }
    if (err) atomicExch(err, 2);
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[128 x N] (+)= A[128 x 32] (u8, tensor memory) x B[N x 32] (s8, shared memory descriptor)
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// shared-memory operand descriptor: K-major, no swizzle; lbo = byte distance between the two 16-byte k-halves,
// sbo = byte distance between groups of 8 rows
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return uint64_t((saddr >> 4) & 0x3FFFu) | (uint64_t((lbo >> 4) & 0x3FFFu) << 16) | (uint64_t((sbo >> 4) & 0x3FFFu) << 32) |
           (uint64_t(1) << 46);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                   "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]) : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}

// Packed fp32 pairs (two IEEE single operations per instruction, each lane rounded as the scalar instruction would)
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float a, float b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void unpk2(f32x2 v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// Four packed bytes (5 trits each) -> five dwords of codes: o[t*stride] = codes at level t of the four bytes, in byte
// order. T_t = (b * 3^(t+1)) >> 8 is the running base-3 prefix of byte b, and trit_t + 1 = T_t - 3 * T_(t-1)
// (the reference decoder's v = (v*3) & 0xFF; trit = (v*3) >> 8, unrolled). The even and odd bytes sit in the 16-bit
// halves of two registers, so one multiply serves two bytes; PRMT gathers the four T bytes of a level, and because
// every byte of T_t - 3 * T_(t-1) lies in 0..2 the subtraction can be done on the whole dword at once.
__device__ __forceinline__ void decode4(uint32_t w, uint32_t *o, int stride) {
    const uint32_t e = __byte_perm(w, 0u, 0x4240u), d = __byte_perm(w, 0u, 0x4341u);
    const uint32_t t0 = __byte_perm(e * 3u, d * 3u, 0x7351u);
    const uint32_t t1 = __byte_perm(e * 9u, d * 9u, 0x7351u);
    const uint32_t t2 = __byte_perm(e * 27u, d * 27u, 0x7351u);
    const uint32_t t3 = __byte_perm(e * 81u, d * 81u, 0x7351u);
    const uint32_t t4 = __byte_perm(e * 243u, d * 243u, 0x7351u);
    o[0] = t0;
    o[stride] = t1 - 3u * t0;
    o[2 * stride] = t2 - 3u * t1;
    o[3 * stride] = t3 - 3u * t2;
    o[4 * stride] = t4 - 3u * t3;
}
// one block's 28 bytes (7 dwords) -> 32 dwords of codes in element order
__device__ __forceinline__ void decode_block(const uint32_t (&r)[7], uint32_t (&o)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) decode4(r[i], o + i, 4);           // elements 16t + 4i .. : dword 4t + i
    decode4(r[4], o + 20, 2);                                      // elements 80 + 8t + 0..3 : dword 20 + 2t
    decode4(r[5], o + 21, 2);                                      // elements 80 + 8t + 4..7 : dword 21 + 2t
    const uint32_t v = __byte_perm(r[6], 0u, 0x4140u);             // bytes 24, 25 (4 trits each) in the two halves
    const uint32_t ta = __byte_perm(v * 3u, v * 9u, 0x7531u);      // [T0(24), T0(25), T1(24), T1(25)]
    const uint32_t tb = __byte_perm(v * 27u, v * 81u, 0x7531u);    // [T2(24), T2(25), T3(24), T3(25)]
    o[30] = ta - 3u * (ta << 16);                                  // elements 120..123
    o[31] = tb - 3u * __byte_perm(ta, tb, 0x5432u);                // elements 124..127
}

// optional cycle accounting of CTA 0 (build with -DGEMM_PROF and pass GemmArgs::prof): where each role's time goes.
// Compiled out by default: even the untaken branches cost a few percent in these short loops.
#ifdef GEMM_PROF
// per-block event times of CTA 0 for blocks 8..23: a.prof[16 + ev * 16 + (g - 8)]
#define PROF_EV(ev, g, cond) do { if (a.prof && blockIdx.x == 0 && (cond) && (g) >= 8 && (g) < 24) a.prof[16 + (ev) * 16 + ((g) - 8)] = clock64(); } while (0)
#define PROF_T0() const long long prof_t0 = a.prof ? clock64() : 0
#define PROF_ADD(slot) do { if (a.prof) prof[slot] += clock64() - prof_t0; } while (0)
#else
#define PROF_T0() do { } while (0)
#define PROF_EV(ev, g, cond) do { } while (0)
#define PROF_ADD(slot) do { } while (0)
#endif

// NCP = 8, 16 or 32 columns = NG groups of 8. The tensor-core instruction always has N = 8 (its issue cost does not
// depend on N); per block there are 4 x NG of them, and each (row quarter, group) has its own epilogue warp that
// fetches the group's 4 x 8 accumulators with one 32-column tensor-memory load.
template <int NCP> struct Cfg {
    static constexpr int NG = NCP / 8;
    static constexpr int BBYTES = BK * NCP * IMG_COL;
    static constexpr int STAGE = WBYTES + BBYTES;
    static constexpr int CTAS = 1;                    // CTAs per SM (two were tried at 8 columns: the halved register file slowed the epilogue 3x)
    static constexpr int STAGES = NG == 4 ? 3 : 4;
    // Hand-offs between the roles cost each role a barrier round trip, so at 8 columns - where a block is little work -
    // NB = 4 blocks (one group of the summation order) travel per hand-off; the wider passes keep one block per hand-off
    // because a block's accumulators already take 64 / 128 tensor-memory columns there.
#ifndef GEMM_NB8
#define GEMM_NB8 4
#endif
    static constexpr int NB = NG == 1 ? GEMM_NB8 : 1;
    // epilogue warps: one per row quarter and CPW columns. 8 columns: two warps per quarter, four columns each.
    static constexpr int EW = 8;
    static constexpr int CPW = NCP / (EW / 4);        // columns per epilogue warp
    static constexpr int GPW = CPW >= 8 ? CPW / 8 : 1;   // column groups an epilogue warp visits
    static constexpr int PPG = CPW >= 8 ? 4 : CPW / 2;   // column pairs it takes from each
#ifndef GEMM_DW8
#define GEMM_DW8 4
#endif
    // decode warps: one per quarter of the rows (GEMM_DW8 = 8: two sets of four that take the slots in turn at 8 columns;
    // measured no faster, because the tensor-core instructions themselves bound the 8-column pass)
    static constexpr int DW = NG == 1 ? GEMM_DW8 : 4;
#ifndef GEMM_MW
#define GEMM_MW 2
#endif
    static constexpr int MW = GEMM_MW;                // MMA issuing threads (one warp each), 4 / MW sub-blocks apiece
    static constexpr int NWARPS = DW + EW + 1 + MW;   // decode, epilogue, producer, MMA issuers: at most 16 warps = 128 registers
    // operand slot i and accumulator slot i belong to the same NB blocks, so one "done" barrier per slot (armed by the
    // MMA issuers' commits) tells the epilogue that the accumulators are ready and the decode warps that the operand
    // slot may be overwritten. Several slots are in flight: each hop (decode -> MMA -> commit -> epilogue -> slot
    // free) costs a few hundred cycles.
    static constexpr int NA = NG == 1 ? 8 / NB : (NG == 2 ? 5 : 3);
    static constexpr int D_COL = NA * NB * 32;
    static constexpr int TMEM_COLS = 512 / CTAS;
    static_assert(D_COL + NA * NB * NG * 32 <= TMEM_COLS && 2 * NA * NB <= DWS && BK % (NB * (DW / 4)) == 0 && NA % (DW / 4) == 0, "tensor memory budget");
    static constexpr size_t SMEM = size_t(STAGES) * STAGE + DWS * 128 * 4 + 512;
};

template <int NCP>
__global__ void __launch_bounds__(Cfg<NCP>::NWARPS * 32, Cfg<NCP>::CTAS) k_ptq_gemm_tc(const GemmArgs a) {
    using C = Cfg<NCP>;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *ring = smem;
    float *dwv = reinterpret_cast<float *>(smem + size_t(C::STAGES) * C::STAGE);      // [DWS][128] block scales of the rows
    uint64_t *bars = reinterpret_cast<uint64_t *>(dwv + DWS * 128);
    uint64_t *full = bars, *empty = bars + 4, *afull = bars + 8, *dfull = bars + 24, *dempty = bars + 32;
    uint64_t *aempty = dfull;                      // "done": all four sub-block MMAs of the slot's block have completed
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 40);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    constexpr int NA = C::NA, NB = C::NB, NG = C::NG, D_COL = C::D_COL, EW = C::EW, DW = C::DW;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef GEMM_PROF
    unsigned long long prof_entry = 0;
    if (a.prof && tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_entry));
#endif
    const int nb = a.K / 128, nkc = nb / BK, ntiles = (a.M + 127) / 128;
    const size_t rowbytes = size_t(nb) * 28;

    if (tid == 0) {
        for (int i = 0; i < C::STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, EW); }
        for (int i = 0; i < NA; ++i) { mbar_init(afull + i, 4); mbar_init(dfull + i, C::MW); mbar_init(dempty + i, EW); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(uint32_t(C::TMEM_COLS)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = *tmem_slot;
#ifdef GEMM_PROF
    if (a.prof && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); a.prof[blockIdx.x == 0 ? 12 : 13] = (long long)(blockIdx.x == 0 ? t - prof_entry : t); }
#endif
    // everything above overlaps the previous kernel's tail; its results (the activation image) are read below
    pdl_sync();

    // work items: a tile over all of K, or (split) a single ring stage of a tile
    const bool split = a.groups != nullptr;
    const int nwork = split ? ntiles * nkc : ntiles;
    int n_items = 0;
    for (int t = blockIdx.x; t < nwork; t += gridDim.x) n_items += split ? 1 : nkc;

    if (warp == DW + EW) {
        // ---- producer ----------------------------------------------------------------------------------
        int s = 0, ph = 1;                         // a fresh barrier passes a wait on parity 1
        for (int tt = blockIdx.x; tt < nwork && !*abort_flag; tt += gridDim.x) {
            const int t = split ? tt / nkc : tt, kc0 = split ? tt - t * nkc : 0, kc1 = split ? kc0 + 1 : nkc;
            for (int kc = kc0; kc < kc1; ++kc) {
                if (!mbar_wait(empty + s, ph, a.err, abort_flag)) break;
                unsigned char *st = ring + size_t(s) * C::STAGE;
                if (a.tiled) {                      // repacked weights: the stage is one contiguous piece
                    if (lane == 0) {
                        mbar_expect_tx(full + s, TBYTES + C::BBYTES);
                        bulk_copy(st, a.W + (size_t(t) * nkc + kc) * TBYTES, TBYTES, full + s);
                    }
                } else {
                    if (lane == 0) mbar_expect_tx(full + s, 128 * (BK * 28) + C::BBYTES);
                    __syncwarp();
#pragma unroll
                    for (int r = lane; r < 128; r += 32) {
                        const int grow = min(t * 128 + r, a.M - 1);
                        bulk_copy(st + r * ROWP, a.W + size_t(grow) * rowbytes + size_t(kc) * (BK * 28), BK * 28, full + s);
                    }
                }
                if (lane == 0) bulk_copy(st + WBYTES, a.image + size_t(kc) * C::BBYTES, C::BBYTES, full + s);
                if (++s == C::STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp > DW + EW) {
        // ---- MMA issue: each of the two threads issues two sub-blocks' MMAs of every block (an issue costs the
        //      thread ~55 cycles whatever its size; two threads keep that far below the other roles' time) --------
        if (lane == 0) {
            constexpr int SPT = 4 / C::MW;          // sub-blocks per issuing thread
            const int sb0 = SPT * (warp - (DW + EW + 1));
            // D s32, A u8, B s8, both K-major, M = 128, N = all the pass's columns: one instruction per 32-weight sub-block.
            // (An instruction costs the tensor core about 190 cycles here whatever N is - measured with N = 8 - so the column
            // groups share one; a block's accumulators are laid out [sub-block][column].)
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (uint32_t(NCP >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            bool ok = true;
            int s = 0, sph = 0, slot = 0, aph = 0, dph = 1;
            long long prof[4] = {0, 0, 0, 0};
            for (int it = 0; it < n_items && ok; ++it) {
                { PROF_T0(); if (!mbar_wait(full + s, sph, a.err, abort_flag)) break; PROF_ADD(0); }
                const uint32_t bbase = smem_u32(ring + size_t(s) * C::STAGE + WBYTES);
                for (int jt = 0; jt < BK / NB; ++jt) {
                    { PROF_T0(); if (!mbar_wait(afull + slot, aph, a.err, abort_flag)) { ok = false; break; } PROF_ADD(1); }
                    PROF_EV(2, it * BK + jt * NB, sb0 == 0);
                    { PROF_T0(); if (!mbar_wait(dempty + slot, dph, a.err, abort_flag)) { ok = false; break; } PROF_ADD(2); }
                    PROF_EV(3, it * BK + jt * NB, sb0 == 0);
                    tc_fence_after();
#pragma unroll
                    for (int jb = 0; jb < NB; ++jb)
#pragma unroll
                        for (int k = 0; k < SPT; ++k)
                            tc_mma_i8(tb + D_COL + (slot * NB + jb) * NG * 32 + (sb0 + k) * NCP, tb + A_COL + (slot * NB + jb) * 32 + (sb0 + k) * 8,
                                      smem_desc(bbase + (jt * NB + jb) * (NCP * IMG_COL) + (sb0 + k) * 256, 128, 1024), idesc, 0u);
                    tc_commit(dfull + slot);
                    PROF_EV(4, it * BK + jt * NB, sb0 == 0);
                    if (++slot == NA) { slot = 0; aph ^= 1; dph ^= 1; }
                }
                if (++s == C::STAGES) { s = 0; sph ^= 1; }
            }
            if (a.prof && blockIdx.x == 0 && sb0 == 0) for (int i = 0; i < 4; ++i) a.prof[4 + i] = prof[i];
        }
    } else if (warp < DW) {
        // ---- decode ------------------------------------------------------------------------------------
        const int q = warp & 3, row = q * 32 + lane;
        const uint32_t lane_base = uint32_t(q * 32) << 16;
        bool ok = true;
        int pending = -1;                          // slot whose tensor-memory store is in flight
        auto publish = [&]() {                     // the store of `pending` is complete: hand the slot to the MMA thread
            if (pending < 0) return;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(afull + pending);
            pending = -1;
        };
        // DSETS sets of four decode warps take the slots (NB blocks each) in turn
        constexpr int DSETS = DW / 4;
        const int set = warp >> 2;
        int s = 0, sph = 0;
        long long prof[4] = {0, 0, 0, 0};
        for (int it = 0; it < n_items && ok; ++it) {
            { PROF_T0(); if (!mbar_wait(full + s, sph, a.err, abort_flag)) break; PROF_ADD(0); }
            const unsigned char *st = ring + size_t(s) * C::STAGE;
#pragma unroll 1
            for (int j = 0; j < BK; ++j) {
                const int g = it * BK + j, bt = g / NB, jb = g % NB, slot = bt % NA;
                if (DSETS > 1 && bt % DSETS != set) continue;
                PROF_EV(0, g, (warp & 3) == 0 && lane == 0);
                uint32_t r[7];
                if (a.tiled) {                      // [block][word][row]: the warp's rows are consecutive dwords
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(st) + j * 7 * 128 + row;
#pragma unroll
                    for (int i = 0; i < 7; ++i) r[i] = src[i * 128];
                } else {
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(st + row * ROWP + j * 28);
#pragma unroll
                    for (int i = 0; i < 7; ++i) r[i] = src[i];
                }
                uint32_t o[32];
                { PROF_T0(); decode_block(r, o); if (a.prof && o[31] == 0xFFFFFFFFu) prof[3]++; PROF_ADD(1); }
                if (jb == 0) {
                    { PROF_T0(); publish(); PROF_ADD(2); }   // the previous slot's stores had this block's arithmetic to finish
                    { PROF_T0(); if (!mbar_wait(aempty + slot, ((bt / NA) & 1) ^ 1, a.err, abort_flag)) { ok = false; break; } PROF_ADD(3); }
                    tc_fence_after();
                }
                const uint32_t ta = tb + lane_base + A_COL + (slot * NB + jb) * 32;
                tmem_st16(ta, o);
                tmem_st16(ta + 16, o + 16);
                PROF_EV(1, g, (warp & 3) == 0 && lane == 0);
                dwv[(g % DWS) * 128 + row] = half_bits_to_float(r[6] >> 16);
                if (jb == NB - 1) {
                    pending = slot;
                    if (DSETS > 1) publish();       // this set's next slot is DSETS slots away: hand over now
                }
            }
            if (++s == C::STAGES) { s = 0; sph ^= 1; }
        }
        publish();
        if (a.prof && blockIdx.x == 0 && warp == 0 && lane == 0) for (int i = 0; i < 4; ++i) a.prof[i] = prof[i];
    } else {
        // ---- epilogue (warps DW .. DW+EW-1): warp (quarter q, group gi) owns 32 rows x 8 columns -------------------
        const int q = warp & 3, part = (warp - DW) >> 2, row = q * 32 + lane;
        const uint32_t lane_base = uint32_t(q * 32) << 16;
        constexpr int GPW = C::GPW, PPG = C::PPG, NCW = C::CPW;
        const int c0 = part * NCW, g0 = c0 / 8, p0 = (c0 % 8) / 2;
        // running sums as column pairs (2p, 2p+1): the arithmetic below is done two columns at a time
        constexpr int NPR = NCW / 2;
        f32x2 acc[NPR], u[NPR], ve[NPR];
#pragma unroll
        for (int c = 0; c < NPR; ++c) { acc[c] = 0ull; u[c] = 0ull; ve[c] = 0ull; }
        const f32x2 magic2 = pk2(12582912.0f, 12582912.0f);
        bool ok = true;
        long long prof[4] = {0, 0, 0, 0};
        int s = 0, sph = 0, g = 0;
        for (int tt = blockIdx.x; tt < nwork && ok; tt += gridDim.x) {
            const int t = split ? tt / nkc : tt, kc0 = split ? tt - t * nkc : 0, kc1 = split ? kc0 + 1 : nkc;
            for (int kc = kc0; kc < kc1 && ok; ++kc) {
                { PROF_T0(); if (!mbar_wait(full + s, sph, a.err, abort_flag)) { ok = false; break; } PROF_ADD(0); }
                const unsigned char *stage_scales = ring + size_t(s) * C::STAGE + WBYTES + NCP * 128 + g0 * 256;
#pragma unroll 1
                for (int j = 0; j < BK; ++j, ++g) {
                    const unsigned char *scales = stage_scales + j * (NCP * IMG_COL);
                    const int bt = g / NB, jb = g % NB, slot = bt % NA;
                    if (jb == 0) {
                        { PROF_T0(); if (!mbar_wait(dfull + slot, (bt / NA) & 1, a.err, abort_flag)) { ok = false; break; } PROF_ADD(0); }
                        PROF_EV(5, g, warp == DW && lane == 0);
                        tc_fence_after();
                    }
                    const float dw = dwv[(g % DWS) * 128 + row];
                    const f32x2 dw2 = pk2(dw, dw);
                    const int b = kc * BK + j, bi = b & 3;
#pragma unroll
                    for (int gw = 0; gw < GPW; ++gw) {
                        constexpr int DS = 2 * PPG;         // this warp's columns per sub-block
                        uint32_t d[4 * DS];                 // [sub-block][column] of one group (or of this warp's half of it)
                        const uint32_t dsrc = tb + lane_base + D_COL + (slot * NB + jb) * NG * 32 + (g0 + gw) * 8;   // [sub-block][column]
#pragma unroll
                        for (int sb = 0; sb < 4; ++sb) {
                            if (PPG == 4) tmem_ld8(dsrc + sb * NCP, d + sb * DS);
                            else tmem_ld4(dsrc + sb * NCP + 2 * p0, d + sb * DS);
                        }
                        // the group's scales, per sub-block and column pair one 16-byte entry (d, d', -s, -s'): they do not
                        // depend on the accumulators and travel while those do
                        ulonglong2 sc[4 * PPG];
#pragma unroll
                        for (int sb = 0; sb < 4; ++sb)
#pragma unroll
                            for (int p = 0; p < PPG; ++p) sc[sb * PPG + p] = *reinterpret_cast<const ulonglong2 *>(scales + gw * 256 + (sb * 4 + p0 + p) * 16);
                        { PROF_T0(); asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); PROF_ADD(1); }
                        if (gw == GPW - 1 && jb == NB - 1) {   // all of this warp's accumulators of the slot are in registers: it is free
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(dempty + slot);
                        }
                        PROF_T0();
                        f32x2 v[PPG];
#pragma unroll
                        for (int p = 0; p < PPG; ++p) {     // straight-line: the pairs' dependency chains interleave
                            f32x2 tt[4];
#pragma unroll
                            for (int sb = 0; sb < 4; ++sb) {
                                const int dc = sb * DS + 2 * p;
                                const f32x2 f = sub2(pk2(__uint_as_float(MAGIC + d[dc]), __uint_as_float(MAGIC + d[dc + 1])), magic2);
                                tt[sb] = fma2(sc[sb * PPG + p].x, f, sc[sb * PPG + p].y);
                            }
                            v[p] = mul2(dw2, add2(add2(tt[0], tt[1]), add2(tt[2], tt[3])));
                        }
                        if (bi == 0 || bi == 2) {
#pragma unroll
                            for (int p = 0; p < PPG; ++p) ve[gw * PPG + p] = v[p];
                        } else if (bi == 1) {
#pragma unroll
                            for (int p = 0; p < PPG; ++p) u[gw * PPG + p] = add2(ve[gw * PPG + p], v[p]);
                        } else if (split) {
                            // the group sum p_g itself goes to memory; the groups are added in order by gemm_sum_groups
                            const int grow = t * 128 + row;
#pragma unroll
                            for (int p = 0; p < PPG; ++p) {
                                const f32x2 q2 = add2(u[gw * PPG + p], add2(ve[gw * PPG + p], v[p]));
                                float lo, hi;
                                unpk2(q2, lo, hi);
                                const int c = (g0 + gw) * 8 + 2 * (p0 + p);
                                if (grow < a.M) {
                                    float *gp = a.groups + (size_t(b >> 2) * NCP + c) * size_t(a.M) + grow;
                                    if (c < a.ncol) gp[0] = lo;
                                    if (c + 1 < a.ncol) gp[a.M] = hi;
                                }
                            }
                        } else {
                            const bool first = b < 4;
#pragma unroll
                            for (int p = 0; p < PPG; ++p) {
                                const f32x2 q2 = add2(u[gw * PPG + p], add2(ve[gw * PPG + p], v[p]));
                                acc[gw * PPG + p] = first ? q2 : add2(acc[gw * PPG + p], q2);
                            }
                        }
                        PROF_ADD(2);
                    }
                    PROF_EV(6, g, warp == DW && lane == 0);
                    if (!split && b == nb - 1) {
                        const int grow = t * 128 + row;
                        if (grow < a.M) {
#pragma unroll
                            for (int c = 0; c < NCW; ++c) {
                                if (c0 + c >= a.ncol) continue;
                                float lo, hi;
                                unpk2(acc[c >> 1], lo, hi);
                                float r = (c & 1) ? hi : lo;
                                if (a.resid) r = __fadd_rn(r, a.resid[size_t(c0 + c) * a.resid_stride + grow]);
                                a.out[size_t(c0 + c) * a.out_stride + grow] = r;
                            }
                        }
                    }
                }
                __syncwarp();
                if (ok && lane == 0) mbar_arrive(empty + s);    // the stage's scales and weights are not needed any more
                if (++s == C::STAGES) { s = 0; sph ^= 1; }
            }
        }
        if (a.prof && blockIdx.x == 0 && warp == DW && lane == 0) for (int i = 0; i < 4; ++i) a.prof[8 + i] = prof[i];
    }
    tc_fence_before();
    __syncthreads();
#ifdef GEMM_PROF
    if (a.prof && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); a.prof[blockIdx.x == 0 ? 14 : 13] = (long long)(blockIdx.x == 0 ? t - prof_entry : t - (unsigned long long)a.prof[13]); }
#endif
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(uint32_t(C::TMEM_COLS)) : "memory");
}

// ---- activation image: [rms norm] -> signs -> Hadamard per hat_block -> q8_1 codes and scales -----------------
// grid (K / chunk, padded columns), 512 threads; chunk = hat_block (or 1024 without rotation)
// chunk = the values one CTA takes: a Hadamard block (hb), or 32 when the Hadamard block is smaller than a q8_1 sub-block
__global__ void __launch_bounds__(512) k_prep_cols(const PrepArgs a, int chunk, int hb, int ncp) {
    pdl_sync();
    extern __shared__ __align__(16) float s[];     // chunk floats
    __shared__ float part[256];
    const int cg = blockIdx.y, tid = threadIdx.x;
    const int c = cg;
    const size_t base = size_t(blockIdx.x) * chunk;
    const size_t blk_bytes = size_t(ncp) * IMG_COL;
    unsigned char *image = a.image;
    if (cg >= a.ncol) {                             // padding column: zero codes and scales
        for (int e = tid * 16; e < chunk; e += 512 * 16) {
            const size_t b = (base + e) / 128;
            const int sb = int((base + e) & 127) >> 5, kh = (e >> 4) & 1;
            *reinterpret_cast<uint4 *>(image + b * blk_bytes + (c / 8) * 1024 + (sb * 2 + kh) * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        for (int e = tid * 32; e < chunk; e += 512 * 32) {
            const size_t b = (base + e) / 128;
            float *ent = reinterpret_cast<float *>(image + b * blk_bytes + size_t(ncp) * 128 + (c / 8) * 256 + (((int((base + e) & 127) >> 5) * 4) + ((c & 7) >> 1)) * 16);
            ent[c & 1] = 0.0f; ent[2 + (c & 1)] = 0.0f;
        }
        return;
    }
    const float *x = a.x + size_t(cg) * a.x_stride;
    float inv = 1.0f;
    const int lane_id = tid & 31, warp_id = tid >> 5;
    if (a.mode == PREP_NORM) {
        // same partial sums as the stand-alone norm kernel: 256 lanes, each its consecutive run, then the fixed tree
        // p[i] += p[i + s], s = 128 .. 1 - run by every warp on its own (the same adds in the same order give the same float
        // in every warp), so one barrier instead of nine
        const int per = (a.K + 255) / 256;
        if (tid < 256) {
            float acc = 0.0f;
            if (per == 16 && a.K == 4096) {
                const float4 *xv = reinterpret_cast<const float4 *>(x + tid * 16);
                const float4 v0 = xv[0], v1 = xv[1], v2 = xv[2], v3 = xv[3];
                const float e[16] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w};
#pragma unroll
                for (int i = 0; i < 16; ++i) acc = __fadd_rn(acc, __fmul_rn(e[i], e[i]));
            } else {
                for (int i = 0; i < per; ++i) {
                    const int d = tid * per + i;
                    if (d < a.K) { const float v = x[d]; acc = __fadd_rn(acc, __fmul_rn(v, v)); }
                }
            }
            part[tid] = acc;
        }
        __syncthreads();
        float v[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) v[w] = part[32 * w + lane_id];
        float t = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[4]), __fadd_rn(v[2], v[6])),
                            __fadd_rn(__fadd_rn(v[1], v[5]), __fadd_rn(v[3], v[7])));
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xFFFFFFFFu, t, s2));
        inv = __frcp_rn(__fsqrt_rn(__fadd_rn(mean_of(t, a.K), a.eps)));
        if (a.inv_out && blockIdx.x == 0 && tid == 0) a.inv_out[size_t(cg) * a.inv_stride] = inv;
    }
    if (a.signs && chunk >= 256) {
        // Sylvester butterflies (a+c, a-c), h ascending, as hat4096.comp:41-60: h = 1, 2, 4 inside a thread's 8
        // consecutive elements, h = 8..128 across lanes; then through shared memory (h = 256..1024 inside a thread and
        // h = 2048 between lanes l and l^16 when the chunk is 4096). Same pairs, same order: bit-identical to the plain loop.
        if (tid < chunk / 8) {
            const size_t tb = base + size_t(tid) * 8;
            const float4 x0 = *reinterpret_cast<const float4 *>(x + tb), x1 = *reinterpret_cast<const float4 *>(x + tb + 4);
            const int4 g0 = *reinterpret_cast<const int4 *>(a.signs + tb), g1 = *reinterpret_cast<const int4 *>(a.signs + tb + 4);
            float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const int sg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            if (a.mode == PREP_NORM) {
                const float4 n0 = *reinterpret_cast<const float4 *>(a.w + tb), n1 = *reinterpret_cast<const float4 *>(a.w + tb + 4);
                const float ne[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                for (int r = 0; r < 8; ++r) v[r] = __fmul_rn(__fmul_rn(v[r], inv), ne[r]);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) v[r] = __fmul_rn(v[r], float(sg[r]));
            fwht_regs_lanes(v, lane_id);
            float4 *dst = reinterpret_cast<float4 *>(s + tid * 8);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
        __syncthreads();
        const float hinv = 1.0f / sqrtf(float(chunk));
        if (chunk == 4096) {
            fwht_4096_tail(s, warp_id, lane_id, hinv);
        } else {
            for (int h = 256; h < chunk; h <<= 1) {
                for (int i = tid; i < (chunk >> 1); i += 512) {
                    const int j = ((i & ~(h - 1)) << 1) | (i & (h - 1));
                    const float p = s[j], r = s[j + h];
                    s[j] = __fadd_rn(p, r);
                    s[j + h] = __fsub_rn(p, r);
                }
                __syncthreads();
            }
            for (int i = tid; i < chunk; i += 512) s[i] = __fmul_rn(s[i], hinv);
        }
    } else {
        for (int i = tid; i < chunk; i += 512) {
            float v = x[base + i];
            if (a.mode == PREP_NORM) v = __fmul_rn(__fmul_rn(v, inv), a.w[base + i]);
            if (a.signs) v = __fmul_rn(v, float(a.signs[base + i]));
            s[i] = v;
        }
        if (a.signs) {
            const float hinv = 1.0f / sqrtf(float(hb));
            for (int h = 1; h < hb; h <<= 1) {
                __syncthreads();
                for (int i = tid; i < (chunk >> 1); i += 512) {
                    const int j = ((i & ~(h - 1)) << 1) | (i & (h - 1));
                    const float p = s[j], r = s[j + h];
                    s[j] = __fadd_rn(p, r);
                    s[j + h] = __fsub_rn(p, r);
                }
            }
            __syncthreads();
            for (int i = tid; i < chunk; i += 512) s[i] = __fmul_rn(s[i], hinv);
        }
    }
    __syncthreads();
    // q8_1 per 32 values: four threads per sub-block, eight consecutive values each (quant8_of32); the eight codes are one
    // 8-byte store into the image, (d, s) rounded to fp16 as the q8_1 record keeps them and stored as fp32 d and -s
    for (int sbk0 = 0; sbk0 < chunk / 32; sbk0 += 128) {
        const int sbk = sbk0 + (tid >> 2), q4 = tid & 3;
        const bool live = sbk < chunk / 32;
        float e[8];
        if (live) {
            const float4 *src = reinterpret_cast<const float4 *>(s + sbk * 32 + q4 * 8);
            const float4 v0 = src[0], v1 = src[1];
            e[0] = v0.x; e[1] = v0.y; e[2] = v0.z; e[3] = v0.w; e[4] = v1.x; e[5] = v1.y; e[6] = v1.z; e[7] = v1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = 0.0f;
        }
        const Q8x8 q = quant8_of32(e);
        if (live) {
            const int e0 = sbk * 32 + q4 * 8;
            const size_t b = (base + e0) / 128;
            const int sb = int((base + e0) & 127) >> 5, kh = (e0 >> 4) & 1;       // (a chunk may be a part of a 128-value block)
            unsigned char *blk = image + b * blk_bytes;
            *reinterpret_cast<uint2 *>(blk + (c / 8) * 1024 + (sb * 2 + kh) * 128 + (c & 7) * 16 + (e0 & 15)) = make_uint2(q.w0, q.w1);
            if (q4 == 0) {
                float *ent = reinterpret_cast<float *>(blk + size_t(ncp) * 128 + (c / 8) * 256 + (sb * 4 + ((c & 7) >> 1)) * 16);
                ent[c & 1] = half_bits_to_float(float_to_half_bits(q.d));
                ent[2 + (c & 1)] = -half_bits_to_float(float_to_half_bits(__fmul_rn(q.d, float(q.sum))));
            }
        }
    }
}

// native row-major PTQ1_0 -> per (tile of 128 rows, 8 blocks of K): [block][word 0..6][row] dwords; rows beyond M are zero
__global__ void k_repack_tiles(const uint32_t *__restrict__ W, int M, int nb, uint32_t *__restrict__ out, size_t total) {
    pdl_sync();
    const int nkc = nb / BK;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const int row = int(i & 127);
        size_t r = i >> 7;
        const int k = int(r % 7); r /= 7;
        const int j = int(r % BK); r /= BK;
        const int kc = int(r % nkc);
        const size_t t = r / nkc;
        const size_t grow = t * 128 + row;
        out[i] = grow < size_t(M) ? W[grow * (size_t(nb) * 7) + (size_t(kc) * BK + j) * 7 + k] : 0u;
    }
}

// out[c][row] = groups[0][c][row] + groups[1][c][row] + ... (ascending), + residual: the tail of a split projection
__global__ void k_gemm_sum_groups(const float *__restrict__ groups, int ngroups, int ncp, int M, int ncol, float *__restrict__ out,
                                  size_t out_stride, const float *__restrict__ resid, size_t resid_stride) {
    pdl_sync();
    const int row = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
    if (row >= M || c >= ncol) return;
    const size_t gs = size_t(ncp) * M;
    const float *gp = groups + size_t(c) * M + row;
    float s = gp[0];
    int g = 1;
    for (; g + 8 <= ngroups; g += 8) {              // eight group sums in flight, added in ascending order
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = gp[size_t(g + u) * gs];
#pragma unroll
        for (int u = 0; u < 8; ++u) s = __fadd_rn(s, v[u]);
    }
    for (; g < ngroups; ++g) s = __fadd_rn(s, gp[size_t(g) * gs]);
    if (resid) s = __fadd_rn(s, resid[size_t(c) * resid_stride + row]);
    out[size_t(c) * out_stride + row] = s;
}

template <int NCP>
cudaError_t launch_t(cudaStream_t st, int sm_count, const GemmArgs &a, bool pdl) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(k_ptq_gemm_tc<NCP>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(Cfg<NCP>::SMEM));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const int ntiles = (a.M + 127) / 128, nwork = a.groups ? ntiles * (a.K / 128 / BK) : ntiles, cap = sm_count * Cfg<NCP>::CTAS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nwork < cap ? nwork : cap);
    cfg.blockDim = dim3(Cfg<NCP>::NWARPS * 32);
    cfg.dynamicSmemBytes = Cfg<NCP>::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    BN_COUNT(1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, k_ptq_gemm_tc<NCP>, a);
    if (e != cudaSuccess || !a.groups) return e;
    launch(k_gemm_sum_groups, dim3((a.M + 255) / 256, a.ncol), dim3(256), 0, st, static_cast<const float *>(a.groups), a.K / 512, NCP, a.M, a.ncol,
           a.out, a.out_stride, a.resid, a.resid_stride);
    return cudaGetLastError();
}

// A wait that nothing will ever satisfy, one round of tries (about 2 ms): exercises the give-up path of mbar_wait
// (error word = 2, abort flag raised, kernel returns) without hanging anything.
__global__ void k_wait_selftest_tc(int *err) {
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(&bar, 0, err, &abort_word, 1);
}

}  // namespace

namespace bnk {

bool gemm_supported(int M, int K, int ncol) {
    return M >= 1 && K >= 1024 && K % 1024 == 0 && ncol >= 1 && ncol <= GEMM_MAX_COLS;
}

bool gemm_wants_split(int sm_count, int M, int K, int ncol) {
    // fewer row tiles than half of what the GPU can hold at once: split over K
    const int ntiles = (M + 127) / 128, cap = sm_count * (gemm_padded_cols(ncol) == 8 ? Cfg<8>::CTAS : 1);
    return K >= 2048 && 2 * ntiles <= cap && getenv("BONSAI_GEMM_NO_SPLIT") == nullptr;
}
size_t gemm_group_floats(int M, int K, int ncol) { return size_t(K / 512) * gemm_padded_cols(ncol) * size_t(M); }

cudaError_t launch_gemm(cudaStream_t st, int sm_count, const GemmArgs &a, bool pdl) {
    const int ncp = gemm_padded_cols(a.ncol);
    if (ncp == 8) return launch_t<8>(st, sm_count, a, pdl);
    if (ncp == 16) return launch_t<16>(st, sm_count, a, pdl);
    return launch_t<32>(st, sm_count, a, pdl);
}

size_t gemm_tiled_bytes(int M, int K) { return size_t((M + 127) / 128) * (K / 128 / BK) * TBYTES; }
void repack_tiles(cudaStream_t st, const uint32_t *W, int M, int K, uint32_t *out) {
    const size_t total = gemm_tiled_bytes(M, K) / 4;
    launch(k_repack_tiles, dim3(unsigned(std::min<size_t>((total + 255) / 256, 148 * 16))), dim3(256), 0, st, W, M, K / 128, out, total);
}

void prep_cols(cudaStream_t st, const PrepArgs &a) {
    const int chunk = a.signs ? (a.hat_block < 32 ? 32 : a.hat_block) : 1024;
    const int ncp = gemm_padded_cols(a.ncol);
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(k_prep_cols, cudaFuncAttributeMaxDynamicSharedMemorySize, 4096 * 4); attr = true; }
    launch(k_prep_cols, dim3(a.K / chunk, ncp), dim3(512), size_t(chunk) * 4, st, a, chunk, a.signs ? a.hat_block : chunk, ncp);
}

cudaError_t launch_wait_selftest_tc(cudaStream_t st, int *err) {
    BN_COUNT(1);
    k_wait_selftest_tc<<<1, 32, 0, st>>>(err);
    return cudaGetLastError();
}

}  // namespace bnk
