// phase_gemv.cu - the fused projection phase as one kernel launch per projection (see phase_body.cuh for the
// kernel's structure). One CTA of 16 compute warps + 1 copy warp per SM. The copies of the first ring stages are
// issued before the kernel waits for the previous grid (programmatic dependent launch) - weights do not depend on it.
#include "phase_body.cuh"

namespace {
using namespace bnk;
using namespace bnk::phase;

template <int EPI>
__global__ void __launch_bounds__(NTHREADS, 1) k_phase_gemv(const PhaseArgs a) {
    const Smem s = carve(dyn_smem());
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, cta = blockIdx.x;
    const Work w = phase_work(a, cta, gridDim.x);

    BN_STAMP(0);
    if (tid == 0) {
        init_barriers(s);
    }
    __syncthreads();

    const bool copy_warp = warp == NWARP;
    if (copy_warp) for (int it = 0; it < min(w.items, STAGES); ++it) issue_item(a, w, s, it, uint32_t(it), lane);

    // constants of the prologue (norm weights, sign vector) do not depend on the previous grid either
    Preload pl;
    pl.on = false;
    if (!copy_warp) {
        preload(a, tid, pl);
        build_btab(s.btab, tid);          // (read after the barriers of the prologue)
    }
    BN_STAMP(1);
    // everything above touched only constant weights; from here on we read the previous grid's output
    asm volatile("griddepcontrol.wait;" ::: "memory");
    BN_STAMP(2);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (copy_warp) {
        // refill a stage as soon as all 16 compute warps have taken its rows into registers
        for (int it = STAGES; it < w.items; ++it) {
            mbar_wait(s.empty + it % STAGES, ((it / STAGES) - 1) & 1, a.err, s.abort);
            issue_item(a, w, s, it, uint32_t(it), lane);
        }
        return;
    }
    prologue<false>(a, s, pl, cta);
    BN_STAMP(5);
    NoFeed nofeed;
    main_loop<EPI>(a, w, s, 0u, cta, nofeed);
}

// silu(gate) * up of the FFN and then the whole input preparation of the down projection (signs, Hadamard, q8_1), done
// ONCE per 4096-wide Hadamard block and written as the activation pack that the projection kernel only has to copy
// (PRO_PACKED) - otherwise every one of the projection's 148 CTAs walks the three Hadamard blocks one after the other.
// Eight CTAs of 512 threads share a Hadamard block for the silu (one double-precision exp per thread); each counts itself
// in, and the one that arrives last (nobody waits) rotates and quantises the block. Same operations per element as the
// projection kernel's own prologue (the helpers are shared), so the same bits.
__global__ void __launch_bounds__(NT) k_swiglu_pack(const float *__restrict__ gate, const float *__restrict__ up,
                                                     const int32_t *__restrict__ signs, float hat_inv,
                                                     float *__restrict__ y, uint32_t *__restrict__ pack, int *__restrict__ count) {
    __shared__ __align__(16) float xs[4096];
    __shared__ __align__(16) int8_t codes[4096];
    __shared__ uint32_t dsw[128];
    __shared__ int last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, hb = blockIdx.x >> 3, tb = hb * 4096 + tid * 8;
    const int4 s0 = *reinterpret_cast<const int4 *>(signs + tb), s1 = *reinterpret_cast<const int4 *>(signs + tb + 4);
    bnk::pdl_sync();
    {
        const int e = blockIdx.x * NT + tid;
        y[e] = __fmul_rn(silu_f(gate[e]), up[e]);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last = atomicAdd(count + hb, 1) == 7;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (tid == 0) count[hb] = 0;                                       // all eight have arrived: ready for the next token
    const float4 y0 = __ldcg(reinterpret_cast<const float4 *>(y + tb)), y1 = __ldcg(reinterpret_cast<const float4 *>(y + tb + 4));
    const int sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float v[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
    for (int r = 0; r < 8; ++r) v[r] = apply_sign(v[r], sg[r]);
    fwht_regs_lanes(v, lane);
    {
        float4 *dst = reinterpret_cast<float4 *>(xs + tid * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    __syncthreads();
    fwht_4096_tail(xs, warp, lane, hat_inv);
    __syncthreads();
    q81_pass(xs, codes, dsw, 128, tid);
    __syncthreads();
    uint32_t *blk = pack + size_t(hb) * 32 * Q81_DWORDS;               // this Hadamard block's 32 blocks of 128
    for (int i = tid; i < 32 * 32; i += NT) blk[(i >> 5) * Q81_DWORDS + 4 + (i & 31)] = reinterpret_cast<const uint32_t *>(codes)[i];
    if (tid < 128) blk[(tid >> 2) * Q81_DWORDS + (tid & 3)] = dsw[tid];
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
    if (threadIdx.x == 0) mbar_wait(&bar, 0, err, nullptr, limit);
}

}  // namespace

namespace bnk {

size_t phase_smem_bytes(int hat_block) { return size_t(phase::smem_bytes(hat_block)); }

bool phase_supported(int M, int K, int hat_block) {
    const int nb = K / 128;
    if (K % 512 || K > phase::MAXK || M < 1) return false;
    if (nb > phase::MAXCH && nb % phase::MAXCH) return false;
    if (hat_block < 16 || hat_block > 4096 || K % hat_block || (hat_block & (hat_block - 1))) return false;
    return true;
}

cudaError_t launch_phase(cudaStream_t st, int sm_count, const PhaseArgs &a, bool pdl) {
    static bool attr_set = false;
    if (!attr_set) {
        const int bytes = int(phase_smem_bytes(4096));
        cudaError_t e = cudaFuncSetAttribute(k_phase_gemv<EPI_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_phase_gemv<EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_phase_gemv<EPI_SILU_FROM>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const int ntiles = (a.M + 15) / 16, nchunks = (a.K / 128 + phase::MAXCH - 1) / phase::MAXCH;
    int grid = ntiles < sm_count ? ntiles : sm_count;
    if (a.epi == EPI_SWIGLU && grid > ntiles / 2) grid = ntiles / 2;              // whole gate / up pairs per CTA
    // multi-chunk projections keep per-tile running sums in shared memory: at most 64 tiles per CTA
    while ((nchunks > 1 || a.epi != EPI_PLAIN) && (ntiles + grid - 1) / grid > 64 - 2) ++grid;
    if (a.epi != EPI_PLAIN && (nchunks > 1 || a.epi == EPI_ARGMAX)) return cudaErrorInvalidValue;   // one chunk of K; the pick runs in the whole-token kernel only
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(phase::NTHREADS);
    cfg.dynamicSmemBytes = phase_smem_bytes(a.hat_block);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    BN_COUNT(1);
    if (a.epi == EPI_SWIGLU) return cudaLaunchKernelEx(&cfg, k_phase_gemv<EPI_SWIGLU>, a);
    if (a.epi == EPI_SILU_FROM) return cudaLaunchKernelEx(&cfg, k_phase_gemv<EPI_SILU_FROM>, a);
    return cudaLaunchKernelEx(&cfg, k_phase_gemv<EPI_PLAIN>, a);
}

bool swiglu_pack_supported(int n, int hat_block) { return hat_block == 4096 && n >= 4096 && n % 4096 == 0 && n / 4096 <= 64; }
void swiglu_pack(cudaStream_t st, const float *gate, const float *up, int n, const int32_t *signs, float hat_inv, float *y, uint32_t *pack, int *count) {
    launch(k_swiglu_pack, dim3(n / phase::NT), dim3(phase::NT), 0, st, gate, up, signs, hat_inv, y, pack, count);
}

cudaError_t launch_wait_selftest_ring(cudaStream_t st, int *err) {
    BN_COUNT(1);
    k_wait_selftest<<<1, 32, 0, st>>>(err, 1 << 10);
    return cudaGetLastError();
}

}  // namespace bnk
