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
    if (!copy_warp) preload(a, tid, pl);
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
    if (hat_block < 32 || hat_block > 4096 || K % hat_block || (hat_block & (hat_block - 1))) return false;
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

cudaError_t launch_wait_selftest_ring(cudaStream_t st, int *err) {
    BN_COUNT(1);
    k_wait_selftest<<<1, 32, 0, st>>>(err, 1 << 10);
    return cudaGetLastError();
}

}  // namespace bnk
