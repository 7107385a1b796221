// common.cuh - shared declarations of libbonsai_cuda (context, error plumbing, device helpers).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "../../include/bonsai_cuda.h"

struct bn_buf {
    void *dptr;
    size_t bytes;
    bool owned;      // false: wraps memory of the caller
};

struct bn_event {
    cudaEvent_t ev;
};

struct bn_ctx {
    int device;
    int sm_count;
    cudaStream_t stream;
    bool own_stream;
    uint64_t launches;
    // library-owned scratch for split-K partials, grown on demand (never during a graph capture)
    float *scratch;
    size_t scratch_bytes;
    // row-tile arrival counters of the split-K finalisation (kept zero between kernels) and the
    // device error word that bounded waits set
    unsigned *counters;
    int *err_dev;
};
constexpr int BN_MAX_TILES = 1 << 16;   // rows / 16 of the largest supported projection

void bn_set_error(const char *fmt, ...);
int bn_cuda_fail(cudaError_t e, const char *what);

#define BN_CUDA(call)                                          \
    do {                                                       \
        cudaError_t e_ = (call);                               \
        if (e_ != cudaSuccess) return bn_cuda_fail(e_, #call); \
    } while (0)

#define BN_REQUIRE(cond, code, ...)  \
    do {                             \
        if (!(cond)) {               \
            bn_set_error(__VA_ARGS__); \
            return (code);           \
        }                            \
    } while (0)

// range check of (buffer, offset, size); alignment in bytes
static inline int bn_check_range(const bn_buf *b, size_t off, size_t n, size_t align, const char *what) {
    if (!b || !b->dptr) { bn_set_error("%s: null buffer", what); return BN_ERR_ARG; }
    if ((reinterpret_cast<uintptr_t>(b->dptr) + off) % align) {      // the address itself: a wrapped pointer may have any base
        bn_set_error("%s: address (base + offset %zu) not %zu-byte aligned", what, off, align);
        return BN_ERR_ARG;
    }
    if (off > b->bytes || n > b->bytes - off) {
        bn_set_error("%s: range [%zu, +%zu) exceeds buffer of %zu bytes", what, off, n, b->bytes);
        return BN_ERR_BOUNDS;
    }
    return BN_OK;
}
#define BN_RANGE(b, off, n, align, what)                                  \
    do {                                                                  \
        int rc_ = bn_check_range((b), (off), (n), (align), (what));       \
        if (rc_ != BN_OK) return rc_;                                     \
    } while (0)

template <class T>
static inline T *bn_ptr(const bn_buf *b, size_t off) {
    return reinterpret_cast<T *>(static_cast<char *>(b->dptr) + off);
}

int bn_scratch_reserve(bn_ctx *ctx, size_t bytes);
// every kernel launch of this library is counted here (one process drives one GPU)
extern unsigned long long g_bn_launches;
#define BN_COUNT(n) (g_bn_launches += (n))
int bn_launch_check(bn_ctx *ctx, const char *what);

// ---- device helpers ---------------------------------------------------------------------------
#ifdef __CUDACC__
// transcendental policy shared with the CPU checker: evaluate in double, round once to float
__device__ __forceinline__ float exp_f(float x) { return float(exp(double(x))); }
__device__ __forceinline__ float log_f(float x) { return float(log(double(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(-x))); }
__device__ __forceinline__ float silu_f(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, exp_f(-x))); }

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)(h & 0xFFFFu)));
}
__device__ __forceinline__ uint32_t float_to_half_bits(float f) {
    return (uint32_t)__half_as_ushort(__float2half_rn(f));
}
#endif
