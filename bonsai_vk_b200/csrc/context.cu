// context.cu - context, memory, transfer and event entry points of libbonsai_cuda.
#include "common.cuh"

#include <stdarg.h>
#include <string.h>

static thread_local char g_err[512] = "";
unsigned long long g_bn_launches = 0;

void bn_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int bn_cuda_fail(cudaError_t e, const char *what) {
    bn_set_error("CUDA error %d (%s) in %s", int(e), cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? BN_ERR_NOMEM : BN_ERR_CUDA;
}

int bn_launch_check(bn_ctx *ctx, const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return bn_cuda_fail(e, what);
    (void)ctx;
    return BN_OK;
}

int bn_scratch_reserve(bn_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return BN_OK;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(ctx->stream, &st);
    BN_REQUIRE(st == cudaStreamCaptureStatusNone, BN_ERR_STATE,
               "scratch must grow to %zu bytes but the stream is capturing; run the op once uncaptured first", bytes);
    BN_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = bytes < (size_t(8) << 20) ? (size_t(8) << 20) : bytes;
    BN_CUDA(cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return BN_OK;
}

extern "C" {

const char *bn_last_error(void) { return g_err; }

int bn_init(int device, bn_ctx **out) {
    BN_REQUIRE(out, BN_ERR_ARG, "bn_init: out is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        bn_set_error("bn_init: no CUDA device (%s); this library has no CPU path",
                     e != cudaSuccess ? cudaGetErrorString(e) : "device count 0");
        return BN_ERR_CUDA;
    }
    BN_REQUIRE(device >= 0 && device < n, BN_ERR_ARG, "bn_init: device %d out of range [0,%d)", device, n);
    // one process drives one GPU (multi-GPU = one process per stage): kernel attributes and the launch counter are
    // kept per process, so a second device in the same process is refused rather than half-supported
    static int g_first_device = -1;
    BN_REQUIRE(g_first_device < 0 || g_first_device == device, BN_ERR_STATE,
               "bn_init: this process already drives device %d; use one process per GPU (asked for device %d)", g_first_device, device);
    g_first_device = device;
    BN_CUDA(cudaSetDevice(device));
    cudaDeviceProp p;
    BN_CUDA(cudaGetDeviceProperties(&p, device));
    BN_REQUIRE(p.major == 10, BN_ERR_STATE,
               "bn_init: device %d is sm_%d%d; this library is built for sm_100a (B200) only", device, p.major, p.minor);
    bn_ctx *c = new bn_ctx();
    c->device = device;
    c->sm_count = p.multiProcessorCount;
    c->launches = 0;
    c->scratch = nullptr;
    c->scratch_bytes = 0;
    e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete c; return bn_cuda_fail(e, "cudaStreamCreate"); }
    c->own_stream = true;
    c->counters = nullptr;
    c->err_dev = nullptr;
    e = cudaMalloc(&c->counters, size_t(BN_MAX_TILES) * 4 + 256);
    if (e != cudaSuccess) { delete c; return bn_cuda_fail(e, "cudaMalloc(counters)"); }
    cudaMemset(c->counters, 0, size_t(BN_MAX_TILES) * 4 + 256);
    c->err_dev = reinterpret_cast<int *>(c->counters + BN_MAX_TILES);
    *out = c;
    g_err[0] = 0;
    return BN_OK;
}

void bn_destroy(bn_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int bn_device_info(bn_ctx *ctx, int *sm_count, size_t *free_bytes, size_t *total_bytes) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_device_info: null context");
    BN_CUDA(cudaSetDevice(ctx->device));
    size_t f = 0, t = 0;
    BN_CUDA(cudaMemGetInfo(&f, &t));
    if (sm_count) *sm_count = ctx->sm_count;
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return BN_OK;
}

int bn_alloc(bn_ctx *ctx, size_t bytes, bn_buf **out) {
    BN_REQUIRE(ctx && out, BN_ERR_ARG, "bn_alloc: null argument");
    BN_REQUIRE(bytes > 0, BN_ERR_ARG, "bn_alloc: zero bytes");
    BN_CUDA(cudaSetDevice(ctx->device));
    void *p = nullptr;
    BN_CUDA(cudaMalloc(&p, bytes));
    bn_buf *b = new bn_buf();
    b->dptr = p;
    b->bytes = bytes;
    b->owned = true;
    *out = b;
    return BN_OK;
}

int bn_free(bn_ctx *ctx, bn_buf *buf) {
    BN_REQUIRE(ctx && buf, BN_ERR_ARG, "bn_free: null argument");
    BN_CUDA(cudaSetDevice(ctx->device));
    BN_CUDA(cudaStreamSynchronize(ctx->stream));
    if (buf->owned) BN_CUDA(cudaFree(buf->dptr));
    delete buf;
    return BN_OK;
}

size_t bn_buf_size(const bn_buf *buf) { return buf ? buf->bytes : 0; }

int bn_wrap(bn_ctx *ctx, void *device_ptr, size_t bytes, bn_buf **out) {
    BN_REQUIRE(ctx && device_ptr && bytes && out, BN_ERR_ARG, "bn_wrap: bad argument");
    bn_buf *b = new bn_buf();
    b->dptr = device_ptr;
    b->bytes = bytes;
    b->owned = false;
    *out = b;
    return BN_OK;
}

int bn_use_stream(bn_ctx *ctx, void *cuda_stream) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_use_stream: null context");
    BN_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    ctx->own_stream = false;
    return BN_OK;
}

int bn_upload(bn_ctx *ctx, bn_buf *dst, size_t off, const void *src, size_t n) {
    BN_REQUIRE(ctx && src, BN_ERR_ARG, "bn_upload: null argument");
    BN_RANGE(dst, off, n, 1, "bn_upload");
    if (n == 0) return BN_OK;
    BN_CUDA(cudaMemcpyAsync(bn_ptr<char>(dst, off), src, n, cudaMemcpyHostToDevice, ctx->stream));
    BN_CUDA(cudaStreamSynchronize(ctx->stream));
    return BN_OK;
}

int bn_upload_async(bn_ctx *ctx, bn_buf *dst, size_t off, const void *src, size_t n) {
    BN_REQUIRE(ctx && src, BN_ERR_ARG, "bn_upload_async: null argument");
    BN_RANGE(dst, off, n, 1, "bn_upload_async");
    if (n == 0) return BN_OK;
    BN_CUDA(cudaMemcpyAsync(bn_ptr<char>(dst, off), src, n, cudaMemcpyHostToDevice, ctx->stream));
    return BN_OK;
}

int bn_download(bn_ctx *ctx, const bn_buf *src, size_t off, void *dst, size_t n) {
    BN_REQUIRE(ctx && dst, BN_ERR_ARG, "bn_download: null argument");
    BN_RANGE(src, off, n, 1, "bn_download");
    if (n == 0) return BN_OK;
    BN_CUDA(cudaMemcpyAsync(dst, bn_ptr<char>(src, off), n, cudaMemcpyDeviceToHost, ctx->stream));
    BN_CUDA(cudaStreamSynchronize(ctx->stream));
    return BN_OK;
}

int bn_memset(bn_ctx *ctx, bn_buf *dst, size_t off, int byte, size_t n) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_memset: null context");
    BN_RANGE(dst, off, n, 1, "bn_memset");
    if (n == 0) return BN_OK;
    BN_CUDA(cudaMemsetAsync(bn_ptr<char>(dst, off), byte, n, ctx->stream));
    return BN_OK;
}

int bn_sync(bn_ctx *ctx) {
    BN_REQUIRE(ctx, BN_ERR_ARG, "bn_sync: null context");
    BN_CUDA(cudaStreamSynchronize(ctx->stream));
    int flag = 0;
    BN_CUDA(cudaMemcpy(&flag, ctx->err_dev, 4, cudaMemcpyDeviceToHost));
    if (flag) {
        cudaMemset(ctx->err_dev, 0, 4);
        if (flag == 3) {
            bn_set_error("a token id read from device memory was outside the vocabulary (id 0 was used in its place); results of that step are invalid");
            return BN_ERR_ARG;
        }
        bn_set_error("a bounded device-side wait gave up (%s); results of the last kernels are invalid",
                     flag == 2 ? "tensor-core projection pipeline" : flag == 4 ? "grid barrier of the whole-token kernel" : "copy ring");
        return BN_ERR_TIMEOUT;
    }
    return BN_OK;
}

int bn_host_alloc(size_t bytes, void **out) {
    BN_REQUIRE(out && bytes, BN_ERR_ARG, "bn_host_alloc: bad argument");
    BN_CUDA(cudaHostAlloc(out, bytes, cudaHostAllocDefault));
    return BN_OK;
}

int bn_host_free(void *p) {
    if (p) BN_CUDA(cudaFreeHost(p));
    return BN_OK;
}

int bn_event_create(bn_ctx *ctx, bn_event **out) {
    BN_REQUIRE(ctx && out, BN_ERR_ARG, "bn_event_create: null argument");
    bn_event *e = new bn_event();
    cudaError_t r = cudaEventCreate(&e->ev);
    if (r != cudaSuccess) { delete e; return bn_cuda_fail(r, "cudaEventCreate"); }
    *out = e;
    return BN_OK;
}

int bn_event_record(bn_ctx *ctx, bn_event *ev) {
    BN_REQUIRE(ctx && ev, BN_ERR_ARG, "bn_event_record: null argument");
    BN_CUDA(cudaEventRecord(ev->ev, ctx->stream));
    return BN_OK;
}

int bn_event_elapsed_ms(bn_ctx *ctx, bn_event *start, bn_event *stop, float *ms) {
    BN_REQUIRE(ctx && start && stop && ms, BN_ERR_ARG, "bn_event_elapsed_ms: null argument");
    BN_CUDA(cudaEventSynchronize(stop->ev));
    BN_CUDA(cudaEventElapsedTime(ms, start->ev, stop->ev));
    return BN_OK;
}

int bn_event_destroy(bn_ctx *ctx, bn_event *ev) {
    BN_REQUIRE(ctx && ev, BN_ERR_ARG, "bn_event_destroy: null argument");
    cudaEventDestroy(ev->ev);
    delete ev;
    return BN_OK;
}

uint64_t bn_launch_count(const bn_ctx *ctx) { (void)ctx; return g_bn_launches; }

}  // extern "C"
