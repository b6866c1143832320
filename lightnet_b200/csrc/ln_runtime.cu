// Context, device-memory pool and tensor handles of liblightnet_b200.
#include <cstdlib>
#include <cstring>

#include "ln_common.h"

static thread_local std::string g_create_error;

int ln_fail(ln_ctx* ctx, int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf;
    else g_create_error = buf;
    return code;
}

// Device-memory pool of a ctx.  Freed blocks are cached by size:
// a request takes the smallest cached block that holds it, provided that block is at most twice the request (so a caller
// whose sizes vary from call to call -- image staging, NMS working memory -- does not force a fresh cudaMalloc, a device-wide
// synchronisation, for every distinct size).  The true size of every live block is remembered, so callers may pass the
// size they asked for when they free.  The cache is trimmed when it exceeds the larger of 2 GiB and the live bytes.
static void pool_drop_cached(ln_ctx* ctx, std::multimap<size_t, void*>::iterator it) {
    cudaFree(it->second);
    ctx->cached_bytes -= it->first;
    ctx->pool_bytes -= it->first;
    ctx->free_blocks.erase(it);
}

void* ln_pool_alloc(ln_ctx* ctx, size_t bytes) {
    bytes = (size_t)ln_round_up((int64_t)(bytes ? bytes : 1), 512);
    auto it = ctx->free_blocks.lower_bound(bytes);
    if (it != ctx->free_blocks.end() && it->first <= 2 * bytes) {
        void* p = it->second;
        ctx->cached_bytes -= it->first;
        ctx->live_blocks[p] = it->first;
        ctx->free_blocks.erase(it);
        return p;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        // release every cached block once and retry
        while (!ctx->free_blocks.empty()) pool_drop_cached(ctx, ctx->free_blocks.begin());
        (void)cudaGetLastError();
        e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) {
            ln_fail(ctx, LN_ERR_CUDA, "cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
            (void)cudaGetLastError();
            return nullptr;
        }
    }
    ctx->pool_bytes += bytes;
    ctx->live_blocks[p] = bytes;
    return p;
}

void ln_pool_free(ln_ctx* ctx, void* p, size_t bytes) {
    if (!p) return;
    auto live = ctx->live_blocks.find(p);
    const size_t real = live != ctx->live_blocks.end() ? live->second : (size_t)ln_round_up((int64_t)(bytes ? bytes : 1), 512);
    if (live != ctx->live_blocks.end()) ctx->live_blocks.erase(live);
    ctx->free_blocks.emplace(real, p);
    ctx->cached_bytes += real;
    // trim: largest blocks first (cudaFree waits for the device, so nothing in flight still uses them)
    const size_t live_bytes = ctx->pool_bytes - ctx->cached_bytes;
    const size_t cap = live_bytes > ((size_t)2 << 30) ? live_bytes : ((size_t)2 << 30);
    while (ctx->cached_bytes > cap && !ctx->free_blocks.empty()) pool_drop_cached(ctx, std::prev(ctx->free_blocks.end()));
}

static size_t storage_bytes(int dtype, int64_t n, int64_t c, int64_t h, int64_t w, int64_t* cstride) {
    if (dtype == LN_Q8 || dtype == LN_F8) {
        *cstride = ln_round_up(c, 32);
        return (size_t)(n * h * w * *cstride);
    }
    if (dtype == LN_F16) {  // NHWC binary16, channels padded to 32: a pixel is a multiple of 64 bytes
        *cstride = 2 * ln_round_up(c, 32);
        return (size_t)(n * h * w * *cstride);
    }
    *cstride = 0;
    return (size_t)(n * c * h * w) * 4;
}

ln_tensor* ln_tensor_new(ln_ctx* ctx, int dtype, int64_t n, int64_t c, int64_t h, int64_t w) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0) {
        ln_fail(ctx, LN_ERR_SHAPE, "tensor shape [%lld,%lld,%lld,%lld] has a non-positive extent", (long long)n, (long long)c,
                (long long)h, (long long)w);
        return nullptr;
    }
    ln_tensor* t = new ln_tensor();
    t->ctx = ctx;
    t->dtype = dtype;
    t->n = n; t->c = c; t->h = h; t->w = w;
    t->bytes = storage_bytes(dtype, n, c, h, w, &t->cstride);
    t->base = ln_pool_alloc(ctx, t->bytes);
    if (!t->base) { delete t; return nullptr; }
    t->ptr = t->base;
    return t;
}

ln_tensor* ln_tensor_view_q(ln_tensor* parent, int64_t channel_offset, int64_t channels) {
    ln_tensor* t = new ln_tensor(*parent);
    t->refcount = 1;
    t->base = nullptr;
    t->bytes = 0;
    t->parent = parent;
    parent->refcount++;
    t->c = channels;
    t->ptr = (char*)parent->ptr + channel_offset;
    return t;
}

// Images [start, start + count) of an f32 NCHW tensor (a contiguous range of the parent's storage).
ln_tensor* ln_tensor_view_batch(ln_tensor* parent, int64_t start, int64_t count) {
    ln_tensor* t = new ln_tensor(*parent);
    t->refcount = 1;
    t->base = nullptr;
    t->bytes = 0;
    t->parent = parent;
    parent->refcount++;
    t->n = count;
    t->ptr = (char*)parent->ptr + (size_t)start * parent->c * parent->h * parent->w * 4;
    return t;
}

extern "C" {

int32_t ln_ctx_create(int32_t device, ln_ctx** out) {
    if (!out) return ln_fail(nullptr, LN_ERR_ARG, "ln_ctx_create: out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        (void)cudaGetLastError();
        return ln_fail(nullptr, LN_ERR_CUDA, "no usable CUDA device (%s); this backend has no CPU fallback",
                       e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    }
    if (device < 0 || device >= count) return ln_fail(nullptr, LN_ERR_ARG, "device %d out of range (%d devices)", device, count);
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return ln_fail(nullptr, LN_ERR_CUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return ln_fail(nullptr, LN_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10) return ln_fail(nullptr, LN_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    ln_ctx* ctx = new ln_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete ctx; return ln_fail(nullptr, LN_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); }
    e = cudaMalloc(&ctx->d_status, 64);
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->d_status, 0, 64, ctx->stream);
    if (e == cudaSuccess) e = cudaMallocHost(&ctx->h_status, 64);
    if (e != cudaSuccess) { delete ctx; return ln_fail(nullptr, LN_ERR_CUDA, "status word allocation: %s", cudaGetErrorString(e)); }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn) { delete ctx; return ln_fail(nullptr, LN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver"); }
    ctx->encode_tiled = (ln_encode_tiled_fn)fn;
    if (const char* e = getenv("LN_NMS_POOL_ENTRIES")) {  // tuning aid: same as ln_ctx_set_nms_pool_entries
        const long long v = atoll(e);
        if (v > 0 && v <= (1ll << 30)) ctx->nms_pool_entries = (int)v;
    }
    if (getenv("LN_DEBUG_CYCLES")) {
        if (cudaMallocManaged(&ctx->debug_cycles, 32 * sizeof(long long)) != cudaSuccess) ctx->debug_cycles = nullptr;
        else memset(ctx->debug_cycles, 0, 32 * sizeof(long long));
    }
    *out = ctx;
    return LN_OK;
}

int32_t ln_ctx_destroy(ln_ctx* ctx) {
    if (!ctx) return LN_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& kv : ctx->free_blocks) cudaFree(kv.second);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return LN_OK;
}

const char* ln_last_error(ln_ctx* ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }

int32_t ln_sync(ln_ctx* ctx) {
    if (!ctx) return LN_ERR_ARG;
    LN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return LN_OK;
}

void* ln_ctx_stream(ln_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

// Debug aid (LN_DEBUG_CYCLES=1 in the environment when the ctx is created, library built with -DLN_CONV_ROLE_TIMING): the 32
// role-timing counters CTA 0 of the last tensor-core convolution wrote.  LN_ERR_UNSUPPORTED when the counters are off.
int32_t ln_ctx_debug_cycles(ln_ctx* ctx, int64_t cycles[32]) {
    if (!ctx || !cycles) return ln_fail(ctx, LN_ERR_ARG, "ln_ctx_debug_cycles: NULL argument");
    if (!ctx->debug_cycles) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_ctx_debug_cycles: role timing is off (set LN_DEBUG_CYCLES=1 before ln_ctx_create)");
    LN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < 32; ++i) cycles[i] = (int64_t)ctx->debug_cycles[i];
    return LN_OK;
}

int32_t ln_ctx_set_exact_epilogue(ln_ctx* ctx, int32_t on) {
    if (!ctx) return LN_ERR_ARG;
    ctx->exact_epilogue = on != 0;
    return LN_OK;
}

int64_t ln_ctx_launch_count(ln_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t ln_ctx_set_kernel_timing(ln_ctx* ctx, int32_t on) {
    if (!ctx) return LN_ERR_ARG;
    cudaSetDevice(ctx->device);
    if (on && !ctx->ev_k0) {
        LN_CUDA(ctx, cudaEventCreate(&ctx->ev_k0));
        LN_CUDA(ctx, cudaEventCreate(&ctx->ev_k1));
    }
    ctx->time_kernels = on != 0;
    ctx->ev_pending = false;
    return LN_OK;
}

int32_t ln_ctx_last_kernel_ms(ln_ctx* ctx, float* ms) {
    if (!ctx || !ms) return ln_fail(ctx, LN_ERR_ARG, "ln_ctx_last_kernel_ms: NULL argument");
    if (!ctx->ev_pending) return ln_fail(ctx, LN_ERR_ARG, "ln_ctx_last_kernel_ms: no kernel has been timed since timing was switched on");
    LN_CUDA(ctx, cudaEventSynchronize(ctx->ev_k1));
    LN_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_k0, ctx->ev_k1));
    return LN_OK;
}

int32_t ln_tensor_upload_f32(ln_ctx* ctx, const int64_t shape[4], const float* host, ln_tensor** out) {
    if (!ctx || !shape || !host || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_f32: NULL argument");
    cudaSetDevice(ctx->device);
    ln_tensor* t = ln_tensor_new(ctx, LN_F32, shape[0], shape[1], shape[2], shape[3]);
    if (!t) return ctx->err.find("cudaMalloc") != std::string::npos ? LN_ERR_CUDA : LN_ERR_SHAPE;
    cudaError_t e = cudaMemcpyAsync(t->ptr, host, (size_t)t->count() * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) { ln_tensor_release(t); return ln_fail(ctx, LN_ERR_CUDA, "upload: %s", cudaGetErrorString(e)); }
    *out = t;
    return LN_OK;
}

int32_t ln_tensor_zeros_f32(ln_ctx* ctx, const int64_t shape[4], ln_tensor** out) {
    if (!ctx || !shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_zeros_f32: NULL argument");
    cudaSetDevice(ctx->device);
    ln_tensor* t = ln_tensor_new(ctx, LN_F32, shape[0], shape[1], shape[2], shape[3]);
    if (!t) return LN_ERR_SHAPE;
    cudaError_t e = cudaMemsetAsync(t->ptr, 0, (size_t)t->count() * 4, ctx->stream);
    if (e != cudaSuccess) { ln_tensor_release(t); return ln_fail(ctx, LN_ERR_CUDA, "memset: %s", cudaGetErrorString(e)); }
    *out = t;
    return LN_OK;
}

int32_t ln_tensor_download_f32(ln_ctx* ctx, const ln_tensor* t, float* host, int64_t count) {
    if (!ctx || !t || !host) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_f32: NULL argument");
    if (t->dtype != LN_F32) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_f32: tensor is not f32");
    if (count != t->count()) return ln_fail(ctx, LN_ERR_SHAPE, "download of %lld elements from a tensor of %lld", (long long)count, (long long)t->count());
    LN_CUDA(ctx, cudaMemcpyAsync(host, t->ptr, (size_t)count * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return LN_OK;
}

int32_t ln_tensor_download_i32(ln_ctx* ctx, const ln_tensor* t, int32_t* host, int64_t count) {
    if (!ctx || !t || !host) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_i32: NULL argument");
    if (t->dtype != LN_I32) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_i32: tensor is not int32");
    if (count != t->count()) return ln_fail(ctx, LN_ERR_SHAPE, "download of %lld elements from a tensor of %lld", (long long)count, (long long)t->count());
    LN_CUDA(ctx, cudaMemcpyAsync(host, t->ptr, (size_t)count * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return LN_OK;
}

int32_t ln_tensor_shape(const ln_tensor* t, int64_t shape[4]) {
    if (!t || !shape) return LN_ERR_ARG;
    shape[0] = t->n; shape[1] = t->c; shape[2] = t->h; shape[3] = t->w;
    return LN_OK;
}

int32_t ln_tensor_dtype(const ln_tensor* t) { return t ? t->dtype : -1; }
float ln_tensor_scale(const ln_tensor* t) { return t ? t->scale : 0.0f; }

int32_t ln_tensor_retain(ln_tensor* t) {
    if (!t) return LN_ERR_ARG;
    t->refcount++;
    return LN_OK;
}

int32_t ln_tensor_release(ln_tensor* t) {
    if (!t) return LN_OK;
    if (--t->refcount > 0) return LN_OK;
    if (t->base) ln_pool_free(t->ctx, t->base, t->bytes);
    ln_tensor* parent = t->parent;
    delete t;
    if (parent) ln_tensor_release(parent);
    return LN_OK;
}

}  // extern "C"
