// Binary16-storage twin of the tensor operators: the methods of trait F16TensorOpsBackend
// (lightnet-cuda/src/lib.rs:6295-6629) that forward_compact_f16 (lightnet-runtime/src/runtime/gpu_f16.rs:21) drives for
// a detector: upload / download / widen / narrow, conv_weights_f16, conv2d_bias_act_f16, maxpool, upsample (both
// directions), route, shortcut (fit + add), per-channel affine.
//
// Storage ("backend-defined, opaque to the caller", lib.rs:6310): NHWC binary16 with channels padded to 32, so that a pixel
// is a multiple of 64 bytes and the tensor-core convolution reads it with the same byte-oriented TMA boxes as the 8-bit
// types (tcgen05.mma kind::f16 consumes 32 bytes of K per instruction, like kind::i8).  Arithmetic follows the reference
// kernels (lightnet-cuda-oxide/src/kernels/half_ops.rs): values widen to binary32, the result is rounded once to
// binary16 (round to nearest even, overflow stays infinite, NaN stays NaN); convolutions accumulate in binary32.
#include <cuda_fp16.h>

#include "ln_conv_plan.h"

namespace {

constexpr int kThreads = 256;

int grid_for(ln_ctx* ctx, int64_t n) {
    int64_t b = (n + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)ctx->sm_count * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

bool is_h(const ln_tensor* t) { return t && t->dtype == LN_F16; }

// f32 NCHW -> binary16 NHWC (pad channels zero)
__global__ void f32_nchw_to_h_nhwc_kernel(const float* __restrict__ x, __half* __restrict__ y, int64_t N, int C, int H, int W, int64_t cs) {
    const int64_t total = N * H * W * cs;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cs);
        const int64_t pix = i / cs, hw = pix % ((int64_t)H * W), n = pix / ((int64_t)H * W);
        y[i] = c < C ? __float2half_rn(x[(n * C + c) * H * W + hw]) : __float2half_rn(0.0f);
    }
}
// binary16 NHWC -> f32 NCHW
__global__ void h_nhwc_to_f32_nchw_kernel(const __half* __restrict__ x, float* __restrict__ y, int64_t N, int C, int H, int W, int64_t cs) {
    const int64_t total = N * C * H * W;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t hw = i % ((int64_t)H * W);
        const int c = (int)((i / ((int64_t)H * W)) % C);
        const int64_t n = i / ((int64_t)H * W * C);
        y[i] = __half2float(x[(n * H * W + hw) * cs + c]);
    }
}
// f32 [F][C][k][k] -> binary16 [fpad][k][k][cpad] (the GEMM B operand, K-major) and the flat rounded copy
__global__ void pack_weights_h_kernel(const float* __restrict__ w, int F, int C, int k, int cpad, int fpad, __half* __restrict__ packed) {
    const int64_t total = (int64_t)fpad * k * k * cpad;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cpad);
        const int tap = (int)((i / cpad) % (k * k));
        const int f = (int)(i / ((int64_t)cpad * k * k));
        packed[i] = (f < F && c < C) ? __float2half_rn(w[((int64_t)f * C + c) * k * k + tap]) : __float2half_rn(0.0f);
    }
}
__global__ void make_mb_unit_kernel(const float* __restrict__ bias, int F, int fpad, float2* __restrict__ mb) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f < fpad) mb[f] = make_float2(f < F ? 1.0f : 0.0f, f < F ? bias[f] : 0.0f);
}

// General convolution on CUDA cores for the geometries the tensor-core kernel does not take (groups, dilation, unequal or
// large strides): one thread per output value, binary32 accumulation in the reference's (channel, ky, kx) order
// (runtime/forward_layers.rs:646-679), weights in their [F][C/g][k][k] order rounded to binary16.
__global__ void conv_h_simt_kernel(const __half* __restrict__ x, int64_t xs, const float* __restrict__ w_f32, const float* __restrict__ bias,
                                   __half* __restrict__ y, int64_t ys, int64_t N, int C, int H, int W, int F, int k, int sx, int sy, int dil, int pad,
                                   int groups, int OH, int OW, int act) {
    const int64_t total = N * OH * OW * F;
    const int cpg = C / groups, fpg = F / groups;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int f = (int)(i % F);
        const int64_t pix = i / F;
        const int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        const int64_t n = pix / ((int64_t)OW * OH);
        const int g = f / fpg;
        float acc = 0.0f;
        for (int ic = 0; ic < cpg; ++ic)
            for (int ky = 0; ky < k; ++ky) {
                const int iy = oy * sy + ky * dil - pad;
                if (iy < 0 || iy >= H) continue;
                for (int kx = 0; kx < k; ++kx) {
                    const int ix = ox * sx + kx * dil - pad;
                    if (ix < 0 || ix >= W) continue;
                    const float xv = __half2float(x[((n * H + iy) * W + ix) * xs + g * cpg + ic]);
                    const float wv = __half2float(__float2half_rn(w_f32[(((int64_t)f * cpg + ic) * k + ky) * k + kx]));
                    acc = fmaf(xv, wv, acc);
                }
            }
        y[pix * ys + f] = __float2half_rn(ln_epilogue_act<false>(act, acc + bias[f]));
    }
}

// max-pool, one thread per (output pixel, 8 channels): window origin o * stride - padding / 2, taps outside the image skipped,
// start value -inf (half_ops.rs maxpool_f16; runtime/layer_ops.rs:1740-1799)
__global__ void maxpool_h_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N, int C8, int H, int W, int OH,
                                 int OW, int size, int sx, int sy, int padding) {
    const int64_t total = N * OH * OW * C8;
    const int off = padding / 2;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C8);
        const int64_t pix = i / C8;
        const int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        const int64_t n = pix / ((int64_t)OW * OH);
        const __half2 ninf = __half2half2(__ushort_as_half((unsigned short)0xFC00));
        __half2 m[4] = {ninf, ninf, ninf, ninf};
        for (int ky = 0; ky < size; ++ky) {
            const int iy = oy * sy + ky - off;
            if (iy < 0 || iy >= H) continue;
            for (int kx = 0; kx < size; ++kx) {
                const int ix = ox * sx + kx - off;
                if (ix < 0 || ix >= W) continue;
                const uint4 v = *reinterpret_cast<const uint4*>(x + ((n * H + iy) * W + ix) * xs + cg * 16);
                const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                for (int j = 0; j < 4; ++j) m[j] = __hmax2(m[j], h[j]);  // a NaN tap never replaces the maximum, as `v > best` in the reference
            }
        }
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = *reinterpret_cast<const uint4*>(m);
    }
}

// nearest up-sample with scale (half_ops.rs upsample_nearest_f16: bits are copied when scale == 1, otherwise f16(scale * x))
__global__ void upsample_h_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N, int C8, int H, int W, int s,
                                  float scale) {
    const int OH = H * s, OW = W * s;
    const int64_t total = N * OH * OW * C8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C8);
        const int64_t pix = i / C8;
        const int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        const int64_t n = pix / ((int64_t)OW * OH);
        uint4 v = *reinterpret_cast<const uint4*>(x + ((n * H + oy / s) * W + ox / s) * xs + cg * 16);
        if (scale != 1.0f) {
            __half* h = reinterpret_cast<__half*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(__fmul_rn(scale, __half2float(h[j])));
        }
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = v;
    }
}
// reverse: out = f16(scale * sum over the stride x stride block), binary32 sum in (dy, dx) order (half_ops.rs upsample_reverse_f16)
__global__ void upsample_reverse_h_kernel(const __half* __restrict__ x, int64_t xs, __half* __restrict__ y, int64_t ys, int64_t N, int C, int H, int W,
                                          int OH, int OW, int s, float scale) {
    const int64_t total = N * OH * OW * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int64_t pix = i / C;
        const int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        const int64_t n = pix / ((int64_t)OW * OH);
        float sum = 0.0f;
        for (int dy = 0; dy < s; ++dy) {
            const int iy = oy * s + dy;
            if (iy >= H) continue;
            for (int dx = 0; dx < s; ++dx) {
                const int ix = ox * s + dx;
                if (ix < W) sum = __fadd_rn(sum, __half2float(x[((n * H + iy) * W + ix) * xs + c]));
            }
        }
        y[pix * ys + c] = __float2half_rn(__fmul_rn(scale, sum));
    }
}

// channel-slice copy between NHWC views (route): 16-byte vectors when everything is aligned, single values otherwise
__global__ void copy_h8_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t pixels, int C8) {
    const int64_t total = pixels * C8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C8);
        const int64_t pix = i / C8;
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = *reinterpret_cast<const uint4*>(x + pix * xs + cg * 16);
    }
}
__global__ void copy_h1_kernel(const __half* __restrict__ x, int64_t xs, __half* __restrict__ y, int64_t ys, int64_t pixels, int C) {
    const int64_t total = pixels * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int64_t pix = i / C;
        y[pix * ys + c] = x[pix * xs + c];
    }
}

// f16(act(a + b)): the sum is formed in binary32 and rounded once (half_ops.rs shortcut_add_act_f16)
__global__ void shortcut_h_kernel(const uint8_t* __restrict__ a, int64_t as, const uint8_t* __restrict__ b, int64_t bs, uint8_t* __restrict__ y, int64_t ys,
                                  int64_t pixels, int C8, int act) {
    const int64_t total = pixels * C8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C8);
        const int64_t pix = i / C8;
        const uint4 va = *reinterpret_cast<const uint4*>(a + pix * as + cg * 16), vb = *reinterpret_cast<const uint4*>(b + pix * bs + cg * 16);
        const __half* ha = reinterpret_cast<const __half*>(&va);
        const __half* hb = reinterpret_cast<const __half*>(&vb);
        uint4 vo;
        __half* ho = reinterpret_cast<__half*>(&vo);
#pragma unroll
        for (int j = 0; j < 8; ++j) ho[j] = __float2half_rn(ln_act_f32(act, __fadd_rn(__half2float(ha[j]), __half2float(hb[j]))));
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = vo;
    }
}

// Flat per-sample crop / zero-pad of a mismatched shortcut source (lib.rs:6494, the f32 rule of lib.rs:4041): element i of a
// sample in NCHW order is element i of the source sample, or zero beyond the source's length.
__global__ void shortcut_fit_h_kernel(const __half* __restrict__ x, int64_t xs, int sc, int sh, int sw, __half* __restrict__ y, int64_t ys, int64_t N, int C,
                                      int H, int W) {
    const int64_t total = N * C * H * W, src_len = (int64_t)sc * sh * sw;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t flat = i % ((int64_t)C * H * W), n = i / ((int64_t)C * H * W);
        const int w = (int)(flat % W), h = (int)((flat / W) % H), c = (int)(flat / ((int64_t)W * H));
        __half v = __float2half_rn(0.0f);
        if (flat < src_len) {
            const int sx = (int)(flat % sw), sy = (int)((flat / sw) % sh), scc = (int)(flat / ((int64_t)sw * sh));
            v = x[((n * sh + sy) * sw + sx) * xs + scc];
        }
        y[((n * H + h) * W + w) * ys + c] = v;
    }
}

// f16(act(x * scale[c] + bias[c])), scale optional (half_ops.rs channel_affine_act_f16: multiply, then add, then activate)
__global__ void channel_affine_h_kernel(const __half* __restrict__ x, int64_t xs, const float* __restrict__ scale, const float* __restrict__ bias,
                                        __half* __restrict__ y, int64_t ys, int64_t pixels, int C, int act) {
    const int64_t total = pixels * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int64_t pix = i / C;
        float v = __half2float(x[pix * xs + c]);
        if (scale) v = __fmul_rn(v, scale[c]);
        y[pix * ys + c] = __float2half_rn(ln_act_f32(act, __fadd_rn(v, bias[c])));
    }
}

int check_launch(ln_ctx* ctx, const char* what) {
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return LN_OK;
}

int64_t hs(const ln_tensor* t) { return t->cstride / 2; }  // pixel stride in binary16 elements

}  // namespace

extern "C" {

int32_t ln_tensor_upload_f16(ln_ctx* ctx, const int64_t shape[4], const float* host, ln_tensor** out) {
    if (!ctx || !shape || !host || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_f16: NULL argument");
    cudaSetDevice(ctx->device);
    ln_tensor* t = ln_tensor_new(ctx, LN_F16, shape[0], shape[1], shape[2], shape[3]);
    if (!t) return LN_ERR_SHAPE;
    const size_t bytes = (size_t)t->count() * 4;
    float* tmp = (float*)ln_pool_alloc(ctx, bytes);
    if (!tmp) { ln_tensor_release(t); return LN_ERR_CUDA; }
    cudaError_t e = cudaMemcpyAsync(tmp, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        f32_nchw_to_h_nhwc_kernel<<<grid_for(ctx, (int64_t)(t->bytes / 2)), kThreads, 0, ctx->stream>>>(tmp, (__half*)t->ptr, t->n, (int)t->c, (int)t->h, (int)t->w, hs(t));
        ctx->launches++;
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // `host` may be pageable and is the caller's to reuse
    ln_pool_free(ctx, tmp, bytes);
    if (e != cudaSuccess) { ln_tensor_release(t); return ln_fail(ctx, LN_ERR_CUDA, "ln_tensor_upload_f16: %s", cudaGetErrorString(e)); }
    *out = t;
    return LN_OK;
}

int32_t ln_tensor_widen_f16(ln_ctx* ctx, const ln_tensor* t, ln_tensor** out_f32) {
    if (!ctx || !out_f32) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_widen_f16: NULL argument");
    if (!is_h(t)) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_widen_f16: binary16 tensor required");
    cudaSetDevice(ctx->device);
    ln_tensor* f = ln_tensor_new(ctx, LN_F32, t->n, t->c, t->h, t->w);
    if (!f) return LN_ERR_CUDA;
    h_nhwc_to_f32_nchw_kernel<<<grid_for(ctx, f->count()), kThreads, 0, ctx->stream>>>((const __half*)t->ptr, (float*)f->ptr, t->n, (int)t->c, (int)t->h, (int)t->w, hs(t));
    int rc = check_launch(ctx, "widen_f16");
    if (rc) { ln_tensor_release(f); return rc; }
    *out_f32 = f;
    return LN_OK;
}

int32_t ln_tensor_narrow_f16(ln_ctx* ctx, const ln_tensor* t, ln_tensor** out_f16) {
    if (!ctx || !out_f16) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_narrow_f16: NULL argument");
    if (!t || t->dtype != LN_F32) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_narrow_f16: f32 tensor required");
    cudaSetDevice(ctx->device);
    ln_tensor* q = ln_tensor_new(ctx, LN_F16, t->n, t->c, t->h, t->w);
    if (!q) return LN_ERR_CUDA;
    f32_nchw_to_h_nhwc_kernel<<<grid_for(ctx, (int64_t)(q->bytes / 2)), kThreads, 0, ctx->stream>>>((const float*)t->ptr, (__half*)q->ptr, t->n, (int)t->c, (int)t->h, (int)t->w, hs(q));
    int rc = check_launch(ctx, "narrow_f32");
    if (rc) { ln_tensor_release(q); return rc; }
    *out_f16 = q;
    return LN_OK;
}

int32_t ln_tensor_download_f16(ln_ctx* ctx, const ln_tensor* t, float* host, int64_t count) {
    if (!ctx || !host) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_f16: NULL argument");
    if (!is_h(t)) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_f16: binary16 tensor required");
    if (count != t->count()) return ln_fail(ctx, LN_ERR_SHAPE, "download of %lld elements from a tensor of %lld", (long long)count, (long long)t->count());
    ln_tensor* f = nullptr;
    int rc = ln_tensor_widen_f16(ctx, t, &f);
    if (rc) return rc;
    rc = ln_tensor_download_f32(ctx, f, host, count);
    ln_tensor_release(f);
    return rc;
}

int32_t ln_conv_weights_f16(ln_ctx* ctx, const ln_tensor* weights_f32, int64_t filters, int64_t per_filter, ln_conv_weights** out) {
    if (!ctx || !weights_f32 || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_conv_weights_f16: NULL argument");
    if (weights_f32->dtype != LN_F32) return ln_fail(ctx, LN_ERR_ARG, "ln_conv_weights_f16: f32 weights required");
    if (filters < 1 || per_filter < 1 || weights_f32->count() != filters * per_filter)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv_weights_f16: weight tensor has %lld elements, expected %lld x %lld", (long long)weights_f32->count(), (long long)filters, (long long)per_filter);
    // The GEMM operand layout needs the kernel size and the channel count, which this call does not carry (per_filter is their
    // product, lib.rs:6311): the f32 weights are kept and packed by the first convolution that names its geometry.
    ln_conv_weights* w = new ln_conv_weights();
    w->ctx = ctx; w->dtype = LN_F16;
    w->filters = filters; w->per_filter = per_filter;
    w->src_f32 = const_cast<ln_tensor*>(weights_f32);
    ln_tensor_retain(w->src_f32);
    *out = w;
    return LN_OK;
}

int32_t ln_conv2d_bias_act_f16(ln_ctx* ctx, const ln_tensor* x, ln_conv_weights* weights, const ln_tensor* bias, const int64_t output_shape[4],
                               int64_t channels, int64_t input_height, int64_t input_width, int64_t filters, int64_t size, int64_t stride_x,
                               int64_t stride_y, int64_t dilation, int64_t padding, int64_t groups, int32_t activation, ln_tensor** out) {
    const char* who = "ln_conv2d_bias_act_f16";
    if (!ctx || !weights || !bias || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "%s: NULL argument", who);
    if (!is_h(x) || weights->dtype != LN_F16) return ln_fail(ctx, LN_ERR_ARG, "%s: binary16 input and weights required", who);
    if (bias->dtype != LN_F32 || bias->count() != filters) return ln_fail(ctx, LN_ERR_SHAPE, "%s: bias must be f32 [filters]", who);
    if (groups < 1 || filters % groups || channels % groups || size < 1 || stride_x < 1 || stride_y < 1 || dilation < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "%s: invalid geometry", who);
    if (x->c != channels || x->h != input_height || x->w != input_width || weights->filters != filters || weights->per_filter != channels / groups * size * size)
        return ln_fail(ctx, LN_ERR_SHAPE, "%s: geometry does not match the tensors", who);
    if (activation < LN_ACT_LINEAR || activation > LN_ACT_RELU) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "%s: activation %d is not on the detector path", who, activation);
    // (the reference's shape rule ignores dilation, model.rs:6472; the taps do not)
    const int64_t oh = (input_height + 2 * padding - size < 0 ? 0 : input_height + 2 * padding - size) / stride_y + 1;
    const int64_t ow = (input_width + 2 * padding - size < 0 ? 0 : input_width + 2 * padding - size) / stride_x + 1;
    if (output_shape[0] != x->n || output_shape[1] != filters || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "%s: output_shape does not match [%lld,%lld,%lld,%lld]", who, (long long)x->n, (long long)filters, (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, x->n, filters, oh, ow);
    if (!y) return LN_ERR_CUDA;
    if (y->cstride != 2 * y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    int rc = LN_OK;
    const int64_t cpad_bytes = x->cstride;  // 2 * channels padded to 32
    const bool tensor_core = groups == 1 && filters <= 4096 && ln_conv_umma_supported(cpad_bytes, size, stride_x, stride_y, dilation, groups, input_width, input_height);
    if (tensor_core) {
        if (!weights->w || weights->channels != channels || weights->k != size) {  // first use with this geometry: pack
            if (weights->w) ln_pool_free(ctx, weights->w, 0);
            weights->channels = channels; weights->k = size;
            weights->cpad = cpad_bytes;
            weights->fpad = ln_round_up(filters, ln_conv_choose_bn(filters));
            const int64_t elems = weights->fpad * size * size * (cpad_bytes / 2);
            weights->w = ln_pool_alloc(ctx, (size_t)elems * 2);
            if (!weights->w) { ln_tensor_release(y); return LN_ERR_CUDA; }
            pack_weights_h_kernel<<<grid_for(ctx, elems), kThreads, 0, ctx->stream>>>((const float*)weights->src_f32->ptr, (int)filters, (int)channels, (int)size, (int)(cpad_bytes / 2),
                                                                                    (int)weights->fpad, (__half*)weights->w);
            rc = check_launch(ctx, "conv_weights_f16");
        }
        float2* mb = (float2*)ln_pool_alloc(ctx, (size_t)weights->fpad * sizeof(float2));
        if (!mb) { ln_tensor_release(y); return LN_ERR_CUDA; }
        if (rc == LN_OK) {
            make_mb_unit_kernel<<<(int)((weights->fpad + 127) / 128), 128, 0, ctx->stream>>>((const float*)bias->ptr, (int)filters, (int)weights->fpad, mb);
            rc = check_launch(ctx, "conv bias table");
        }
        ln_conv_geom g;
        g.kind = LN_KIND_F16;
        g.x = x->ptr; g.x_pixel_stride = x->cstride;
        g.N = (int)x->n; g.H = (int)x->h; g.W = (int)x->w; g.C = (int)cpad_bytes; g.cpad = (int)cpad_bytes;
        g.w = weights->w; g.F = (int)filters; g.fpad = (int)weights->fpad; g.k = (int)size; g.stride = (int)stride_x; g.pad = (int)padding;
        g.OH = (int)oh; g.OW = (int)ow; g.act = activation; g.out_kind = LN_OUT_Q;
        g.out = y->ptr; g.out_pixel_stride = y->cstride;
        if (rc == LN_OK) {
            ln_conv_umma_plan plan;
            plan.mb = mb;
            rc = ln_conv_umma_plan_build(ctx, &plan, g);
            if (rc == LN_OK) rc = ln_conv_umma_launch(ctx, &plan);
            if (rc == LN_OK) rc = ln_check_status(ctx, who);
            ln_conv_umma_plan_release(ctx, &plan);
        }
        ln_pool_free(ctx, mb, (size_t)weights->fpad * sizeof(float2));
    } else {
        conv_h_simt_kernel<<<grid_for(ctx, y->count()), kThreads, 0, ctx->stream>>>((const __half*)x->ptr, hs(x), (const float*)weights->src_f32->ptr, (const float*)bias->ptr,
                                                                                  (__half*)y->ptr, hs(y), x->n, (int)channels, (int)input_height, (int)input_width, (int)filters,
                                                                                  (int)size, (int)stride_x, (int)stride_y, (int)dilation, (int)padding, (int)groups, (int)oh, (int)ow,
                                                                                  activation);
        rc = check_launch(ctx, "conv2d_bias_act_f16");
    }
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_maxpool_f16(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height, int64_t input_width,
                       int64_t size, int64_t stride_x, int64_t stride_y, int64_t padding, ln_tensor** out) {
    if (!ctx || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_maxpool_f16: NULL argument");
    if (!is_h(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_maxpool_f16: binary16 tensor required");
    if (x->c != channels || x->h != input_height || x->w != input_width || size < 1 || stride_x < 1 || stride_y < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_maxpool_f16: geometry does not match the input tensor");
    const int64_t oh = (input_height + padding - size < 0 ? 0 : input_height + padding - size) / stride_y + 1;
    const int64_t ow = (input_width + padding - size < 0 ? 0 : input_width + padding - size) / stride_x + 1;
    if (output_shape[0] != x->n || output_shape[1] != channels || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_maxpool_f16: output_shape does not match pool_dim (%lld x %lld)", (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, x->n, channels, oh, ow);
    if (!y) return LN_ERR_CUDA;
    const int C8 = (int)(y->cstride / 16);
    maxpool_h_kernel<<<grid_for(ctx, x->n * oh * ow * C8), kThreads, 0, ctx->stream>>>((const uint8_t*)x->ptr, x->cstride, (uint8_t*)y->ptr, y->cstride, x->n, C8, (int)input_height,
                                                                                      (int)input_width, (int)oh, (int)ow, (int)size, (int)stride_x, (int)stride_y, (int)padding);
    int rc = check_launch(ctx, "maxpool_f16");
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_upsample_f16(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height, int64_t input_width,
                        int64_t stride, float scale, int32_t reverse, ln_tensor** out) {
    if (!ctx || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_upsample_f16: NULL argument");
    if (!is_h(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_upsample_f16: binary16 tensor required");
    if (stride < 1) return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_f16: upsample stride cannot be zero");
    if (x->c != channels || x->h != input_height || x->w != input_width) return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_f16: geometry does not match the input tensor");
    const int64_t oh = reverse ? input_height / stride : input_height * stride, ow = reverse ? input_width / stride : input_width * stride;
    if (output_shape[0] != x->n || output_shape[1] != channels || output_shape[2] != oh || output_shape[3] != ow || oh < 1 || ow < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_f16: output_shape does not match");
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, x->n, channels, oh, ow);
    if (!y) return LN_ERR_CUDA;
    if (reverse) {
        if (y->cstride != 2 * y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
        upsample_reverse_h_kernel<<<grid_for(ctx, y->count()), kThreads, 0, ctx->stream>>>((const __half*)x->ptr, hs(x), (__half*)y->ptr, hs(y), x->n, (int)channels, (int)input_height,
                                                                                        (int)input_width, (int)oh, (int)ow, (int)stride, scale);
    } else {
        const int C8 = (int)(y->cstride / 16);
        upsample_h_kernel<<<grid_for(ctx, x->n * oh * ow * C8), kThreads, 0, ctx->stream>>>((const uint8_t*)x->ptr, x->cstride, (uint8_t*)y->ptr, y->cstride, x->n, C8, (int)input_height,
                                                                                           (int)input_width, (int)stride, scale);
    }
    int rc = check_launch(ctx, "upsample_f16");
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_route_concat_f16(ln_ctx* ctx, const ln_tensor* const* inputs, int32_t n_inputs, const int64_t* input_channel_offsets, const int64_t* input_channels,
                            const int64_t* input_total_channels, const int64_t output_shape[4], int64_t channel_stride, ln_tensor** out) {
    if (!ctx || !inputs || !input_channel_offsets || !input_channels || !input_total_channels || !output_shape || !out || n_inputs < 1)
        return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_f16: NULL argument");
    int64_t total_c = 0;
    for (int i = 0; i < n_inputs; ++i) {
        const ln_tensor* t = inputs[i];
        if (!is_h(t)) return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_f16: input %d is not a binary16 tensor", i);
        if (t->c != input_total_channels[i] || input_channel_offsets[i] < 0 || input_channels[i] < 1 || input_channel_offsets[i] + input_channels[i] > t->c)
            return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_f16: channel slice of input %d is outside its %lld channels", i, (long long)t->c);
        if (t->n != output_shape[0] || t->h != output_shape[2] || t->w != output_shape[3] || t->h * t->w != channel_stride)
            return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_f16: input %d does not match the output's batch / spatial shape", i);
        total_c += input_channels[i];
    }
    if (total_c != output_shape[1]) return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_f16: slices add up to %lld channels, output has %lld", (long long)total_c, (long long)output_shape[1]);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, output_shape[0], output_shape[1], output_shape[2], output_shape[3]);
    if (!y) return LN_ERR_CUDA;
    if (y->cstride != 2 * y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    const int64_t pixels = y->n * y->h * y->w;
    int64_t off = 0;
    int rc = LN_OK;
    for (int i = 0; i < n_inputs && rc == LN_OK; ++i) {
        const ln_tensor* t = inputs[i];
        const uint8_t* src = (const uint8_t*)t->ptr + 2 * input_channel_offsets[i];
        uint8_t* dst = (uint8_t*)y->ptr + 2 * off;
        if (input_channel_offsets[i] % 8 == 0 && off % 8 == 0 && input_channels[i] % 8 == 0)
            copy_h8_kernel<<<grid_for(ctx, pixels * (input_channels[i] / 8)), kThreads, 0, ctx->stream>>>(src, t->cstride, dst, y->cstride, pixels, (int)(input_channels[i] / 8));
        else
            copy_h1_kernel<<<grid_for(ctx, pixels * input_channels[i]), kThreads, 0, ctx->stream>>>((const __half*)src, hs(t), (__half*)dst, hs(y), pixels, (int)input_channels[i]);
        rc = check_launch(ctx, "route_concat_f16");
        off += input_channels[i];
    }
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_shortcut_fit_f16(ln_ctx* ctx, const ln_tensor* x, int64_t batch, const int64_t output_shape[4], ln_tensor** out) {
    if (!ctx || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_fit_f16: NULL argument");
    if (!is_h(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_fit_f16: binary16 tensor required");
    if (batch != x->n || output_shape[0] != batch) return ln_fail(ctx, LN_ERR_SHAPE, "ln_shortcut_fit_f16: batch mismatch");
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, output_shape[0], output_shape[1], output_shape[2], output_shape[3]);
    if (!y) return LN_ERR_SHAPE;
    if (y->cstride != 2 * y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    shortcut_fit_h_kernel<<<grid_for(ctx, y->count()), kThreads, 0, ctx->stream>>>((const __half*)x->ptr, hs(x), (int)x->c, (int)x->h, (int)x->w, (__half*)y->ptr, hs(y), y->n, (int)y->c,
                                                                                 (int)y->h, (int)y->w);
    int rc = check_launch(ctx, "shortcut_fit_f16");
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_shortcut_add_act_f16(ln_ctx* ctx, const ln_tensor* a, const ln_tensor* b, int32_t activation, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_act_f16: NULL argument");
    if (!is_h(a) || !is_h(b)) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_act_f16: binary16 tensors required");
    if (a->n != b->n || a->c != b->c || a->h != b->h || a->w != b->w) return ln_fail(ctx, LN_ERR_SHAPE, "ln_shortcut_add_act_f16: shapes differ");
    if (activation < LN_ACT_LINEAR || activation > LN_ACT_RELU) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_shortcut_add_act_f16: activation %d is not on the detector path", activation);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, a->n, a->c, a->h, a->w);
    if (!y) return LN_ERR_CUDA;
    const int C8 = (int)(y->cstride / 16);
    const int64_t pixels = a->n * a->h * a->w;
    shortcut_h_kernel<<<grid_for(ctx, pixels * C8), kThreads, 0, ctx->stream>>>((const uint8_t*)a->ptr, a->cstride, (const uint8_t*)b->ptr, b->cstride, (uint8_t*)y->ptr, y->cstride, pixels,
                                                                               C8, activation);
    int rc = check_launch(ctx, "shortcut_add_act_f16");
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_channel_affine_act_f16(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* scale, const ln_tensor* bias, int64_t channels, int64_t channel_stride,
                                  int32_t activation, ln_tensor** out) {
    if (!ctx || !bias || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_channel_affine_act_f16: NULL argument");
    if (!is_h(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_channel_affine_act_f16: binary16 tensor required");
    if (x->c != channels || x->h * x->w != channel_stride || bias->dtype != LN_F32 || bias->count() != channels || (scale && (scale->dtype != LN_F32 || scale->count() != channels)))
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_channel_affine_act_f16: per-channel parameters do not match %lld channels of %lld values", (long long)channels, (long long)channel_stride);
    if (activation < LN_ACT_LINEAR || activation > LN_ACT_RELU) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_channel_affine_act_f16: activation %d is not on the detector path", activation);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F16, x->n, x->c, x->h, x->w);
    if (!y) return LN_ERR_CUDA;
    if (y->cstride != 2 * y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    const int64_t pixels = x->n * x->h * x->w;
    channel_affine_h_kernel<<<grid_for(ctx, pixels * channels), kThreads, 0, ctx->stream>>>((const __half*)x->ptr, hs(x), scale ? (const float*)scale->ptr : nullptr, (const float*)bias->ptr,
                                                                                          (__half*)y->ptr, hs(y), pixels, (int)channels, activation);
    int rc = check_launch(ctx, "channel_affine_act_f16");
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

}  // extern "C"
