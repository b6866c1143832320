// f32 NCHW operators: the F32TensorOpsBackend subset on the detector path
// (lightnet-cuda/src/lib.rs:460).  Plain CUDA-core kernels: this path exists for
// trait fidelity, for calibration and as the f32 parity target; the throughput path
// is the 8-bit one.
#include "ln_common.h"

namespace {

constexpr int kThreads = 256;
inline int blocks_for(int64_t n, int per_block = kThreads) { return (int)((n + per_block - 1) / per_block); }

// Direct convolution, one thread per (pixel, group of FPT filters).  Semantics of
// runtime/forward_layers.rs:646-695: taps outside the image are skipped, groups partition
// channels, weights are [filters][C/groups][k][k].
template <int FPT>
__global__ void conv2d_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int B, int C,
                                  int H, int W, int F, int k, int sx, int sy, int dil, int pad, int groups, int OH, int OW) {
    const int fgroups = (F + FPT - 1) / FPT;
    const int64_t total = (int64_t)B * fgroups * OH * OW;
    const int cpg = C / groups, fpg = F / groups;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int ox = (int)(idx % OW);
        int oy = (int)((idx / OW) % OH);
        int fg = (int)((idx / ((int64_t)OW * OH)) % fgroups);
        int b = (int)(idx / ((int64_t)OW * OH * fgroups));
        float acc[FPT];
#pragma unroll
        for (int j = 0; j < FPT; ++j) acc[j] = 0.0f;
        const int f0 = fg * FPT;
        // all FPT filters share a group only when FPT divides fpg; otherwise fall back to per-filter groups
        const bool same_group = (fpg % FPT) == 0;
        if (same_group) {
            const int g = f0 / fpg;
            for (int ic = 0; ic < cpg; ++ic) {
                const float* xp = x + ((int64_t)b * C + g * cpg + ic) * H * W;
                for (int ky = 0; ky < k; ++ky) {
                    int iy = oy * sy + ky * dil - pad;
                    if (iy < 0 || iy >= H) continue;
                    for (int kx = 0; kx < k; ++kx) {
                        int ix = ox * sx + kx * dil - pad;
                        if (ix < 0 || ix >= W) continue;
                        float xv = xp[(int64_t)iy * W + ix];
#pragma unroll
                        for (int j = 0; j < FPT; ++j)
                            if (f0 + j < F) acc[j] = fmaf(xv, w[(((int64_t)(f0 + j) * cpg + ic) * k + ky) * k + kx], acc[j]);
                    }
                }
            }
        } else {
            for (int j = 0; j < FPT; ++j) {
                int f = f0 + j;
                if (f >= F) break;
                const int g = f / fpg;
                for (int ic = 0; ic < cpg; ++ic) {
                    const float* xp = x + ((int64_t)b * C + g * cpg + ic) * H * W;
                    for (int ky = 0; ky < k; ++ky) {
                        int iy = oy * sy + ky * dil - pad;
                        if (iy < 0 || iy >= H) continue;
                        for (int kx = 0; kx < k; ++kx) {
                            int ix = ox * sx + kx * dil - pad;
                            if (ix < 0 || ix >= W) continue;
                            acc[j] = fmaf(xp[(int64_t)iy * W + ix], w[(((int64_t)f * cpg + ic) * k + ky) * k + kx], acc[j]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < FPT; ++j)
            if (f0 + j < F) y[(((int64_t)b * F + f0 + j) * OH + oy) * OW + ox] = acc[j];
    }
}

// bias_add / activation / bias_activation: channel = (i / channel_stride) % channels (lightnet-kernels-shared/src/lib.rs:10-40)
__global__ void bias_act_f32_kernel(const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y, int64_t n,
                                    int64_t channels, int64_t channel_stride, int act) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (bias) v += bias[(i / channel_stride) % channels];
        y[i] = ln_act_f32(act, v);
    }
}

__global__ void channel_scale_f32_kernel(const float* __restrict__ x, const float* __restrict__ scale, float* __restrict__ y, int64_t n, int64_t channels,
                                         int64_t channel_stride) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = __fmul_rn(x[i], scale[(i / channel_stride) % channels]);
}

// [region] forward (lightnet-cuda/src/host_ops.rs:73-116): channel-major NCHW entries -> spatial-major [batch, spatial, anchor, entry],
// logistic objectness (entry 4), optional softmax over the class entries.  One thread per (batch, cell, anchor).
__global__ void region_forward_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t batch, int spatial, int anchors, int entries, int classes,
                                          int softmax_classes) {
    const int64_t total = batch * spatial * anchors;
    const int64_t channels = (int64_t)anchors * entries;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int a = (int)(i % anchors);
        const int64_t s = (i / anchors) % spatial, b = i / ((int64_t)anchors * spatial);
        float* out = y + (b * spatial + s) * channels + (int64_t)a * entries;
        const float* in = x + (b * channels + (int64_t)a * entries) * spatial + s;
        for (int e = 0; e < entries; ++e) out[e] = in[(int64_t)e * spatial];
        out[4] = 1.0f / (1.0f + expf(-out[4]));
        if (softmax_classes) {
            float mx = -INFINITY;
            for (int c = 0; c < classes; ++c) mx = fmaxf(mx, out[5 + c]);
            float sum = 0.0f;
            for (int c = 0; c < classes; ++c) {
                const float v = expf(out[5 + c] - mx);
                out[5 + c] = v;
                sum += v;
            }
            if (sum > 0.0f)
                for (int c = 0; c < classes; ++c) out[5 + c] = out[5 + c] / sum;
        }
    }
}

// modern_yolo_forward_f32 (lightnet-cuda/src/lib.rs:4884-4915): every entry sanitised, the trailing 1 + classes planes through a
// sigmoid of the logit clamped to [-30, 30].
__global__ void modern_activate_f32_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, long long spatial, int channels, int class_begin) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)((i / spatial) % channels);
        float v = ln_finite_or_zero(x[i]);
        if (c >= class_begin) v = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-fminf(fmaxf(v, -30.0f), 30.0f))));
        y[i] = v;
    }
}

// modern_yolo_predecode (lightnet-cuda-oxide/src/kernels/dense_loss.rs:788-812): one thread per cell; the softmax expectation of
// each side's bins (modern_yolo/cpu.rs:283-308), corners to a sanitised centre-size box (cpu.rs:340-387), then the objectness
// and class planes copied behind it.
__global__ void modern_predecode_f32_kernel(const float* __restrict__ x, float* __restrict__ y, long long cells, int w, int h, int classes, int coords) {
    const long long s = (long long)w * h;
    const int bins = coords / 4 > 2 ? coords / 4 : 2, cin = coords + 1 + classes, cout = 5 + classes;
    for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < cells; g += (long long)gridDim.x * blockDim.x) {
        const long long b = g / s, loc = g - b * s;
        const float* px = x + b * cin * s + loc;
        float side[4];
        for (int sd = 0; sd < 4; ++sd) {
            float mx = -INFINITY;
            for (int k = 0; k < bins; ++k) mx = fmaxf(mx, ln_finite_or_zero(px[(long long)(sd * bins + k) * s]));
            float denom = 0.0f, expected = 0.0f;
            for (int k = 0; k < bins; ++k) {
                const float e = expf(fminf(fmaxf(__fsub_rn(ln_finite_or_zero(px[(long long)(sd * bins + k) * s]), mx), -60.0f), 60.0f));
                denom = __fadd_rn(denom, e);
                expected = __fadd_rn(expected, __fmul_rn((float)k, e));
            }
            side[sd] = __fdiv_rn(expected, fmaxf(denom, 1e-8f));
        }
        const int row = (int)(loc / w), col = (int)(loc - (long long)row * w);
        const float cx = (float)col + 0.5f, cy = (float)row + 0.5f;
        float left = ln_finite_or_zero(__fdiv_rn(__fsub_rn(cx, side[0]), (float)w)), top = ln_finite_or_zero(__fdiv_rn(__fsub_rn(cy, side[1]), (float)h));
        float right = ln_finite_or_zero(__fdiv_rn(__fadd_rn(cx, side[2]), (float)w)), bottom = ln_finite_or_zero(__fdiv_rn(__fadd_rn(cy, side[3]), (float)h));
        if (right < left) { const float t = left; left = right; right = t; }
        if (bottom < top) { const float t = top; top = bottom; bottom = t; }
        float* py = y + b * cout * s + loc;
        py[0] = ln_finite_or_zero(__fmul_rn(0.5f, __fadd_rn(left, right)));
        py[s] = ln_finite_or_zero(__fmul_rn(0.5f, __fadd_rn(top, bottom)));
        py[2 * s] = fmaxf(ln_finite_or_zero(fmaxf(__fsub_rn(right, left), 1e-6f)), 1e-6f);
        py[3 * s] = fmaxf(ln_finite_or_zero(fmaxf(__fsub_rn(bottom, top), 1e-6f)), 1e-6f);
        for (int e = 0; e < classes + 1; ++e) py[(long long)(4 + e) * s] = px[(long long)(coords + e) * s];
    }
}

// Classic [yolo] head activation on anchor-major NCHW entries (lightnet-cuda/src/lib.rs:4951-4966): logistic on every entry but w / h
// (none when new_coords), then x, y scaled: v * scale_xy - 0.5 * (scale_xy - 1).
__global__ void yolo_activate_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n, int64_t plane, int entries, float scale_xy,
                                         int new_coords) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int entry = (int)((i / plane) % entries);
        float v = x[i];
        if (!new_coords && entry != 2 && entry != 3) v = 1.0f / (1.0f + expf(-v));
        if (entry < 2) v = __fsub_rn(__fmul_rn(v, scale_xy), __fmul_rn(0.5f, __fsub_rn(scale_xy, 1.0f)));
        y[i] = v;
    }
}

__global__ void add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = a[i] + b[i];
}

// shortcut_fit: flat per-sample crop / zero-pad (lightnet-cuda/src/lib.rs:4036-4056)
__global__ void shortcut_fit_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t batch, int64_t in_len,
                                        int64_t out_len) {
    int64_t n = batch * out_len;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t b = i / out_len, j = i % out_len;
        y[i] = j < in_len ? x[b * in_len + j] : 0.0f;
    }
}

// route copy of one source's channel slice (runtime/layer_ops.rs:1850-1883)
__global__ void route_copy_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t batch, int64_t src_total_c,
                                      int64_t src_c0, int64_t chunk_c, int64_t dst_total_c, int64_t dst_c0, int64_t plane) {
    int64_t n = batch * chunk_c * plane;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t p = i % plane, c = (i / plane) % chunk_c, b = i / (plane * chunk_c);
        y[(b * dst_total_c + dst_c0 + c) * plane + p] = x[(b * src_total_c + src_c0 + c) * plane + p];
    }
}

// Darknet max-pool: window origin o*stride - padding/2, taps outside skipped, start at -inf
// (runtime/layer_ops.rs:1740-1799; lightnet-kernels-shared/src/lib.rs:95-140)
__global__ void maxpool_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t BC, int H, int W, int OH, int OW,
                                   int size, int sx, int sy, int padding) {
    int64_t n = BC * OH * OW;
    const int off = padding / 2;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int ox = (int)(i % OW), oy = (int)((i / OW) % OH);
        int64_t bc = i / ((int64_t)OW * OH);
        const float* xp = x + bc * H * W;
        float m = -INFINITY;
        for (int ky = 0; ky < size; ++ky) {
            int iy = oy * sy + ky - off;
            if (iy < 0 || iy >= H) continue;
            for (int kx = 0; kx < size; ++kx) {
                int ix = ox * sx + kx - off;
                if (ix < 0 || ix >= W) continue;
                m = fmaxf(m, xp[(int64_t)iy * W + ix]);
            }
        }
        y[i] = m;
    }
}

// nearest up-sample: out[y,x] = scale * in[y/s, x/s] (runtime/layer_ops.rs:2208-2256)
__global__ void upsample_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t BC, int H, int W, int s, float scale) {
    const int OH = H * s, OW = W * s;
    int64_t n = BC * OH * OW;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int ox = (int)(i % OW), oy = (int)((i / OW) % OH);
        int64_t bc = i / ((int64_t)OW * OH);
        y[i] = scale * x[(bc * H + oy / s) * W + ox / s];
    }
}

// reverse up-sample: out[y/s, x/s] += scale * in[y, x]; gather form (each output sums its s*s block in the
// row-major order the reference visits them)
__global__ void upsample_reverse_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t BC, int H, int W, int s,
                                            float scale) {
    const int OH = H / s, OW = W / s;
    int64_t n = BC * OH * OW;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int ox = (int)(i % OW), oy = (int)((i / OW) % OH);
        int64_t bc = i / ((int64_t)OW * OH);
        float acc = 0.0f;
        for (int dy = 0; dy < s; ++dy)
            for (int dx = 0; dx < s; ++dx) acc += scale * x[(bc * H + oy * s + dy) * W + ox * s + dx];
        y[i] = acc;
    }
}

__global__ void bn_fold_kernel(const float* gamma, const float* mean, const float* var, const float* bias, float eps, float* scale,
                               float* bias_out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    // single IEEE operations in the order of weights_io.rs:32-92 (no fused multiply-add), so the result has the host fold's bits
    float s = __fdiv_rn(gamma[i], __fsqrt_rn(__fadd_rn(var[i], eps)));
    scale[i] = s;
    bias_out[i] = __fsub_rn(bias[i], __fmul_rn(mean[i], s));
}

int grid_for(ln_ctx* ctx, int64_t n) {
    int64_t b = (n + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)ctx->sm_count * 32;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

bool is_f32(const ln_tensor* t) { return t && t->dtype == LN_F32; }

}  // namespace

extern "C" {

int32_t ln_conv2d_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* weights, const int64_t output_shape[4],
                      int64_t input_channels, int64_t input_height, int64_t input_width, int64_t filters, int64_t kernel_size,
                      int64_t stride_x, int64_t stride_y, int64_t dilation, int64_t padding, int64_t groups, ln_tensor** out) {
    if (!ctx || !out || !output_shape) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_f32: NULL argument");
    if (!is_f32(x) || !is_f32(weights)) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_f32: f32 tensors required");
    if (groups < 1 || filters % groups || input_channels % groups || kernel_size < 1 || stride_x < 1 || stride_y < 1 || dilation < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_f32: invalid geometry (groups %lld filters %lld channels %lld)", (long long)groups,
                       (long long)filters, (long long)input_channels);
    if (x->c != input_channels || x->h != input_height || x->w != input_width)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_f32: input tensor is [%lld,%lld,%lld,%lld], geometry says C=%lld H=%lld W=%lld",
                       (long long)x->n, (long long)x->c, (long long)x->h, (long long)x->w, (long long)input_channels,
                       (long long)input_height, (long long)input_width);
    if (weights->count() != filters * (input_channels / groups) * kernel_size * kernel_size)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_f32: weight tensor has %lld elements, expected %lld", (long long)weights->count(),
                       (long long)(filters * (input_channels / groups) * kernel_size * kernel_size));
    // lightnet-model model.rs:6472 conv_dim (dilation does not enter the extent)
    int64_t oh = (input_height + 2 * padding - kernel_size < 0 ? 0 : input_height + 2 * padding - kernel_size) / stride_y + 1;
    int64_t ow = (input_width + 2 * padding - kernel_size < 0 ? 0 : input_width + 2 * padding - kernel_size) / stride_x + 1;
    if (output_shape[0] != x->n || output_shape[1] != filters || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_f32: output_shape [%lld,%lld,%lld,%lld] does not match [%lld,%lld,%lld,%lld]",
                       (long long)output_shape[0], (long long)output_shape[1], (long long)output_shape[2], (long long)output_shape[3],
                       (long long)x->n, (long long)filters, (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, filters, oh, ow);
    if (!y) return LN_ERR_CUDA;
    int64_t total = x->n * ((filters + 3) / 4) * oh * ow;
    conv2d_f32_kernel<4><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, (const float*)weights->ptr, (float*)y->ptr, (int)x->n, (int)input_channels, (int)input_height,
        (int)input_width, (int)filters, (int)kernel_size, (int)stride_x, (int)stride_y, (int)dilation, (int)padding, (int)groups,
        (int)oh, (int)ow);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "conv2d_f32 launch: %s", cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

static int32_t bias_act_impl(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* bias, int64_t channels, int64_t channel_stride,
                             int32_t activation, ln_tensor** out, const char* who) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "%s: NULL argument", who);
    if (!is_f32(x) || (bias && !is_f32(bias))) return ln_fail(ctx, LN_ERR_ARG, "%s: f32 tensors required", who);
    if (bias && (channels < 1 || channel_stride < 1 || bias->count() != channels))
        return ln_fail(ctx, LN_ERR_SHAPE, "%s: bias has %lld elements for %lld channels", who, (long long)bias->count(), (long long)channels);
    if (activation < LN_ACT_LINEAR || activation > LN_ACT_RELU) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "%s: activation %d is not on the detector path", who, activation);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, x->c, x->h, x->w);
    if (!y) return LN_ERR_CUDA;
    bias_act_f32_kernel<<<grid_for(ctx, x->count()), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, bias ? (const float*)bias->ptr : nullptr, (float*)y->ptr, x->count(), channels > 0 ? channels : 1,
        channel_stride > 0 ? channel_stride : 1, activation);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "%s launch: %s", who, cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

int32_t ln_bias_add_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* bias, int64_t channels, int64_t channel_stride, ln_tensor** out) {
    if (!bias) return ln_fail(ctx, LN_ERR_ARG, "ln_bias_add_f32: bias is NULL");
    return bias_act_impl(ctx, x, bias, channels, channel_stride, LN_ACT_LINEAR, out, "ln_bias_add_f32");
}
int32_t ln_activation_f32(ln_ctx* ctx, const ln_tensor* x, int32_t activation, ln_tensor** out) {
    return bias_act_impl(ctx, x, nullptr, 1, 1, activation, out, "ln_activation_f32");
}
int32_t ln_bias_activation_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* bias, int64_t channels, int64_t channel_stride,
                               int32_t activation, ln_tensor** out) {
    if (!bias) return ln_fail(ctx, LN_ERR_ARG, "ln_bias_activation_f32: bias is NULL");
    return bias_act_impl(ctx, x, bias, channels, channel_stride, activation, out, "ln_bias_activation_f32");
}

int32_t ln_channel_scale_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* scale, int64_t channels, int64_t channel_stride, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_channel_scale_f32: NULL argument");
    if (!is_f32(x) || !is_f32(scale)) return ln_fail(ctx, LN_ERR_ARG, "ln_channel_scale_f32: f32 tensors required");
    if (channels < 1 || channel_stride < 1 || scale->count() != channels)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_channel_scale_f32: scale has %lld elements for %lld channels", (long long)scale->count(), (long long)channels);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, x->c, x->h, x->w);
    if (!y) return LN_ERR_CUDA;
    channel_scale_f32_kernel<<<grid_for(ctx, x->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (const float*)scale->ptr, (float*)y->ptr, x->count(), channels, channel_stride);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "channel_scale launch: %s", cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

int32_t ln_region_forward_f32(ln_ctx* ctx, const ln_tensor* x, int64_t anchors, int64_t entries, int64_t classes, int32_t softmax_classes, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_region_forward_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_region_forward_f32: f32 tensor required");
    if (anchors < 1 || classes < 0 || entries < classes + 5 || x->c != anchors * entries)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_region_forward_f32: %lld channels do not hold %lld anchors of %lld entries (>= classes + 5)", (long long)x->c, (long long)anchors, (long long)entries);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, x->c, x->h, x->w);  // same element count; the layout is [batch, spatial, anchor, entry]
    if (!y) return LN_ERR_CUDA;
    region_forward_f32_kernel<<<grid_for(ctx, x->n * x->h * x->w * anchors), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)y->ptr, x->n, (int)(x->h * x->w), (int)anchors,
                                                                                                         (int)entries, (int)classes, softmax_classes);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "region_forward launch: %s", cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

int32_t ln_yolo_activate_f32(ln_ctx* ctx, const ln_tensor* x, int64_t classes, float scale_xy, int32_t new_coords, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_yolo_activate_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_yolo_activate_f32: f32 tensor required");
    if (classes < 0 || x->c % (classes + 5)) return ln_fail(ctx, LN_ERR_SHAPE, "YOLO head tensor length mismatch: %lld channels are not a multiple of %lld entries", (long long)x->c, (long long)(classes + 5));
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, x->c, x->h, x->w);
    if (!y) return LN_ERR_CUDA;
    yolo_activate_f32_kernel<<<grid_for(ctx, x->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)y->ptr, x->count(), x->h * x->w, (int)(classes + 5), scale_xy, new_coords);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "yolo_activate launch: %s", cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

int32_t ln_modern_yolo_forward_f32(ln_ctx* ctx, const ln_tensor* x, int64_t classes, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_modern_yolo_forward_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_modern_yolo_forward_f32: f32 tensor required");
    if (classes < 0) return ln_fail(ctx, LN_ERR_ARG, "ln_modern_yolo_forward_f32: negative class count");
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, x->c, x->h, x->w);
    if (!y) return LN_ERR_CUDA;
    const long long class_begin = x->c - (classes + 1) > 0 ? x->c - (classes + 1) : 0;  // saturating_sub, lib.rs:4898
    modern_activate_f32_kernel<<<grid_for(ctx, x->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)y->ptr, x->count(), x->h * x->w, (int)x->c, (int)class_begin);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "modern_yolo_forward launch: %s", cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

int32_t ln_modern_yolo_predecode_f32(ln_ctx* ctx, const ln_tensor* x, int64_t classes, int64_t coords, int32_t kind, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_modern_yolo_predecode_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_modern_yolo_predecode_f32: f32 tensor required");
    if (kind != 1 && kind != 2) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_modern_yolo_predecode_f32: kind %d is not a distribution head (1 = ppyoloe, 2 = yolonas)", kind);
    if (classes < 1 || coords < 8 || coords % 4) return ln_fail(ctx, LN_ERR_ARG, "ln_modern_yolo_predecode_f32: %lld classes, %lld box entries", (long long)classes, (long long)coords);
    if (x->c != coords + 1 + classes) return ln_fail(ctx, LN_ERR_SHAPE, "distribution head tensor length mismatch: %lld channels, expected %lld", (long long)x->c, (long long)(coords + 1 + classes));
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, LN_F32, x->n, 5 + classes, x->h, x->w);
    if (!y) return LN_ERR_CUDA;
    const long long cells = x->n * x->h * x->w;
    modern_predecode_f32_kernel<<<grid_for(ctx, cells), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)y->ptr, cells, (int)x->w, (int)x->h, (int)classes, (int)coords);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(y); return ln_fail(ctx, LN_ERR_CUDA, "modern_yolo_predecode launch: %s", cudaGetErrorString(e)); }
    *out = y;
    return LN_OK;
}

int32_t ln_shortcut_add_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* y, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_f32: NULL argument");
    if (!is_f32(x) || !is_f32(y)) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_f32: f32 tensors required");
    if (x->count() != y->count()) return ln_fail(ctx, LN_ERR_SHAPE, "ln_shortcut_add_f32: %lld vs %lld elements", (long long)x->count(), (long long)y->count());
    cudaSetDevice(ctx->device);
    ln_tensor* o = ln_tensor_new(ctx, LN_F32, x->n, x->c, x->h, x->w);
    if (!o) return LN_ERR_CUDA;
    add_f32_kernel<<<grid_for(ctx, x->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (const float*)y->ptr, (float*)o->ptr, x->count());
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(o); return ln_fail(ctx, LN_ERR_CUDA, "shortcut_add launch: %s", cudaGetErrorString(e)); }
    *out = o;
    return LN_OK;
}

int32_t ln_shortcut_fit_f32(ln_ctx* ctx, const ln_tensor* x, int64_t batch, const int64_t output_shape[4], ln_tensor** out) {
    if (!ctx || !out || !output_shape) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_fit_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_fit_f32: f32 tensor required");
    if (batch < 1 || x->count() % batch || output_shape[0] != batch) return ln_fail(ctx, LN_ERR_SHAPE, "ln_shortcut_fit_f32: batch %lld does not divide the tensors", (long long)batch);
    cudaSetDevice(ctx->device);
    ln_tensor* o = ln_tensor_new(ctx, LN_F32, output_shape[0], output_shape[1], output_shape[2], output_shape[3]);
    if (!o) return LN_ERR_CUDA;
    shortcut_fit_f32_kernel<<<grid_for(ctx, o->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)o->ptr, batch,
                                                                                    x->count() / batch, o->count() / batch);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(o); return ln_fail(ctx, LN_ERR_CUDA, "shortcut_fit launch: %s", cudaGetErrorString(e)); }
    *out = o;
    return LN_OK;
}

int32_t ln_route_concat_f32(ln_ctx* ctx, const ln_tensor* const* inputs, int32_t n_inputs, const int64_t* input_channel_offsets,
                            const int64_t* input_channels, const int64_t* input_total_channels, const int64_t output_shape[4],
                            int64_t channel_stride, ln_tensor** out) {
    if (!ctx || !out || !inputs || !input_channel_offsets || !input_channels || !input_total_channels || !output_shape || n_inputs < 1)
        return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_f32: NULL argument");
    int64_t sum = 0;
    for (int i = 0; i < n_inputs; ++i) {
        if (!is_f32(inputs[i])) return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_f32: input %d is not f32", i);
        if (inputs[i]->c != input_total_channels[i] || input_channel_offsets[i] + input_channels[i] > input_total_channels[i] ||
            inputs[i]->h * inputs[i]->w != channel_stride || inputs[i]->n != output_shape[0])
            return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_f32: input %d does not match its channel slice / plane size", i);
        sum += input_channels[i];
    }
    if (sum != output_shape[1] || output_shape[2] * output_shape[3] != channel_stride)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_f32: slices sum to %lld channels, output has %lld", (long long)sum, (long long)output_shape[1]);
    cudaSetDevice(ctx->device);
    ln_tensor* o = ln_tensor_new(ctx, LN_F32, output_shape[0], output_shape[1], output_shape[2], output_shape[3]);
    if (!o) return LN_ERR_CUDA;
    int64_t c0 = 0;
    for (int i = 0; i < n_inputs; ++i) {
        int64_t n = o->n * input_channels[i] * channel_stride;
        route_copy_f32_kernel<<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>((const float*)inputs[i]->ptr, (float*)o->ptr, o->n,
                                                                             input_total_channels[i], input_channel_offsets[i],
                                                                             input_channels[i], o->c, c0, channel_stride);
        ctx->launches++;
        c0 += input_channels[i];
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(o); return ln_fail(ctx, LN_ERR_CUDA, "route_concat launch: %s", cudaGetErrorString(e)); }
    *out = o;
    return LN_OK;
}

int32_t ln_maxpool_f32(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height,
                       int64_t input_width, int64_t size, int64_t stride_x, int64_t stride_y, int64_t padding, ln_tensor** out) {
    if (!ctx || !out || !output_shape) return ln_fail(ctx, LN_ERR_ARG, "ln_maxpool_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_maxpool_f32: f32 tensor required");
    if (x->c != channels || x->h != input_height || x->w != input_width || size < 1 || stride_x < 1 || stride_y < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_maxpool_f32: geometry does not match the input tensor");
    // lightnet-model model.rs:8854 pool_dim
    int64_t oh = (input_height + padding - size < 0 ? 0 : input_height + padding - size) / stride_y + 1;
    int64_t ow = (input_width + padding - size < 0 ? 0 : input_width + padding - size) / stride_x + 1;
    if (output_shape[0] != x->n || output_shape[1] != channels || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_maxpool_f32: output_shape does not match pool_dim (%lld x %lld)", (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    ln_tensor* o = ln_tensor_new(ctx, LN_F32, x->n, channels, oh, ow);
    if (!o) return LN_ERR_CUDA;
    maxpool_f32_kernel<<<grid_for(ctx, o->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)o->ptr, x->n * channels,
                                                                                (int)input_height, (int)input_width, (int)oh, (int)ow,
                                                                                (int)size, (int)stride_x, (int)stride_y, (int)padding);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(o); return ln_fail(ctx, LN_ERR_CUDA, "maxpool launch: %s", cudaGetErrorString(e)); }
    *out = o;
    return LN_OK;
}

int32_t ln_upsample_f32(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height,
                        int64_t input_width, int64_t stride, float scale, int32_t reverse, ln_tensor** out) {
    if (!ctx || !out || !output_shape) return ln_fail(ctx, LN_ERR_ARG, "ln_upsample_f32: NULL argument");
    if (!is_f32(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_upsample_f32: f32 tensor required");
    if (stride < 1) return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_f32: upsample stride cannot be zero");
    if (x->c != channels || x->h != input_height || x->w != input_width)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_f32: geometry does not match the input tensor");
    int64_t oh = reverse ? input_height / stride : input_height * stride;
    int64_t ow = reverse ? input_width / stride : input_width * stride;
    if (output_shape[0] != x->n || output_shape[1] != channels || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_f32: output_shape does not match (%lld x %lld)", (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    ln_tensor* o = ln_tensor_new(ctx, LN_F32, x->n, channels, oh, ow);
    if (!o) return LN_ERR_CUDA;
    if (reverse)
        upsample_reverse_f32_kernel<<<grid_for(ctx, o->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)o->ptr,
                                                                                             x->n * channels, (int)input_height,
                                                                                             (int)input_width, (int)stride, scale);
    else
        upsample_f32_kernel<<<grid_for(ctx, o->count()), kThreads, 0, ctx->stream>>>((const float*)x->ptr, (float*)o->ptr, x->n * channels,
                                                                                     (int)input_height, (int)input_width, (int)stride, scale);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(o); return ln_fail(ctx, LN_ERR_CUDA, "upsample launch: %s", cudaGetErrorString(e)); }
    *out = o;
    return LN_OK;
}

int32_t ln_batchnorm_fold_f32(ln_ctx* ctx, const ln_tensor* gamma, const ln_tensor* mean, const ln_tensor* variance,
                              const ln_tensor* bias, float eps, ln_tensor** scale_out, ln_tensor** bias_out) {
    if (!ctx || !scale_out || !bias_out) return ln_fail(ctx, LN_ERR_ARG, "ln_batchnorm_fold_f32: NULL argument");
    if (!is_f32(gamma) || !is_f32(mean) || !is_f32(variance) || !is_f32(bias)) return ln_fail(ctx, LN_ERR_ARG, "ln_batchnorm_fold_f32: f32 tensors required");
    int64_t n = gamma->count();
    if (mean->count() != n || variance->count() != n || bias->count() != n) return ln_fail(ctx, LN_ERR_SHAPE, "ln_batchnorm_fold_f32: parameter length mismatch for %lld filters", (long long)n);
    cudaSetDevice(ctx->device);
    ln_tensor* s = ln_tensor_new(ctx, LN_F32, 1, n, 1, 1);
    ln_tensor* b = ln_tensor_new(ctx, LN_F32, 1, n, 1, 1);
    if (!s || !b) { ln_tensor_release(s); ln_tensor_release(b); return LN_ERR_CUDA; }
    bn_fold_kernel<<<blocks_for(n), kThreads, 0, ctx->stream>>>((const float*)gamma->ptr, (const float*)mean->ptr, (const float*)variance->ptr,
                                                                (const float*)bias->ptr, eps, (float*)s->ptr, (float*)b->ptr, (int)n);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(s); ln_tensor_release(b); return ln_fail(ctx, LN_ERR_CUDA, "bn_fold launch: %s", cudaGetErrorString(e)); }
    *scale_out = s;
    *bias_out = b;
    return LN_OK;
}

}  // extern "C"
