// Image pre-processing on the device: the step in front of the network.
//
// Reference (lightnet-runtime/src/image.rs): PlanarRgbImage::from_interleaved_rgb_u8 (:57) turns interleaved 8-bit RGB into
// planar f32 (byte / 255); resize (:95) is Darknet's float bilinear resize (align-corners, horizontal pass then vertical);
// resize_linear_exact (:157) is OpenCV's INTER_LINEAR_EXACT in fixed point on the bytes; letterbox (:203) resizes to fit
// and pads with 0.5 at integer offsets.  Here a batch of 8-bit images of different sizes goes to one f32 NCHW tensor of the
// network's size in a single kernel; every output value is computed with the reference's operations in the reference's
// order (single IEEE-754 operations, no contraction), so the result is bit-identical to the CPU path.
#include "ln_common.h"

namespace {

struct ImageMeta {
    long long offset;  // of the image's first byte in the staged pixel buffer
    int sw, sh;        // source size
    int nw, nh;        // size after the resize (letterbox: fitted inside the destination)
    int xo, yo;        // where the resized image sits in the destination
};

// byte / 255.0f for every byte value, filled once per block (an IEEE division per source tap would dominate the kernel)
__device__ __forceinline__ void fill_unit_table(float* table) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) table[i] = __fdiv_rn((float)i, 255.0f);
    __syncthreads();
}

__device__ __forceinline__ float src_value(const float* table, const uint8_t* img, int sw, int y, int x, int c) {
    return table[img[((size_t)y * sw + x) * 3 + c]];
}

// image.rs:108-127: one value of the horizontally resized plane
__device__ __forceinline__ float horizontal(const float* table, const uint8_t* img, int sw, int nw, float w_scale, int y, int col, int c) {
    if (col == nw - 1 || sw == 1) return src_value(table, img, sw, y, sw - 1, c);
    const float sx = __fmul_rn((float)col, w_scale);
    const int ix = (int)sx;  // NaN -> 0, like the reference's saturating cast
    const float dx = __fsub_rn(sx, (float)ix);
    // the indices are clamped for memory safety only: for every size the reference accepts they are in range already
    const int i0 = min(max(ix, 0), sw - 1), i1 = min(i0 + 1, sw - 1);
    return __fadd_rn(__fmul_rn(__fsub_rn(1.0f, dx), src_value(table, img, sw, y, i0, c)), __fmul_rn(dx, src_value(table, img, sw, y, i1, c)));
}

constexpr int kPixelsPerThread = 8;  // destination pixels per thread (amortises the table fill and the per-image scales)

// Darknet float resize (modes letterbox and resize): a thread takes kPixelsPerThread destination pixels, three channels each.
__global__ void __launch_bounds__(256) image_float_resize_kernel(const uint8_t* __restrict__ pixels, const ImageMeta* __restrict__ meta, int W, int H,
                                                                 float* __restrict__ out) {
    __shared__ float table[256];
    fill_unit_table(table);
    const int n = blockIdx.y;
    const ImageMeta m = meta[n];
    const uint8_t* img = pixels + m.offset;
    const float w_scale = __fdiv_rn(__fsub_rn((float)m.sw, 1.0f), __fsub_rn((float)m.nw, 1.0f));
    const float h_scale = __fdiv_rn(__fsub_rn((float)m.sh, 1.0f), __fsub_rn((float)m.nh, 1.0f));
    for (int k = 0; k < kPixelsPerThread; ++k) {
    const int p = (blockIdx.x * kPixelsPerThread + k) * blockDim.x + threadIdx.x;
    if (p >= W * H) return;
    const int y = p / W, x = p - y * W;
    float* o = out + (size_t)n * 3 * W * H + p;
    const int ry = y - m.yo, rx = x - m.xo;
    if (ry < 0 || ry >= m.nh || rx < 0 || rx >= m.nw) {
        o[0] = 0.5f; o[(size_t)W * H] = 0.5f; o[(size_t)2 * W * H] = 0.5f;  // letterbox padding (image.rs:216)
        continue;
    }
    if (m.sw == m.nw && m.sh == m.nh) {  // resize returns the source unchanged (image.rs:102-104)
        for (int c = 0; c < 3; ++c) o[(size_t)c * W * H] = src_value(table, img, m.sw, ry, rx, c);
        continue;
    }
    const float sy = m.sh == 1 ? 0.0f : __fmul_rn((float)ry, h_scale);
    const int iy = (int)sy;
    const float dy = __fsub_rn(sy, (float)iy);
    const bool last_row = ry == m.nh - 1 || m.sh == 1;
    const int y0 = min(max(iy, 0), m.sh - 1), y1 = min(y0 + 1, m.sh - 1);  // clamped for memory safety only
    for (int c = 0; c < 3; ++c) {
        float v = __fmul_rn(__fsub_rn(1.0f, dy), horizontal(table, img, m.sw, m.nw, w_scale, y0, rx, c));
        if (!last_row) v = __fadd_rn(v, __fmul_rn(dy, horizontal(table, img, m.sw, m.nw, w_scale, y1, rx, c)));
        o[(size_t)c * W * H] = v;
    }
    }
}

// image.rs:307-327 exact_coeffs for one destination index: taps (x0, x1) and weights (256 - c1, c1)
__device__ __forceinline__ void exact_tap(int d, int src, int dst, int* x0, int* x1, unsigned* c0, unsigned* c1) {
    const double fsx = __dsub_rn(__ddiv_rn(__dmul_rn(__dadd_rn((double)d, 0.5), (double)src), (double)dst), 0.5);
    double f0 = floor(fsx);
    double fx = __dsub_rn(fsx, f0);
    if (f0 < 0.0) { f0 = 0.0; fx = 0.0; }
    if (f0 >= (double)src - 1.0) { f0 = (double)src - 1.0; fx = 0.0; }
    *x0 = (int)f0;
    *x1 = min(*x0 + 1, src - 1);
    *c1 = (unsigned)floor(__dadd_rn(__dmul_rn(fx, 256.0), 0.5));
    *c0 = 256u - *c1;
}

// OpenCV INTER_LINEAR_EXACT on the bytes (image.rs:157-190), then byte / 255: one thread per destination pixel.
__global__ void __launch_bounds__(256) image_exact_resize_kernel(const uint8_t* __restrict__ pixels, const ImageMeta* __restrict__ meta, int W, int H,
                                                                 float* __restrict__ out) {
    __shared__ float table[256];
    fill_unit_table(table);
    const int n = blockIdx.y;
    const ImageMeta m = meta[n];
    const uint8_t* img = pixels + m.offset;
    for (int k = 0; k < kPixelsPerThread; ++k) {
    const int p = (blockIdx.x * kPixelsPerThread + k) * blockDim.x + threadIdx.x;
    if (p >= W * H) return;
    const int y = p / W, x = p - y * W;
    float* o = out + (size_t)n * 3 * W * H + p;
    if (m.sw == W && m.sh == H) {
        for (int c = 0; c < 3; ++c) o[(size_t)c * W * H] = src_value(table, img, m.sw, y, x, c);
        continue;
    }
    int x0, x1, y0, y1;
    unsigned cx0, cx1, cy0, cy1;
    exact_tap(x, m.sw, W, &x0, &x1, &cx0, &cx1);
    exact_tap(y, m.sh, H, &y0, &y1, &cy0, &cy1);
    for (int c = 0; c < 3; ++c) {
        const unsigned t0 = (unsigned)img[((size_t)y0 * m.sw + x0) * 3 + c] * cx0 + (unsigned)img[((size_t)y0 * m.sw + x1) * 3 + c] * cx1;
        const unsigned t1 = (unsigned)img[((size_t)y1 * m.sw + x0) * 3 + c] * cx0 + (unsigned)img[((size_t)y1 * m.sw + x1) * 3 + c] * cx1;
        const unsigned v = (t0 * cy0 + t1 * cy1 + 32768u) >> 16;
        o[(size_t)c * W * H] = table[v & 0xFFu];
    }
    }
}

// image.rs:329-341 fit_inside
void fit_inside(int sw, int sh, int dw, int dh, int* nw, int* nh) {
    if (((float)dw / (float)sw) < ((float)dh / (float)sh)) {
        *nw = dw > 1 ? dw : 1;
        const long long v = (long long)sh * dw / sw;
        *nh = v > 1 ? (int)v : 1;
    } else {
        const long long v = (long long)sw * dh / sh;
        *nw = v > 1 ? (int)v : 1;
        *nh = dh > 1 ? dh : 1;
    }
}

}  // namespace

// Enqueues upload + resize of `count` images on `stream` without synchronising.  The staging memory (metadata + pixels) comes
// from the ctx pool and is handed back through *staging / *staging_bytes: the caller frees it once the stream has passed this work.
int ln_image_preprocess_enqueue(ln_ctx* ctx, cudaStream_t stream, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths,
                                const int32_t* heights, int32_t count, int32_t mode, int32_t dst_w, int32_t dst_h, float* dst, void** staging,
                                size_t* staging_bytes) {
    *staging = nullptr;
    *staging_bytes = 0;
    if (mode < LN_PRE_LETTERBOX || mode > LN_PRE_RESIZE_EXACT) return ln_fail(ctx, LN_ERR_ARG, "image pre-processing: unknown mode %d", mode);
    if (dst_w < 1 || dst_h < 1) return ln_fail(ctx, LN_ERR_ARG, "resize dimensions must be non-zero");
    std::vector<ImageMeta> meta((size_t)count);
    int64_t first = -1, last = 0;  // byte range of the pixel buffer these images occupy
    for (int i = 0; i < count; ++i) {
        if (widths[i] < 1 || heights[i] < 1) return ln_fail(ctx, LN_ERR_ARG, "source image dimensions must be non-zero");
        if (offsets[i] < 0) return ln_fail(ctx, LN_ERR_ARG, "image pre-processing: negative offset for image %d", i);
        const int64_t end = offsets[i] + (int64_t)widths[i] * heights[i] * 3;
        if (first < 0 || offsets[i] < first) first = offsets[i];
        if (end > last) last = end;
    }
    for (int i = 0; i < count; ++i) {
        ImageMeta& m = meta[i];
        m.offset = offsets[i] - first; m.sw = widths[i]; m.sh = heights[i];
        if (mode == LN_PRE_LETTERBOX) {
            fit_inside(m.sw, m.sh, dst_w, dst_h, &m.nw, &m.nh);
            m.xo = (dst_w - m.nw) / 2; m.yo = (dst_h - m.nh) / 2;
        } else { m.nw = dst_w; m.nh = dst_h; m.xo = 0; m.yo = 0; }
    }
    const int64_t total = last - first;
    cudaSetDevice(ctx->device);
    const size_t meta_bytes = (size_t)ln_round_up((int64_t)(count * sizeof(ImageMeta)), 256);
    const size_t bytes = meta_bytes + (size_t)total;
    unsigned char* dev = (unsigned char*)ln_pool_alloc(ctx, bytes);
    if (!dev) return LN_ERR_CUDA;
    *staging = dev;
    *staging_bytes = bytes;
    // `meta` is pageable host memory: this copy is complete (staged by the driver) when the call returns
    cudaError_t e = cudaMemcpyAsync(dev, meta.data(), count * sizeof(ImageMeta), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dev + meta_bytes, pixels_host + first, (size_t)total, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) {
        const dim3 grid((unsigned)(((int64_t)dst_w * dst_h + 256 * kPixelsPerThread - 1) / (256 * kPixelsPerThread)), (unsigned)count);
        if (mode == LN_PRE_RESIZE_EXACT) image_exact_resize_kernel<<<grid, 256, 0, stream>>>(dev + meta_bytes, (const ImageMeta*)dev, dst_w, dst_h, dst);
        else image_float_resize_kernel<<<grid, 256, 0, stream>>>(dev + meta_bytes, (const ImageMeta*)dev, dst_w, dst_h, dst);
        ctx->launches++;
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "image pre-processing: %s", cudaGetErrorString(e));
    return LN_OK;
}

// Shared by the entry point below and by ln_net_detect_u8: fills `dst` (f32 [count, 3, dst_h, dst_w] on the device) and waits for it.
int ln_image_preprocess_into(ln_ctx* ctx, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths, const int32_t* heights,
                             int32_t count, int32_t mode, int32_t dst_w, int32_t dst_h, float* dst) {
    void* staging = nullptr;
    size_t staging_bytes = 0;
    int rc = ln_image_preprocess_enqueue(ctx, ctx->stream, pixels_host, offsets, widths, heights, count, mode, dst_w, dst_h, dst, &staging, &staging_bytes);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);  // the caller's pixels may go away after this
    if (staging) ln_pool_free(ctx, staging, staging_bytes);
    if (rc) return rc;
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "image pre-processing: %s", cudaGetErrorString(e));
    return LN_OK;
}

extern "C" int32_t ln_image_preprocess_u8(ln_ctx* ctx, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths,
                                          const int32_t* heights, int32_t count, int32_t mode, int32_t dst_w, int32_t dst_h, ln_tensor** out) {
    if (!ctx || !pixels_host || !offsets || !widths || !heights || !out || count < 1) return ln_fail(ctx, LN_ERR_ARG, "ln_image_preprocess_u8: NULL argument");
    ln_tensor* t = ln_tensor_new(ctx, LN_F32, count, 3, dst_h, dst_w);
    if (!t) return LN_ERR_CUDA;
    int rc = ln_image_preprocess_into(ctx, pixels_host, offsets, widths, heights, count, mode, dst_w, dst_h, (float*)t->ptr);
    if (rc) { ln_tensor_release(t); return rc; }
    *out = t;
    return LN_OK;
}
