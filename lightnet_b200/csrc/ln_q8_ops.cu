// 8-bit (int8 / FP8 E4M3) NHWC operators: quantise / dequantise / layout, weight packing, max-pool,
// up-sample, route, shortcut, and the CUDA-core convolutions (first layer with C <= 4, and a general
// fallback for geometries the tensor-core kernel does not take).  All of these are HBM-bound byte
// work: one thread moves 16 bytes of channels of one pixel, loads and stores are 16-byte vectors,
// grids are sized in multiples of the SM count.
#include <cuda_fp8.h>

#include "ln_conv_plan.h"

namespace {

constexpr int kThreads = 256;

int grid_for(ln_ctx* ctx, int64_t n) {
    int64_t b = (n + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)ctx->sm_count * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&hr));
}
__device__ __forceinline__ uint8_t float_to_e4m3(float v) { return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }

template <int KIND>
__device__ __forceinline__ float code_to_float(uint8_t c) {
    return KIND == LN_KIND_I8 ? (float)(int8_t)c : e4m3_to_float(c);
}
template <int KIND>
__device__ __forceinline__ uint8_t quantize_code(float a, float inv_s) {
    if (KIND == LN_KIND_I8) return (uint8_t)(ln_quant_i8(a, inv_s) & 0xFF);
    return float_to_e4m3(__fmul_rn(a, inv_s));
}

// f32 NCHW -> 8-bit NHWC (pad channels written as zero)
template <int KIND>
__global__ void quantize_nchw_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, int64_t N, int C, int H, int W, int64_t cstride,
                                     float inv_s) {
    const int64_t total = N * H * W * cstride;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i % cstride);
        int64_t pix = i / cstride;
        int64_t hw = pix % ((int64_t)H * W), n = pix / ((int64_t)H * W);
        y[i] = c < C ? quantize_code<KIND>(x[(n * C + c) * H * W + hw], inv_s) : 0;
    }
}

// 8-bit NHWC view -> f32 NCHW (value = code * scale)
template <int KIND>
__global__ void dequantize_nhwc_kernel(const uint8_t* __restrict__ x, float* __restrict__ y, int64_t N, int C, int H, int W, int64_t cstride,
                                       float scale) {
    const int64_t total = N * C * H * W;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t hw = i % ((int64_t)H * W);
        int c = (int)((i / ((int64_t)H * W)) % C);
        int64_t n = i / ((int64_t)H * W * C);
        y[i] = code_to_float<KIND>(x[(n * H * W + hw) * cstride + c]) * scale;
    }
}

// raw codes: NHWC view <-> NCHW dense
__global__ void codes_nhwc_to_nchw_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, int64_t N, int C, int H, int W, int64_t cstride) {
    const int64_t total = N * C * H * W;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t hw = i % ((int64_t)H * W);
        int c = (int)((i / ((int64_t)H * W)) % C);
        int64_t n = i / ((int64_t)H * W * C);
        y[i] = x[(n * H * W + hw) * cstride + c];
    }
}
__global__ void codes_nchw_to_nhwc_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, int64_t N, int C, int H, int W, int64_t cstride) {
    const int64_t total = N * H * W * cstride;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i % cstride);
        int64_t pix = i / cstride;
        int64_t hw = pix % ((int64_t)H * W), n = pix / ((int64_t)H * W);
        y[i] = c < C ? x[(n * C + c) * H * W + hw] : 0;
    }
}

// Weight packing: one block per (padded) filter.  s = max|w| / qmax, code = quantise(w / s);
// layout [fpad][k][k][cpad] plus the reference's [F][C][k][k] order for the CUDA-core kernels.
template <int KIND>
__global__ void pack_weights_kernel(const float* __restrict__ w, int F, int C, int k, int cpad, uint8_t* __restrict__ packed,
                                    uint8_t* __restrict__ oihw, float* __restrict__ wscale) {
    const int f = blockIdx.x;
    const int per = C * k * k;
    __shared__ float red[32];
    __shared__ float s_scale;
    float m = 0.0f;
    if (f < F)
        for (int i = threadIdx.x; i < per; i += blockDim.x) m = fmaxf(m, fabsf(w[(int64_t)f * per + i]));
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) mm = fmaxf(mm, red[i]);
        const float qmax = KIND == LN_KIND_I8 ? 127.0f : 448.0f;
        float s = (mm > 0.0f && isfinite(mm)) ? __fdiv_rn(mm, qmax) : 1.0f;
        s_scale = s;
        wscale[f] = f < F ? s : 0.0f;
    }
    __syncthreads();
    const float s = s_scale;
    const int row = k * k * cpad;
    int l1 = 0;
    for (int i = threadIdx.x; i < row; i += blockDim.x) {
        int c = i % cpad, tap = i / cpad;
        uint8_t code = 0;
        if (f < F && c < C) {
            float v = __fdiv_rn(w[((int64_t)f * C + c) * k * k + tap], s);
            code = KIND == LN_KIND_I8 ? (uint8_t)(ln_quant_i8(v, 1.0f) & 0xFF) : float_to_e4m3(v);
            oihw[((int64_t)f * C + c) * k * k + tap] = code;
            l1 += abs((int)(int8_t)code);
        }
        packed[(int64_t)f * row + i] = code;
    }
    // sum of |code| of the filter: 127 * this bounds the magnitude of any int8 accumulator
    for (int o = 16; o > 0; o >>= 1) l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = (float)l1;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
        wscale[gridDim.x + f] = t;
    }
}

// ---- glue ------------------------------------------------------------------------------------

// order-preserving key of an E4M3 byte under signed byte comparison (an involution)
__device__ __forceinline__ uint32_t f8_key4(uint32_t v) {
    uint32_t neg = (v >> 7) & 0x01010101u;  // 1 in each negative byte
    return v ^ (neg * 0x7Fu);
}

template <int KIND>
__device__ __forceinline__ uint4 max16(uint4 a, uint4 b) {
    if (KIND == LN_KIND_I8) return make_uint4(__vmaxs4(a.x, b.x), __vmaxs4(a.y, b.y), __vmaxs4(a.z, b.z), __vmaxs4(a.w, b.w));
    return make_uint4(f8_key4(__vmaxs4(f8_key4(a.x), f8_key4(b.x))), f8_key4(__vmaxs4(f8_key4(a.y), f8_key4(b.y))),
                      f8_key4(__vmaxs4(f8_key4(a.z), f8_key4(b.z))), f8_key4(__vmaxs4(f8_key4(a.w), f8_key4(b.w))));
}

// Max-pool, NHWC, one thread per (output pixel, 16 channels).  Window origin o*stride - padding/2, taps outside the
// image skipped (runtime/layer_ops.rs:1740-1799); a window with no tap inside gives the most negative code.
template <int KIND>
__global__ void maxpool_q_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N, int C16, int H,
                                 int W, int OH, int OW, int size, int sx, int sy, int padding) {
    const int64_t total = N * OH * OW * C16;
    const int off = padding / 2;
    const uint32_t lowest = KIND == LN_KIND_I8 ? 0x81818181u : 0xFEFEFEFEu;  // -127 / -448
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int cg = (int)(i % C16);
        int64_t pix = i / C16;
        int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        int64_t n = pix / ((int64_t)OW * OH);
        uint4 m = make_uint4(lowest, lowest, lowest, lowest);
        for (int ky = 0; ky < size; ++ky) {
            int iy = oy * sy + ky - off;
            if (iy < 0 || iy >= H) continue;
            for (int kx = 0; kx < size; ++kx) {
                int ix = ox * sx + kx - off;
                if (ix < 0 || ix >= W) continue;
                uint4 v = *reinterpret_cast<const uint4*>(x + ((n * H + iy) * W + ix) * xs + cg * 16);
                m = max16<KIND>(m, v);
            }
        }
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = m;
    }
}

// The SPP case: 5x5 window, stride 1, output the size of the input.  Every window meets the image, so taps outside are
// replaced by the nearest pixel inside (which the window holds already): no branches.  One thread walks down a column
// segment of one (image, x, 16 channels) keeping the horizontal 5-tap maxima of the last five rows: 5 loads per output
// instead of 25.
template <int KIND>
__global__ void __launch_bounds__(256) maxpool5_same_q_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N,
                                                             int C16, int H, int W, int off, int seg_rows) {
    const int64_t total = N * W * C16;
    const int oy0 = blockIdx.y * seg_rows, oy1 = min(oy0 + seg_rows, H);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C16);
        const int ox = (int)((i / C16) % W);
        const int64_t n = i / ((int64_t)C16 * W);
        const uint8_t* xn = x + n * H * W * xs + cg * 16;
        uint8_t* yn = y + n * H * W * ys + cg * 16;
        int64_t col[5];
#pragma unroll
        for (int k = 0; k < 5; ++k) col[k] = (int64_t)min(max(ox + k - off, 0), W - 1) * xs;
        auto row_max = [&](int iy) {
            const uint8_t* row = xn + (int64_t)min(max(iy, 0), H - 1) * W * xs;
            uint4 v[5];
#pragma unroll
            for (int k = 0; k < 5; ++k) v[k] = *reinterpret_cast<const uint4*>(row + col[k]);
            return max16<KIND>(max16<KIND>(max16<KIND>(v[0], v[1]), max16<KIND>(v[2], v[3])), v[4]);
        };
        uint4 r0 = row_max(oy0 - off), r1 = row_max(oy0 - off + 1), r2 = row_max(oy0 - off + 2), r3 = row_max(oy0 - off + 3);
        for (int oy = oy0; oy < oy1; ++oy) {
            const uint4 r4 = row_max(oy - off + 4);
            *reinterpret_cast<uint4*>(yn + ((int64_t)oy * W + ox) * ys) = max16<KIND>(max16<KIND>(max16<KIND>(r0, r1), max16<KIND>(r2, r3)), r4);
            r0 = r1; r1 = r2; r2 = r3; r3 = r4;
        }
    }
}

// The down-sampling case: 2x2 window, stride 2, window origin at (2 oy, 2 ox).  The first tap is always inside the image; a
// second tap beyond the last row / column (odd sizes) is replaced by the first: four independent loads, no branches.
template <int KIND>
__global__ void __launch_bounds__(256) maxpool2_s2_q_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N,
                                                           int C16, int H, int W, int OH, int OW) {
    const int64_t total = N * OH * OW * C16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C16);
        const int64_t pix = i / C16;
        const int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        const int64_t n = pix / ((int64_t)OW * OH);
        const int x0 = 2 * ox, x1 = min(x0 + 1, W - 1), y0 = 2 * oy, y1 = min(y0 + 1, H - 1);
        const uint8_t* xn = x + n * H * W * xs + cg * 16;
        const uint4 a = *reinterpret_cast<const uint4*>(xn + ((int64_t)y0 * W + x0) * xs), b = *reinterpret_cast<const uint4*>(xn + ((int64_t)y0 * W + x1) * xs);
        const uint4 c = *reinterpret_cast<const uint4*>(xn + ((int64_t)y1 * W + x0) * xs), d = *reinterpret_cast<const uint4*>(xn + ((int64_t)y1 * W + x1) * xs);
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = max16<KIND>(max16<KIND>(a, b), max16<KIND>(c, d));
    }
}

// nearest up-sample, NHWC (runtime/layer_ops.rs:2208-2256, scale folded into the tensor scale)
__global__ void upsample_q_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N, int C16, int H, int W,
                                  int s) {
    const int OH = H * s, OW = W * s;
    const int64_t total = N * OH * OW * C16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int cg = (int)(i % C16);
        int64_t pix = i / C16;
        int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        int64_t n = pix / ((int64_t)OW * OH);
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) =
            *reinterpret_cast<const uint4*>(x + ((n * H + oy / s) * W + ox / s) * xs + cg * 16);
    }
}

// Up-sample that requantises (runtime/layer_ops.rs:2208-2256 on codes): nearest with a scale, or reverse = scale times the sum of each
// stride x stride block ((dy, dx) order; the sum of int8 codes is exact), written as quantise(value * r), r = s_in * scale / s_out.
template <int KIND>
__global__ void upsample_requant_q_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t N, int C, int H, int W,
                                          int OH, int OW, int s, int reverse, float r) {
    const int64_t total = N * OH * OW * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int64_t pix = i / C;
        const int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        const int64_t n = pix / ((int64_t)OW * OH);
        float v;
        if (reverse) {
            int isum = 0;
            float fsum = 0.0f;
            for (int dy = 0; dy < s; ++dy)
                for (int dx = 0; dx < s; ++dx) {
                    const int iy = oy * s + dy, ix = ox * s + dx;
                    if (iy >= H || ix >= W) continue;
                    const uint8_t code = x[((n * H + iy) * W + ix) * xs + c];
                    if (KIND == LN_KIND_I8) isum += (int)(int8_t)code;
                    else fsum = __fadd_rn(fsum, e4m3_to_float(code));
                }
            v = KIND == LN_KIND_I8 ? __int2float_rn(isum) : fsum;
        } else v = code_to_float<KIND>(x[((n * H + oy / s) * W + ox / s) * xs + c]);
        y[pix * ys + c] = quantize_code<KIND>(v, r);
    }
}

// shortcut_fit on codes (lightnet-cuda/src/lib.rs:4041 / :6494): element i of a sample, in NCHW order, is element i of the source sample,
// zero beyond the source's length
__global__ void shortcut_fit_q_kernel(const uint8_t* __restrict__ x, int64_t xs, int sc, int sh, int sw, uint8_t* __restrict__ y, int64_t ys, int64_t N, int C,
                                      int H, int W) {
    const int64_t total = N * C * H * W, src_len = (int64_t)sc * sh * sw;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t flat = i % ((int64_t)C * H * W), n = i / ((int64_t)C * H * W);
        const int w = (int)(flat % W), h = (int)((flat / W) % H), c = (int)(flat / ((int64_t)W * H));
        uint8_t v = 0;
        if (flat < src_len) {
            const int sx = (int)(flat % sw), sy = (int)((flat / sw) % sh), scc = (int)(flat / ((int64_t)sw * sh));
            v = x[((n * sh + sy) * sw + sx) * xs + scc];
        }
        y[((n * H + h) * W + w) * ys + c] = v;
    }
}

// channel-slice copy between NHWC views (route); 16-byte and byte variants
__global__ void copy_q16_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t pixels, int C16) {
    const int64_t total = pixels * C16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int cg = (int)(i % C16);
        int64_t pix = i / C16;
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = *reinterpret_cast<const uint4*>(x + pix * xs + cg * 16);
    }
}
__global__ void copy_q1_kernel(const uint8_t* __restrict__ x, int64_t xs, uint8_t* __restrict__ y, int64_t ys, int64_t pixels, int C) {
    const int64_t total = pixels * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i % C);
        int64_t pix = i / C;
        y[pix * ys + c] = x[pix * xs + c];
    }
}

// shortcut: code = quantise(act(a*sa + b*sb) / sy); 16 channels (one 16-byte vector) per thread
template <int KIND, bool EXACT>
__global__ void shortcut_q_kernel(const uint8_t* __restrict__ a, int64_t as, float sa, const uint8_t* __restrict__ b, int64_t bs, float sb,
                                  uint8_t* __restrict__ y, int64_t ys, int64_t pixels, int C16, int act, float inv_sy) {
    const int64_t total = pixels * C16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C16);
        const int64_t pix = i / C16;
        const uint4 va = *reinterpret_cast<const uint4*>(a + pix * as + cg * 16);
        const uint4 vb = *reinterpret_cast<const uint4*>(b + pix * bs + cg * 16);
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t wo[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t out = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float v = __fmul_rn(code_to_float<KIND>((uint8_t)(wa[w] >> (8 * j))), sa);
                v = __fmaf_rn(code_to_float<KIND>((uint8_t)(wb[w] >> (8 * j))), sb, v);
                out |= (uint32_t)quantize_code<KIND>(ln_epilogue_act<EXACT>(act, v), inv_sy) << (8 * j);
            }
            wo[w] = out;
        }
        *reinterpret_cast<uint4*>(y + pix * ys + cg * 16) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
}

// ---- CUDA-core convolutions ------------------------------------------------------------------

// General fallback: one thread per (output pixel, filter); NHWC input, weights [fpad][k][k][cpad].
template <int KIND, bool EXACT>
__global__ void conv_simt_kernel(ln_conv_geom g, const float2* __restrict__ mb) {
    const int64_t total = (int64_t)g.N * g.OH * g.OW * g.F;
    const uint8_t* x = (const uint8_t*)g.x;
    const uint8_t* w = (const uint8_t*)g.w;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int f = (int)(i % g.F);
        int64_t pix = i / g.F;
        int ox = (int)(pix % g.OW), oy = (int)((pix / g.OW) % g.OH);
        int64_t n = pix / ((int64_t)g.OW * g.OH);
        int iacc = 0;
        float facc = 0.0f;
        // a group's channels: all of them (padded, where the pad bytes of both operands are zero) when there is one group
        const int w_cpad = g.w_cpad ? g.w_cpad : g.cpad;
        const int cpg = g.groups > 1 ? g.C / g.groups : g.cpad, cbase = g.groups > 1 ? (f / (g.F / g.groups)) * cpg : 0;
        const bool words = (cpg & 3) == 0 && (cbase & 3) == 0;
        for (int ky = 0; ky < g.k; ++ky) {
            int iy = oy * g.stride + ky - g.pad;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.k; ++kx) {
                int ix = ox * g.stride + kx - g.pad;
                if (ix < 0 || ix >= g.W) continue;
                const uint8_t* xp = x + ((n * g.H + iy) * g.W + ix) * g.x_pixel_stride + cbase;
                const uint8_t* wp = w + (((int64_t)f * g.k + ky) * g.k + kx) * w_cpad;
                if (words) {
                    for (int c = 0; c < cpg; c += 4) {
                        uint32_t xv = *reinterpret_cast<const uint32_t*>(xp + c), wv = *reinterpret_cast<const uint32_t*>(wp + c);
                        if (KIND == LN_KIND_I8) iacc = __dp4a((int)xv, (int)wv, iacc);
                        else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                facc = fmaf(e4m3_to_float((uint8_t)(xv >> (8 * j))), e4m3_to_float((uint8_t)(wv >> (8 * j))), facc);
                        }
                    }
                } else {
                    for (int c = 0; c < cpg; ++c) {
                        if (KIND == LN_KIND_I8) iacc += (int)(int8_t)xp[c] * (int)(int8_t)wp[c];
                        else facc = fmaf(e4m3_to_float(xp[c]), e4m3_to_float(wp[c]), facc);
                    }
                }
            }
        }
        if (g.out_kind == LN_OUT_ACC) {
            int32_t* o = (int32_t*)g.out;
            o[(((int64_t)n * g.F + f) * g.OH + oy) * g.OW + ox] = KIND == LN_KIND_I8 ? iacc : __float_as_int(facc);
            continue;
        }
        const float2 m = mb[f];
        float a = ln_epilogue_act<EXACT>(g.act, __fmaf_rn(KIND == LN_KIND_I8 ? __int2float_rn(iacc) : facc, m.x, m.y));
        if (g.out_kind == LN_OUT_F32) ((float*)g.out)[(((int64_t)n * g.F + f) * g.OH + oy) * g.OW + ox] = a;
        else ((uint8_t*)g.out)[pix * g.out_pixel_stride + f] = quantize_code<KIND>(a, g.inv_sy);
    }
}

// Depthwise convolution (groups = channels = filters; lightnet-cuda-oxide/src/kernels/conv_direct.rs:19 with one channel per
// group): HBM-bound byte work.  One thread per (output pixel, 16 channels): every tap is one 16-byte load of the input and one
// 16-byte load of the weights, which are staged in shared memory tap-major ([k*k][C]) once per block; the 16 outputs leave as
// one 16-byte store.
template <int KIND, bool EXACT>
__global__ void __launch_bounds__(256) conv_dw_q_kernel(ln_conv_geom g, const float2* __restrict__ mb) {
    extern __shared__ uint8_t s_dw[];  // [k*k][C16*16]
    const int kk = g.k * g.k, C16 = (g.C + 15) / 16, w_cpad = g.w_cpad ? g.w_cpad : g.cpad;
    const uint8_t* w = (const uint8_t*)g.w;
    for (int i = threadIdx.x; i < kk * C16 * 16; i += blockDim.x) {
        const int tap = i / (C16 * 16), c = i - tap * (C16 * 16);
        s_dw[i] = c < g.C ? w[((int64_t)c * kk + tap) * w_cpad] : 0;
    }
    __syncthreads();
    const uint8_t* x = (const uint8_t*)g.x;
    const int64_t total = (int64_t)g.N * g.OH * g.OW * C16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C16);
        const int64_t pix = i / C16;
        const int ox = (int)(pix % g.OW), oy = (int)((pix / g.OW) % g.OH);
        const int64_t n = pix / ((int64_t)g.OW * g.OH);
        int iacc[16];
        float facc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) { iacc[j] = 0; facc[j] = 0.0f; }
        for (int ky = 0; ky < g.k; ++ky) {
            const int iy = oy * g.stride + ky - g.pad;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.k; ++kx) {
                const int ix = ox * g.stride + kx - g.pad;
                if (ix < 0 || ix >= g.W) continue;
                const uint4 xv = *reinterpret_cast<const uint4*>(x + ((n * g.H + iy) * g.W + ix) * g.x_pixel_stride + cg * 16);
                const uint4 wv = *reinterpret_cast<const uint4*>(s_dw + (ky * g.k + kx) * C16 * 16 + cg * 16);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint8_t xb = (uint8_t)(xw[j >> 2] >> (8 * (j & 3))), wb = (uint8_t)(ww[j >> 2] >> (8 * (j & 3)));
                    if (KIND == LN_KIND_I8) iacc[j] += (int)(int8_t)xb * (int)(int8_t)wb;
                    else facc[j] = fmaf(e4m3_to_float(xb), e4m3_to_float(wb), facc[j]);
                }
            }
        }
        uint32_t packed[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int f = cg * 16 + j;
            if (f >= g.F) continue;
            if (g.out_kind == LN_OUT_ACC) {
                ((int32_t*)g.out)[(((int64_t)n * g.F + f) * g.OH + oy) * g.OW + ox] = KIND == LN_KIND_I8 ? iacc[j] : __float_as_int(facc[j]);
                continue;
            }
            const float2 m = mb[f];
            const float a = ln_epilogue_act<EXACT>(g.act, __fmaf_rn(KIND == LN_KIND_I8 ? __int2float_rn(iacc[j]) : facc[j], m.x, m.y));
            if (g.out_kind == LN_OUT_F32) ((float*)g.out)[(((int64_t)n * g.F + f) * g.OH + oy) * g.OW + ox] = a;
            else packed[j >> 2] |= (uint32_t)quantize_code<KIND>(a, g.inv_sy) << (8 * (j & 3));
        }
        if (g.out_kind == LN_OUT_Q) *reinterpret_cast<uint4*>((uint8_t*)g.out + pix * g.out_pixel_stride + cg * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// First layer (C <= 4): f32 NCHW image -> quantise -> k x k convolution -> epilogue -> 8-bit NHWC.
// One thread per (output pixel, group of 16 filters); the quantised patch is packed 4 codes per word
// (tap-major, channel-minor, zero padded) and each filter costs ceil(k*k*C/4) dp4a with its weights
// read from shared memory.
constexpr int kStemMaxWords = 13;  // k*k*C <= 52 (e.g. 3x3x3 = 27 -> 7 words; 7x7x1 = 49 -> 13 words)
template <int KIND, bool EXACT>
__global__ void conv_stem_kernel(const float* __restrict__ x, float inv_sx, int N, int C, int H, int W, const uint8_t* __restrict__ w_oihw,
                                 const float2* __restrict__ mb, int F, int k, int stride, int pad, int OH, int OW, int act, float inv_sy,
                                 uint8_t* __restrict__ out, int64_t out_pixel_stride) {
    extern __shared__ uint32_t s_w[];  // [F16*16][words]
    const int taps = k * k * C, words = (taps + 3) / 4;
    const int F16 = (F + 15) / 16;
    float2* s_mb = reinterpret_cast<float2*>(s_w + F16 * 16 * words);
    for (int i = threadIdx.x; i < F16 * 16 * words; i += blockDim.x) {
        int f = i / words, wd = i % words;
        uint32_t v = 0;
        for (int j = 0; j < 4; ++j) {
            int t = wd * 4 + j;  // t = (ky*k + kx)*C + c
            if (f < F && t < taps) {
                int c = t % C, tap = t / C;
                v |= (uint32_t)w_oihw[((int64_t)f * C + c) * k * k + tap] << (8 * j);
            }
        }
        s_w[i] = v;
    }
    for (int i = threadIdx.x; i < F16 * 16; i += blockDim.x) s_mb[i] = i < F ? mb[i] : make_float2(0.0f, 0.0f);
    __syncthreads();
    const int64_t total = (int64_t)N * OH * OW * F16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        // consecutive threads take consecutive pixels (coalesced NCHW reads); filter group is the slow index
        int64_t pix = i % ((int64_t)N * OH * OW);
        int fg = (int)(i / ((int64_t)N * OH * OW));
        int ox = (int)(pix % OW), oy = (int)((pix / OW) % OH);
        int64_t n = pix / ((int64_t)OW * OH);
        uint32_t patch[kStemMaxWords];
#pragma unroll
        for (int wd = 0; wd < kStemMaxWords; ++wd) patch[wd] = 0;
        for (int t = 0; t < taps; ++t) {
            int c = t % C, tap = t / C, ky = tap / k, kx = tap % k;
            int iy = oy * stride + ky - pad, ix = ox * stride + kx - pad;
            uint32_t code = 0;
            if (iy >= 0 && iy < H && ix >= 0 && ix < W) code = quantize_code<KIND>(x[((n * C + c) * H + iy) * W + ix], inv_sx);
            // static indexing keeps `patch` in registers
#pragma unroll
            for (int wd = 0; wd < kStemMaxWords; ++wd)
                if (wd == (t >> 2)) patch[wd] |= code << (8 * (t & 3));
        }
        uint32_t packed[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t v = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int f = fg * 16 + q * 4 + b;
                const uint32_t* wf = s_w + f * words;
                int iacc = 0;
                float facc = 0.0f;
#pragma unroll
                for (int wd = 0; wd < kStemMaxWords; ++wd) {
                    if (wd < words) {
                        if (KIND == LN_KIND_I8) iacc = __dp4a((int)patch[wd], (int)wf[wd], iacc);
                        else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                facc = fmaf(e4m3_to_float((uint8_t)(patch[wd] >> (8 * j))), e4m3_to_float((uint8_t)(wf[wd] >> (8 * j))), facc);
                        }
                    }
                }
                const float2 m = s_mb[f];
                float a = ln_epilogue_act<EXACT>(act, __fmaf_rn(KIND == LN_KIND_I8 ? __int2float_rn(iacc) : facc, m.x, m.y));
                uint32_t code = f < F ? quantize_code<KIND>(a, inv_sy) : 0u;
                v |= code << (8 * b);
            }
            packed[q] = v;
        }
        *reinterpret_cast<uint4*>(out + pix * out_pixel_stride + fg * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// rne(a * inv_s) clamped to +-127 in the low byte of the result, on the FMA pipe only (no conversion unit).
__device__ __forceinline__ uint32_t quant_i8_magic(float a, float inv_s) {
    float t = __fmul_rn(a, inv_s);
    t = fminf(fmaxf(t, -127.0f), 127.0f);  // NaN -> -127
    return __float_as_uint(__fadd_rn(t, 12582912.0f));
}
__device__ __forceinline__ uint32_t pack4_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// The usual first layer: 3x3 convolution of a 3-channel f32 NCHW image, int8.  One thread per pair of adjacent output
// pixels: the 27 input values of each are quantised once into 7 packed words held in registers, then every filter costs
// 7 dp4a per pixel against weights read (broadcast) from shared memory once for both, and each group of 16 filters
// leaves as one 16-byte store per pixel.
template <int ACT, bool EXACT>
__global__ void __launch_bounds__(256) conv_stem_k3c3_i8_kernel(const float* __restrict__ x, float inv_sx, int N, int H, int W,
                                                                const uint8_t* __restrict__ w_oihw, const float2* __restrict__ mb, int F, int stride,
                                                                int pad, int OH, int OW, float inv_sy, uint8_t* __restrict__ out,
                                                                int64_t out_pixel_stride, int s2d) {
    extern __shared__ uint4 s_w4[];  // [F16*16][2]: 8 words per filter, 7 used; byte t of a filter = tap (t/3), channel (t%3)
    const int F16 = (F + 15) / 16;
    float2* s_mb = reinterpret_cast<float2*>(s_w4 + F16 * 16 * 2);
    uint32_t* s_w = reinterpret_cast<uint32_t*>(s_w4);
    for (int i = threadIdx.x; i < F16 * 16 * 8; i += blockDim.x) {
        const int f = i >> 3, wd = i & 7;
        uint32_t v = 0;
        for (int j = 0; j < 4; ++j) {
            const int t = wd * 4 + j;
            if (f < F && t < 27) v |= (uint32_t)w_oihw[((int64_t)f * 3 + (t % 3)) * 9 + (t / 3)] << (8 * j);
        }
        s_w[i] = v;
    }
    for (int i = threadIdx.x; i < F16 * 16; i += blockDim.x) s_mb[i] = i < F ? mb[i] : make_float2(0.0f, 0.0f);
    __syncthreads();
    // one thread per pair of horizontally adjacent output pixels: every weight word read from shared memory serves both
    const int OWP = (OW + 1) / 2;
    const int64_t total = (int64_t)N * OH * OWP;
    for (int64_t pp = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; pp < total; pp += (int64_t)gridDim.x * blockDim.x) {
        const int ox0 = (int)(pp % OWP) * 2, oy = (int)((pp / OWP) % OH);
        const int64_t n = pp / ((int64_t)OWP * OH);
        const bool second = ox0 + 1 < OW;
        // taps outside the image contribute nothing: every load goes to a clamped (valid) address and the code is masked, so the
        // loads carry no branches
        uint32_t patch[2][7] = {{0, 0, 0, 0, 0, 0, 0}, {0, 0, 0, 0, 0, 0, 0}};
        const float* xn = x + n * 3 * (int64_t)H * W;
        int rowoff[3];
        bool rowok[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const int iy = oy * stride + k - pad;
            rowok[k] = iy >= 0 && iy < H;
            rowoff[k] = min(max(iy, 0), H - 1) * W;
        }
#pragma unroll
        for (int px = 0; px < 2; ++px) {
            int coloff[3];
            bool colok[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const int ix = (ox0 + px) * stride + k - pad;
                colok[k] = ix >= 0 && ix < W;
                coloff[k] = min(max(ix, 0), W - 1);
            }
#pragma unroll
            for (int t = 0; t < 27; ++t) {
                const int c = t % 3, ky = (t / 3) / 3, kx = (t / 3) % 3;
                const uint32_t q = quant_i8_magic(__ldg(xn + (int64_t)c * H * W + rowoff[ky] + coloff[kx]), inv_sx) & 0xFFu;
                patch[px][t >> 2] |= (rowok[ky] && colok[kx] ? q : 0u) << (8 * (t & 3));
            }
        }
        const uint4* wp = s_w4;      // 16 filters x 2 words of 16 bytes per group: constant offsets inside the group
        const float2* mp = s_mb;
        // s2d: the 32 channels of pixel (y, x) go to sub-pixel (y & 1) * 2 + (x & 1) of the 128-byte pixel (y / 2, x / 2); the pair
        // of this thread (x even, x + 1) lands in consecutive 32-byte slots either way
        uint8_t* op = s2d ? out + ((((int64_t)n * (OH >> 1) + (oy >> 1)) * (OW >> 1) + (ox0 >> 1)) * 4 + (oy & 1) * 2) * out_pixel_stride
                          : out + (((int64_t)n * OH + oy) * OW + ox0) * out_pixel_stride;
        const __half2 inv_h = __float2half2_rn(inv_sy);
        for (int fg = 0; fg < F16; ++fg, wp += 32, mp += 16, op += 16) {
            uint32_t packed[2][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float v[2][4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint4 w0 = wp[(q * 4 + b) * 2], w1 = wp[(q * 4 + b) * 2 + 1];
                    const float2 m = mp[q * 4 + b];
#pragma unroll
                    for (int px = 0; px < 2; ++px) {
                        int acc = __dp4a((int)patch[px][0], (int)w0.x, 0);
                        acc = __dp4a((int)patch[px][1], (int)w0.y, acc);
                        acc = __dp4a((int)patch[px][2], (int)w0.z, acc);
                        acc = __dp4a((int)patch[px][3], (int)w0.w, acc);
                        acc = __dp4a((int)patch[px][4], (int)w1.x, acc);
                        acc = __dp4a((int)patch[px][5], (int)w1.y, acc);
                        acc = __dp4a((int)patch[px][6], (int)w1.z, acc);
                        // |acc| <= 27*127*127 < 2^22: adding it to the bits of 1.5*2^23 converts exactly
                        const float xf = __fadd_rn(__int_as_float(0x4B400000 + acc), -12582912.0f);
                        v[px][b] = __fmaf_rn(xf, m.x, m.y);  // filters beyond F have m = {0, 0}: their code is act(0) and is masked below
                    }
                }
#pragma unroll
                for (int px = 0; px < 2; ++px) {
                    if (EXACT) {
                        uint32_t u[4];
#pragma unroll
                        for (int b = 0; b < 4; ++b) u[b] = fg * 16 + q * 4 + b < F ? quant_i8_magic(ln_epilogue_act<true>(ACT, v[px][b]), inv_sy) : 0u;
                        packed[px][q] = pack4_low_bytes(u[0], u[1], u[2], u[3]);
                    } else {
                        uint32_t w = ln_h2_pack(ln_h2_act_quant<ACT>(v[px][0], v[px][1], inv_h), ln_h2_act_quant<ACT>(v[px][2], v[px][3], inv_h));
                        const int valid = F - (fg * 16 + q * 4);  // keep only the codes of real filters
                        if (valid < 4) w = valid <= 0 ? 0u : (w & (0xFFFFFFFFu >> (8 * (4 - valid))));
                        packed[px][q] = w;
                    }
                }
            }
            *reinterpret_cast<uint4*>(op) = make_uint4(packed[0][0], packed[0][1], packed[0][2], packed[0][3]);
            if (second) *reinterpret_cast<uint4*>(op + out_pixel_stride) = make_uint4(packed[1][0], packed[1][1], packed[1][2], packed[1][3]);
        }
    }
}

// The first layer on the warp-level tensor-core instruction (mma.sync m16n8k32, s8 x s8 -> s32): K = 27 taps padded to 32 is
// one instruction deep, so there is no pipeline to build -- what the layer costs is quantising the 27 inputs of a pixel and the
// epilogue of its F outputs.  A warp takes 64 output pixels (two horizontally adjacent ones per thread, as the CUDA-core kernel
// does): every thread quantises its two patches into a [64 pixels][32 bytes] tile of shared memory, ldmatrix hands the tile to
// the tensor core 16 pixels at a time, and a thread receives, for two pixels of the 16, the accumulators of filters 8 j + 2 q
// and 8 j + 2 q + 1 (q = lane % 4): adjacent filters of one pixel, which is what the packed-binary16 epilogue wants, with the
// {multiplier, bias} of its eight filters in registers for the whole kernel.  Codes go back through the same tile (a pixel's
// row holds its patch before and its F codes after), so every thread stores the 16-byte pieces of its own two pixels.
// F = 8 * GROUPS (16 or 32 are instantiated).  Bit-exact accumulators; the epilogue is the one of conv_umma_kernel (exact or fast).
// KIND = LN_KIND_F8: the same with E4M3 codes and f32 accumulation (mma.sync ... f32.e4m3.e4m3.f32); the epilogue is the general one
// (activation in f32, exact or with the hardware exponential, E4M3 code of a / s_y).
template <int KIND, int ACT, bool EXACT, int GROUPS>
__global__ void __launch_bounds__(256) conv_stem_mma_kernel(const float* __restrict__ x, float inv_sx, int N, int H, int W,
                                                               const uint8_t* __restrict__ w_oihw, const float2* __restrict__ mb, int F, int stride,
                                                               int pad, int OH, int OW, float inv_sy, uint8_t* __restrict__ out,
                                                               int64_t out_pixel_stride, int s2d) {
    __shared__ __align__(16) uint32_t s_w[32 * 8];          // [filter][8 words]: byte t of a filter = tap (t / 3), channel (t % 3)
    __shared__ __align__(16) uint8_t s_tile[8][64 * 32];    // per warp
    for (int i = threadIdx.x; i < 32 * 8; i += blockDim.x) {
        const int f = i >> 3, wd = i & 7;
        uint32_t v = 0;
        for (int j = 0; j < 4; ++j) {
            const int t = wd * 4 + j;
            if (f < F && t < 27) v |= (uint32_t)w_oihw[((int64_t)f * 3 + (t % 3)) * 9 + (t / 3)] << (8 * j);
        }
        s_w[i] = v;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q = lane & 3, r8 = lane >> 2;
    constexpr int groups = GROUPS;  // filter groups of 8 (F = 8 * GROUPS)
    // B fragments (32 x 8, "col": filter r8 of the group, K words q and q + 4) and the epilogue constants of this thread's filters
    uint32_t bfrag[4][2];
    float cm[4][2], cb[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int fb = 8 * j + r8;
        bfrag[j][0] = j < groups ? s_w[fb * 8 + q] : 0u;
        bfrag[j][1] = j < groups ? s_w[fb * 8 + q + 4] : 0u;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int f = 8 * j + 2 * q + e;
            const float2 m = f < F ? mb[f] : make_float2(0.0f, 0.0f);
            if (EXACT || KIND != LN_KIND_I8) { cm[j][e] = m.x; cb[j][e] = m.y; }
            else {  // folded: fma(float with the bits 0x4B400000 + acc, m / s_y, b / s_y - 1.5 * 2^23 * m / s_y) is the pre-activation in code units
                cm[j][e] = __fmul_rn(m.x, inv_sy);
                cb[j][e] = __fmaf_rn(-12582912.0f, cm[j][e], __fmul_rn(m.y, inv_sy));
            }
        }
    }
    uint8_t* tile = s_tile[warp];
    const uint32_t tile_s = (uint32_t)__cvta_generic_to_shared(tile);
    const __half2 kh = __float2half2_rn(1.44269504f / inv_sy), inv_h = __float2half2_rn(inv_sy);
    const int OWP = (OW + 1) / 2;
    const int total = N * OH * OWP;  // pixel pairs (the launcher checks that this fits 31 bits)
    const int warps_total = (int)gridDim.x * (int)(blockDim.x >> 5);
    for (int wbase = ((int)blockIdx.x * (int)(blockDim.x >> 5) + warp) * 32; wbase < total; wbase += warps_total * 32) {
        const int pp = wbase + lane;
        const bool have = pp < total;
        const unsigned ppc = (unsigned)(have ? pp : total - 1);
        const unsigned rowi = ppc / (unsigned)OWP;  // n * OH + oy
        const int ox0 = (int)(ppc - rowi * (unsigned)OWP) * 2;
        const int n = (int)(rowi / (unsigned)OH), oy = (int)(rowi - (unsigned)n * (unsigned)OH);
        const bool second = ox0 + 1 < OW;
        // ---- quantise the inputs of the two patches once (they share 3 - stride of their three columns), as one word of three
        // channel codes per input pixel; taps outside the image contribute nothing: clamped loads, masked words
        const float* xn = x + (int64_t)n * 3 * H * W;
        const int plane = H * W;
        uint32_t trip[3][5];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const int iy = oy * stride + ky - pad;
            const bool rok = iy >= 0 && iy < H;
            const int roff = min(max(iy, 0), H - 1) * W;
#pragma unroll
            for (int j = 0; j < 5; ++j) {
                if (j < 3 + stride) {  // (stride is 1 or 2)
                    const int ix = ox0 * stride + j - pad;
                    const float* px = xn + roff + min(max(ix, 0), W - 1);
                    uint32_t c0, c1, c2;
                    if (KIND == LN_KIND_I8) {
                        c0 = quant_i8_magic(__ldg(px), inv_sx) & 0xFFu;
                        c1 = quant_i8_magic(__ldg(px + plane), inv_sx) & 0xFFu;
                        c2 = quant_i8_magic(__ldg(px + 2 * plane), inv_sx) & 0xFFu;
                    } else {
                        c0 = float_to_e4m3(__fmul_rn(__ldg(px), inv_sx));
                        c1 = float_to_e4m3(__fmul_rn(__ldg(px + plane), inv_sx));
                        c2 = float_to_e4m3(__fmul_rn(__ldg(px + 2 * plane), inv_sx));
                    }
                    trip[ky][j] = rok && ix >= 0 && ix < W ? (c0 | (c1 << 8) | (c2 << 16)) : 0u;
                } else trip[ky][j] = 0u;
            }
        }
        // the patch is the byte stream of nine such triples (tap major); word w takes bytes 4 w .. 4 w + 3 of it
#pragma unroll
        for (int px = 0; px < 2; ++px) {
            uint32_t t9[10];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) t9[tap] = stride == 1 ? trip[tap / 3][tap % 3 + px] : trip[tap / 3][tap % 3 + 2 * px];
            t9[9] = 0u;
            uint32_t patch[8];
            patch[7] = 0u;
#pragma unroll
            for (int wd = 0; wd < 7; ++wd) {
                const int b0 = 4 * wd, ta = b0 / 3, off = b0 % 3;  // first byte of the word is byte `off` of triple `ta`
                // bytes off .. 2 of triple ta, then the first 1 + off bytes of triple ta + 1 (a triple's fourth byte is 0, and so is triple 9)
                patch[wd] = off == 0 ? __byte_perm(t9[ta], t9[ta + 1], 0x4210) : (off == 1 ? __byte_perm(t9[ta], t9[ta + 1], 0x5421) : __byte_perm(t9[ta], t9[ta + 1], 0x6542));
            }
            // (the two 16-byte halves of a row are swapped in rows 4..7 mod 8: rows r and r + 4 then sit in different banks)
            const int rr = 2 * lane + px, sw = (rr >> 2) & 1;
            uint4* row = reinterpret_cast<uint4*>(tile + rr * 32);
            row[sw] = make_uint4(patch[0], patch[1], patch[2], patch[3]);
            row[sw ^ 1] = make_uint4(patch[4], patch[5], patch[6], patch[7]);
        }
        __syncwarp();
        // ---- 16 pixels at a time through the tensor core, then the epilogue of this thread's 2 x 8 values of the group
#pragma unroll 1
        for (int g = 0; g < 4; ++g) {
            uint32_t a0, a1, a2, a3;
            // ldmatrix x4: lanes 0-7 address rows 0-7 (bytes 0-15), 8-15 rows 8-15 (bytes 0-15), 16-23 rows 0-7 (bytes 16-31), 24-31 rows 8-15 (bytes 16-31)
            const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
            const uint32_t addr = tile_s + (uint32_t)((16 * g + lrow) * 32 + (((lane >> 4) ^ (lrow >> 2)) & 1) * 16);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(addr));
            __syncwarp();  // every lane has its fragment: the rows of this group may now take the codes
            int acc[4][4];  // int32 accumulators, or the bits of f32 ones
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
                if (j < groups) {
                    if (KIND == LN_KIND_I8)
                        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                                     : "+r"(acc[j][0]), "+r"(acc[j][1]), "+r"(acc[j][2]), "+r"(acc[j][3])
                                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bfrag[j][0]), "r"(bfrag[j][1]));
                    else
                        asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                                     : "+r"(acc[j][0]), "+r"(acc[j][1]), "+r"(acc[j][2]), "+r"(acc[j][3])
                                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bfrag[j][0]), "r"(bfrag[j][1]));
                }
            }
            // this thread: pixel rows r8 and r8 + 8 of the group, filters 8 j + 2 q, 8 j + 2 q + 1
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                uint8_t* orow = tile + (16 * g + r8 + 8 * hrow) * 32;
                const int osw = ((r8 >> 2) & 1) << 4;  // (16 g and 8 hrow do not change bit 2 of the row)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j >= groups) continue;
                    const int a_lo = acc[j][2 * hrow], a_hi = acc[j][2 * hrow + 1];
                    uint32_t two;  // the two code bytes, filter 8 j + 2 q in the low one
                    if (KIND != LN_KIND_I8) {
                        const float v0 = ln_epilogue_act<EXACT>(ACT, __fmaf_rn(__int_as_float(a_lo), cm[j][0], cb[j][0]));
                        const float v1 = ln_epilogue_act<EXACT>(ACT, __fmaf_rn(__int_as_float(a_hi), cm[j][1], cb[j][1]));
                        two = (uint32_t)float_to_e4m3(__fmul_rn(v0, inv_sy)) | ((uint32_t)float_to_e4m3(__fmul_rn(v1, inv_sy)) << 8);
                    } else if (EXACT) {
                        // |acc| <= 27 * 127 * 127 < 2^22: adding it to the bits of 1.5 * 2^23 converts exactly
                        const float v0 = __fmaf_rn(__fadd_rn(__int_as_float(0x4B400000 + a_lo), -12582912.0f), cm[j][0], cb[j][0]);
                        const float v1 = __fmaf_rn(__fadd_rn(__int_as_float(0x4B400000 + a_hi), -12582912.0f), cm[j][1], cb[j][1]);
                        const uint32_t u0 = quant_i8_magic(ln_epilogue_act<true>(ACT, v0), inv_sy), u1 = quant_i8_magic(ln_epilogue_act<true>(ACT, v1), inv_sy);
                        two = (u0 & 0xFFu) | ((u1 & 0xFFu) << 8);
                    } else {
                        const float t0 = __fmaf_rn(__int_as_float(0x4B400000 + a_lo), cm[j][0], cb[j][0]);
                        const float t1 = __fmaf_rn(__int_as_float(0x4B400000 + a_hi), cm[j][1], cb[j][1]);
                        const uint32_t c2 = ln_h2_code<ACT>(t0, t1, kh, inv_h);  // code bytes in the low byte of each half
                        two = __byte_perm(c2, 0u, 0x4420);
                    }
                    *reinterpret_cast<uint16_t*>(orow + ((8 * j + 2 * q) ^ osw)) = (uint16_t)two;
                }
            }
        }
        __syncwarp();
        // ---- every thread stores the codes of its own two pixels
        if (have) {
            uint8_t* op = s2d ? out + ((((int64_t)n * (OH >> 1) + (oy >> 1)) * (OW >> 1) + (ox0 >> 1)) * 4 + (oy & 1) * 2) * out_pixel_stride
                              : out + (((int64_t)n * OH + oy) * OW + ox0) * out_pixel_stride;
            const uint4* r0 = reinterpret_cast<const uint4*>(tile + (2 * lane) * 32);
            const uint4* r1 = reinterpret_cast<const uint4*>(tile + (2 * lane + 1) * 32);
            const int sw0 = ((2 * lane) >> 2) & 1;  // rows 2 lane and 2 lane + 1 share their bit 2
            for (int fg = 0; fg * 16 < F; ++fg) {
                uint4 v0 = r0[fg ^ sw0], v1 = r1[fg ^ sw0];
                if (F - fg * 16 < 16) { v0.z = v0.w = 0u; v1.z = v1.w = 0u; }  // eight real filters in this half: the rest of the 16 bytes is padding
                *reinterpret_cast<uint4*>(op + fg * 16) = v0;
                if (second) *reinterpret_cast<uint4*>(op + out_pixel_stride + fg * 16) = v1;
            }
        }
        __syncwarp();
    }
}

// The same first layer in FP8 E4M3, one thread per pair of adjacent output pixels: the 27 input values of each are rounded
// to E4M3 once and kept as floats (products of two E4M3 values are exact in f32), every filter costs 27 FMAs per pixel
// against decoded weights read (broadcast) from shared memory once for both.
template <int ACT, bool EXACT>
__global__ void __launch_bounds__(256) conv_stem_k3c3_f8_kernel(const float* __restrict__ x, float inv_sx, int N, int H, int W,
                                                                const uint8_t* __restrict__ w_oihw, const float2* __restrict__ mb, int F, int stride,
                                                                int pad, int OH, int OW, float inv_sy, uint8_t* __restrict__ out,
                                                                int64_t out_pixel_stride, int s2d) {
    extern __shared__ uint4 s_w4[];  // [F16*16][7] float4: 28 floats per filter, 27 used; float t of a filter = tap (t/3), channel (t%3)
    const int F16 = (F + 15) / 16;
    float* s_w = reinterpret_cast<float*>(s_w4);
    float2* s_mb = reinterpret_cast<float2*>(s_w + F16 * 16 * 28);
    for (int i = threadIdx.x; i < F16 * 16 * 28; i += blockDim.x) {
        const int f = i / 28, t = i % 28;
        s_w[i] = (f < F && t < 27) ? e4m3_to_float(w_oihw[((int64_t)f * 3 + (t % 3)) * 9 + (t / 3)]) : 0.0f;
    }
    for (int i = threadIdx.x; i < F16 * 16; i += blockDim.x) s_mb[i] = i < F ? mb[i] : make_float2(0.0f, 0.0f);
    __syncthreads();
    const float4* s_wv = reinterpret_cast<const float4*>(s_w);
    const int OWP = (OW + 1) / 2;
    const int64_t total = (int64_t)N * OH * OWP;
    for (int64_t pp = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; pp < total; pp += (int64_t)gridDim.x * blockDim.x) {
        const int ox0 = (int)(pp % OWP) * 2, oy = (int)((pp / OWP) % OH);
        const int64_t n = pp / ((int64_t)OWP * OH);
        const bool second = ox0 + 1 < OW;
        // taps outside the image contribute nothing: every load goes to a clamped (valid) address and the value is masked
        float patch[2][28];
        patch[0][27] = patch[1][27] = 0.0f;
        const float* xn = x + n * 3 * (int64_t)H * W;
        int rowoff[3];
        bool rowok[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const int iy = oy * stride + k - pad;
            rowok[k] = iy >= 0 && iy < H;
            rowoff[k] = min(max(iy, 0), H - 1) * W;
        }
#pragma unroll
        for (int px = 0; px < 2; ++px) {
            int coloff[3];
            bool colok[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const int ix = (ox0 + px) * stride + k - pad;
                colok[k] = ix >= 0 && ix < W;
                coloff[k] = min(max(ix, 0), W - 1);
            }
#pragma unroll
            for (int t = 0; t < 27; ++t) {
                const int c = t % 3, ky = (t / 3) / 3, kx = (t / 3) % 3;
                const float v = e4m3_to_float(float_to_e4m3(__fmul_rn(__ldg(xn + (int64_t)c * H * W + rowoff[ky] + coloff[kx]), inv_sx)));
                patch[px][t] = rowok[ky] && colok[kx] ? v : 0.0f;
            }
        }
        uint8_t* op = s2d ? out + ((((int64_t)n * (OH >> 1) + (oy >> 1)) * (OW >> 1) + (ox0 >> 1)) * 4 + (oy & 1) * 2) * out_pixel_stride
                          : out + (((int64_t)n * OH + oy) * OW + ox0) * out_pixel_stride;
        for (int fg = 0; fg < F16; ++fg, op += 16) {
            uint32_t packed[2][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t word[2] = {0, 0};
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int f = fg * 16 + q * 4 + b;
                    float acc[2] = {0.0f, 0.0f};
#pragma unroll
                    for (int j = 0; j < 7; ++j) {
                        const float4 w = s_wv[f * 7 + j];
#pragma unroll
                        for (int px = 0; px < 2; ++px) {
                            acc[px] = __fmaf_rn(patch[px][4 * j], w.x, acc[px]);
                            acc[px] = __fmaf_rn(patch[px][4 * j + 1], w.y, acc[px]);
                            acc[px] = __fmaf_rn(patch[px][4 * j + 2], w.z, acc[px]);
                            acc[px] = __fmaf_rn(patch[px][4 * j + 3], w.w, acc[px]);
                        }
                    }
                    const float2 m = s_mb[f];
#pragma unroll
                    for (int px = 0; px < 2; ++px) {
                        const float a = ln_epilogue_act<EXACT>(ACT, __fmaf_rn(acc[px], m.x, m.y));
                        if (f < F) word[px] |= (uint32_t)float_to_e4m3(__fmul_rn(a, inv_sy)) << (8 * b);
                    }
                }
                packed[0][q] = word[0];
                packed[1][q] = word[1];
            }
            *reinterpret_cast<uint4*>(op) = make_uint4(packed[0][0], packed[0][1], packed[0][2], packed[0][3]);
            if (second) *reinterpret_cast<uint4*>(op + out_pixel_stride) = make_uint4(packed[1][0], packed[1][1], packed[1][2], packed[1][3]);
        }
    }
}

bool is_q(const ln_tensor* t) { return t && (t->dtype == LN_Q8 || t->dtype == LN_F8); }
int kind_of(int dtype) { return dtype == LN_F8 ? LN_KIND_F8 : LN_KIND_I8; }

}  // namespace

int ln_check_status(ln_ctx* ctx, const char* where) {
    LN_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    LN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int s = *ctx->h_status;
    if (s == LN_STATUS_OK) return LN_OK;
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
    return ln_fail(ctx, LN_ERR_TIMEOUT, "%s: a bounded device-side wait gave up (status %d: %s)", where, s,
                   s == LN_STATUS_PRODUCER_TIMEOUT ? "TMA producer" : s == LN_STATUS_MMA_TIMEOUT ? "MMA issuer" : s == LN_STATUS_EPILOGUE_TIMEOUT ? "epilogue" : "unknown");
}

int ln_conv_simt_launch(ln_ctx* ctx, const ln_conv_geom& g, const void* w_unused, const float2* mb) {
    (void)w_unused;
    const int64_t total = (int64_t)g.N * g.OH * g.OW * g.F;
    const bool exact = ctx->exact_epilogue;
    // depthwise: the vectorised kernel (16 channels per thread, weights tap-major in shared memory)
    const size_t dw_smem = (size_t)g.k * g.k * ((g.C + 15) / 16) * 16;
    if (g.groups > 1 && g.groups == g.C && g.F == g.C && dw_smem <= 48 * 1024 && (g.x_pixel_stride & 15) == 0 && (((uintptr_t)g.x) & 15) == 0 &&
        (g.out_kind != LN_OUT_Q || ((g.out_pixel_stride & 15) == 0 && (((uintptr_t)g.out) & 15) == 0))) {
        const int dgrid = grid_for(ctx, (int64_t)g.N * g.OH * g.OW * ((g.C + 15) / 16));
        if (g.kind == LN_KIND_I8) {
            if (exact) conv_dw_q_kernel<LN_KIND_I8, true><<<dgrid, kThreads, dw_smem, ctx->stream>>>(g, mb);
            else conv_dw_q_kernel<LN_KIND_I8, false><<<dgrid, kThreads, dw_smem, ctx->stream>>>(g, mb);
        } else {
            if (exact) conv_dw_q_kernel<LN_KIND_F8, true><<<dgrid, kThreads, dw_smem, ctx->stream>>>(g, mb);
            else conv_dw_q_kernel<LN_KIND_F8, false><<<dgrid, kThreads, dw_smem, ctx->stream>>>(g, mb);
        }
        LN_LAUNCHED(ctx);
        return LN_OK;
    }
    const int grid = grid_for(ctx, total);
    if (g.kind == LN_KIND_I8) {
        if (exact) conv_simt_kernel<LN_KIND_I8, true><<<grid, kThreads, 0, ctx->stream>>>(g, mb);
        else conv_simt_kernel<LN_KIND_I8, false><<<grid, kThreads, 0, ctx->stream>>>(g, mb);
    } else {
        if (exact) conv_simt_kernel<LN_KIND_F8, true><<<grid, kThreads, 0, ctx->stream>>>(g, mb);
        else conv_simt_kernel<LN_KIND_F8, false><<<grid, kThreads, 0, ctx->stream>>>(g, mb);
    }
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_conv_stem_launch(ln_ctx* ctx, int kind, const float* x_nchw, float inv_sx, int N, int C, int H, int W, const void* w_oihw,
                        const float2* mb, int F, int k, int stride, int pad, int OH, int OW, int act, float inv_sy, void* out,
                        long long out_pixel_stride, int s2d_out) {
    if (s2d_out && !(k == 3 && C == 3 && F == 32 && out_pixel_stride == 32 && OH % 2 == 0 && OW % 2 == 0))
        return ln_fail(ctx, LN_ERR_UNSUPPORTED, "first-layer convolution: the space-to-depth output needs 3x3 over 3 channels, 32 filters and even output sizes");
    const int taps = k * k * C, words = (taps + 3) / 4;
    if (words > kStemMaxWords) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "first-layer convolution: k*k*C = %d exceeds %d", taps, kStemMaxWords * 4);
    const int F16 = (F + 15) / 16;
    const size_t smem = (size_t)F16 * 16 * words * 4 + (size_t)F16 * 16 * sizeof(float2);
    if (smem > 48 * 1024) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "first-layer convolution: %d filters do not fit shared memory", F);
    const int64_t total = (int64_t)N * OH * OW * F16;
    const int grid = grid_for(ctx, total);
    const bool exact = ctx->exact_epilogue;
    if (k == 3 && C == 3 && (kind == LN_KIND_I8 || F16 * 16 * 28 * 4 <= 40 * 1024)) {
        const size_t smem3 = (size_t)F16 * 16 * (kind == LN_KIND_I8 ? 32 : 28 * 4) + (size_t)F16 * 16 * sizeof(float2);
        // both kernels take two horizontally adjacent output pixels per thread
        const int grid3 = grid_for(ctx, (int64_t)N * OH * ((OW + 1) / 2));
#define LN_STEM3(A, E)                                                                                                                             \
    do {                                                                                                                                           \
        if (kind == LN_KIND_I8)                                                                                                                    \
            conv_stem_k3c3_i8_kernel<A, E><<<grid3, kThreads, smem3, ctx->stream>>>(x_nchw, inv_sx, N, H, W, (const uint8_t*)w_oihw, mb, F, stride, pad, \
                                                                                   OH, OW, inv_sy, (uint8_t*)out, out_pixel_stride, s2d_out);     \
        else                                                                                                                                       \
            conv_stem_k3c3_f8_kernel<A, E><<<grid3, kThreads, smem3, ctx->stream>>>(x_nchw, inv_sx, N, H, W, (const uint8_t*)w_oihw, mb, F, stride, pad, \
                                                                                   OH, OW, inv_sy, (uint8_t*)out, out_pixel_stride, s2d_out);     \
    } while (0)
        // 16 or 32 filters: the tensor-core form (LN_STEM_MMA=0 keeps the CUDA-core kernels, for A/B measurements)
        const char* stem_env = getenv("LN_STEM_MMA");
        // (its fast epilogue drops the lower clamp of the activations that are bounded below: needs 0.31 / s_y <= 127)
        if ((F == 32 || F == 16) && (stride == 1 || stride == 2) && (int64_t)N * OH * ((OW + 1) / 2) < (1ll << 30) &&
            (kind != LN_KIND_I8 || exact || inv_sy <= 400.0f) && !(stem_env && atoi(stem_env) == 0)) {
            const int64_t warps = ((int64_t)N * OH * ((OW + 1) / 2) + 31) / 32;
            int64_t blocks = (warps + 7) / 8;
            const int64_t cap = (int64_t)ctx->sm_count * 8;
            if (blocks > cap) blocks = cap;
#define LN_STEM_MMA(A, E)                                                                                                                          \
    do {                                                                                                                                           \
        if (kind == LN_KIND_I8 && F == 32)                                                                                                         \
            conv_stem_mma_kernel<LN_KIND_I8, A, E, 4><<<(int)blocks, 256, 0, ctx->stream>>>(x_nchw, inv_sx, N, H, W, (const uint8_t*)w_oihw, mb, F, stride, pad, OH, \
                                                                                           OW, inv_sy, (uint8_t*)out, out_pixel_stride, s2d_out); \
        else if (kind == LN_KIND_I8)                                                                                                               \
            conv_stem_mma_kernel<LN_KIND_I8, A, E, 2><<<(int)blocks, 256, 0, ctx->stream>>>(x_nchw, inv_sx, N, H, W, (const uint8_t*)w_oihw, mb, F, stride, pad, OH, \
                                                                                           OW, inv_sy, (uint8_t*)out, out_pixel_stride, s2d_out); \
        else if (F == 32)                                                                                                                          \
            conv_stem_mma_kernel<LN_KIND_F8, A, E, 4><<<(int)blocks, 256, 0, ctx->stream>>>(x_nchw, inv_sx, N, H, W, (const uint8_t*)w_oihw, mb, F, stride, pad, OH, \
                                                                                           OW, inv_sy, (uint8_t*)out, out_pixel_stride, s2d_out); \
        else                                                                                                                                       \
            conv_stem_mma_kernel<LN_KIND_F8, A, E, 2><<<(int)blocks, 256, 0, ctx->stream>>>(x_nchw, inv_sx, N, H, W, (const uint8_t*)w_oihw, mb, F, stride, pad, OH, \
                                                                                           OW, inv_sy, (uint8_t*)out, out_pixel_stride, s2d_out); \
    } while (0)
            switch (act) {
                case LN_ACT_LINEAR: if (exact) LN_STEM_MMA(LN_ACT_LINEAR, true); else LN_STEM_MMA(LN_ACT_LINEAR, false); break;
                case LN_ACT_LEAKY: if (exact) LN_STEM_MMA(LN_ACT_LEAKY, true); else LN_STEM_MMA(LN_ACT_LEAKY, false); break;
                case LN_ACT_RELU: if (exact) LN_STEM_MMA(LN_ACT_RELU, true); else LN_STEM_MMA(LN_ACT_RELU, false); break;
                case LN_ACT_MISH: if (exact) LN_STEM_MMA(LN_ACT_MISH, true); else LN_STEM_MMA(LN_ACT_MISH, false); break;
                case LN_ACT_SWISH: if (exact) LN_STEM_MMA(LN_ACT_SWISH, true); else LN_STEM_MMA(LN_ACT_SWISH, false); break;
                case LN_ACT_LOGISTIC: if (exact) LN_STEM_MMA(LN_ACT_LOGISTIC, true); else LN_STEM_MMA(LN_ACT_LOGISTIC, false); break;
                default: return ln_fail(ctx, LN_ERR_UNSUPPORTED, "first-layer convolution: activation %d", act);
            }
#undef LN_STEM_MMA
            LN_LAUNCHED(ctx);
            return LN_OK;
        }
        switch (act) {
            case LN_ACT_LINEAR: if (exact) LN_STEM3(LN_ACT_LINEAR, true); else LN_STEM3(LN_ACT_LINEAR, false); break;
            case LN_ACT_LEAKY: if (exact) LN_STEM3(LN_ACT_LEAKY, true); else LN_STEM3(LN_ACT_LEAKY, false); break;
            case LN_ACT_RELU: if (exact) LN_STEM3(LN_ACT_RELU, true); else LN_STEM3(LN_ACT_RELU, false); break;
            case LN_ACT_MISH: if (exact) LN_STEM3(LN_ACT_MISH, true); else LN_STEM3(LN_ACT_MISH, false); break;
            case LN_ACT_SWISH: if (exact) LN_STEM3(LN_ACT_SWISH, true); else LN_STEM3(LN_ACT_SWISH, false); break;
            case LN_ACT_LOGISTIC: if (exact) LN_STEM3(LN_ACT_LOGISTIC, true); else LN_STEM3(LN_ACT_LOGISTIC, false); break;
            default: return ln_fail(ctx, LN_ERR_UNSUPPORTED, "first-layer convolution: activation %d", act);
        }
#undef LN_STEM3
        LN_LAUNCHED(ctx);
        return LN_OK;
    }
#define LN_STEM(K, E)                                                                                                                   \
    conv_stem_kernel<K, E><<<grid, kThreads, smem, ctx->stream>>>(x_nchw, inv_sx, N, C, H, W, (const uint8_t*)w_oihw, mb, F, k, stride, pad, \
                                                                 OH, OW, act, inv_sy, (uint8_t*)out, out_pixel_stride)
    if (kind == LN_KIND_I8) { if (exact) LN_STEM(LN_KIND_I8, true); else LN_STEM(LN_KIND_I8, false); }
    else { if (exact) LN_STEM(LN_KIND_F8, true); else LN_STEM(LN_KIND_F8, false); }
#undef LN_STEM
    LN_LAUNCHED(ctx);
    return LN_OK;
}

// ---- internal helpers used by the network executor ------------------------------------------

int ln_q_maxpool_launch(ln_ctx* ctx, int kind, const void* x, int64_t xs, void* y, int64_t ys, int64_t N, int C, int H, int W, int OH, int OW,
                        int size, int sx, int sy, int padding) {
    const int C16 = (int)(ln_round_up(C, 16) / 16);
    const int64_t total = N * OH * OW * C16;
    const int off = padding / 2;
    if (size == 5 && sx == 1 && sy == 1 && OH == H && OW == W && off >= 0 && off <= 4) {
        // columns are split into row segments until there are about two blocks per SM (a segment re-reads four rows)
        const int64_t cols = N * W * C16;
        int segs = (int)((2ll * ctx->sm_count * kThreads + cols - 1) / cols);
        segs = segs < 1 ? 1 : (segs > (H + 3) / 4 ? (H + 3) / 4 : segs);
        const int seg_rows = (H + segs - 1) / segs;
        const dim3 grid((unsigned)grid_for(ctx, cols), (unsigned)((H + seg_rows - 1) / seg_rows));
        if (kind == LN_KIND_I8) maxpool5_same_q_kernel<LN_KIND_I8><<<grid, kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, off, seg_rows);
        else maxpool5_same_q_kernel<LN_KIND_F8><<<grid, kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, off, seg_rows);
        LN_LAUNCHED(ctx);
        return LN_OK;
    }
    if (size == 2 && sx == 2 && sy == 2 && off == 0 && 2 * (OH - 1) < H && 2 * (OW - 1) < W) {
        if (kind == LN_KIND_I8) maxpool2_s2_q_kernel<LN_KIND_I8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, OH, OW);
        else maxpool2_s2_q_kernel<LN_KIND_F8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, OH, OW);
        LN_LAUNCHED(ctx);
        return LN_OK;
    }
    if (kind == LN_KIND_I8)
        maxpool_q_kernel<LN_KIND_I8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, OH, OW, size, sx, sy, padding);
    else
        maxpool_q_kernel<LN_KIND_F8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, OH, OW, size, sx, sy, padding);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_q_upsample_requant_launch(ln_ctx* ctx, int kind, const void* x, int64_t xs, void* y, int64_t ys, int64_t N, int C, int H, int W, int stride, int reverse,
                                 float r) {
    const int OH = reverse ? H / stride : H * stride, OW = reverse ? W / stride : W * stride;
    const int64_t total = N * OH * OW * C;
    if (kind == LN_KIND_I8)
        upsample_requant_q_kernel<LN_KIND_I8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C, H, W, OH, OW, stride, reverse, r);
    else
        upsample_requant_q_kernel<LN_KIND_F8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C, H, W, OH, OW, stride, reverse, r);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_q_shortcut_fit_launch(ln_ctx* ctx, const void* x, int64_t xs, int sc, int sh, int sw, void* y, int64_t ys, int64_t N, int C, int H, int W) {
    shortcut_fit_q_kernel<<<grid_for(ctx, N * C * H * W), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, sc, sh, sw, (uint8_t*)y, ys, N, C, H, W);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_q_upsample_launch(ln_ctx* ctx, const void* x, int64_t xs, void* y, int64_t ys, int64_t N, int C, int H, int W, int stride) {
    const int C16 = (int)(ln_round_up(C, 16) / 16);
    const int64_t total = N * H * stride * W * stride * C16;
    upsample_q_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, N, C16, H, W, stride);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_q_copy_launch(ln_ctx* ctx, const void* x, int64_t xs, void* y, int64_t ys, int64_t pixels, int C) {
    const bool vec = (C % 16 == 0) && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)xs | (uintptr_t)ys) % 16 == 0);
    if (vec) copy_q16_kernel<<<grid_for(ctx, pixels * (C / 16)), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, pixels, C / 16);
    else copy_q1_kernel<<<grid_for(ctx, pixels * C), kThreads, 0, ctx->stream>>>((const uint8_t*)x, xs, (uint8_t*)y, ys, pixels, C);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_q_shortcut_launch(ln_ctx* ctx, int kind, const void* a, int64_t as, float sa, const void* b, int64_t bs, float sb, void* y, int64_t ys,
                         int64_t pixels, int C, int act, float inv_sy) {
    const int C4 = (int)(ln_round_up(C, 16) / 16);  // 16-channel vectors (tensors are padded to 32 channels)
    const int64_t total = pixels * C4;
    const int grid = grid_for(ctx, total);
    const bool exact = ctx->exact_epilogue;
#define LN_SC(K, E)                                                                                                                            \
    shortcut_q_kernel<K, E><<<grid, kThreads, 0, ctx->stream>>>((const uint8_t*)a, as, sa, (const uint8_t*)b, bs, sb, (uint8_t*)y, ys, pixels, C4, \
                                                               act, inv_sy)
    if (kind == LN_KIND_I8) { if (exact) LN_SC(LN_KIND_I8, true); else LN_SC(LN_KIND_I8, false); }
    else { if (exact) LN_SC(LN_KIND_F8, true); else LN_SC(LN_KIND_F8, false); }
#undef LN_SC
    LN_LAUNCHED(ctx);
    return LN_OK;
}

int ln_q_quantize_launch(ln_ctx* ctx, int kind, const float* x, void* y, int64_t N, int C, int H, int W, int64_t cstride, float inv_s) {
    const int64_t total = N * H * W * cstride;
    if (kind == LN_KIND_I8) quantize_nchw_kernel<LN_KIND_I8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(x, (uint8_t*)y, N, C, H, W, cstride, inv_s);
    else quantize_nchw_kernel<LN_KIND_F8><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(x, (uint8_t*)y, N, C, H, W, cstride, inv_s);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

// ---- C ABI -----------------------------------------------------------------------------------

extern "C" {

int32_t ln_tensor_upload_q(ln_ctx* ctx, const int64_t shape[4], const float* host, float scale, int32_t dtype, ln_tensor** out) {
    if (!ctx || !shape || !host || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_q: NULL argument");
    if (dtype != LN_Q8 && dtype != LN_F8) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_q: dtype must be LN_Q8 or LN_F8");
    if (!(scale > 0.0f)) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_q: scale must be positive");
    ln_tensor* f = nullptr;
    int rc = ln_tensor_upload_f32(ctx, shape, host, &f);
    if (rc) return rc;
    rc = ln_tensor_narrow_f32(ctx, f, scale, dtype, out);
    ln_tensor_release(f);
    return rc;
}

int32_t ln_tensor_narrow_f32(ln_ctx* ctx, const ln_tensor* t, float scale, int32_t dtype, ln_tensor** out_q) {
    if (!ctx || !t || !out_q) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_narrow_f32: NULL argument");
    if (t->dtype != LN_F32) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_narrow_f32: f32 tensor required");
    if (dtype != LN_Q8 && dtype != LN_F8) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_narrow_f32: dtype must be LN_Q8 or LN_F8");
    if (!(scale > 0.0f)) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_narrow_f32: scale must be positive");
    cudaSetDevice(ctx->device);
    ln_tensor* q = ln_tensor_new(ctx, dtype, t->n, t->c, t->h, t->w);
    if (!q) return LN_ERR_CUDA;
    q->scale = scale;
    int rc = ln_q_quantize_launch(ctx, kind_of(dtype), (const float*)t->ptr, q->ptr, t->n, (int)t->c, (int)t->h, (int)t->w, q->cstride, 1.0f / scale);
    if (rc) { ln_tensor_release(q); return rc; }
    *out_q = q;
    return LN_OK;
}

int32_t ln_tensor_widen_q(ln_ctx* ctx, const ln_tensor* t, ln_tensor** out_f32) {
    if (!ctx || !out_f32) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_widen_q: NULL argument");
    if (!is_q(t)) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_widen_q: 8-bit tensor required");
    cudaSetDevice(ctx->device);
    ln_tensor* f = ln_tensor_new(ctx, LN_F32, t->n, t->c, t->h, t->w);
    if (!f) return LN_ERR_CUDA;
    if (t->dtype == LN_Q8)
        dequantize_nhwc_kernel<LN_KIND_I8><<<grid_for(ctx, f->count()), kThreads, 0, ctx->stream>>>((const uint8_t*)t->ptr, (float*)f->ptr, t->n, (int)t->c, (int)t->h, (int)t->w, t->cstride, t->scale);
    else
        dequantize_nhwc_kernel<LN_KIND_F8><<<grid_for(ctx, f->count()), kThreads, 0, ctx->stream>>>((const uint8_t*)t->ptr, (float*)f->ptr, t->n, (int)t->c, (int)t->h, (int)t->w, t->cstride, t->scale);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ln_tensor_release(f); return ln_fail(ctx, LN_ERR_CUDA, "widen launch: %s", cudaGetErrorString(e)); }
    *out_f32 = f;
    return LN_OK;
}

int32_t ln_tensor_download_q(ln_ctx* ctx, const ln_tensor* t, void* host_codes, int64_t count, float* scale) {
    if (!ctx || !host_codes) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_q: NULL argument");
    if (!is_q(t)) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_download_q: 8-bit tensor required");
    if (count != t->count()) return ln_fail(ctx, LN_ERR_SHAPE, "download of %lld codes from a tensor of %lld", (long long)count, (long long)t->count());
    cudaSetDevice(ctx->device);
    void* tmp = ln_pool_alloc(ctx, (size_t)count);
    if (!tmp) return LN_ERR_CUDA;
    codes_nhwc_to_nchw_kernel<<<grid_for(ctx, count), kThreads, 0, ctx->stream>>>((const uint8_t*)t->ptr, (uint8_t*)tmp, t->n, (int)t->c, (int)t->h, (int)t->w, t->cstride);
    ctx->launches++;
    cudaError_t e = cudaMemcpyAsync(host_codes, tmp, (size_t)count, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    ln_pool_free(ctx, tmp, (size_t)count);
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "download_q: %s", cudaGetErrorString(e));
    if (scale) *scale = t->scale;
    return LN_OK;
}

int32_t ln_tensor_upload_codes(ln_ctx* ctx, const int64_t shape[4], const void* host_codes, float scale, int32_t dtype, ln_tensor** out) {
    if (!ctx || !shape || !host_codes || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_codes: NULL argument");
    if (dtype != LN_Q8 && dtype != LN_F8) return ln_fail(ctx, LN_ERR_ARG, "ln_tensor_upload_codes: dtype must be LN_Q8 or LN_F8");
    cudaSetDevice(ctx->device);
    ln_tensor* q = ln_tensor_new(ctx, dtype, shape[0], shape[1], shape[2], shape[3]);
    if (!q) return LN_ERR_SHAPE;
    q->scale = scale;
    const int64_t count = q->count();
    void* tmp = ln_pool_alloc(ctx, (size_t)count);
    if (!tmp) { ln_tensor_release(q); return LN_ERR_CUDA; }
    cudaError_t e = cudaMemcpyAsync(tmp, host_codes, (size_t)count, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        codes_nchw_to_nhwc_kernel<<<grid_for(ctx, q->n * q->h * q->w * q->cstride), kThreads, 0, ctx->stream>>>((const uint8_t*)tmp, (uint8_t*)q->ptr, q->n, (int)q->c, (int)q->h, (int)q->w, q->cstride);
        ctx->launches++;
        e = cudaGetLastError();
    }
    ln_pool_free(ctx, tmp, (size_t)count);
    if (e != cudaSuccess) { ln_tensor_release(q); return ln_fail(ctx, LN_ERR_CUDA, "upload_codes: %s", cudaGetErrorString(e)); }
    *out = q;
    return LN_OK;
}

int32_t ln_conv_weights_q(ln_ctx* ctx, const ln_tensor* weights_f32, int64_t filters, int64_t channels, int64_t kernel_size, int32_t dtype,
                          ln_conv_weights** out) {
    if (!ctx || !weights_f32 || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_conv_weights_q: NULL argument");
    if (weights_f32->dtype != LN_F32) return ln_fail(ctx, LN_ERR_ARG, "ln_conv_weights_q: f32 weights required");
    if (dtype != LN_Q8 && dtype != LN_F8) return ln_fail(ctx, LN_ERR_ARG, "ln_conv_weights_q: dtype must be LN_Q8 or LN_F8");
    if (filters < 1 || channels < 1 || kernel_size < 1 || weights_f32->count() != filters * channels * kernel_size * kernel_size)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv_weights_q: weight tensor has %lld elements, expected %lld", (long long)weights_f32->count(),
                       (long long)(filters * channels * kernel_size * kernel_size));
    cudaSetDevice(ctx->device);
    ln_conv_weights* w = new ln_conv_weights();
    w->ctx = ctx; w->dtype = dtype;
    w->filters = filters; w->channels = channels; w->k = kernel_size;
    w->cpad = ln_round_up(channels, 32);
    w->fpad = ln_round_up(filters, ln_conv_choose_bn(filters));
    const size_t packed_bytes = (size_t)(w->fpad * kernel_size * kernel_size * w->cpad);
    const size_t oihw_bytes = (size_t)(filters * channels * kernel_size * kernel_size);
    w->w = ln_pool_alloc(ctx, packed_bytes);
    w->w_oihw = ln_pool_alloc(ctx, oihw_bytes);
    w->wscale = (float*)ln_pool_alloc(ctx, (size_t)w->fpad * 8);  // [fpad] scales, then [fpad] sums of |code|
    if (!w->w || !w->w_oihw || !w->wscale) { ln_conv_weights_release(w); return LN_ERR_CUDA; }
    if (dtype == LN_Q8)
        pack_weights_kernel<LN_KIND_I8><<<(int)w->fpad, 256, 0, ctx->stream>>>((const float*)weights_f32->ptr, (int)filters, (int)channels, (int)kernel_size, (int)w->cpad, (uint8_t*)w->w, (uint8_t*)w->w_oihw, w->wscale);
    else
        pack_weights_kernel<LN_KIND_F8><<<(int)w->fpad, 256, 0, ctx->stream>>>((const float*)weights_f32->ptr, (int)filters, (int)channels, (int)kernel_size, (int)w->cpad, (uint8_t*)w->w, (uint8_t*)w->w_oihw, w->wscale);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    w->h_wscale.resize((size_t)w->fpad * 2);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->h_wscale.data(), w->wscale, (size_t)w->fpad * 8, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    w->max_l1 = 0.0f;
    for (int64_t f = 0; f < w->fpad; ++f) w->max_l1 = w->h_wscale[(size_t)(w->fpad + f)] > w->max_l1 ? w->h_wscale[(size_t)(w->fpad + f)] : w->max_l1;
    w->h_wscale.resize((size_t)w->fpad);
    w->max_scale = 0.0f;
    for (float v : w->h_wscale) w->max_scale = v > w->max_scale ? v : w->max_scale;
    if (e != cudaSuccess) { ln_conv_weights_release(w); return ln_fail(ctx, LN_ERR_CUDA, "weight packing: %s", cudaGetErrorString(e)); }
    *out = w;
    return LN_OK;
}

int32_t ln_conv_weights_release(ln_conv_weights* w) {
    if (!w) return LN_OK;
    ln_ctx* ctx = w->ctx;
    if (w->w) ln_pool_free(ctx, w->w, (size_t)(w->fpad * w->k * w->k * w->cpad));
    if (w->w_oihw) ln_pool_free(ctx, w->w_oihw, (size_t)(w->filters * w->channels * w->k * w->k));
    if (w->wscale) ln_pool_free(ctx, w->wscale, (size_t)w->fpad * 8);
    ln_tensor_release(w->src_f32);
    delete w;
    return LN_OK;
}

int32_t ln_conv2d_bias_act_q(ln_ctx* ctx, const ln_tensor* x, const ln_conv_weights* weights, const ln_tensor* bias, const int64_t output_shape[4],
                             int64_t channels, int64_t input_height, int64_t input_width, int64_t filters, int64_t kernel_size, int64_t stride_x,
                             int64_t stride_y, int64_t dilation, int64_t padding, int64_t groups, int32_t activation, float y_scale, int32_t out_kind,
                             ln_tensor** out) {
    if (!ctx || !weights || !bias || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_bias_act_q: NULL argument");
    if (!is_q(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_bias_act_q: 8-bit input required");
    if (x->dtype != weights->dtype) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_bias_act_q: input and weights have different 8-bit types");
    if (bias->dtype != LN_F32 || bias->count() != filters) return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_bias_act_q: bias must be f32 [filters]");
    if (dilation != 1) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_conv2d_bias_act_q: dilation must be 1");
    if (groups < 1 || channels % groups || filters % groups) return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_bias_act_q: groups do not divide channels / filters");
    if (stride_x != stride_y || stride_x < 1) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_conv2d_bias_act_q: stride_x must equal stride_y");
    if (x->c != channels || x->h != input_height || x->w != input_width || weights->channels != channels / groups || weights->filters != filters || weights->k != kernel_size)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_bias_act_q: geometry does not match the tensors");
    if (activation < LN_ACT_LINEAR || activation > LN_ACT_RELU) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_conv2d_bias_act_q: activation %d is not on the detector path", activation);
    if (out_kind < LN_OUT_Q || out_kind > LN_OUT_ACC) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_bias_act_q: bad out_kind");
    if (out_kind == LN_OUT_Q && !(y_scale > 0.0f)) return ln_fail(ctx, LN_ERR_ARG, "ln_conv2d_bias_act_q: y_scale must be positive");
    int64_t oh = (input_height + 2 * padding - kernel_size < 0 ? 0 : input_height + 2 * padding - kernel_size) / stride_y + 1;
    int64_t ow = (input_width + 2 * padding - kernel_size < 0 ? 0 : input_width + 2 * padding - kernel_size) / stride_x + 1;
    if (output_shape[0] != x->n || output_shape[1] != filters || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_conv2d_bias_act_q: output_shape does not match [%lld,%lld,%lld,%lld]", (long long)x->n, (long long)filters, (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    const int kind = kind_of(x->dtype);
    int out_dtype = out_kind == LN_OUT_Q ? x->dtype : (out_kind == LN_OUT_F32 ? LN_F32 : (kind == LN_KIND_I8 ? LN_I32 : LN_F32));
    ln_tensor* y = ln_tensor_new(ctx, out_dtype, x->n, filters, oh, ow);
    if (!y) return LN_ERR_CUDA;
    if (out_kind == LN_OUT_Q) {
        y->scale = y_scale;
        if (y->cstride != y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    }
    float2* mb = (float2*)ln_pool_alloc(ctx, (size_t)weights->fpad * sizeof(float2));
    if (!mb) { ln_tensor_release(y); return LN_ERR_CUDA; }
    int rc = ln_conv_umma_make_mb(ctx, weights->wscale, (const float*)bias->ptr, x->scale, (int)filters, (int)weights->fpad, mb);
    ln_conv_geom g;
    g.kind = kind;
    g.x = x->ptr; g.x_pixel_stride = x->cstride;
    g.N = (int)x->n; g.H = (int)x->h; g.W = (int)x->w; g.C = (int)x->c; g.cpad = (int)weights->cpad;
    g.w = weights->w; g.F = (int)filters; g.fpad = (int)weights->fpad; g.k = (int)kernel_size; g.stride = (int)stride_x; g.pad = (int)padding;
    g.OH = (int)oh; g.OW = (int)ow; g.act = activation; g.out_kind = out_kind;
    g.inv_sy = out_kind == LN_OUT_Q ? 1.0f / y_scale : 1.0f;
    g.small_acc = kind == LN_KIND_I8 && 127.0f * weights->max_l1 < 4194304.0f;
    g.acc_shift = kind == LN_KIND_I8 && out_kind == LN_OUT_Q ? ln_acc_shift(weights->max_l1, x->scale, weights->max_scale, g.inv_sy) : -1;
    g.out = y->ptr; g.out_pixel_stride = y->cstride;
    g.groups = (int)groups;
    if (groups > 1) { g.cpad = (int)ln_round_up(channels, 32); g.w_cpad = (int)weights->cpad; }
    if (rc == LN_OK) {
        if (groups == 1 && x->cstride >= weights->cpad && filters <= 4096 && ln_conv_umma_supported(weights->cpad, kernel_size, stride_x, stride_y, dilation, groups, input_width, input_height)) {
            ln_conv_umma_plan plan;
            plan.mb = mb;
            rc = ln_conv_umma_plan_build(ctx, &plan, g);
            if (rc == LN_OK && ctx->time_kernels) cudaEventRecord(ctx->ev_k0, ctx->stream);
            if (rc == LN_OK) rc = ln_conv_umma_launch(ctx, &plan);
            if (rc == LN_OK && ctx->time_kernels) { cudaEventRecord(ctx->ev_k1, ctx->stream); ctx->ev_pending = true; }
            if (rc == LN_OK) rc = ln_check_status(ctx, "ln_conv2d_bias_act_q");
            ln_conv_umma_plan_release(ctx, &plan);
        } else {
            rc = ln_conv_simt_launch(ctx, g, nullptr, mb);
        }
    }
    ln_pool_free(ctx, mb, (size_t)weights->fpad * sizeof(float2));
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_maxpool_q(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height, int64_t input_width,
                     int64_t size, int64_t stride_x, int64_t stride_y, int64_t padding, ln_tensor** out) {
    if (!ctx || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_maxpool_q: NULL argument");
    if (!is_q(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_maxpool_q: 8-bit tensor required");
    if (x->c != channels || x->h != input_height || x->w != input_width || size < 1 || stride_x < 1 || stride_y < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_maxpool_q: geometry does not match the input tensor");
    int64_t oh = (input_height + padding - size < 0 ? 0 : input_height + padding - size) / stride_y + 1;
    int64_t ow = (input_width + padding - size < 0 ? 0 : input_width + padding - size) / stride_x + 1;
    if (output_shape[0] != x->n || output_shape[1] != channels || output_shape[2] != oh || output_shape[3] != ow)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_maxpool_q: output_shape does not match pool_dim (%lld x %lld)", (long long)oh, (long long)ow);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, x->dtype, x->n, channels, oh, ow);
    if (!y) return LN_ERR_CUDA;
    y->scale = x->scale;
    int rc = ln_q_maxpool_launch(ctx, kind_of(x->dtype), x->ptr, x->cstride, y->ptr, y->cstride, x->n, (int)channels, (int)input_height, (int)input_width,
                                 (int)oh, (int)ow, (int)size, (int)stride_x, (int)stride_y, (int)padding);
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_upsample_q(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height, int64_t input_width,
                      int64_t stride, float scale, int32_t reverse, ln_tensor** out) {
    if (!ctx || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_upsample_q: NULL argument");
    if (!is_q(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_upsample_q: 8-bit tensor required");
    if (stride < 1) return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_q: upsample stride cannot be zero");
    if (!(scale > 0.0f)) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_upsample_q: scale must be positive");
    if (x->c != channels || x->h != input_height || x->w != input_width) return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_q: geometry does not match the input tensor");
    const int64_t oh = reverse ? input_height / stride : input_height * stride, ow = reverse ? input_width / stride : input_width * stride;
    if (output_shape[0] != x->n || output_shape[1] != channels || output_shape[2] != oh || output_shape[3] != ow || oh < 1 || ow < 1)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_upsample_q: output_shape does not match");
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, x->dtype, x->n, channels, oh, ow);
    if (!y) return LN_ERR_CUDA;
    int rc;
    if (reverse) {
        // out = scale * (sum of a stride x stride block): the code is the block's mean, the tensor scale carries scale * stride^2
        if (y->cstride != y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
        y->scale = x->scale * scale * (float)(stride * stride);
        rc = ln_q_upsample_requant_launch(ctx, kind_of(x->dtype), x->ptr, x->cstride, y->ptr, y->cstride, x->n, (int)channels, (int)input_height, (int)input_width, (int)stride, 1,
                                          1.0f / (float)(stride * stride));
    } else {
        y->scale = x->scale * scale;  // out = scale * in: the codes are unchanged, the tensor scale carries the factor
        rc = ln_q_upsample_launch(ctx, x->ptr, x->cstride, y->ptr, y->cstride, x->n, (int)channels, (int)input_height, (int)input_width, (int)stride);
    }
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_shortcut_fit_q(ln_ctx* ctx, const ln_tensor* x, int64_t batch, const int64_t output_shape[4], ln_tensor** out) {
    if (!ctx || !output_shape || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_fit_q: NULL argument");
    if (!is_q(x)) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_fit_q: 8-bit tensor required");
    if (batch != x->n || output_shape[0] != batch) return ln_fail(ctx, LN_ERR_SHAPE, "ln_shortcut_fit_q: batch mismatch");
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, x->dtype, output_shape[0], output_shape[1], output_shape[2], output_shape[3]);
    if (!y) return LN_ERR_SHAPE;
    y->scale = x->scale;
    if (y->cstride != y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    int rc = ln_q_shortcut_fit_launch(ctx, x->ptr, x->cstride, (int)x->c, (int)x->h, (int)x->w, y->ptr, y->cstride, y->n, (int)y->c, (int)y->h, (int)y->w);
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

int32_t ln_route_concat_q(ln_ctx* ctx, const ln_tensor* const* inputs, int32_t n_inputs, const int64_t* input_channel_offsets,
                          const int64_t* input_channels, const int64_t* input_total_channels, const int64_t output_shape[4], int64_t channel_stride,
                          ln_tensor** out) {
    if (!ctx || !out || !inputs || !input_channel_offsets || !input_channels || !input_total_channels || !output_shape || n_inputs < 1)
        return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_q: NULL argument");
    int64_t sum = 0;
    for (int i = 0; i < n_inputs; ++i) {
        if (!is_q(inputs[i]) || inputs[i]->dtype != inputs[0]->dtype) return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_q: input %d is not an 8-bit tensor of the common type", i);
        if (inputs[i]->scale != inputs[0]->scale) return ln_fail(ctx, LN_ERR_ARG, "ln_route_concat_q: inputs must share one scale (input %d has %g, input 0 has %g)", i, inputs[i]->scale, inputs[0]->scale);
        if (inputs[i]->c != input_total_channels[i] || input_channel_offsets[i] + input_channels[i] > input_total_channels[i] ||
            inputs[i]->h * inputs[i]->w != channel_stride || inputs[i]->n != output_shape[0])
            return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_q: input %d does not match its channel slice / plane size", i);
        sum += input_channels[i];
    }
    if (sum != output_shape[1] || output_shape[2] * output_shape[3] != channel_stride)
        return ln_fail(ctx, LN_ERR_SHAPE, "ln_route_concat_q: slices sum to %lld channels, output has %lld", (long long)sum, (long long)output_shape[1]);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, inputs[0]->dtype, output_shape[0], output_shape[1], output_shape[2], output_shape[3]);
    if (!y) return LN_ERR_CUDA;
    y->scale = inputs[0]->scale;
    if (y->cstride != y->c) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    int64_t c0 = 0;
    for (int i = 0; i < n_inputs; ++i) {
        int rc = ln_q_copy_launch(ctx, (const uint8_t*)inputs[i]->ptr + input_channel_offsets[i], inputs[i]->cstride, (uint8_t*)y->ptr + c0, y->cstride,
                                  y->n * channel_stride, (int)input_channels[i]);
        if (rc) { ln_tensor_release(y); return rc; }
        c0 += input_channels[i];
    }
    *out = y;
    return LN_OK;
}

int32_t ln_shortcut_add_act_q(ln_ctx* ctx, const ln_tensor* a, const ln_tensor* b, int32_t activation, float y_scale, ln_tensor** out) {
    if (!ctx || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_act_q: NULL argument");
    if (!is_q(a) || !is_q(b) || a->dtype != b->dtype) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_act_q: two 8-bit tensors of one type required");
    if (a->n != b->n || a->c != b->c || a->h != b->h || a->w != b->w) return ln_fail(ctx, LN_ERR_SHAPE, "ln_shortcut_add_act_q: shapes differ (use the f32 path to fit mismatched sources)");
    if (!(y_scale > 0.0f)) return ln_fail(ctx, LN_ERR_ARG, "ln_shortcut_add_act_q: y_scale must be positive");
    if (activation < LN_ACT_LINEAR || activation > LN_ACT_RELU) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_shortcut_add_act_q: activation %d is not on the detector path", activation);
    cudaSetDevice(ctx->device);
    ln_tensor* y = ln_tensor_new(ctx, a->dtype, a->n, a->c, a->h, a->w);
    if (!y) return LN_ERR_CUDA;
    y->scale = y_scale;
    if (y->cstride != ln_round_up(y->c, 16)) cudaMemsetAsync(y->ptr, 0, y->bytes, ctx->stream);
    int rc = ln_q_shortcut_launch(ctx, kind_of(a->dtype), a->ptr, a->cstride, a->scale, b->ptr, b->cstride, b->scale, y->ptr, y->cstride, a->n * a->h * a->w,
                                  (int)a->c, activation, 1.0f / y_scale);
    if (rc) { ln_tensor_release(y); return rc; }
    *out = y;
    return LN_OK;
}

}  // extern "C"
