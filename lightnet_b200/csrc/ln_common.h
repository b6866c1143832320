// Internal declarations shared by the translation units of liblightnet_b200.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../../include/lightnet_b200.h"

// cuTensorMapEncodeTiled is resolved at run time through cudaGetDriverEntryPoint so that the library
// has no link-time dependency on the driver library (it must load on a machine without a GPU).
typedef CUresult (*ln_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct ln_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string err;
    bool exact_epilogue = false;
    int nms_pool_entries = 0;  // capacity of one NMS candidate pool, 0 = automatic
    int64_t launches = 0;
    int sm_count = 0;
    std::multimap<size_t, void*> free_blocks;  // size-keyed cache of freed blocks; reuse is stream ordered
    std::map<void*, size_t> live_blocks;       // true size of every block handed out
    size_t pool_bytes = 0;                     // bytes held from the device: live + cached
    size_t cached_bytes = 0;
    int* d_status = nullptr;  // device status word written by kernels whose bounded waits give up
    int* h_status = nullptr;  // pinned mirror
    ln_encode_tiled_fn encode_tiled = nullptr;
    long long* debug_cycles = nullptr;  // when set (LN_DEBUG_CYCLES=1), the tensor-core convolution records role timings of CTA 0
    std::set<const void*> configured_kernels;  // kernels whose dynamic shared memory limit has been raised
    // ln_ctx_set_kernel_timing: the operator-level convolution brackets its main kernel with these events
    // pinned host staging for result read-backs (grown on demand by the entry points that may allocate)
    void* h_stage = nullptr;
    size_t h_stage_bytes = 0;
    bool time_kernels = false;
    cudaEvent_t ev_k0 = nullptr, ev_k1 = nullptr;
    bool ev_pending = false;
};

struct ln_tensor {
    ln_ctx* ctx = nullptr;
    int refcount = 1;
    int dtype = LN_F32;
    int64_t n = 0, c = 0, h = 0, w = 0;  // logical shape [batch, channels, height, width]
    void* ptr = nullptr;                 // first element of the view
    void* base = nullptr;                // pool block (nullptr for a view onto `parent`)
    size_t bytes = 0;
    ln_tensor* parent = nullptr;         // keeps the owner of a view alive
    int64_t cstride = 0;                 // 8-bit and binary16 NHWC tensors: bytes between consecutive pixels
    float scale = 1.0f;                  // 8-bit tensors: value = code * scale
    int64_t count() const { return n * c * h * w; }
};

struct ln_conv_weights {
    ln_ctx* ctx = nullptr;
    int dtype = LN_Q8;
    int64_t filters = 0, channels = 0, k = 0;
    int64_t fpad = 0, cpad = 0;     // filters padded to a multiple of 16 (>= 64 multiple of 64), channels to 32
    void* w = nullptr;              // [fpad][k][k][cpad] 8-bit codes
    float* wscale = nullptr;        // [fpad] per-filter scale (device)
    std::vector<float> h_wscale;    // host copy
    float max_l1 = 0.0f;            // max over filters of the sum of |code| (bounds the int8 accumulators)
    float max_scale = 0.0f;         // largest per-filter scale
    void* w_oihw = nullptr;         // [filters][channels][k][k] codes in the reference's weight order (SIMT path)
    // binary16 weights (dtype LN_F16): the f32 source is kept and packed by the first convolution that names kernel size and channels
    ln_tensor* src_f32 = nullptr;
    int64_t per_filter = 0;
};

int ln_fail(ln_ctx* ctx, int code, const char* fmt, ...);
int ln_image_preprocess_enqueue(ln_ctx* ctx, cudaStream_t stream, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths,
                                const int32_t* heights, int32_t count, int32_t mode, int32_t dst_w, int32_t dst_h, float* dst, void** staging,
                                size_t* staging_bytes);
int ln_image_preprocess_into(ln_ctx* ctx, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths, const int32_t* heights,
                             int32_t count, int32_t mode, int32_t dst_w, int32_t dst_h, float* dst);
void* ln_pool_alloc(ln_ctx* ctx, size_t bytes);
void ln_pool_free(ln_ctx* ctx, void* p, size_t bytes);
ln_tensor* ln_tensor_new(ln_ctx* ctx, int dtype, int64_t n, int64_t c, int64_t h, int64_t w);  // allocates storage
ln_tensor* ln_tensor_view_q(ln_tensor* parent, int64_t channel_offset, int64_t channels);      // channel slice of an NHWC tensor
ln_tensor* ln_tensor_view_batch(ln_tensor* parent, int64_t start, int64_t count);               // image range of an f32 NCHW tensor
inline int64_t ln_round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

#define LN_CUDA(ctx, call)                                                                                   \
    do {                                                                                                     \
        cudaError_t e__ = (call);                                                                            \
        if (e__ != cudaSuccess) return ln_fail((ctx), LN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

#define LN_LAUNCHED(ctx)                                                                                             \
    do {                                                                                                             \
        (ctx)->launches++;                                                                                           \
        cudaError_t e__ = cudaGetLastError();                                                                        \
        if (e__ != cudaSuccess) return ln_fail((ctx), LN_ERR_CUDA, "kernel launch failed at %s:%d: %s", __FILE__, __LINE__, \
                                               cudaGetErrorString(e__));                                             \
    } while (0)

// ---- device-side numerics shared by the kernels --------------------------------------------------

#ifdef __CUDACC__
// exp built only from IEEE-754 binary32 operations (fma where written): a CPU evaluating the same
// sequence gets the same bits.  Accuracy: a few ulp.
// f32::is_finite ? v : 0 (finite_or_zero of lightnet-layers/src/modern_yolo/cpu.rs:199)
__device__ __forceinline__ float ln_finite_or_zero(float v) { return (__float_as_uint(v) & 0x7F800000u) == 0x7F800000u ? 0.0f : v; }

__device__ __forceinline__ float ln_det_expf(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    float n = rintf(__fmul_rn(x, 1.44269502e+00f));
    float r = __fmaf_rn(n, -6.93145752e-01f, x);
    r = __fmaf_rn(n, -1.42860677e-06f, r);
    float p = 1.98412698e-04f;
    p = __fmaf_rn(p, r, 1.38888889e-03f);
    p = __fmaf_rn(p, r, 8.33333377e-03f);
    p = __fmaf_rn(p, r, 4.16666679e-02f);
    p = __fmaf_rn(p, r, 1.66666672e-01f);
    p = __fmaf_rn(p, r, 5.00000000e-01f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int e = (int)n;
    int e1 = e / 2, e2 = e - e1;
    float s1 = __int_as_float((e1 + 127) << 23), s2 = __int_as_float((e2 + 127) << 23);
    return __fmul_rn(__fmul_rn(p, s1), s2);
}
__device__ __forceinline__ float ln_det_sigmoid(float v) {
    // for v >= 17, exp(-v) < 2^-24 and 1 + exp(-v) rounds to 1: the quotient is exactly 1 (same bits as the full evaluation)
    if (v >= 17.0f) return 1.0f;
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, ln_det_expf(-v)));
}

__device__ __forceinline__ float ln_ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float ln_rcp_ftz(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Activation of the 8-bit epilogues.  EXACT: IEEE-only operations (bit-reproducible); otherwise the
// hardware ex2/rcp approximations (about 2 ulp each).
template <bool EXACT>
__device__ __forceinline__ float ln_epilogue_act(int act, float v) {
    switch (act) {
        case LN_ACT_LINEAR: return v;
        case LN_ACT_LEAKY: return fmaxf(v, __fmul_rn(0.1f, v));  // v>0 ? v : 0.1v
        case LN_ACT_RELU: return fmaxf(v, 0.0f);
        case LN_ACT_MISH: {
            if (EXACT) {
                if (v > 20.0f) return v;
                float e = ln_det_expf(v);
                float w = __fmul_rn(e, __fadd_rn(e, 2.0f));
                return __fmul_rn(v, __fdiv_rn(w, __fadd_rn(w, 2.0f)));
            } else {
                const float e = ln_ex2_ftz(fminf(v, 20.0f) * 1.44269504f);
                const float w = e * (e + 2.0f);
                return v * (w * ln_rcp_ftz(w + 2.0f));
            }
        }
        case LN_ACT_SWISH:
            if (EXACT) return __fdiv_rn(v, __fadd_rn(1.0f, ln_det_expf(-v)));
            return v * ln_rcp_ftz(1.0f + ln_ex2_ftz(fmaxf(v, -60.0f) * -1.44269504f));
        case LN_ACT_LOGISTIC:
            if (EXACT) return ln_det_sigmoid(v);
            return ln_rcp_ftz(1.0f + ln_ex2_ftz(fmaxf(v, -60.0f) * -1.44269504f));
    }
    return v;
}

// ---- packed-half epilogue (fast mode) ---------------------------------------------------------
// The fast int8 epilogue evaluates activation and requantisation two values at a time in binary16: the
// output has 8 bits, binary16 carries 11, and one packed instruction does the work of two.  The result can
// differ from the exact epilogue by one code (a few percent of the codes do).  `v` holds two pre-activation
// values; the return value holds, in the low byte of each half, the int8 code clamp(rne(act(v) * inv_s), +-127).
__device__ __forceinline__ __half2 ln_h2_ex2(__half2 x) {
    uint32_t xi = *reinterpret_cast<uint32_t*>(&x), yi;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(yi) : "r"(xi));
    return *reinterpret_cast<__half2*>(&yi);
}
// 1/d for both halves, d in [1, 32000]: bit-trick seed (12% error) and two Newton steps (0.02%), no conversion unit.
__device__ __forceinline__ __half2 ln_h2_rcp(__half2 d) {
    const uint32_t seed = 0x77987798u - *reinterpret_cast<uint32_t*>(&d);  // no borrow between halves for d in range
    __half2 r = *reinterpret_cast<const __half2*>(&seed);
    const __half2 two = __float2half2_rn(2.0f);
    r = __hmul2(r, __hfma2(__hneg2(d), r, two));
    r = __hmul2(r, __hfma2(__hneg2(d), r, two));
    return r;
}
template <int ACT>
__device__ __forceinline__ __half2 ln_h2_act(__half2 v) {
    if (ACT == LN_ACT_LEAKY) return __hmax2(v, __hmul2(v, __float2half2_rn(0.1f)));
    if (ACT == LN_ACT_RELU) return __hmax2(v, __float2half2_rn(0.0f));
    if (ACT == LN_ACT_MISH) {
        // v * w/(w+2), w = e^v (e^v + 2); the ratio is evaluated at min(v, 5) (it is 1 - 9e-5 there and rises to 1)
        const __half2 e = ln_h2_ex2(__hmul2(__hmin2(v, __float2half2_rn(5.0f)), __float2half2_rn(1.44269504f)));
        const __half2 w = __hfma2(e, e, __hadd2(e, e));
        return __hmul2(v, __hmul2(w, ln_h2_rcp(__hadd2(w, __float2half2_rn(2.0f)))));
    }
    if (ACT == LN_ACT_SWISH || ACT == LN_ACT_LOGISTIC) {
        // 1 / (1 + e^-v), with v clamped to >= -10 (the sigmoid is below 5e-5 there)
        const __half2 e = ln_h2_ex2(__hmul2(__hmax2(v, __float2half2_rn(-10.0f)), __float2half2_rn(-1.44269504f)));
        const __half2 s = ln_h2_rcp(__hadd2(e, __float2half2_rn(1.0f)));
        return ACT == LN_ACT_SWISH ? __hmul2(v, s) : s;
    }
    return v;
}
template <int ACT>
__device__ __forceinline__ uint32_t ln_h2_act_quant(float v0, float v1, __half2 inv_s) {
    // pre-activations beyond the binary16 range saturate to its largest finite value in the conversion itself (their codes saturate anyway)
    uint32_t vb;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(vb) : "f"(v1), "f"(v0));  // first source -> upper half
    const __half2 v = *reinterpret_cast<const __half2*>(&vb);
    __half2 t = __hmul2(ln_h2_act<ACT>(v), inv_s);
    t = __hmin2(__hmax2(t, __float2half2_rn(-127.0f)), __float2half2_rn(127.0f));
    t = __hadd2(t, __float2half2_rn(1536.0f));  // ulp is 1 in [1024, 2048): the low mantissa bits are rne(t)
    return *reinterpret_cast<uint32_t*>(&t);
}
// The same with the two pre-activations already in units of the output scale (t = v / s; the caller folds 1 / s into its
// per-filter multiplier and bias, so no multiply by 1 / s is left here).  `k` holds s * log2(e) in both halves: t * k is the
// exponent argument of the transcendental activations; `inv_s` is used by the logistic only.  Activations that are bounded
// below by a small multiple of s (mish >= -0.31, swish >= -0.28, relu, logistic) need no lower clamp as long as
// s >= 0.31 / 127, which the caller checks.
template <int ACT>
__device__ __forceinline__ uint32_t ln_h2_code(float t0, float t1, __half2 k, __half2 inv_s) {
    uint32_t tb;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(tb) : "f"(t1), "f"(t0));  // first source -> upper half
    const __half2 t = *reinterpret_cast<const __half2*>(&tb);
    const __half2 lo = __float2half2_rn(-127.0f);
    __half2 y;
    if (ACT == LN_ACT_LEAKY) y = __hmax2(__hmax2(t, __hmul2(t, __float2half2_rn(0.1f))), lo);
    else if (ACT == LN_ACT_RELU) y = __hmax2(t, __float2half2_rn(0.0f));
    else if (ACT == LN_ACT_MISH) {
        // t * w / (w + 2), w = e^v (e^v + 2), the ratio evaluated at min(v, 5)
        const __half2 e = ln_h2_ex2(__hmin2(__hmul2(t, k), __float2half2_rn(5.0f * 1.44269504f)));
        const __half2 w = __hmul2(e, __hadd2(e, __float2half2_rn(2.0f)));
        y = __hmul2(t, __hmul2(w, ln_h2_rcp(__hadd2(w, __float2half2_rn(2.0f)))));
    } else if (ACT == LN_ACT_SWISH || ACT == LN_ACT_LOGISTIC) {
        // 1 / (1 + e^-v) with v clamped to >= -10
        const __half2 e = ln_h2_ex2(__hmin2(__hmul2(t, __hneg2(k)), __float2half2_rn(10.0f * 1.44269504f)));
        const __half2 sg = ln_h2_rcp(__hadd2(e, __float2half2_rn(1.0f)));
        y = ACT == LN_ACT_SWISH ? __hmul2(t, sg) : __hmul2(sg, inv_s);
    } else y = __hmax2(t, lo);
    y = __hadd2(__hmin2(y, __float2half2_rn(127.0f)), __float2half2_rn(1536.0f));  // ulp is 1 in [1024, 2048): the low mantissa bits are rne(y)
    return *reinterpret_cast<uint32_t*>(&y);
}
// The activation alone for two pre-activations that are already in units of the output scale (see ln_h2_code): the value in
// those units, unrounded and unclamped.  Used where the conversion that follows saturates by itself (FP8 output).
template <int ACT>
__device__ __forceinline__ __half2 ln_h2_value(float t0, float t1, __half2 k, __half2 inv_s) {
    uint32_t tb;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(tb) : "f"(t1), "f"(t0));  // first source -> upper half
    const __half2 t = *reinterpret_cast<const __half2*>(&tb);
    if (ACT == LN_ACT_LEAKY) return __hmax2(t, __hmul2(t, __float2half2_rn(0.1f)));
    if (ACT == LN_ACT_RELU) return __hmax2(t, __float2half2_rn(0.0f));
    if (ACT == LN_ACT_MISH) {
        const __half2 e = ln_h2_ex2(__hmin2(__hmul2(t, k), __float2half2_rn(5.0f * 1.44269504f)));
        const __half2 w = __hmul2(e, __hadd2(e, __float2half2_rn(2.0f)));
        return __hmul2(t, __hmul2(w, ln_h2_rcp(__hadd2(w, __float2half2_rn(2.0f)))));
    }
    if (ACT == LN_ACT_SWISH || ACT == LN_ACT_LOGISTIC) {
        const __half2 e = ln_h2_ex2(__hmin2(__hmul2(t, __hneg2(k)), __float2half2_rn(10.0f * 1.44269504f)));
        const __half2 sg = ln_h2_rcp(__hadd2(e, __float2half2_rn(1.0f)));
        return ACT == LN_ACT_SWISH ? __hmul2(t, sg) : __hmul2(sg, inv_s);
    }
    return t;
}
// two binary16 values -> two E4M3 codes (round to nearest even, saturating to +-448), lower half in the lower byte
__device__ __forceinline__ uint32_t ln_h2_to_e4m3x2(__half2 v) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(d) : "r"(*reinterpret_cast<const uint32_t*>(&v)));
    return (uint32_t)d;
}
// {a.lo, a.hi, b.lo, b.hi} code bytes of two ln_h2_act_quant results -> one packed word
__device__ __forceinline__ uint32_t ln_h2_pack(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x6420); }

// f32 path activations (libm-accurate device functions)
__device__ __forceinline__ float ln_act_f32(int act, float v) {
    switch (act) {
        case LN_ACT_LINEAR: return v;
        case LN_ACT_LOGISTIC: return 1.0f / (1.0f + expf(-v));
        case LN_ACT_LEAKY: return v > 0.0f ? v : 0.1f * v;
        case LN_ACT_MISH: return v * tanhf(logf(1.0f + expf(v)));
        case LN_ACT_SWISH: return v / (1.0f + expf(-v));
        case LN_ACT_RELU: return fmaxf(v, 0.0f);
    }
    return v;
}

// int8 quantiser of the epilogues: rne(a * inv_s), clamped to +-127.
__device__ __forceinline__ int ln_quant_i8(float a, float inv_s) {
    float t = __fmul_rn(a, inv_s);
    t = fminf(fmaxf(t, -127.0f), 127.0f);  // NaN -> -127
    return __float2int_rn(t);
}
#endif
