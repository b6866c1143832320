// Launch plan of one reduced-precision convolution (tensor-core path and CUDA-core path).
#pragma once
#include <cstring>

#include "ln_common.h"

// operand type of the tensor-core convolution: int8 (int32 accumulate), FP8 E4M3 or binary16 (f32 accumulate).  The kernel and its
// planner count channels in BYTES per pixel (cpad, x_pixel_stride); binary16 callers pass two bytes per channel.
enum { LN_KIND_I8 = 0, LN_KIND_F8 = 1, LN_KIND_F16 = 2 };

// status word values written by kernels whose bounded waits gave up
enum {
    LN_STATUS_OK = 0,
    LN_STATUS_PRODUCER_TIMEOUT = 101,
    LN_STATUS_MMA_TIMEOUT = 102,
    LN_STATUS_EPILOGUE_TIMEOUT = 103
};

struct ln_conv_umma_params {
    CUtensorMap tmA[4];  // activations; stride-2 convolutions use one map per input parity class
    CUtensorMap tmB;     // weights as a [fpad][k*k*cpad] matrix
    int bk, bn, stages, nbuf;
    int subs;  // an accumulator tile is handed to the epilogue as `subs` units of bn / subs columns
    int b_resident;  // the weights of the (single) filter tile stay in shared memory for the whole kernel
    int small_acc;  // every accumulator is known to stay below 2^22 in magnitude
    int acc_shift;  // fast int8 epilogue: low accumulator bits dropped so that what is left stays below 2^22 (0 = none)
    int R, S, stride, pad;
    int cblocks, cpad;
    int OW, OH, N, F, fpad_used;
    int TW, TH, TN, log_tw, log_th;
    int tiles_w, tiles_h, tiles_n, tiles_f, num_tiles;
    int num_units;  // work units of the persistent loop (= num_tiles)
    // pipelines (1 or 2): producer / MMA-issuer pairs that take the CTA's tiles alternately, each with stages / pipes stages
    int pipes;
    unsigned long long magic_f, magic_w, magic_h;  // ceil(2^40 / tiles_*) for division-free tile decoding
    int act, out_kind;
    float inv_sy;
    const float2* mb;  // [fpad] {x_scale * w_scale[f], bias[f]}
    // [fpad / 2] float4 {m 2i, m 2i+1, b 2i, b 2i+1}, m = mult / s_y, b = bias / s_y - 1.5 * 2^23 * m: lets the fast epilogue take
    // the pre-activation, in units of the output scale, straight from the float whose bits are 0x4B400000 + accumulator
    // (= 1.5 * 2^23 + accumulator); null when accumulators can exceed 2^22
    const float2* mb_folded;
    float sy_log2e;  // output scale * log2(e): exponent argument per code unit (folded fast epilogue)
    int tab_bytes;   // bytes of the {multiplier, bias} table the epilogue warps copy to shared memory (all filter tiles)
    int out_esize;   // bytes per element of an LN_OUT_Q output (1, or 2 for binary16)
    void* out;
    long long out_pixel_stride;  // bytes between pixels of an 8-bit NHWC output
    // fused shortcut (null = none): out = quant((code * s_c + residual_code * s_res) * inv_sy2), code = the convolution's own int8 output
    const void* res;
    long long res_pixel_stride;
    float s_c, s_res, inv_sy2;
    // Pixel-group packing of 1x1 convolutions with few channels (pack > 1): an accumulator row is `pack` consecutive pixels,
    // its column j * f_real + f is filter f of the j-th of them (see ln_conv_umma_plan_build).
    int pack, f_real;
    // Row-shifted boxes for 3x3 stride-1 convolutions (halo = 1): per channel block the producer loads three boxes of
    // TW x (TH + 2) pixels, shifted by 0, 1, 2 pixels in x; the tap (r, s) reads box s from row r on.  a_stages such sets
    // are in flight; the weight tiles have their own ring (`stages`) unless they are resident.
    int halo, a_stages, box_bytes;
    int* status;
    long long* debug;  // optional: role timing of CTA 0 (32 counters), null = off
};

struct ln_conv_umma_plan {
    ln_conv_umma_params p;
    float2* mb = nullptr;
    // device storage the plan owns when it packs pixel groups: the block-diagonal weight matrix and its {mult, bias} pairs
    void* aux_w = nullptr;
    float2* aux_mb = nullptr;
    float2* aux_mbf = nullptr;  // the folded table of mb_folded
    size_t aux_w_bytes = 0, aux_mb_bytes = 0, aux_mbf_bytes = 0;
    size_t smem = 0;
    int grid = 0;
    int kind = LN_KIND_I8;
};

// Geometry of one convolution as the planners see it.
struct ln_conv_geom {
    int kind = LN_KIND_I8;
    const void* x = nullptr;      // NHWC 8-bit input view
    long long x_pixel_stride = 0; // bytes
    int N = 0, H = 0, W = 0, C = 0, cpad = 0;
    const void* w = nullptr;      // [fpad][k][k][cpad]
    int F = 0, fpad = 0, k = 1, stride = 1, pad = 0;
    // grouped convolution (CUDA-core kernels only): filter f reads the C / groups channels of group f / (F / groups); the weights
    // are [fpad][k][k][w_cpad] with C / groups real channels per row (w_cpad = 0 means cpad, the ungrouped layout)
    int groups = 1, w_cpad = 0;
    int OH = 0, OW = 0;
    int act = 0, out_kind = 0;
    float inv_sy = 1.0f;
    bool small_acc = false;  // 127 * max over filters of sum|w code| < 2^22
    // Larger accumulators in the fast epilogue: this many low bits are dropped first (see ln_acc_shift); 0 = none, -1 = not allowed
    int acc_shift = 0;
    // x is the 2x2 space-to-depth image of the 32-channel input ([H/2][W/2][4 * 32], sub-pixel (y & 1) * 2 + (x & 1) major):
    // the 3x3 stride-2 pad-1 convolution described here is then run as a 2x2 stride-1 one over 128-byte rows
    bool s2d_input = false;
    void* out = nullptr;
    long long out_pixel_stride = 0;
    // fused linear shortcut that follows the convolution (see ln_conv_umma_params)
    const void* res = nullptr;
    long long res_pixel_stride = 0;
    float s_c = 1.0f, s_res = 1.0f, inv_sy2 = 1.0f;
};

inline int ln_conv_choose_bn(int64_t F) {
    int bn = 32;
    int64_t best = -1;
    const int cand[4] = {32, 64, 128, 256};
    for (int c : cand) {
        int64_t fp = ln_round_up(F, c);
        if (best < 0 || fp <= best) { best = fp; bn = c; }
    }
    return bn;
}

bool ln_conv_umma_supported(int64_t channels_padded, int64_t k, int64_t stride_x, int64_t stride_y, int64_t dilation, int64_t groups,
                            int64_t in_w, int64_t in_h);
// plan->mb must point at device storage for fpad float2 before the build.
int ln_conv_umma_plan_build(ln_ctx* ctx, ln_conv_umma_plan* plan, const ln_conv_geom& g);
int ln_conv_umma_make_mb(ln_ctx* ctx, const float* wscale_dev, const float* bias_dev, float x_scale, int F, int fpad, float2* mb_dev);
int ln_conv_umma_launch(ln_ctx* ctx, const ln_conv_umma_plan* plan);
// Returns the storage a plan owns (aux_w / aux_mb) to the ctx pool.
void ln_conv_umma_plan_release(ln_ctx* ctx, ln_conv_umma_plan* plan);

// CUDA-core int8 / FP8 convolution for shapes the tensor-core kernel does not take (any C, stride, padding).
// Weights in the reference's [F][C][k][k] order.
int ln_conv_simt_launch(ln_ctx* ctx, const ln_conv_geom& g, const void* w_oihw, const float2* mb);

// First layer: f32 NCHW image in, quantise on the fly, 8-bit NHWC out (C <= 4).
int ln_conv_stem_launch(ln_ctx* ctx, int kind, const float* x_nchw, float inv_sx, int N, int C, int H, int W, const void* w_oihw,
                        const float2* mb, int F, int k, int stride, int pad, int OH, int OW, int act, float inv_sy, void* out,
                        long long out_pixel_stride, int s2d_out = 0);

// Reads the device status word; returns LN_OK or LN_ERR_TIMEOUT (and clears the word).
int ln_check_status(ln_ctx* ctx, const char* where);

// The fast int8 epilogue converts an accumulator to binary32 by adding it to the bits of 1.5 * 2^23, which needs |accumulator| < 2^22.
// Where the bound 127 * max_l1 (max_l1 = largest sum of |weight code| of a filter) is larger, the low `shift` bits are dropped
// first; that moves a pre-activation by at most 2^(shift - 1) accumulator units (the mean is put back into the bias), i.e.
// 2^(shift - 1) * s_x * s_w / s_y output codes, which has to stay at or under 0.02 of a code for every filter.
// Returns the shift (0 when none is needed) or -1 when no shift up to 8 bits meets both conditions.
inline int ln_acc_shift(float max_l1, float x_scale, float max_w_scale, float inv_sy) {
    const float bound = 127.0f * max_l1;
    for (int sh = 0; sh <= 8; ++sh) {
        if (bound >= 4194304.0f * (float)(1 << sh)) continue;
        if (sh == 0) return 0;
        return (float)(1 << (sh - 1)) * x_scale * max_w_scale * inv_sy <= 0.02f ? sh : -1;
    }
    return -1;
}
