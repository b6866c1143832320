/*
 * lightnet_b200.h -- C ABI of the B200 (sm_100a) backend for lightnet's detector
 * inference path: [convolutional] forward + route/shortcut/upsample/maxpool glue +
 * [yolo] decode + per-class greedy NMS.
 *
 * The entry points map one to one onto the methods a Rust backend crate implements
 * for the lightnet runtime (trait F32TensorOpsBackend, src/lightnet-cuda/src/lib.rs:460,
 * and a reduced-precision trait shaped like F16TensorOpsBackend, lib.rs:6295).  Each
 * declaration cites the trait method it stands behind.  All shapes are
 * [batch, channels, height, width] as in runtime/weights_io.rs:758
 * (tensor_backend_shape); host f32 data is planar NCHW (lightnet-model model.rs:98).
 *
 * Conventions
 *   - every function returns an int32 status: LN_OK or an LN_ERR_* code; nothing aborts
 *     or throws across the boundary; ln_last_error(ctx) gives the message
 *     (maps to `Result<_, Self::Error>`, Error: Display)
 *   - tensors are opaque ref-counted handles; every op returns a NEW tensor and never
 *     mutates its inputs (maps to `type Tensor: Clone`; retain = Clone, release = Drop)
 *   - one ctx = one device + one stream; all work is stream ordered; a ctx is
 *     thread-compatible, not thread-safe (the runtime's executor is !Sync:
 *     runtime/gpu_types.rs:227-244).  Multi-GPU = one ctx per device.
 *   - there is no CPU fallback: without a usable CUDA device ln_ctx_create fails.
 */
#ifndef LIGHTNET_B200_H
#define LIGHTNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ln_ctx ln_ctx;
typedef struct ln_tensor ln_tensor;
typedef struct ln_conv_weights ln_conv_weights;
typedef struct ln_net ln_net;

enum ln_status {
    LN_OK = 0,
    LN_ERR_SHAPE = 1,       /* OxideError::Shape analogue (lightnet-cuda-oxide/src/lib.rs:177-192) */
    LN_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed */
    LN_ERR_TIMEOUT = 3,     /* a bounded device-side wait gave up; the context stays usable */
    LN_ERR_UNSUPPORTED = 4, /* OxideError::NotImplemented analogue */
    LN_ERR_ARG = 5,
    LN_ERR_PARSE = 6
};

/* F32ActivationKind (lightnet-cuda/src/lib.rs:23-55), hot-path subset. */
enum ln_activation { LN_ACT_LINEAR = 0, LN_ACT_LOGISTIC = 1, LN_ACT_LEAKY = 2, LN_ACT_MISH = 3, LN_ACT_SWISH = 4, LN_ACT_RELU = 5 };

enum ln_dtype { LN_F32 = 0, LN_Q8 = 1, LN_I32 = 2, LN_F8 = 3, LN_F16 = 4 };

/* What a reduced-precision convolution writes. */
enum ln_conv_out {
    LN_OUT_Q = 0,   /* same 8-bit storage type as the input, requantised with y_scale */
    LN_OUT_F32 = 1, /* f32 NCHW: the convolution feeding a detection head (ConvPrecision::NoLowPrecision policy,
                       lightnet-cuda/src/lib.rs:161, runtime/types.rs:146-170) */
    LN_OUT_ACC = 2  /* raw int32 accumulators, NCHW (parity checks only; int8 inputs only) */
};

/* ---- context ------------------------------------------------------------------- */
/* OxideBackend::with_device (lightnet-cuda-oxide/src/lib.rs:643) */
int32_t ln_ctx_create(int32_t device, ln_ctx** out);
int32_t ln_ctx_destroy(ln_ctx* ctx);
const char* ln_last_error(ln_ctx* ctx); /* ctx may be NULL: message of the last failed create */
int32_t ln_sync(ln_ctx* ctx);
/* The ctx's cudaStream_t, for callers that time with CUDA events. */
void* ln_ctx_stream(ln_ctx* ctx);
/* 1 = activation epilogues use only IEEE-exact operations (bit-reproducible on a CPU), 0 = fast hardware
   approximations (default).  Affects mish / swish / logistic in reduced-precision convolutions. */
int32_t ln_ctx_set_exact_epilogue(ln_ctx* ctx, int32_t on);
/* Tuning knob of ln_yolo_decode_nms (no counterpart in the reference): capacity, in candidates per image, of the
   compact pool the NMS selection works in.  0 (default) = automatic.  A small pool costs extra passes over the head
   tensors when very many candidates tie; the records do not depend on it. */
int32_t ln_ctx_set_nms_pool_entries(ln_ctx* ctx, int64_t entries);
/* Measurement aid (no counterpart in the reference): while on, ln_conv2d_bias_act_q brackets its convolution kernel with
   CUDA events on the ctx stream; ln_ctx_last_kernel_ms returns the duration of the most recent one. */
int32_t ln_ctx_set_kernel_timing(ln_ctx* ctx, int32_t on);
int32_t ln_ctx_last_kernel_ms(ln_ctx* ctx, float* ms);
/* Number of kernels this library has launched on the ctx since creation. */
int64_t ln_ctx_launch_count(ln_ctx* ctx);

/* ---- f32 tensors: F32TensorOpsBackend ---------------------------------------------- */
/* upload_f32 / zeros_f32 / download_f32 / tensor_shape (lib.rs:464-469) */
int32_t ln_tensor_upload_f32(ln_ctx* ctx, const int64_t shape[4], const float* host, ln_tensor** out);
int32_t ln_tensor_zeros_f32(ln_ctx* ctx, const int64_t shape[4], ln_tensor** out);
int32_t ln_tensor_download_f32(ln_ctx* ctx, const ln_tensor* t, float* host, int64_t count);
int32_t ln_tensor_shape(const ln_tensor* t, int64_t shape[4]);
int32_t ln_tensor_dtype(const ln_tensor* t);
int32_t ln_tensor_retain(ln_tensor* t);
int32_t ln_tensor_release(ln_tensor* t);

/* conv2d_f32 (lib.rs:1776); weights are f32 [filters, C/groups, k, k] */
int32_t ln_conv2d_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* weights, const int64_t output_shape[4],
                      int64_t input_channels, int64_t input_height, int64_t input_width, int64_t filters,
                      int64_t kernel_size, int64_t stride_x, int64_t stride_y, int64_t dilation, int64_t padding,
                      int64_t groups, ln_tensor** out);
/* bias_add_f32 (lib.rs:477), activation_f32 (lib.rs:500), bias_activation_f32 (lib.rs:546) */
int32_t ln_bias_add_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* bias, int64_t channels, int64_t channel_stride,
                        ln_tensor** out);
int32_t ln_activation_f32(ln_ctx* ctx, const ln_tensor* x, int32_t activation, ln_tensor** out);
int32_t ln_bias_activation_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* bias, int64_t channels,
                               int64_t channel_stride, int32_t activation, ln_tensor** out);
/* shortcut_add_f32 (lib.rs:803), shortcut_fit_f32 (lib.rs:4041) */
int32_t ln_shortcut_add_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* y, ln_tensor** out);
int32_t ln_shortcut_fit_f32(ln_ctx* ctx, const ln_tensor* x, int64_t batch, const int64_t output_shape[4], ln_tensor** out);
/* route_concat_f32 (lib.rs:937) */
int32_t ln_route_concat_f32(ln_ctx* ctx, const ln_tensor* const* inputs, int32_t n_inputs,
                            const int64_t* input_channel_offsets, const int64_t* input_channels,
                            const int64_t* input_total_channels, const int64_t output_shape[4], int64_t channel_stride,
                            ln_tensor** out);
/* maxpool_f32 (lib.rs:2036), upsample_f32 (lib.rs:3963) */
int32_t ln_maxpool_f32(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels,
                       int64_t input_height, int64_t input_width, int64_t size, int64_t stride_x, int64_t stride_y,
                       int64_t padding, ln_tensor** out);
int32_t ln_upsample_f32(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels,
                        int64_t input_height, int64_t input_width, int64_t stride, float scale, int32_t reverse,
                        ln_tensor** out);
/* channel_scale_f32 (lib.rs:485): out[i] = x[i] * scale[(i / channel_stride) % channels] */
int32_t ln_channel_scale_f32(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* scale, int64_t channels, int64_t channel_stride,
                             ln_tensor** out);
/* region_forward_f32 (lib.rs:5090; host_ops.rs:73-116): the [region] head's forward.  x is [batch, anchors * entries, h, w]; the result
   holds the same values in spatial-major order [batch, h * w, anchors, entries] with the objectness (entry 4) through the logistic and,
   when softmax_classes != 0, a softmax over entries 5 .. 5 + classes. */
int32_t ln_region_forward_f32(ln_ctx* ctx, const ln_tensor* x, int64_t anchors, int64_t entries, int64_t classes, int32_t softmax_classes,
                              ln_tensor** out);
/* yolo_activate_f32 (lib.rs:4951): classic [yolo] head activation in place order: logistic on every entry but w / h (none with
   new_coords), then x, y become v * scale_xy - 0.5 * (scale_xy - 1). */
int32_t ln_yolo_activate_f32(ln_ctx* ctx, const ln_tensor* x, int64_t classes, float scale_xy, int32_t new_coords, ln_tensor** out);
/* batchnorm_fold_f32 (lib.rs:6208): returns (scale, bias') */
int32_t ln_batchnorm_fold_f32(ln_ctx* ctx, const ln_tensor* gamma, const ln_tensor* mean, const ln_tensor* variance,
                              const ln_tensor* bias, float eps, ln_tensor** scale_out, ln_tensor** bias_out);

/* ---- 8-bit tensors (int8 / FP8 E4M3): twins of F16TensorOpsBackend ------------------ */
/* Storage is NHWC, channels padded to a multiple of 32, one f32 scale per tensor (value = q * scale).
   upload_f16 (lib.rs:6300) analogue: quantise host f32 NCHW data with `scale` (int8: rne, clamp +-127;
   FP8: cvt.rn.satfinite e4m3). */
int32_t ln_tensor_upload_q(ln_ctx* ctx, const int64_t shape[4], const float* host, float scale, int32_t dtype, ln_tensor** out);
/* Raw 8-bit codes of a Q8 / F8 tensor in NCHW order (parity checks), and its scale. */
int32_t ln_tensor_download_q(ln_ctx* ctx, const ln_tensor* t, void* host_codes, int64_t count, float* scale);
/* Raw 8-bit codes (NCHW order) -> device tensor with the given scale. */
int32_t ln_tensor_upload_codes(ln_ctx* ctx, const int64_t shape[4], const void* host_codes, float scale, int32_t dtype,
                               ln_tensor** out);
/* int32 accumulators of an LN_OUT_ACC convolution, NCHW. */
int32_t ln_tensor_download_i32(ln_ctx* ctx, const ln_tensor* t, int32_t* host, int64_t count);
/* widen_f16 (lib.rs:6304) / narrow_f32 (lib.rs:6308) analogues, on device. */
int32_t ln_tensor_widen_q(ln_ctx* ctx, const ln_tensor* t, ln_tensor** out_f32);
int32_t ln_tensor_narrow_f32(ln_ctx* ctx, const ln_tensor* t, float scale, int32_t dtype, ln_tensor** out_q);
float ln_tensor_scale(const ln_tensor* t);

/* conv_weights_f16 (lib.rs:6311) analogue: f32 [filters, per_filter = C*k*k] BN-folded weights ->
   the backend's GEMM operand ([filters][k][k][C] 8-bit, channels padded) plus per-filter scales
   (int8: s = max|w|/127 per filter; FP8: s = max|w|/448 per filter). */
int32_t ln_conv_weights_q(ln_ctx* ctx, const ln_tensor* weights_f32, int64_t filters, int64_t channels, int64_t kernel_size,
                          int32_t dtype, ln_conv_weights** out);
int32_t ln_conv_weights_release(ln_conv_weights* w);
/* conv2d_bias_act_f16 (lib.rs:6342) analogue:
     int8: acc = sum(xq*wq) (int32);  v = fma(float(acc), x.scale*w.scale[f], bias[f]);  a = act(v)
     FP8 : acc = sum(xq*wq) (f32);    v = fma(acc,        x.scale*w.scale[f], bias[f]);  a = act(v)
   LN_OUT_Q stores quantise(a / y_scale); LN_OUT_F32 stores a; LN_OUT_ACC stores acc.
   groups must be 1 and dilation 1 (all detector cfgs on the path). */
int32_t ln_conv2d_bias_act_q(ln_ctx* ctx, const ln_tensor* x, const ln_conv_weights* weights, const ln_tensor* bias,
                             const int64_t output_shape[4], int64_t channels, int64_t input_height, int64_t input_width,
                             int64_t filters, int64_t kernel_size, int64_t stride_x, int64_t stride_y, int64_t dilation,
                             int64_t padding, int64_t groups, int32_t activation, float y_scale, int32_t out_kind,
                             ln_tensor** out);
/* maxpool_f16 (lib.rs:6384), upsample_f16 (lib.rs:6405), route_concat_f16 (lib.rs:6417),
   shortcut_add_act_f16 (lib.rs:6502) analogues.  Max-pool, up-sample and route keep the codes (route inputs must share one
   scale; a forward up-sample multiplies the tensor scale by `scale`); a reverse up-sample stores the mean code of each
   stride x stride block and carries scale * stride^2 in the tensor scale; shortcut requantises act(a*sa + b*sb) with y_scale. */
int32_t ln_maxpool_q(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height,
                     int64_t input_width, int64_t size, int64_t stride_x, int64_t stride_y, int64_t padding, ln_tensor** out);
int32_t ln_upsample_q(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height,
                      int64_t input_width, int64_t stride, float scale, int32_t reverse, ln_tensor** out);
int32_t ln_route_concat_q(ln_ctx* ctx, const ln_tensor* const* inputs, int32_t n_inputs, const int64_t* input_channel_offsets,
                          const int64_t* input_channels, const int64_t* input_total_channels, const int64_t output_shape[4],
                          int64_t channel_stride, ln_tensor** out);
int32_t ln_shortcut_add_act_q(ln_ctx* ctx, const ln_tensor* a, const ln_tensor* b, int32_t activation, float y_scale,
                              ln_tensor** out);
/* shortcut_fit_f16 (lib.rs:6494) analogue: flat per-sample crop / zero-pad of a mismatched shortcut source, on the codes (the scale is kept). */
int32_t ln_shortcut_fit_q(ln_ctx* ctx, const ln_tensor* x, int64_t batch, const int64_t output_shape[4], ln_tensor** out);

/* ---- binary16 storage: trait F16TensorOpsBackend (lib.rs:6295-6629) ------------------------ */
/* The twin that forward_compact_f16 (lightnet-runtime/src/runtime/gpu_f16.rs:21) drives, method for method.  TensorF16 is an
   ln_tensor of dtype LN_F16 (storage backend-defined: NHWC, channels padded to 32); values are rounded once to binary16 (nearest
   even, overflow stays infinite); convolutions run tcgen05.mma kind::f16 with binary32 accumulation.
   upload_f16 (lib.rs:6300), download_f16 (:6302, widened to f32 NCHW), widen_f16 (:6304), narrow_f32 (:6308). */
int32_t ln_tensor_upload_f16(ln_ctx* ctx, const int64_t shape[4], const float* host, ln_tensor** out);
int32_t ln_tensor_download_f16(ln_ctx* ctx, const ln_tensor* t, float* host, int64_t count);
int32_t ln_tensor_widen_f16(ln_ctx* ctx, const ln_tensor* t, ln_tensor** out_f32);
int32_t ln_tensor_narrow_f16(ln_ctx* ctx, const ln_tensor* t_f32, ln_tensor** out_f16);
/* conv_weights_f16 (lib.rs:6311): f32 [filters, per_filter] BN-folded weights -> the backend's GEMM operand.  Released with
   ln_conv_weights_release. */
int32_t ln_conv_weights_f16(ln_ctx* ctx, const ln_tensor* weights_f32, int64_t filters, int64_t per_filter, ln_conv_weights** out);
/* conv2d_bias_act_f16 (lib.rs:6342): f16(activation(conv(x, weights) + bias)), bias f32 [filters].  groups = 1, dilation = 1 and
   stride_x = stride_y in {1, 2} run on the tensor cores; every other geometry runs a CUDA-core kernel with the same arithmetic.
   (`weights` is not const: the operand layout is built by the first call that names the geometry.) */
int32_t ln_conv2d_bias_act_f16(ln_ctx* ctx, const ln_tensor* x, ln_conv_weights* weights, const ln_tensor* bias,
                               const int64_t output_shape[4], int64_t channels, int64_t input_height, int64_t input_width,
                               int64_t filters, int64_t size, int64_t stride_x, int64_t stride_y, int64_t dilation, int64_t padding,
                               int64_t groups, int32_t activation, ln_tensor** out);
/* maxpool_f16 (lib.rs:6384), upsample_f16 (:6405; reverse != 0 sums stride x stride blocks), route_concat_f16 (:6417),
   shortcut_fit_f16 (:6494), shortcut_add_act_f16 (:6502), channel_affine_act_f16 (:6619; scale may be NULL). */
int32_t ln_maxpool_f16(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height,
                       int64_t input_width, int64_t size, int64_t stride_x, int64_t stride_y, int64_t padding, ln_tensor** out);
int32_t ln_upsample_f16(ln_ctx* ctx, const ln_tensor* x, const int64_t output_shape[4], int64_t channels, int64_t input_height,
                        int64_t input_width, int64_t stride, float scale, int32_t reverse, ln_tensor** out);
int32_t ln_route_concat_f16(ln_ctx* ctx, const ln_tensor* const* inputs, int32_t n_inputs, const int64_t* input_channel_offsets,
                            const int64_t* input_channels, const int64_t* input_total_channels, const int64_t output_shape[4],
                            int64_t channel_stride, ln_tensor** out);
int32_t ln_shortcut_fit_f16(ln_ctx* ctx, const ln_tensor* x, int64_t batch, const int64_t output_shape[4], ln_tensor** out);
int32_t ln_shortcut_add_act_f16(ln_ctx* ctx, const ln_tensor* a, const ln_tensor* b, int32_t activation, ln_tensor** out);
int32_t ln_channel_affine_act_f16(ln_ctx* ctx, const ln_tensor* x, const ln_tensor* scale, const ln_tensor* bias, int64_t channels,
                                  int64_t channel_stride, int32_t activation, ln_tensor** out);

/* ---- [yolo] decode + NMS on the device ---------------------------------------------- */
/* Optional device path for decode_network_detections (lightnet-train/src/detect.rs:113-244): the Rust shim
   returns Ok(None) when this is absent (the idiom of yolo_loss_f32, lightnet-cuda/src/lib.rs:4918), so detect.rs
   and the CLI stay unchanged.  Semantics: decode_yolo_head (detect.rs:934-1016) over every head in order,
   stable sort by confidence (detect.rs:107), greedy per-class NMS (apply_nms, detect.rs:1449-1484, on the
   sorted list), records in confidence-descending order; top_k > 0 truncates the result (extension).
   The IoU>1.0 pre-pass of detect.rs:127-128 is not run (it can only fire for coincident boxes). */
typedef struct ln_yolo_head {
    const ln_tensor* raw;  /* f32 [batch, n_anchor*(5+classes), gh, gw] raw head (YoloHeadOutput, runtime/types.rs:107) */
    int32_t classes;
    int32_t n_anchor;
    float anchors[2 * 8];  /* (w,h) per masked anchor, already selected through `mask` (detection_geometry.rs:100) */
    float scale_x_y;
    int32_t new_coords;
    /* 0 = [yolo] / [gaussian_yolo] (the fields above); 1 = an activated [yolox] head (classes + 5 channels: cxcywh logits,
       objectness, classes; box by decode_yolox_box, lightnet-layers/src/modern_yolo/cpu.rs:461, score objectness * class);
       2 = a [ppyoloe] / [yolonas] head after ln_modern_yolo_predecode_f32 (final box, objectness, classes; score
       max(class, objectness * class), lightnet-train/src/detect.rs:1158-1162).  Kinds 1 and 2 take n_anchor = 1, ignore
       anchors / scale_x_y / new_coords, and expect the probabilities ln_modern_yolo_forward_f32 produces (in [0, 1]). */
    int32_t kind;
} ln_yolo_head;

typedef struct ln_detection { /* Detection (detect.rs:21-27): bbox centre/size in image pixels */
    float class_id, confidence, objectness, x, y, w, h;
} ln_detection;

typedef struct ln_detect_options { /* DetectionOptions (detect.rs:47-61) + top_k */
    float confidence_threshold;
    float nms_threshold;
    int32_t letterbox;
    int32_t top_k;        /* 0 = unlimited */
    int32_t max_per_image; /* capacity of the caller's record array per image */
} ln_detect_options;

/* records_host: [batch][max_per_image] ln_detection; counts_host: [batch] kept count (clamped to max_per_image).
   image_w/image_h: per image original size (batch entries). */
int32_t ln_yolo_decode_nms(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t net_w, int32_t net_h,
                           const int32_t* image_w, const int32_t* image_h, const ln_detect_options* opts,
                           ln_detection* records_host, int32_t* counts_host);
/* Same result as ln_yolo_decode_nms, for callers that must not allocate device memory.  (No counterpart in the
   reference: its decode and NMS run on the host.)  Some hosts of this library cannot call cudaMalloc while they
   serve requests -- a serving loop that has promised its memory budget to other tenants at start-up, a process whose
   allocator is frozen after initialisation, a thread that may not take the device-wide synchronisation cudaMalloc
   and cudaFree imply.  This entry point therefore keeps its working memory in a fixed 64 MiB array that belongs to
   the loaded library (every GPU that loads the library holds those 64 MiB until the process ends) and calls no
   cudaMalloc, cudaFree or other allocating routine; the caller still owns and passes the head tensors and the two
   result arrays.
   Limits and rules:
     - a call whose working set (it grows with batch x grid cells x anchors x classes, and with max_per_image) does
       not fit in the 64 MiB is refused with LN_ERR_UNSUPPORTED and a message that names both sizes; nothing is
       truncated.  For scale: three YOLOv4-608 heads with 80 classes fit for batches up to 4 (8 bytes for every
       (cell, anchor, class) slot of an image, 1.82 million of them at that size);
     - the first call on each device looks up the device address of the array; make that first call during set-up,
       before any stream capture begins;
     - all calls on a device share the one array, which still holds what the previous call left; the parts that must
       start at zero are cleared on entry.  Two calls that overlap in time on the same GPU (two contexts, two
       threads) race on it: serialise them. */
int32_t ln_yolo_decode_nms_noalloc(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t net_w, int32_t net_h,
                                   const int32_t* image_w, const int32_t* image_h, const ln_detect_options* opts,
                                   ln_detection* records_host, int32_t* counts_host);
/* Decode only: candidates of one image in emission order (parity with decode_yolo_head). */
int32_t ln_yolo_decode_only(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t image_index, int32_t net_w,
                            int32_t net_h, int32_t image_w, int32_t image_h, float confidence_threshold, int32_t letterbox,
                            ln_detection* records_host, int64_t capacity, int64_t* count);

/* ---- image pre-processing: the step in front of the network ---------------------------- */
/* PlanarRgbImage::{from_interleaved_rgb_u8, letterbox, resize, resize_linear_exact} (lightnet-runtime/src/image.rs:57, 203,
   95, 157) for a batch: `count` interleaved 8-bit RGB images of sizes widths[i] x heights[i], image i starting at
   pixels_host + offsets[i], become one f32 [count, 3, dst_h, dst_w] tensor.  Bit-identical to the reference's CPU code. */
#define LN_PRE_LETTERBOX 0    /* Darknet float resize to fit inside, 0.5 padding, offsets (dst - new) / 2 */
#define LN_PRE_RESIZE 1       /* Darknet float resize to exactly dst_w x dst_h (align-corners bilinear) */
#define LN_PRE_RESIZE_EXACT 2 /* OpenCV INTER_LINEAR_EXACT on the bytes, then byte / 255 */
int32_t ln_image_preprocess_u8(ln_ctx* ctx, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths,
                               const int32_t* heights, int32_t count, int32_t mode, int32_t dst_w, int32_t dst_h, ln_tensor** out);

/* ---- whole network: GpuExecutableNetwork<B> ------------------------------------------ */
/* GpuExecutableNetwork::new (runtime/gpu_state.rs:8) from cfg text; `batch` > 0 overrides [net] batch
   (Network::with_batch, model.rs:3256).  precision: LN_F32 (trait-faithful f32 NCHW path), LN_F16 (the operator sequence of
   forward_compact_f16 over the binary16 twin), LN_Q8 or LN_F8. */
int32_t ln_net_create(ln_ctx* ctx, const char* cfg_text, int32_t batch, int32_t precision, ln_net** out);
int32_t ln_net_destroy(ln_net* net);
int32_t ln_net_num_layers(const ln_net* net);
/* info[20]: kind(0 conv,1 maxpool,2 route,3 shortcut,4 upsample,5 yolo), in w,h,c,b, out w,h,c,b,
   filters,size,stride_x,stride_y,padding,batch_normalize,activation,groups,dilation, two reserved (0) */
int32_t ln_net_layer_info(const ln_net* net, int32_t layer, int32_t info[20]);
int64_t ln_net_weight_count(const ln_net* net);
/* load_weights_file payload (runtime/weights_io.rs:227-235): per conv biases, [scales, mean, variance], weights. */
int32_t ln_net_load_weights(ln_net* net, const float* blob, int64_t count);
/* Darknet .weights file with header (runtime/weights_io.rs:911-928). */
int32_t ln_net_load_weights_file(ln_net* net, const char* path);
/* One f32 forward of `input` (host NCHW, net batch) recording amax of every layer output, then per-tensor
   scales (amax/127 or amax/448; tensors joined by route/maxpool/upsample share one).  Needed before an
   8-bit forward unless ln_net_set_scales is used. */
int32_t ln_net_calibrate(ln_net* net, const float* input_host);
/* scales[num_layers+1]: [0] network input, [1+i] output of layer i. */
int32_t ln_net_get_scales(const ln_net* net, float* scales, int32_t count);
int32_t ln_net_set_scales(ln_net* net, const float* scales, int32_t count);
/* Layers of the batch run `micro_batch` images at a time so that activations stay in L2 (0 = whole batch).  The two part
   networks of the host-input pipeline (ln_net_set_host_pipeline) always run their part whole. */
int32_t ln_net_set_micro_batch(ln_net* net, int32_t micro_batch);
/* forward_compact (runtime/gpu_forward_compact.rs:8): host f32 NCHW input -> heads resident on the device. */
int32_t ln_net_forward(ln_net* net, const float* input_host);
/* Same with the input already on the device (f32 NCHW tensor of the net's input shape). */
int32_t ln_net_forward_device(ln_net* net, const ln_tensor* input);
int32_t ln_net_num_heads(const ln_net* net);
/* Head tensor (f32 NCHW raw logits) of the last forward; retained for the caller. */
int32_t ln_net_head(ln_net* net, int32_t head_index, ln_tensor** out);
/* Output of layer `layer` from the last forward (whole-batch forwards with micro_batch = 0 only). */
int32_t ln_net_layer_output(ln_net* net, int32_t layer, ln_tensor** out);
/* forward + device decode + NMS; what `lightnet-rs detect-image` does per batch (lightnet-cli/src/main.rs:249-459). */
int32_t ln_net_detect(ln_net* net, const float* input_host, const int32_t* image_w, const int32_t* image_h,
                      const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host);
int32_t ln_net_detect_device(ln_net* net, const ln_tensor* input, const int32_t* image_w, const int32_t* image_h,
                             const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host);
/* The same work as ln_net_detect split in two calls so that a caller with a stream of batches overlaps the upload of the next
   batch with the layers of the current one (what a serving loop over GpuExecutableNetwork::forward_compact,
   lightnet-runtime/src/runtime/gpu_forward_compact.rs:8, does with a second input tensor).  ln_net_submit enqueues the
   host-to-device copy of one f32 NCHW batch on the network's copy stream and returns at once; at most two batches may be in
   flight, and `input_host` must stay unchanged until the matching ln_net_collect returns (pinned memory for a copy that really
   is asynchronous).  ln_net_collect runs the oldest submitted batch (layers, decode, NMS) and returns its records like
   ln_net_detect.  LN_ERR_ARG when a third batch is submitted or nothing is left to collect. */
int32_t ln_net_submit(ln_net* net, const float* input_host);
/* ln_net_submit for a batch of 8-bit RGB images (the arguments of ln_image_preprocess_u8): the upload of the pixels and the
   resize to the network's input run on the copy stream, under the layers of the batch submitted before.  `pixels_host` must stay
   unchanged until the matching ln_net_collect returns; pass that call the images' own widths / heights as image_w / image_h. */
int32_t ln_net_submit_u8(ln_net* net, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths, const int32_t* heights,
                         int32_t mode);
int32_t ln_net_collect(ln_net* net, const int32_t* image_w, const int32_t* image_h, const ln_detect_options* opts,
                       ln_detection* records_host, int32_t* counts_host);
/* ln_image_preprocess_u8 (to the network's input size) followed by ln_net_detect_device; the records are scaled to each
   image's own size (widths / heights), as `lightnet-rs detect-image` does (lightnet-cli/src/main.rs: load, letterbox, detect). */
int32_t ln_net_detect_u8(ln_net* net, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths, const int32_t* heights,
                         int32_t mode, const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host);
/* Device time in ms of the most recent ln_net_forward* / ln_net_detect* call, by phase
   (0 = layers, 1 = decode+NMS), measured with CUDA events on the ctx stream. */
int32_t ln_net_last_times(const ln_net* net, float times_ms[2]);
/* Per-kernel timing of 8-bit forwards.  With profiling on, every launch of the plan is bracketed by CUDA events on
   the ctx stream (the forward then synchronises).  ln_net_profile returns, for the last forward, device ms per layer
   (per_layer_ms[num_layers]) and per kernel class (per_op_ms[8]: 0 tensor-core conv, 1 CUDA-core conv, 2 first-layer
   conv, 3 max-pool, 4 up-sample, 5 route copy, 6 shortcut, 7 input quantise) and the launch count per class. */
/* 8-bit plans run a linear [shortcut] in the epilogue of the convolution in front of it when nobody else reads that
   convolution (same arithmetic on the same int8 codes, so results do not change); 0 = keep every layer separate. */
int32_t ln_net_set_fusion(ln_net* net, int32_t on);
int32_t ln_net_set_profile(ln_net* net, int32_t on);
/* Host-input pipeline (default on; 8-bit precisions, even batch >= 8): ln_net_detect uploads the batch in two parts (a quarter,
   then three quarters) on a copy stream and runs them through two networks of those batch sizes with the same weights and
   scales, so the upload of the second part overlaps the layers of the first; both write their image ranges of one set of head
   tensors, and one decode + NMS runs over the whole batch.  Detections are the same as with the pipeline off.  No counterpart
   in the reference. */
int32_t ln_net_set_host_pipeline(ln_net* net, int32_t on);
/* 8-bit forwards replay one captured CUDA graph of the whole batch (default on); 0 = launch kernel by kernel. */
int32_t ln_net_set_cuda_graph(ln_net* net, int32_t on);
int32_t ln_net_profile(const ln_net* net, float* per_layer_ms, int32_t num_layers, float per_op_ms[8], int32_t per_op_launches[8]);


/* ---- modern anchor-free heads ------------------------------------------------------------- */
/* modern_yolo_forward_f32 (lightnet-cuda/src/lib.rs:4884): the shared [yolox] / [ppyoloe] / [yolonas] output activation in NCHW:
   every entry sanitised (non-finite -> 0), the trailing 1 + classes planes through a sigmoid of the logit clamped to [-30, 30]. */
int32_t ln_modern_yolo_forward_f32(ln_ctx* ctx, const ln_tensor* x, int64_t classes, ln_tensor** out);
/* modern_yolo_predecode_f32 (lib.rs:4936; kernel lightnet-cuda-oxide/src/kernels/dense_loss.rs:788): device box decode of an
   activated [ppyoloe] / [yolonas] head (kind 1 or 2, the trait's numbering) of coords = 4 * (reg_max + 1) box entries:
   returns [batch, 5 + classes, H, W] holding the final centre-size box, then the objectness and class planes.  Hand the
   result to ln_yolo_decode_nms as a head of kind 2 (decode_modern_detections, lightnet-train/src/detect.rs:1035, through
   decode_network_detections). */
int32_t ln_modern_yolo_predecode_f32(ln_ctx* ctx, const ln_tensor* x, int64_t classes, int64_t coords, int32_t kind, ln_tensor** out);

/* ---- debug aids (no counterpart in the reference) ------------------------------------------- */
/* Largest distance, in units of the 32-bit confidence key, between the approximate (hardware ex2 / rcp) score the head passes
   classify candidates with and the exact one, over a sweep of n_obj objectness logits in [obj_lo, obj_hi] times n_x class
   logits in [x_lo, x_hi].  The passes trust the approximation only beyond 256 units from a decision boundary. */
int32_t ln_debug_score_key_error(ln_ctx* ctx, float obj_lo, float obj_hi, float x_lo, float x_hi, int32_t n_obj, int32_t n_x,
                                 uint32_t* worst);
/* Sustained tensor-core rate of this GPU, in TOP/s (TFLOP/s for binary16): every SM issues `iters` x 4 tcgen05.mma instructions
   (M = 128, N = 256, 32 bytes of K each) on operands resident in shared memory, timed with CUDA events on the ctx stream.  The
   measured denominator of the convolution's roofline.  dtype: LN_Q8, LN_F8 or LN_F16. */
int32_t ln_debug_mma_peak(ln_ctx* ctx, int32_t dtype, int32_t iters, float* tops);
/* The same loop with another instruction shape: N = n filters per instruction (a multiple of 32 up to 256) and, with pair != 0,
   clusters of two CTAs issuing M = 256 instructions for both SMs (tcgen05.mma.cta_group::2).  Shows what a filter tile narrower
   than 256 costs at the issue port.  Bits 1 and 2 of `pair` select variants of the loop: 2 = a tcgen05.commit after every
   four instructions (as a pipelined main loop releases its stages), 4 = the operands rotate through four tile sets, 8 = two
   warps issue, each into its own accumulator. */
int32_t ln_debug_mma_peak_shape(ln_ctx* ctx, int32_t dtype, int32_t n, int32_t pair, int32_t iters, float* tops);
/* Role-timing counters (clock cycles) that CTA 0 of the most recent tensor-core convolution recorded: [0..1] producer total /
   waiting, [2..5] MMA issuer total / waiting for an accumulator / waiting for operands / tiles, [6..] epilogue warps.  Only with
   a library built with -DLN_CONV_ROLE_TIMING and LN_DEBUG_CYCLES=1 in the environment at ln_ctx_create; LN_ERR_UNSUPPORTED
   otherwise. */
int32_t ln_ctx_debug_cycles(ln_ctx* ctx, int64_t cycles[32]);

#ifdef __cplusplus
}
#endif
#endif /* LIGHTNET_B200_H */
