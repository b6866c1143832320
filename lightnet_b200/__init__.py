"""lightnet_b200 -- B200 (sm_100a) backend for lightnet's detector inference path.

This module is the Python binding of the C ABI in include/lightnet_b200.h.  The class and method
names mirror the reference's backend seam (trait F32TensorOpsBackend, src/lightnet-cuda/src/lib.rs:460,
and the reduced-precision twin shaped like F16TensorOpsBackend, lib.rs:6295) and its executor
(GpuExecutableNetwork, src/lightnet-runtime/src/runtime/gpu_types.rs:220), so that tests read like
the reference's own.  There is no CPU fallback: everything here needs the compiled CUDA library and a
B200; a missing library or device raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# the in-tree library; LIGHTNET_B200_LIB names another build of it (e.g. one compiled with extra -D switches for an A/B run)
LIB_PATH = os.environ.get("LIGHTNET_B200_LIB") or os.path.join(_HERE, "liblightnet_b200.so")

LN_F32, LN_Q8, LN_I32, LN_F8, LN_F16 = 0, 1, 2, 3, 4
LN_OUT_Q, LN_OUT_F32, LN_OUT_ACC = 0, 1, 2
ACTIVATIONS = {"linear": 0, "logistic": 1, "leaky": 2, "mish": 3, "swish": 4, "relu": 5}
STATUS = {0: "ok", 1: "shape", 2: "cuda", 3: "timeout", 4: "unsupported", 5: "argument", 6: "parse"}


LN_PRE_LETTERBOX, LN_PRE_RESIZE, LN_PRE_RESIZE_EXACT = 0, 1, 2


def pack_u8_images(images):
    """Concatenates interleaved u8 RGB images into one byte buffer; returns (bytes, offsets int64, widths int32, heights int32)."""
    images = [np.ascontiguousarray(im, np.uint8) for im in images]
    for im in images:
        if im.ndim != 3 or im.shape[2] != 3:
            raise ValueError("expected [height, width, 3] uint8 images")
    sizes = [im.size for im in images]
    offsets = np.zeros(len(images), np.int64)
    offsets[1:] = np.cumsum(sizes[:-1])
    flat = np.concatenate([im.ravel() for im in images]) if images else np.zeros(0, np.uint8)
    widths = np.array([im.shape[1] for im in images], np.int32)
    heights = np.array([im.shape[0] for im in images], np.int32)
    return flat, offsets, widths, heights


class BackendError(RuntimeError):
    """Non-zero status from the C ABI (maps to `Result::Err(Self::Error)` of the reference traits)."""

    def __init__(self, code, message):
        super().__init__("%s error: %s" % (STATUS.get(code, str(code)), message))
        self.code = code
        self.kind = STATUS.get(code, str(code))


class ln_yolo_head(C.Structure):
    _fields_ = [("raw", C.c_void_p), ("classes", C.c_int32), ("n_anchor", C.c_int32), ("anchors", C.c_float * 16),
                ("scale_x_y", C.c_float), ("new_coords", C.c_int32), ("kind", C.c_int32)]


class ln_detect_options(C.Structure):
    _fields_ = [("confidence_threshold", C.c_float), ("nms_threshold", C.c_float), ("letterbox", C.c_int32),
                ("top_k", C.c_int32), ("max_per_image", C.c_int32)]


_lib = None

# name -> (restype, argtypes); every symbol include/lightnet_b200.h declares
_I64P = C.POINTER(C.c_int64)
_VP = C.c_void_p
_PP = C.POINTER(C.c_void_p)
SYMBOLS = {
    "ln_ctx_create": (C.c_int32, [C.c_int32, _PP]),
    "ln_ctx_destroy": (C.c_int32, [_VP]),
    "ln_last_error": (C.c_char_p, [_VP]),
    "ln_sync": (C.c_int32, [_VP]),
    "ln_ctx_stream": (C.c_void_p, [_VP]),
    "ln_ctx_set_exact_epilogue": (C.c_int32, [_VP, C.c_int32]),
    "ln_ctx_set_nms_pool_entries": (C.c_int32, [_VP, C.c_int64]),
    "ln_image_preprocess_u8": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _VP]),
    "ln_net_detect_u8": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_int32, _VP, _VP, _VP]),
    "ln_ctx_set_kernel_timing": (C.c_int32, [_VP, C.c_int32]),
    "ln_ctx_last_kernel_ms": (C.c_int32, [_VP, C.POINTER(C.c_float)]),
    "ln_ctx_launch_count": (C.c_int64, [_VP]),
    "ln_tensor_upload_f32": (C.c_int32, [_VP, _I64P, _VP, _PP]),
    "ln_tensor_zeros_f32": (C.c_int32, [_VP, _I64P, _PP]),
    "ln_tensor_download_f32": (C.c_int32, [_VP, _VP, _VP, C.c_int64]),
    "ln_tensor_shape": (C.c_int32, [_VP, _I64P]),
    "ln_tensor_dtype": (C.c_int32, [_VP]),
    "ln_tensor_retain": (C.c_int32, [_VP]),
    "ln_tensor_release": (C.c_int32, [_VP]),
    "ln_conv2d_f32": (C.c_int32, [_VP, _VP, _VP, _I64P] + [C.c_int64] * 10 + [_PP]),
    "ln_bias_add_f32": (C.c_int32, [_VP, _VP, _VP, C.c_int64, C.c_int64, _PP]),
    "ln_activation_f32": (C.c_int32, [_VP, _VP, C.c_int32, _PP]),
    "ln_bias_activation_f32": (C.c_int32, [_VP, _VP, _VP, C.c_int64, C.c_int64, C.c_int32, _PP]),
    "ln_shortcut_add_f32": (C.c_int32, [_VP, _VP, _VP, _PP]),
    "ln_shortcut_fit_f32": (C.c_int32, [_VP, _VP, C.c_int64, _I64P, _PP]),
    "ln_route_concat_f32": (C.c_int32, [_VP, _PP, C.c_int32, _I64P, _I64P, _I64P, _I64P, C.c_int64, _PP]),
    "ln_maxpool_f32": (C.c_int32, [_VP, _VP, _I64P] + [C.c_int64] * 7 + [_PP]),
    "ln_upsample_f32": (C.c_int32, [_VP, _VP, _I64P] + [C.c_int64] * 4 + [C.c_float, C.c_int32, _PP]),
    "ln_batchnorm_fold_f32": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_float, _PP, _PP]),
    "ln_tensor_upload_q": (C.c_int32, [_VP, _I64P, _VP, C.c_float, C.c_int32, _PP]),
    "ln_tensor_download_q": (C.c_int32, [_VP, _VP, _VP, C.c_int64, C.POINTER(C.c_float)]),
    "ln_tensor_upload_codes": (C.c_int32, [_VP, _I64P, _VP, C.c_float, C.c_int32, _PP]),
    "ln_tensor_download_i32": (C.c_int32, [_VP, _VP, _VP, C.c_int64]),
    "ln_tensor_widen_q": (C.c_int32, [_VP, _VP, _PP]),
    "ln_tensor_narrow_f32": (C.c_int32, [_VP, _VP, C.c_float, C.c_int32, _PP]),
    "ln_tensor_scale": (C.c_float, [_VP]),
    "ln_conv_weights_q": (C.c_int32, [_VP, _VP, C.c_int64, C.c_int64, C.c_int64, C.c_int32, _PP]),
    "ln_conv_weights_release": (C.c_int32, [_VP]),
    "ln_conv2d_bias_act_q": (C.c_int32, [_VP, _VP, _VP, _VP, _I64P] + [C.c_int64] * 10 + [C.c_int32, C.c_float, C.c_int32, _PP]),
    "ln_maxpool_q": (C.c_int32, [_VP, _VP, _I64P] + [C.c_int64] * 7 + [_PP]),
    "ln_upsample_q": (C.c_int32, [_VP, _VP, _I64P] + [C.c_int64] * 4 + [C.c_float, C.c_int32, _PP]),
    "ln_route_concat_q": (C.c_int32, [_VP, _PP, C.c_int32, _I64P, _I64P, _I64P, _I64P, C.c_int64, _PP]),
    "ln_shortcut_add_act_q": (C.c_int32, [_VP, _VP, _VP, C.c_int32, C.c_float, _PP]),
    "ln_shortcut_fit_q": (C.c_int32, [_VP, _VP, C.c_int64, _I64P, _PP]),
    "ln_yolo_decode_nms": (C.c_int32, [_VP, _VP, C.c_int32, C.c_int32, C.c_int32, _VP, _VP, _VP, _VP, _VP]),
    "ln_yolo_decode_nms_noalloc": (C.c_int32, [_VP, _VP, C.c_int32, C.c_int32, C.c_int32, _VP, _VP, _VP, _VP, _VP]),
    "ln_yolo_decode_only": (C.c_int32, [_VP, _VP, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                        C.c_int32, _VP, C.c_int64, C.POINTER(C.c_int64)]),
    "ln_net_create": (C.c_int32, [_VP, C.c_char_p, C.c_int32, C.c_int32, _PP]),
    "ln_net_destroy": (C.c_int32, [_VP]),
    "ln_net_num_layers": (C.c_int32, [_VP]),
    "ln_net_layer_info": (C.c_int32, [_VP, C.c_int32, _VP]),
    "ln_net_weight_count": (C.c_int64, [_VP]),
    "ln_net_load_weights": (C.c_int32, [_VP, _VP, C.c_int64]),
    "ln_net_load_weights_file": (C.c_int32, [_VP, C.c_char_p]),
    "ln_net_calibrate": (C.c_int32, [_VP, _VP]),
    "ln_net_get_scales": (C.c_int32, [_VP, _VP, C.c_int32]),
    "ln_net_set_scales": (C.c_int32, [_VP, _VP, C.c_int32]),
    "ln_net_set_micro_batch": (C.c_int32, [_VP, C.c_int32]),
    "ln_net_forward": (C.c_int32, [_VP, _VP]),
    "ln_net_forward_device": (C.c_int32, [_VP, _VP]),
    "ln_net_num_heads": (C.c_int32, [_VP]),
    "ln_net_head": (C.c_int32, [_VP, C.c_int32, _PP]),
    "ln_net_layer_output": (C.c_int32, [_VP, C.c_int32, _PP]),
    "ln_net_detect": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "ln_net_detect_device": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "ln_net_submit": (C.c_int32, [_VP, _VP]),
    "ln_net_submit_u8": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_int32]),
    "ln_net_collect": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, _VP]),
    "ln_net_last_times": (C.c_int32, [_VP, _VP]),
    "ln_net_set_profile": (C.c_int32, [_VP, C.c_int32]),
    "ln_net_set_fusion": (C.c_int32, [_VP, C.c_int32]),
    "ln_net_set_host_pipeline": (C.c_int32, [_VP, C.c_int32]),
    "ln_net_set_cuda_graph": (C.c_int32, [_VP, C.c_int32]),
    "ln_net_profile": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP]),
    "ln_channel_scale_f32": (C.c_int32, [_VP, _VP, _VP, C.c_int64, C.c_int64, _PP]),
    "ln_region_forward_f32": (C.c_int32, [_VP, _VP, C.c_int64, C.c_int64, C.c_int64, C.c_int32, _PP]),
    "ln_yolo_activate_f32": (C.c_int32, [_VP, _VP, C.c_int64, C.c_float, C.c_int32, _PP]),
    "ln_tensor_upload_f16": (C.c_int32, [_VP, _I64P, _VP, _PP]),
    "ln_tensor_download_f16": (C.c_int32, [_VP, _VP, _VP, C.c_int64]),
    "ln_tensor_widen_f16": (C.c_int32, [_VP, _VP, _PP]),
    "ln_tensor_narrow_f16": (C.c_int32, [_VP, _VP, _PP]),
    "ln_conv_weights_f16": (C.c_int32, [_VP, _VP, C.c_int64, C.c_int64, _PP]),
    "ln_conv2d_bias_act_f16": (C.c_int32, [_VP, _VP, _VP, _VP, _I64P] + [C.c_int64] * 10 + [C.c_int32, _PP]),
    "ln_maxpool_f16": (C.c_int32, [_VP, _VP, _I64P] + [C.c_int64] * 7 + [_PP]),
    "ln_upsample_f16": (C.c_int32, [_VP, _VP, _I64P] + [C.c_int64] * 4 + [C.c_float, C.c_int32, _PP]),
    "ln_route_concat_f16": (C.c_int32, [_VP, _PP, C.c_int32, _I64P, _I64P, _I64P, _I64P, C.c_int64, _PP]),
    "ln_shortcut_fit_f16": (C.c_int32, [_VP, _VP, C.c_int64, _I64P, _PP]),
    "ln_shortcut_add_act_f16": (C.c_int32, [_VP, _VP, _VP, C.c_int32, _PP]),
    "ln_channel_affine_act_f16": (C.c_int32, [_VP, _VP, _VP, _VP, C.c_int64, C.c_int64, C.c_int32, _PP]),
    "ln_debug_score_key_error": (C.c_int32, [_VP, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int32, C.c_int32, C.POINTER(C.c_uint32)]),
    "ln_ctx_debug_cycles": (C.c_int32, [_VP, _I64P]),
    "ln_modern_yolo_forward_f32": (C.c_int32, [_VP, _VP, C.c_int64, _VP]),
    "ln_modern_yolo_predecode_f32": (C.c_int32, [_VP, _VP, C.c_int64, C.c_int64, C.c_int32, _VP]),
    "ln_debug_mma_peak": (C.c_int32, [_VP, C.c_int32, C.c_int32, C.POINTER(C.c_float)]),
    "ln_debug_mma_peak_shape": (C.c_int32, [_VP, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_float)]),
}


def load_library():
    """dlopen the in-tree CUDA library; raises if it has not been built (python -m lightnet_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m lightnet_b200.build` (needs nvcc); "
                              "this package has no CPU fallback" % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _shape4(shape):
    s = tuple(int(v) for v in shape)
    if len(s) != 4:
        raise ValueError("shapes are [batch, channels, height, width]")
    return (C.c_int64 * 4)(*s)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _act(a):
    return ACTIVATIONS[a] if isinstance(a, str) else int(a)


class Tensor:
    """Opaque ref-counted device tensor (`type Tensor: Clone`); dropping the object releases the handle."""

    def __init__(self, backend, handle):
        self.backend = backend
        self.h = handle

    def __del__(self):
        # a handle that outlives its (closed) backend has nothing left to release: the context took its memory with it
        if getattr(self, "h", None) and _lib is not None and getattr(self.backend, "ctx", None):
            _lib.ln_tensor_release(self.h)
        self.h = None

    @property
    def shape(self):
        s = (C.c_int64 * 4)()
        _lib.ln_tensor_shape(self.h, s)
        return tuple(int(v) for v in s)

    @property
    def dtype(self):
        return int(_lib.ln_tensor_dtype(self.h))

    @property
    def scale(self):
        return float(_lib.ln_tensor_scale(self.h))


class ConvWeights:
    def __init__(self, backend, handle):
        self.backend = backend
        self.h = handle

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None and getattr(self.backend, "ctx", None):
            _lib.ln_conv_weights_release(self.h)
        self.h = None


class B200Backend:
    """One device + one stream (`OxideBackend::with_device`, lightnet-cuda-oxide/src/lib.rs:643)."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.ln_ctx_create(device, C.byref(h))
        if rc:
            raise BackendError(rc, self.lib.ln_last_error(None).decode())
        self.ctx = h
        self.device = device

    def close(self):
        if getattr(self, "ctx", None):
            self.lib.ln_ctx_destroy(self.ctx)
            self.ctx = None

    def _check(self, rc):
        if rc:
            raise BackendError(rc, self.lib.ln_last_error(self.ctx).decode())

    def _out(self, fn, *args):
        h = C.c_void_p()
        self._check(fn(self.ctx, *args, C.byref(h)))
        return Tensor(self, h)

    def sync(self):
        self._check(self.lib.ln_sync(self.ctx))

    @property
    def stream(self):
        return self.lib.ln_ctx_stream(self.ctx)

    @property
    def launch_count(self):
        return int(self.lib.ln_ctx_launch_count(self.ctx))

    def set_exact_epilogue(self, on: bool):
        self._check(self.lib.ln_ctx_set_exact_epilogue(self.ctx, int(on)))

    def set_kernel_timing(self, on: bool):
        self._check(self.lib.ln_ctx_set_kernel_timing(self.ctx, int(on)))

    def last_kernel_ms(self) -> float:
        ms = C.c_float()
        self._check(self.lib.ln_ctx_last_kernel_ms(self.ctx, C.byref(ms)))
        return float(ms.value)

    # ---- image pre-processing (PlanarRgbImage::letterbox / resize / resize_linear_exact) ---------------
    def preprocess_u8(self, images, dst_w, dst_h, mode=LN_PRE_LETTERBOX):
        """images: list of uint8 arrays [h, w, 3] (interleaved RGB, any sizes) -> f32 Tensor [n, 3, dst_h, dst_w]."""
        flat, offsets, widths, heights = pack_u8_images(images)
        return self._out(self.lib.ln_image_preprocess_u8, _ptr(flat), _ptr(offsets), _ptr(widths), _ptr(heights), len(images), mode,
                         dst_w, dst_h)

    def set_nms_pool_entries(self, entries: int):
        """Candidates per image the NMS selection pool holds (0 = automatic); results do not depend on it."""
        self._check(self.lib.ln_ctx_set_nms_pool_entries(self.ctx, int(entries)))

    def debug_score_key_error(self, obj_lo, obj_hi, x_lo, x_hi, n_obj, n_x):
        """Largest distance, in confidence-key units, between the approximate and the exact candidate score over a sweep."""
        worst = C.c_uint32()
        self._check(self.lib.ln_debug_score_key_error(self.ctx, obj_lo, obj_hi, x_lo, x_hi, n_obj, n_x, C.byref(worst)))
        return int(worst.value)

    def mma_peak(self, dtype=LN_Q8, iters=4096, n=256, pair=False):
        """Measured tensor-core rate (TOP/s) of a tcgen05.mma-only loop on every SM: M = 128 (256 over a CTA pair), N = n."""
        t = C.c_float()
        if n == 256 and not pair:
            self._check(self.lib.ln_debug_mma_peak(self.ctx, dtype, iters, C.byref(t)))
        else:
            self._check(self.lib.ln_debug_mma_peak_shape(self.ctx, dtype, n, 1 if pair else 0, iters, C.byref(t)))
        return float(t.value)

    def debug_cycles(self):
        """The 32 role-timing counters of the last tensor-core convolution (needs a -DLN_CONV_ROLE_TIMING build and LN_DEBUG_CYCLES=1)."""
        out = (C.c_int64 * 32)()
        self._check(self.lib.ln_ctx_debug_cycles(self.ctx, out))
        return list(out)

    # ---- F32TensorOpsBackend ------------------------------------------------------------------
    def upload_f32(self, shape, host):
        host = np.ascontiguousarray(host, np.float32)
        if host.size != int(np.prod(shape)):
            raise BackendError(1, "host data has %d values for shape %s" % (host.size, tuple(shape)))
        return self._out(self.lib.ln_tensor_upload_f32, _shape4(shape), _ptr(host))

    def zeros_f32(self, shape):
        return self._out(self.lib.ln_tensor_zeros_f32, _shape4(shape))

    def download_f32(self, t):
        out = np.empty(t.shape, np.float32)
        self._check(self.lib.ln_tensor_download_f32(self.ctx, t.h, _ptr(out), out.size))
        return out

    def tensor_shape(self, t):
        return t.shape

    def conv2d_f32(self, x, weights, output_shape, input_channels, input_height, input_width, filters, kernel_size, stride_x,
                   stride_y, dilation, padding, groups):
        return self._out(self.lib.ln_conv2d_f32, x.h, weights.h, _shape4(output_shape), input_channels, input_height, input_width,
                         filters, kernel_size, stride_x, stride_y, dilation, padding, groups)

    def bias_add_f32(self, x, bias, channels, channel_stride):
        return self._out(self.lib.ln_bias_add_f32, x.h, bias.h, channels, channel_stride)

    def activation_f32(self, x, activation):
        return self._out(self.lib.ln_activation_f32, x.h, _act(activation))

    def bias_activation_f32(self, x, bias, channels, channel_stride, activation):
        return self._out(self.lib.ln_bias_activation_f32, x.h, bias.h, channels, channel_stride, _act(activation))

    def shortcut_add_f32(self, x, y):
        return self._out(self.lib.ln_shortcut_add_f32, x.h, y.h)

    def shortcut_fit_f32(self, x, batch, output_shape):
        return self._out(self.lib.ln_shortcut_fit_f32, x.h, batch, _shape4(output_shape))

    def _route(self, fn, inputs, input_channel_offsets, input_channels, input_total_channels, output_shape, channel_stride):
        n = len(inputs)
        arr = (C.c_void_p * n)(*[t.h for t in inputs])
        i64 = lambda v: (C.c_int64 * n)(*[int(x) for x in v])
        return self._out(fn, arr, n, i64(input_channel_offsets), i64(input_channels), i64(input_total_channels),
                         _shape4(output_shape), channel_stride)

    def route_concat_f32(self, inputs, input_channel_offsets, input_channels, input_total_channels, output_shape, channel_stride):
        return self._route(self.lib.ln_route_concat_f32, inputs, input_channel_offsets, input_channels, input_total_channels,
                           output_shape, channel_stride)

    def maxpool_f32(self, x, output_shape, channels, input_height, input_width, size, stride_x, stride_y, padding):
        return self._out(self.lib.ln_maxpool_f32, x.h, _shape4(output_shape), channels, input_height, input_width, size, stride_x,
                         stride_y, padding)

    def upsample_f32(self, x, output_shape, channels, input_height, input_width, stride, scale, reverse):
        return self._out(self.lib.ln_upsample_f32, x.h, _shape4(output_shape), channels, input_height, input_width, stride,
                         float(scale), int(reverse))

    def batchnorm_fold_f32(self, gamma, mean, variance, bias, eps):
        s, b = C.c_void_p(), C.c_void_p()
        self._check(self.lib.ln_batchnorm_fold_f32(self.ctx, gamma.h, mean.h, variance.h, bias.h, float(eps), C.byref(s), C.byref(b)))
        return Tensor(self, s), Tensor(self, b)

    def channel_scale_f32(self, x, scale, channels, channel_stride):
        return self._out(self.lib.ln_channel_scale_f32, x.h, scale.h, channels, channel_stride)

    def region_forward_f32(self, x, anchors, entries, classes, softmax_classes):
        return self._out(self.lib.ln_region_forward_f32, x.h, anchors, entries, classes, int(bool(softmax_classes)))

    def yolo_activate_f32(self, x, classes, scale_xy, new_coords):
        return self._out(self.lib.ln_yolo_activate_f32, x.h, classes, float(scale_xy), int(bool(new_coords)))

    def modern_yolo_forward_f32(self, x, classes):
        """The output activation of [yolox] / [ppyoloe] / [yolonas] heads (lightnet-cuda/src/lib.rs:4884)."""
        return self._out(self.lib.ln_modern_yolo_forward_f32, x.h, int(classes))

    def modern_yolo_predecode_f32(self, x, classes, coords, kind):
        """Device box decode of an activated distribution head (lib.rs:4936): [B, coords + 1 + classes, H, W] -> [B, 5 + classes, H, W]."""
        return self._out(self.lib.ln_modern_yolo_predecode_f32, x.h, int(classes), int(coords), int(kind))

    # ---- F16TensorOpsBackend (binary16 storage) ---------------------------------------------------
    def upload_f16(self, shape, host):
        host = np.ascontiguousarray(host, np.float32)
        return self._out(self.lib.ln_tensor_upload_f16, _shape4(shape), _ptr(host))

    def download_f16(self, t):
        out = np.empty(t.shape, np.float32)
        self._check(self.lib.ln_tensor_download_f16(self.ctx, t.h, _ptr(out), out.size))
        return out

    def widen_f16(self, t):
        return self._out(self.lib.ln_tensor_widen_f16, t.h)

    def narrow_f32_f16(self, t):
        """narrow_f32 of the binary16 trait: an f32 device tensor rounded to binary16 storage."""
        return self._out(self.lib.ln_tensor_narrow_f16, t.h)

    def conv_weights_f16(self, weights, filters, per_filter):
        h = C.c_void_p()
        self._check(self.lib.ln_conv_weights_f16(self.ctx, weights.h, filters, per_filter, C.byref(h)))
        return ConvWeights(self, h)

    def conv2d_bias_act_f16(self, x, weights, bias, output_shape, channels, input_height, input_width, filters, size, stride_x, stride_y,
                            dilation, padding, groups, activation):
        return self._out(self.lib.ln_conv2d_bias_act_f16, x.h, weights.h, bias.h, _shape4(output_shape), channels, input_height, input_width,
                         filters, size, stride_x, stride_y, dilation, padding, groups, _act(activation))

    def maxpool_f16(self, x, output_shape, channels, input_height, input_width, size, stride_x, stride_y, padding):
        return self._out(self.lib.ln_maxpool_f16, x.h, _shape4(output_shape), channels, input_height, input_width, size, stride_x, stride_y, padding)

    def upsample_f16(self, x, output_shape, channels, input_height, input_width, stride, scale, reverse):
        return self._out(self.lib.ln_upsample_f16, x.h, _shape4(output_shape), channels, input_height, input_width, stride, float(scale), int(bool(reverse)))

    def route_concat_f16(self, inputs, input_channel_offsets, input_channels, input_total_channels, output_shape, channel_stride):
        return self._route(self.lib.ln_route_concat_f16, inputs, input_channel_offsets, input_channels, input_total_channels, output_shape, channel_stride)

    def shortcut_fit_f16(self, x, batch, output_shape):
        return self._out(self.lib.ln_shortcut_fit_f16, x.h, batch, _shape4(output_shape))

    def shortcut_add_act_f16(self, a, b, activation):
        return self._out(self.lib.ln_shortcut_add_act_f16, a.h, b.h, _act(activation))

    def channel_affine_act_f16(self, x, scale, bias, channels, channel_stride, activation):
        return self._out(self.lib.ln_channel_affine_act_f16, x.h, scale.h if scale is not None else None, bias.h, channels, channel_stride, _act(activation))

    # ---- 8-bit twins (int8 / FP8 E4M3) ---------------------------------------------------------
    def upload_q(self, shape, host, scale, dtype=LN_Q8):
        host = np.ascontiguousarray(host, np.float32)
        return self._out(self.lib.ln_tensor_upload_q, _shape4(shape), _ptr(host), float(scale), dtype)

    def upload_codes(self, shape, codes, scale, dtype=LN_Q8):
        codes = np.ascontiguousarray(codes).view(np.uint8)
        return self._out(self.lib.ln_tensor_upload_codes, _shape4(shape), _ptr(codes), float(scale), dtype)

    def download_q(self, t):
        """Raw codes in NCHW order (int8 for LN_Q8, uint8 E4M3 bytes for LN_F8) and the tensor scale."""
        out = np.empty(t.shape, np.int8 if t.dtype == LN_Q8 else np.uint8)
        s = C.c_float()
        self._check(self.lib.ln_tensor_download_q(self.ctx, t.h, _ptr(out), out.size, C.byref(s)))
        return out, float(s.value)

    def download_i32(self, t):
        out = np.empty(t.shape, np.int32)
        self._check(self.lib.ln_tensor_download_i32(self.ctx, t.h, _ptr(out), out.size))
        return out

    def widen_q(self, t):
        return self._out(self.lib.ln_tensor_widen_q, t.h)

    def narrow_f32(self, t, scale, dtype=LN_Q8):
        return self._out(self.lib.ln_tensor_narrow_f32, t.h, float(scale), dtype)

    def conv_weights_q(self, weights, filters, channels, kernel_size, dtype=LN_Q8):
        h = C.c_void_p()
        self._check(self.lib.ln_conv_weights_q(self.ctx, weights.h, filters, channels, kernel_size, dtype, C.byref(h)))
        return ConvWeights(self, h)

    def conv2d_bias_act_q(self, x, weights, bias, output_shape, channels, input_height, input_width, filters, kernel_size,
                          stride_x, stride_y, dilation, padding, groups, activation, y_scale=1.0, out_kind=LN_OUT_Q):
        return self._out(self.lib.ln_conv2d_bias_act_q, x.h, weights.h, bias.h, _shape4(output_shape), channels, input_height,
                         input_width, filters, kernel_size, stride_x, stride_y, dilation, padding, groups, _act(activation),
                         float(y_scale), out_kind)

    def maxpool_q(self, x, output_shape, channels, input_height, input_width, size, stride_x, stride_y, padding):
        return self._out(self.lib.ln_maxpool_q, x.h, _shape4(output_shape), channels, input_height, input_width, size, stride_x,
                         stride_y, padding)

    def upsample_q(self, x, output_shape, channels, input_height, input_width, stride, scale, reverse):
        return self._out(self.lib.ln_upsample_q, x.h, _shape4(output_shape), channels, input_height, input_width, stride,
                         float(scale), int(reverse))

    def route_concat_q(self, inputs, input_channel_offsets, input_channels, input_total_channels, output_shape, channel_stride):
        return self._route(self.lib.ln_route_concat_q, inputs, input_channel_offsets, input_channels, input_total_channels,
                           output_shape, channel_stride)

    def shortcut_fit_q(self, x, batch, output_shape):
        return self._out(self.lib.ln_shortcut_fit_q, x.h, batch, _shape4(output_shape))

    def shortcut_add_act_q(self, a, b, activation, y_scale):
        return self._out(self.lib.ln_shortcut_add_act_q, a.h, b.h, _act(activation), float(y_scale))

    # ---- [yolo] decode + NMS ---------------------------------------------------------------------
    @staticmethod
    def _heads(heads):
        arr = (ln_yolo_head * len(heads))()
        for k, h in enumerate(heads):
            arr[k].raw = h["raw"].h
            arr[k].classes = h["classes"]
            arr[k].n_anchor = len(h["anchors"])
            flat = [v for a in h["anchors"] for v in a]
            for i, v in enumerate(flat):
                arr[k].anchors[i] = v
            arr[k].scale_x_y = h.get("scale_x_y", 1.0)
            arr[k].new_coords = int(h.get("new_coords", 0))
            arr[k].kind = int(h.get("kind", 0))  # 1 = activated [yolox] head, 2 = predecoded distribution head (one dummy anchor)
        return arr

    def yolo_decode_nms(self, heads, net_w, net_h, image_w, image_h, confidence_threshold=0.25, nms_threshold=0.45,
                        letterbox=True, top_k=0, max_per_image=1024, noalloc=False):
        """heads: list of dicts {raw: Tensor f32 [B, A*(5+cls), gh, gw], classes, anchors [(w,h)...], scale_x_y, new_coords}.
        Returns a list (one per image) of (n,7) arrays {class, conf, obj, x, y, w, h}, confidence descending."""
        arr = self._heads(heads)
        batch = heads[0]["raw"].shape[0]
        iw = np.ascontiguousarray(np.broadcast_to(np.asarray(image_w, np.int32), (batch,)))
        ih = np.ascontiguousarray(np.broadcast_to(np.asarray(image_h, np.int32), (batch,)))
        opts = ln_detect_options(confidence_threshold, nms_threshold, int(letterbox), top_k, max_per_image)
        rec = np.empty((batch, max_per_image, 7), np.float32)
        cnt = np.zeros(batch, np.int32)
        # noalloc=True takes the entry point that keeps its working memory in a fixed array of the library (for hosts
        # that may not allocate device memory while serving); same records, bounded problem size
        fn = self.lib.ln_yolo_decode_nms_noalloc if noalloc else self.lib.ln_yolo_decode_nms
        self._check(fn(self.ctx, arr, len(heads), net_w, net_h, _ptr(iw), _ptr(ih), C.byref(opts), _ptr(rec), _ptr(cnt)))
        return [rec[b, :cnt[b]].copy() for b in range(batch)]

    def yolo_decode_only(self, heads, image_index, net_w, net_h, image_w, image_h, confidence_threshold, letterbox, capacity=1 << 22):
        arr = self._heads(heads)
        rec = np.zeros((capacity, 7), np.float32)
        n = C.c_int64()
        self._check(self.lib.ln_yolo_decode_only(self.ctx, arr, len(heads), image_index, net_w, net_h, image_w, image_h,
                                                 confidence_threshold, int(letterbox), _ptr(rec), capacity, C.byref(n)))
        if n.value > capacity:
            raise BackendError(1, "decode produced %d candidates, capacity %d" % (n.value, capacity))
        return rec[: n.value].copy()


class GpuExecutableNetwork:
    """`GpuExecutableNetwork<B>` of the reference runtime: cfg -> layers, Darknet weights, forward, detect."""

    KINDS = {0: "conv", 1: "maxpool", 2: "route", 3: "shortcut", 4: "upsample", 5: "yolo"}

    def __init__(self, backend: B200Backend, cfg_text: str, batch: int = 0, precision: int = LN_F32):
        self.backend = backend
        self.lib = backend.lib
        h = C.c_void_p()
        backend._check(self.lib.ln_net_create(backend.ctx, cfg_text.encode(), batch, precision, C.byref(h)))
        self.h = h
        self.precision = precision
        self.num_layers = self.lib.ln_net_num_layers(self.h)
        i0 = self.layer_info(0)
        self.batch, self.channels, self.height, self.width = i0["in_b"], i0["in_c"], i0["in_h"], i0["in_w"]

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None and getattr(self.backend, "ctx", None):
            self.lib.ln_net_destroy(self.h)
            self.h = None

    def layer_info(self, i):
        v = np.zeros(20, np.int32)
        if self.lib.ln_net_layer_info(self.h, i, _ptr(v)):
            raise IndexError(i)
        keys = ["kind", "in_w", "in_h", "in_c", "in_b", "out_w", "out_h", "out_c", "out_b", "filters", "size", "stride_x", "stride_y",
                "padding", "bn", "act", "groups", "dilation"]
        d = dict(zip(keys, (int(x) for x in v)))
        d["kind"] = self.KINDS[d["kind"]]
        return d

    def layers(self):
        return [self.layer_info(i) for i in range(self.num_layers)]

    def weight_count(self):
        return int(self.lib.ln_net_weight_count(self.h))

    def load_weights(self, blob):
        blob = np.ascontiguousarray(blob, np.float32)
        self.backend._check(self.lib.ln_net_load_weights(self.h, _ptr(blob), blob.size))

    def load_weights_file(self, path):
        self.backend._check(self.lib.ln_net_load_weights_file(self.h, os.fsencode(path)))

    def calibrate(self, x):
        x = np.ascontiguousarray(x, np.float32)
        self.backend._check(self.lib.ln_net_calibrate(self.h, _ptr(x)))

    def scales(self):
        out = np.zeros(self.num_layers + 1, np.float32)
        self.backend._check(self.lib.ln_net_get_scales(self.h, _ptr(out), out.size))
        return out

    def set_scales(self, s):
        s = np.ascontiguousarray(s, np.float32)
        self.backend._check(self.lib.ln_net_set_scales(self.h, _ptr(s), s.size))

    def set_micro_batch(self, mb):
        self.backend._check(self.lib.ln_net_set_micro_batch(self.h, mb))

    def forward(self, x):
        """`forward_compact`: host f32 NCHW in, heads stay on the device."""
        x = np.ascontiguousarray(x, np.float32)
        assert x.size == self.batch * self.channels * self.height * self.width
        self.backend._check(self.lib.ln_net_forward(self.h, _ptr(x)))

    def forward_device(self, t: Tensor):
        self.backend._check(self.lib.ln_net_forward_device(self.h, t.h))

    def num_heads(self):
        return self.lib.ln_net_num_heads(self.h)

    def head(self, k):
        h = C.c_void_p()
        self.backend._check(self.lib.ln_net_head(self.h, k, C.byref(h)))
        return Tensor(self.backend, h)

    def layer_output(self, i):
        h = C.c_void_p()
        self.backend._check(self.lib.ln_net_layer_output(self.h, i, C.byref(h)))
        return Tensor(self.backend, h)

    def _out_buffers(self, max_per_image, out):
        """(records [batch, max_per_image, 7] f32, counts [batch] i32): fresh arrays, or the caller's own (`out`, e.g. page-locked ones
        that the records then reach by DMA; the returned per-image arrays are views into them, valid until the buffers are reused)."""
        if out is None:
            return np.empty((self.batch, max_per_image, 7), np.float32), np.zeros(self.batch, np.int32), True
        rec, cnt = out
        if rec.shape != (self.batch, max_per_image, 7) or rec.dtype != np.float32 or not rec.flags["C_CONTIGUOUS"] or \
                cnt.shape != (self.batch,) or cnt.dtype != np.int32:
            raise ValueError("out must be (float32 [batch, max_per_image, 7], int32 [batch]) C-contiguous arrays")
        return rec, cnt, False

    def _detect(self, fn, src, image_w, image_h, confidence_threshold, nms_threshold, letterbox, top_k, max_per_image, out=None):
        iw = np.ascontiguousarray(np.broadcast_to(np.asarray(image_w, np.int32), (self.batch,)))
        ih = np.ascontiguousarray(np.broadcast_to(np.asarray(image_h, np.int32), (self.batch,)))
        opts = ln_detect_options(confidence_threshold, nms_threshold, int(letterbox), top_k, max_per_image)
        rec, cnt, own = self._out_buffers(max_per_image, out)
        self.backend._check(fn(self.h, src, _ptr(iw), _ptr(ih), C.byref(opts), _ptr(rec), _ptr(cnt)))
        return [rec[b, :cnt[b]].copy() if own else rec[b, :cnt[b]] for b in range(self.batch)]

    def detect(self, x, image_w, image_h, confidence_threshold=0.25, nms_threshold=0.45, letterbox=True, top_k=0,
               max_per_image=1024, out=None):
        """forward + device decode + NMS for a host batch (what `lightnet-rs detect-image` does per image)."""
        x = np.ascontiguousarray(x, np.float32)
        return self._detect(self.lib.ln_net_detect, _ptr(x), image_w, image_h, confidence_threshold, nms_threshold, letterbox,
                            top_k, max_per_image, out)

    def submit(self, x):
        """Enqueues the upload of one host batch (f32 NCHW, C-contiguous; keep it alive and unchanged until the matching collect
        returns; pinned memory makes the copy asynchronous).  At most two batches may be in flight."""
        if not (isinstance(x, np.ndarray) and x.dtype == np.float32 and x.flags["C_CONTIGUOUS"]):
            raise ValueError("submit needs a C-contiguous float32 array (it is read after this call returns)")
        self._in_flight = getattr(self, "_in_flight", [])
        self.backend._check(self.lib.ln_net_submit(self.h, _ptr(x)))
        self._in_flight.append(x)

    def submit_u8(self, images, mode=LN_PRE_LETTERBOX, packed=None):
        """submit() for a batch of uint8 [h, w, 3] images (or `packed` = pack_u8_images(images), kept alive and unchanged until
        the matching collect returns): upload and resize run under the layers of the batch submitted before.  Pass the images'
        own widths / heights to collect()."""
        packed = packed if packed is not None else pack_u8_images(images)
        flat, offsets, widths, heights = packed
        self._in_flight = getattr(self, "_in_flight", [])
        self.backend._check(self.lib.ln_net_submit_u8(self.h, _ptr(flat), _ptr(offsets), _ptr(widths), _ptr(heights), mode))
        self._in_flight.append(packed)

    def collect(self, image_w, image_h, confidence_threshold=0.25, nms_threshold=0.45, letterbox=True, top_k=0, max_per_image=1024,
                out=None):
        """Runs the oldest submitted batch and returns its detections, like detect()."""
        iw = np.ascontiguousarray(np.broadcast_to(np.asarray(image_w, np.int32), (self.batch,)))
        ih = np.ascontiguousarray(np.broadcast_to(np.asarray(image_h, np.int32), (self.batch,)))
        opts = ln_detect_options(confidence_threshold, nms_threshold, int(letterbox), top_k, max_per_image)
        rec, cnt, own = self._out_buffers(max_per_image, out)
        try:
            self.backend._check(self.lib.ln_net_collect(self.h, _ptr(iw), _ptr(ih), C.byref(opts), _ptr(rec), _ptr(cnt)))
        finally:
            if getattr(self, "_in_flight", None):
                self._in_flight.pop(0)
        return [rec[b, :cnt[b]].copy() if own else rec[b, :cnt[b]] for b in range(self.batch)]

    def detect_device(self, t: Tensor, image_w, image_h, confidence_threshold=0.25, nms_threshold=0.45, letterbox=True, top_k=0,
                      max_per_image=1024, out=None):
        return self._detect(self.lib.ln_net_detect_device, t.h, image_w, image_h, confidence_threshold, nms_threshold, letterbox,
                            top_k, max_per_image, out)

    def detect_u8(self, images, confidence_threshold=0.25, nms_threshold=0.45, letterbox=True, top_k=0, max_per_image=1024,
                  mode=LN_PRE_LETTERBOX, packed=None, out=None):
        """Pre-processing on the device + detect for a batch of uint8 [h, w, 3] images (or `packed` = pack_u8_images(images),
        e.g. kept in pinned memory by a caller that reuses it); boxes come back in each image's own pixel coordinates."""
        flat, offsets, widths, heights = packed if packed is not None else pack_u8_images(images)
        opts = ln_detect_options(confidence_threshold, nms_threshold, int(letterbox), top_k, max_per_image)
        rec, cnt, own = self._out_buffers(max_per_image, out)
        self.backend._check(self.lib.ln_net_detect_u8(self.h, _ptr(flat), _ptr(offsets), _ptr(widths), _ptr(heights), mode, C.byref(opts),
                                                      _ptr(rec), _ptr(cnt)))
        return [rec[b, :cnt[b]].copy() if own else rec[b, :cnt[b]] for b in range(self.batch)]

    def set_cuda_graph(self, on: bool):
        self.backend._check(self.lib.ln_net_set_cuda_graph(self.h, int(on)))

    def set_host_pipeline(self, on: bool):
        """detect() on host buffers uploads and runs the batch in two overlapping halves (default on)."""
        self.backend._check(self.lib.ln_net_set_host_pipeline(self.h, int(on)))

    def set_fusion(self, on: bool):
        self.backend._check(self.lib.ln_net_set_fusion(self.h, int(on)))

    def set_profile(self, on: bool):
        self.backend._check(self.lib.ln_net_set_profile(self.h, int(on)))

    OP_CLASSES = ["conv_umma", "conv_simt", "conv_stem", "maxpool", "upsample", "route_copy", "shortcut", "quantize"]

    def profile(self):
        """(per-layer ms, {kernel class: (ms, launches)}) of the last profiled 8-bit forward."""
        per_layer = np.zeros(self.num_layers, np.float32)
        per_op = np.zeros(8, np.float32)
        launches = np.zeros(8, np.int32)
        self.backend._check(self.lib.ln_net_profile(self.h, _ptr(per_layer), self.num_layers, _ptr(per_op), _ptr(launches)))
        return per_layer, {n: (float(per_op[i]), int(launches[i])) for i, n in enumerate(self.OP_CLASSES)}

    def last_times_ms(self):
        t = np.zeros(2, np.float32)
        self.lib.ln_net_last_times(self.h, _ptr(t))
        return float(t[0]), float(t[1])
