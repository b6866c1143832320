"""ctypes binding of the CPU oracle (oracle/lightnet_oracle.cpp).

Test infrastructure only: imported by tests/, by the smoke entry and by the bench's
cpu_baseline / reference legs as the checker.  The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "build", "liblightnet_oracle.so")

ACT = {"linear": 0, "logistic": 1, "leaky": 2, "mish": 3, "swish": 4, "relu": 5}
KIND = {0: "conv", 1: "maxpool", 2: "route", 3: "shortcut", 4: "upsample", 5: "yolo"}


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the library is missing or stale."""
    src = os.path.join(_HERE, "lightnet_oracle.cpp")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.orc_last_error.restype = C.c_char_p
        L.orc_net_create.restype = C.c_void_p
        L.orc_net_create.argtypes = [C.c_char_p, C.c_int]
        L.orc_net_destroy.argtypes = [C.c_void_p]
        L.orc_net_num_layers.argtypes = [C.c_void_p]
        L.orc_net_layer_info.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_net_dims.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_net_layer_sources.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.orc_net_weight_count.restype = C.c_longlong
        L.orc_net_weight_count.argtypes = [C.c_void_p]
        L.orc_net_set_weights.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong]
        L.orc_net_forward_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.orc_net_layer_output_f32.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_net_calibrate.argtypes = [C.c_void_p]
        L.orc_net_get_amax.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_net_get_scales.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_net_set_scales.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.orc_net_forward_q8.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_net_forward_f8.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_net_calibrate_qmax.argtypes = [C.c_void_p, C.c_float]
        L.orc_net_layer_output_f8.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_net_head_f8.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_f32_to_e4m3_fast.restype = C.c_ubyte
        L.orc_f32_to_e4m3_fast.argtypes = [C.c_float]
        L.orc_net_layer_output_q8.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_net_head_q8.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_net_conv_quant.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_net_detect.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int,
                                     C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_decode_nms.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_decode_only.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_nms_records.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_int]
        L.orc_nms_records_by_class.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_int]
        L.orc_nms_records_first_k.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int]
        L.orc_conv_q8_acc.argtypes = [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p] + [C.c_int] * 5 + [C.c_void_p]
        L.orc_conv_q8_acc_grouped.argtypes = [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p]
        L.orc_image_from_u8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.orc_image_resize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_image_resize_exact_u8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_image_letterbox.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_image_fit_inside.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_f8_epilogue.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        L.orc_conv_f8_acc.argtypes = [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p, C.c_void_p]
        L.orc_q8_epilogue.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_float,
                                      C.c_void_p, C.c_void_p]
        L.orc_conv_f32.argtypes = [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p, C.c_void_p] + [C.c_int] * 7 + [C.c_void_p]
        L.orc_maxpool_f32.argtypes = [C.c_void_p] + [C.c_int] * 8 + [C.c_void_p]
        for name in ("orc_activate", "orc_det_activate"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_int, C.c_float]
        L.orc_det_expf.restype = C.c_float
        L.orc_det_expf.argtypes = [C.c_float]
        L.orc_bbox_iou.restype = C.c_float
        L.orc_bbox_iou.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_f32_to_e4m3.restype = C.c_ubyte
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_ubyte]
        L.orc_quant_i8.restype = C.c_int8
        L.orc_quant_i8.argtypes = [C.c_float, C.c_float]
        L.orc_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _err():
    return lib().orc_last_error().decode()


class OracleError(RuntimeError):
    pass


class Net:
    """The oracle's executable network: cfg text -> layers -> f32 / int8 forward -> detections."""

    def __init__(self, cfg_text: str, batch: int = 0):
        self.h = lib().orc_net_create(cfg_text.encode(), batch)
        if not self.h:
            raise OracleError(_err())
        d = np.zeros(4, np.int32)
        lib().orc_net_dims(self.h, _p(d))
        self.width, self.height, self.channels, self.batch = (int(v) for v in d)
        self.num_layers = lib().orc_net_num_layers(self.h)

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_net_destroy(self.h)
            self.h = None

    def layer_info(self, i):
        v = np.zeros(20, np.int32)
        if lib().orc_net_layer_info(self.h, i, _p(v)):
            raise IndexError(i)
        keys = ["kind", "in_w", "in_h", "in_c", "in_b", "out_w", "out_h", "out_c", "out_b", "filters", "size", "stride_x",
                "stride_y", "padding", "bn", "act", "groups", "dilation"]
        d = dict(zip(keys, (int(x) for x in v)))
        d["kind"] = KIND[d["kind"]]
        src = np.zeros(16, np.int32)
        n = lib().orc_net_layer_sources(self.h, i, _p(src), 16)
        d["sources"] = [int(x) for x in src[:n]]
        return d

    def layers(self):
        return [self.layer_info(i) for i in range(self.num_layers)]

    def weight_count(self) -> int:
        return int(lib().orc_net_weight_count(self.h))

    def set_weights(self, w: np.ndarray):
        w = np.ascontiguousarray(w, np.float32)
        if lib().orc_net_set_weights(self.h, _p(w), w.size):
            raise OracleError(_err())

    def forward_f32(self, x: np.ndarray, folded: bool = False):
        x = np.ascontiguousarray(x, np.float32)
        assert x.size == self.batch * self.channels * self.height * self.width
        if lib().orc_net_forward_f32(self.h, _p(x), 1 if folded else 0):
            raise OracleError(_err())

    def out_shape(self, i):
        d = self.layer_info(i)
        return (d["out_b"], d["out_c"], d["out_h"], d["out_w"])

    def layer_output_f32(self, i):
        out = np.zeros(self.out_shape(i), np.float32)
        if lib().orc_net_layer_output_f32(self.h, i, _p(out)):
            raise OracleError("no f32 output for layer %d" % i)
        return out

    def calibrate(self):
        if lib().orc_net_calibrate(self.h):
            raise OracleError(_err())

    def amax(self):
        out = np.zeros(self.num_layers + 1, np.float32)
        lib().orc_net_get_amax(self.h, _p(out))
        return out

    def scales(self):
        out = np.zeros(self.num_layers + 1, np.float32)
        lib().orc_net_get_scales(self.h, _p(out))
        return out

    def set_scales(self, s):
        s = np.ascontiguousarray(s, np.float32)
        if lib().orc_net_set_scales(self.h, _p(s), s.size):
            raise OracleError("scale count mismatch")

    def calibrate_f8(self):
        if lib().orc_net_calibrate_qmax(self.h, 448.0):
            raise OracleError(_err())

    def forward_f8(self, x):
        x = np.ascontiguousarray(x, np.float32)
        if lib().orc_net_forward_f8(self.h, _p(x)):
            raise OracleError(_err())

    def layer_output_f8(self, i):
        out = np.zeros(self.out_shape(i), np.uint8)
        if lib().orc_net_layer_output_f8(self.h, i, _p(out)):
            raise OracleError("no fp8 output for layer %d" % i)
        return out

    def head_f8(self, i):
        out = np.zeros(self.out_shape(i), np.float32)
        if lib().orc_net_head_f8(self.h, i, _p(out)):
            raise OracleError("layer %d is not a head of the fp8 run" % i)
        return out

    def forward_q8(self, x):
        x = np.ascontiguousarray(x, np.float32)
        if lib().orc_net_forward_q8(self.h, _p(x)):
            raise OracleError(_err())

    def layer_output_q8(self, i):
        out = np.zeros(self.out_shape(i), np.int8)
        if lib().orc_net_layer_output_q8(self.h, i, _p(out)):
            raise OracleError("no int8 output for layer %d" % i)
        return out

    def head_q8(self, i):
        out = np.zeros(self.out_shape(i), np.float32)
        if lib().orc_net_head_q8(self.h, i, _p(out)):
            raise OracleError("layer %d is not a head of the int8 run" % i)
        return out

    def conv_quant(self, i):
        d = self.layer_info(i)
        n = d["filters"] * d["in_c"] * d["size"] * d["size"]
        wq = np.zeros(n, np.int8)
        ws = np.zeros(d["filters"], np.float32)
        fb = np.zeros(d["filters"], np.float32)
        if lib().orc_net_conv_quant(self.h, i, _p(wq), _p(ws), _p(fb)):
            raise OracleError("layer %d is not a convolution" % i)
        return wq.reshape(d["filters"], d["in_c"], d["size"], d["size"]), ws, fb

    def detect(self, source, b, img_w, img_h, thr=0.25, nms=0.45, letterbox=True, top_k=0, det_exp=False,
               skip_pass1=False, max_out=1 << 20):
        """source: 'f32' or 'q8'.  Returns an (n,7) array {class, conf, obj, x, y, w, h}."""
        out = np.zeros((max_out, 7), np.float32)
        n = lib().orc_net_detect(self.h, 0 if source == "f32" else 1, b, img_w, img_h, thr, nms, int(letterbox), top_k,
                                 int(det_exp), int(skip_pass1), _p(out), max_out)
        if n < 0:
            raise OracleError(_err())
        return out[: min(n, max_out)].copy()


def _head_args(heads, specs):
    """heads: list of float32 arrays (one image each, [A*(5+cls), gh, gw]); specs: list of dicts
    {gw, gh, classes, anchors:[(w,h),...], scale_x_y, new_coords, kind}; kind 1 = an activated [yolox] head, 2 = a distribution
    head after modern_predecode (both take one dummy anchor)."""
    arrs = [np.ascontiguousarray(h, np.float32) for h in heads]
    ptrs = (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    meta = np.zeros((len(specs), 8), np.float32)
    anchors = []
    for k, s in enumerate(specs):
        meta[k, :7] = [s["gw"], s["gh"], s["classes"], len(s["anchors"]), s.get("scale_x_y", 1.0), s.get("new_coords", 0), s.get("kind", 0)]
        for a in s["anchors"]:
            anchors += [a[0], a[1]]
    return arrs, ptrs, meta, np.asarray(anchors, np.float32)


def decode_nms(heads, specs, net_w, net_h, img_w, img_h, thr, nms, letterbox=False, top_k=0, det_exp=False,
               skip_pass1=False, max_out=1 << 20):
    arrs, ptrs, meta, anchors = _head_args(heads, specs)
    out = np.zeros((max_out, 7), np.float32)
    n = lib().orc_decode_nms(len(arrs), ptrs, _p(meta), _p(anchors), net_w, net_h, img_w, img_h, thr, nms, int(letterbox),
                             top_k, int(det_exp), int(skip_pass1), _p(out), max_out)
    if n < 0:
        raise OracleError(_err())
    return out[: min(n, max_out)].copy()


def decode_only(heads, specs, net_w, net_h, img_w, img_h, thr, letterbox=False, det_exp=False, max_out=1 << 22):
    arrs, ptrs, meta, anchors = _head_args(heads, specs)
    out = np.zeros((max_out, 7), np.float32)
    n = lib().orc_decode_only(len(arrs), ptrs, _p(meta), _p(anchors), net_w, net_h, img_w, img_h, thr, int(letterbox),
                              int(det_exp), _p(out), max_out)
    if n < 0:
        raise OracleError(_err())
    if n > max_out:
        raise OracleError("decode_only: %d candidates exceed max_out" % n)
    return out[:n].copy()


def modern_activate(x, classes):
    """modern_yolo_forward_f32 (lightnet-cuda/src/lib.rs:4884): NCHW head -> sanitised, objectness and classes through a sigmoid."""
    y = np.ascontiguousarray(x, np.float32).copy()
    b, c, h, w = y.shape
    L = lib()
    L.orc_modern_activate.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
    L.orc_modern_activate(_p(y), b, c, h * w, classes)
    return y


def modern_predecode(act, classes, coords):
    """modern_yolo_predecode (lightnet-cuda-oxide/src/kernels/dense_loss.rs:788): [B, coords + 1 + classes, H, W] -> [B, 5 + classes, H, W]."""
    a = np.ascontiguousarray(act, np.float32)
    b, c, h, w = a.shape
    assert c == coords + 1 + classes
    out = np.zeros((b, 5 + classes, h, w), np.float32)
    L = lib()
    L.orc_modern_predecode.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    L.orc_modern_predecode(_p(a), _p(out), b, w, h, classes, coords)
    return out


def nms_records(recs, nms, top_k=0, skip_pass1=False, by_class=False):
    """The NMS sequence of decode_network_detections on records in emission order.  by_class=True runs it class by
    class (classes never interact in apply_nms): same result, cost quadratic in the class sizes instead of the total."""
    r = np.ascontiguousarray(recs, np.float32).copy()
    fn = lib().orc_nms_records_by_class if by_class else lib().orc_nms_records
    n = fn(_p(r), r.shape[0], nms, top_k, int(skip_pass1))
    return r[:n].copy()


def nms_records_first_k(recs, nms, k):
    """First k records of the sorted-list NMS pass (no thr = 1.0 pre-pass), stopping once k rows are kept."""
    r = np.ascontiguousarray(recs, np.float32).copy()
    n = lib().orc_nms_records_first_k(_p(r), r.shape[0], nms, k)
    return r[:n].copy()


def region_forward(x, anchors, entries, classes, softmax_classes):
    """lightnet-cuda/src/host_ops.rs:73-116 region_forward, loop for loop (small cases): [B, A*E, H, W] -> [B, H*W, A, E] flat."""
    x = np.asarray(x, np.float32)
    B, Cc, H, W = x.shape
    assert Cc == anchors * entries and entries >= classes + 5
    spatial = H * W
    flat = x.reshape(B, Cc, spatial)
    out = np.zeros((B, spatial, anchors, entries), np.float32)
    for b in range(B):
        for s in range(spatial):
            for a in range(anchors):
                row = flat[b, a * entries:(a + 1) * entries, s].copy()
                row[4] = np.float32(1.0) / (np.float32(1.0) + np.exp(-row[4], dtype=np.float32))
                if softmax_classes:
                    cls = row[5:5 + classes]
                    mx = np.float32(-np.inf) if classes == 0 else cls.max()
                    e = np.exp(cls - mx, dtype=np.float32)
                    total = np.float32(0)
                    for v in e:
                        total = np.float32(total + v)
                    row[5:5 + classes] = e / total if total > 0 else e
                out[b, s, a] = row
    return out


def yolo_activate(x, classes, scale_xy, new_coords):
    """lightnet-cuda/src/lib.rs:4951-4966 yolo_activate_f32 default body."""
    x = np.asarray(x, np.float32)
    B, Cc, H, W = x.shape
    entries = classes + 5
    out = x.copy().reshape(B, Cc // entries, entries, H * W)
    if not new_coords:
        keep = [e for e in range(entries) if e not in (2, 3)]
        out[:, :, keep] = np.float32(1.0) / (np.float32(1.0) + np.exp(-out[:, :, keep], dtype=np.float32))
    s = np.float32(scale_xy)
    out[:, :, :2] = out[:, :, :2] * s - np.float32(0.5) * (s - np.float32(1.0))
    return out.reshape(x.shape)


def conv_q8_acc(x, wq, stride=1, pad=0, groups=1):
    """x int8 NCHW, wq int8 [F, C/groups, k, k] -> int32 NCHW accumulators."""
    x = np.ascontiguousarray(x, np.int8)
    wq = np.ascontiguousarray(wq, np.int8)
    B, Cc, H, W = x.shape
    F, cpg, k, _ = wq.shape
    assert cpg * groups == Cc and F % groups == 0
    OH = (H + 2 * pad - k) // stride + 1
    OW = (W + 2 * pad - k) // stride + 1
    acc = np.zeros((B, F, OH, OW), np.int32)
    lib().orc_conv_q8_acc_grouped(_p(x), B, Cc, H, W, _p(wq), F, k, stride, stride, pad, groups, _p(acc))
    return acc


def q8_epilogue(acc, mult, bias, act, inv_sy):
    acc = np.ascontiguousarray(acc, np.int32)
    B, F, OH, OW = acc.shape
    mult = np.ascontiguousarray(mult, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    of = np.zeros(acc.shape, np.float32)
    oq = np.zeros(acc.shape, np.int8)
    lib().orc_q8_epilogue(_p(acc), B, F, OH * OW, _p(mult), _p(bias), ACT[act] if isinstance(act, str) else act,
                          float(inv_sy), _p(of), _p(oq))
    return of, oq


def f8_epilogue(acc, mult, bias, act, inv_sy):
    acc = np.ascontiguousarray(acc, np.float32)
    B, F, OH, OW = acc.shape
    mult = np.ascontiguousarray(mult, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    of = np.zeros(acc.shape, np.float32)
    oq = np.zeros(acc.shape, np.uint8)
    lib().orc_f8_epilogue(_p(acc), B, F, OH * OW, _p(mult), _p(bias), ACT[act] if isinstance(act, str) else act,
                          float(inv_sy), _p(of), _p(oq))
    return of, oq


def conv_f8_acc(x, w, stride, pad):
    """E4M3 code convolution in double: returns (acc, l1), both float64 NCHW."""
    x = np.ascontiguousarray(x, np.uint8)
    w = np.ascontiguousarray(w, np.uint8)
    B, Cc, H, W = x.shape
    F, _, k, _ = w.shape
    OH = (H + 2 * pad - k) // stride + 1
    OW = (W + 2 * pad - k) // stride + 1
    acc = np.zeros((B, F, OH, OW), np.float64)
    l1 = np.zeros((B, F, OH, OW), np.float64)
    lib().orc_conv_f8_acc(_p(x), B, Cc, H, W, _p(w), F, k, stride, pad, _p(acc), _p(l1))
    return acc, l1


def f32_to_e4m3_array(v):
    v = np.ascontiguousarray(v, np.float32)
    return np.array([f32_to_e4m3_fast(t) for t in v.ravel()], np.uint8).reshape(v.shape)


def conv_f32(x, w, bias, stride=1, pad=0, groups=1, act="linear", stride_y=None):
    """`stride` is the stride in x; stride_y defaults to it (the reference's geometry case sx2_sy1 has two)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    B, Cc, H, W = x.shape
    F, _, k, _ = w.shape
    sy = stride if stride_y is None else stride_y
    OH = (H + 2 * pad - k) // sy + 1
    OW = (W + 2 * pad - k) // stride + 1
    y = np.zeros((B, F, OH, OW), np.float32)
    lib().orc_conv_f32(_p(x), B, Cc, H, W, _p(w), _p(bias), F, k, stride, sy, pad, groups, ACT[act], _p(y))
    return y


def maxpool_f32(x, size, stride_x, stride_y, padding):
    x = np.ascontiguousarray(x, np.float32)
    B, Cc, H, W = x.shape
    OH = max(H + padding - size, 0) // stride_y + 1
    OW = max(W + padding - size, 0) // stride_x + 1
    y = np.zeros((B, Cc, OH, OW), np.float32)
    lib().orc_maxpool_f32(_p(x), B, Cc, H, W, size, stride_x, stride_y, padding, _p(y))
    return y


def activate(act, v):
    return float(lib().orc_activate(ACT[act], float(v)))


def det_activate(act, v):
    return float(lib().orc_det_activate(ACT[act], float(v)))


def det_expf(v):
    return float(lib().orc_det_expf(float(v)))


def bbox_iou(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return float(lib().orc_bbox_iou(_p(a), _p(b)))


def f32_to_e4m3(v):
    return int(lib().orc_f32_to_e4m3(float(v)))


def e4m3_to_f32(b):
    return float(lib().orc_e4m3_to_f32(int(b)))


def f32_to_e4m3_fast(v):
    return int(lib().orc_f32_to_e4m3_fast(float(v)))


def e4m3_table():
    """Value of every E4M3 code (NaN codes as nan)."""
    return np.array([e4m3_to_f32(c) for c in range(256)], np.float32)


def image_from_u8(rgb):
    """u8 [H, W, 3] interleaved -> f32 [3, H, W] (PlanarRgbImage::from_interleaved_rgb_u8)."""
    rgb = np.ascontiguousarray(rgb, np.uint8)
    h, w, _ = rgb.shape
    out = np.zeros((3, h, w), np.float32)
    lib().orc_image_from_u8(_p(rgb), w, h, _p(out))
    return out


def image_resize(planar, w, h):
    """Darknet float resize of f32 [C, H, W] (PlanarRgbImage::resize)."""
    planar = np.ascontiguousarray(planar, np.float32)
    c, sh, sw = planar.shape
    out = np.zeros((c, h, w), np.float32)
    lib().orc_image_resize(_p(planar), sw, sh, c, w, h, _p(out))
    return out


def image_resize_exact_u8(rgb, w, h):
    """OpenCV INTER_LINEAR_EXACT on u8 [H, W, 3] (PlanarRgbImage::resize_linear_exact)."""
    rgb = np.ascontiguousarray(rgb, np.uint8)
    sh, sw, _ = rgb.shape
    out = np.zeros((h, w, 3), np.uint8)
    lib().orc_image_resize_exact_u8(_p(rgb), sw, sh, w, h, _p(out))
    return out


def image_letterbox(planar, w, h):
    planar = np.ascontiguousarray(planar, np.float32)
    c, sh, sw = planar.shape
    out = np.zeros((c, h, w), np.float32)
    lib().orc_image_letterbox(_p(planar), sw, sh, c, w, h, _p(out))
    return out


def image_fit_inside(sw, sh, dw, dh):
    nw, nh = C.c_int(), C.c_int()
    lib().orc_image_fit_inside(sw, sh, dw, dh, C.byref(nw), C.byref(nh))
    return nw.value, nh.value


def set_threads(n):
    lib().orc_set_threads(int(n))
