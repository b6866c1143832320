"""The binary16-storage twin (trait F16TensorOpsBackend, lightnet-cuda/src/lib.rs:6295-6629) through the C ABI, against the
CPU oracle and numpy.  Tolerances are the reference's own: one binary16 rounding for element operators
(docs/OXIDE_BENCH.md:70, 5.2e-4 * |ref| + 1e-7), 1e-3 + 1e-3 * |ref| for a convolution
(lightnet-cuda-oxide/tests/oxide_conv_parity.rs:12), and max|d| <= 5e-3 * max|ref| for the heads of a whole network against
the f32 forward (lightnet-cuda-oxide/tests/oxide_runtime_f16.rs:1-11, 113-133).  Needs a B200: run with -m gpu."""
import numpy as np
import pytest

import lightnet_b200 as ln
from lightnet_b200 import synth, zoo
from oracle import oracle_api as orc

pytestmark = pytest.mark.gpu

F16_ELEMENT = lambda ref: 5.2e-4 * np.abs(ref) + 1e-7
HEAD_TOL = 5e-3


@pytest.fixture(scope="module")
def be():
    b = ln.B200Backend(0)
    yield b
    b.close()


def h(x):
    """binary16 rounding of f32 values, back in f32"""
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def test_upload_download_widen_narrow(be):
    rng = np.random.default_rng(1)
    x = rng.normal(0, 3, (2, 37, 9, 11)).astype(np.float32)     # 37 channels: padded to 64 in storage
    x[0, 0, 0, :4] = [1e6, -1e6, np.inf, 65504.0]               # overflow stays infinite (lib.rs:6307)
    t = be.upload_f16(x.shape, x)
    assert t.dtype == ln.LN_F16 and t.shape == x.shape
    got = be.download_f16(t)
    assert np.array_equal(got, h(x))
    assert np.isinf(got[0, 0, 0, 0]) and got[0, 0, 0, 1] == -np.inf and got[0, 0, 0, 3] == 65504.0
    wide = be.widen_f16(t)
    assert wide.dtype == ln.LN_F32 and np.array_equal(be.download_f32(wide), h(x))
    again = be.narrow_f32_f16(be.upload_f32(x.shape, x))
    assert np.array_equal(be.download_f16(again), h(x))
    with pytest.raises(ln.BackendError):
        be.widen_f16(wide)


# (b, c, h, w, f, k, sx, sy, dil, pad, groups): the geometry cases of lightnet-cuda-oxide/tests/oxide_conv_parity.rs:106-121 (the
# tensor-core kernel takes groups = 1, dilation = 1, sx = sy in {1, 2}; the rest exercise the CUDA-core kernel) and layer shapes
F16_CONV_CASES = [
    (2, 5, 7, 9, 6, 1, 1, 1, 1, 0, 1), (2, 3, 9, 11, 5, 3, 1, 1, 1, 1, 1), (1, 2, 8, 8, 3, 3, 1, 1, 1, 0, 1), (1, 4, 13, 13, 6, 3, 2, 2, 1, 1, 1),
    (2, 3, 10, 12, 4, 3, 2, 1, 1, 1, 1), (3, 3, 15, 13, 5, 5, 2, 2, 1, 2, 1), (2, 4, 9, 7, 6, 3, 1, 1, 1, 1, 2), (2, 6, 9, 9, 6, 3, 1, 1, 1, 1, 6),
    (2, 16, 10, 10, 70, 3, 1, 1, 1, 1, 1),
    (1, 128, 38, 38, 256, 3, 1, 1, 1, 1, 1), (2, 256, 26, 26, 255, 1, 1, 1, 1, 0, 1), (1, 64, 52, 52, 128, 3, 2, 2, 1, 1, 1), (2, 32, 40, 40, 64, 1, 1, 1, 1, 0, 1),
    (1, 16, 64, 64, 32, 3, 1, 1, 1, 1, 1),
]


@pytest.mark.parametrize("case", F16_CONV_CASES)
@pytest.mark.parametrize("act", ["leaky", "mish"])
def test_conv2d_bias_act_f16(be, case, act):
    b, c, hh, w, f, k, sx, sy, dil, pad, g = case
    rng = np.random.default_rng(hash(case) & 0xFFFF)
    x = rng.normal(0, 1, (b, c, hh, w)).astype(np.float32)
    wt = rng.normal(0, np.sqrt(2.0 / (c // g * k * k)), (f, c // g, k, k)).astype(np.float32)
    bias = rng.normal(0, 0.1, f).astype(np.float32)
    oh, ow = (hh + 2 * pad - k) // sy + 1, (w + 2 * pad - k) // sx + 1
    tx = be.upload_f16(x.shape, x)
    w16 = be.conv_weights_f16(be.upload_f32(wt.shape, wt), f, c // g * k * k)
    tb = be.upload_f32((1, f, 1, 1), bias)
    y = be.download_f16(be.conv2d_bias_act_f16(tx, w16, tb, (b, f, oh, ow), c, hh, w, f, k, sx, sy, dil, pad, g, act))
    ref = orc.conv_f32(h(x), h(wt), bias, stride=sx, stride_y=sy, pad=pad, groups=g, act=act)   # binary16 operands, f32 arithmetic
    assert y.shape == ref.shape
    assert np.array_equal(y, h(y))                                # values are binary16
    assert np.all(np.abs(y - ref) <= 1e-3 + 1e-3 * np.abs(ref)), float(np.abs(y - ref).max())
    # a second call reuses the packed operand
    y2 = be.download_f16(be.conv2d_bias_act_f16(tx, w16, tb, (b, f, oh, ow), c, hh, w, f, k, sx, sy, dil, pad, g, act))
    assert np.array_equal(y, y2)


def test_f16_glue(be):
    rng = np.random.default_rng(2)
    x = h(rng.normal(0, 1, (2, 40, 9, 11)))
    tx = be.upload_f16(x.shape, x)
    for size, sx, sy, padding in [(2, 2, 2, 1), (2, 1, 1, 1), (5, 1, 1, 4), (3, 2, 1, 1)]:
        ref = orc.maxpool_f32(x, size, sx, sy, padding)
        y = be.download_f16(be.maxpool_f16(tx, ref.shape, 40, 9, 11, size, sx, sy, padding))
        assert np.array_equal(y, ref)
    up = be.download_f16(be.upsample_f16(tx, (2, 40, 18, 22), 40, 9, 11, 2, 1.0, False))
    assert np.array_equal(up, np.repeat(np.repeat(x, 2, 2), 2, 3))
    up = be.download_f16(be.upsample_f16(tx, (2, 40, 18, 22), 40, 9, 11, 2, 0.3, False))
    assert np.array_equal(up, h(np.float32(0.3) * np.repeat(np.repeat(x, 2, 2), 2, 3)))
    # reverse: binary32 sum of each 2x2 block in (dy, dx) order, times scale, one rounding (half_ops.rs upsample_reverse_f16)
    xe = x[:, :, :8, :10]
    te = be.upload_f16(xe.shape, xe)
    s = ((xe[:, :, 0::2, 0::2] + xe[:, :, 0::2, 1::2]) + xe[:, :, 1::2, 0::2]) + xe[:, :, 1::2, 1::2]
    rv = be.download_f16(be.upsample_f16(te, (2, 40, 4, 5), 40, 8, 10, 2, 0.5, True))
    assert np.array_equal(rv, h(np.float32(0.5) * s))
    with pytest.raises(ln.BackendError) as e:
        be.upsample_f16(tx, (2, 40, 9, 11), 40, 9, 11, 0, 1.0, False)
    assert "stride cannot be zero" in str(e.value)
    # route: whole tensors, and a channel slice that is not a multiple of 8 (groups = 5, group_id = 3)
    x2 = h(rng.normal(0, 1, (2, 24, 9, 11)))
    t2 = be.upload_f16(x2.shape, x2)
    r = be.download_f16(be.route_concat_f16([tx, t2], [0, 0], [40, 24], [40, 24], (2, 64, 9, 11), 99))
    assert np.array_equal(r, np.concatenate([x, x2], 1))
    r = be.download_f16(be.route_concat_f16([t2, tx], [0, 24], [24, 8], [24, 40], (2, 32, 9, 11), 99))
    assert np.array_equal(r, np.concatenate([x2, x[:, 24:32]], 1))
    # shortcut: f16(act(a + b)), the sum in binary32 (half_ops.rs shortcut_add_act_f16)
    x3 = h(rng.normal(0, 1, x.shape))
    t3 = be.upload_f16(x3.shape, x3)
    for act in ("linear", "leaky"):
        ref = x + x3
        ref = ref if act == "linear" else np.where(ref > 0, ref, np.float32(0.1) * ref)
        assert np.array_equal(be.download_f16(be.shortcut_add_act_f16(tx, t3, act)), h(ref))
    sw = be.download_f16(be.shortcut_add_act_f16(tx, t3, "swish"))
    ref = np.array([orc.activate("swish", v) for v in (x + x3).ravel()], np.float32).reshape(x.shape)
    assert np.all(np.abs(sw - ref) <= F16_ELEMENT(ref))
    # shortcut_fit: flat per-sample crop / zero-pad in NCHW order (lib.rs:4041, :6494)
    fit = be.download_f16(be.shortcut_fit_f16(t2, 2, (2, 40, 9, 11)))
    want = np.zeros((2, 40 * 99), np.float32)
    want[:, :24 * 99] = x2.reshape(2, -1)
    assert np.array_equal(fit.reshape(2, -1), want)
    crop = be.download_f16(be.shortcut_fit_f16(tx, 2, (2, 7, 5, 6)))
    assert np.array_equal(crop.reshape(2, -1), x.reshape(2, -1)[:, :7 * 30])
    # per-channel affine (batch-norm inference on binary16, gpu_f16.rs:405-426): f16(act(x * scale[c] + bias[c]))
    sc = rng.normal(1, 0.2, 40).astype(np.float32)
    bi = rng.normal(0, 0.5, 40).astype(np.float32)
    ts, tb = be.upload_f32((1, 40, 1, 1), sc), be.upload_f32((1, 40, 1, 1), bi)
    aff = be.download_f16(be.channel_affine_act_f16(tx, ts, tb, 40, 99, "linear"))
    assert np.array_equal(aff, h((x * sc[None, :, None, None]).astype(np.float32) + bi[None, :, None, None]))
    aff = be.download_f16(be.channel_affine_act_f16(tx, None, tb, 40, 99, "relu"))
    assert np.array_equal(aff, h(np.maximum(x + bi[None, :, None, None], 0)))
    # channel_scale_f32 (lib.rs:485) of the f32 trait
    xf = rng.normal(0, 1, (2, 40, 9, 11)).astype(np.float32)
    got = be.download_f32(be.channel_scale_f32(be.upload_f32(xf.shape, xf), ts, 40, 99))
    assert np.array_equal(got, xf * sc[None, :, None, None])


def run_f16_network(be, cfg, batch, seed, size):
    o = orc.Net(cfg, batch)
    blob = synth.he_weights(o.layers(), seed, bn_identity=False)
    o.set_weights(blob)
    x = synth.uniform_images(batch, 3, size[1], size[0], seed + 1)
    o.forward_f32(x, folded=False)
    net = ln.GpuExecutableNetwork(be, cfg, batch, ln.LN_F16)
    net.load_weights(blob)
    net.forward(x)
    return o, net, x


def test_yolov3_tiny_f16_heads(be):
    """forward_compact_f16 replayed over the twin: heads within the reference's whole-network bound of the f32 CPU forward."""
    cfg = zoo.yolov3_tiny_cfg()
    o, net, x = run_f16_network(be, cfg, 1, 61, (416, 416))
    worst = 0.0
    for k, layer in enumerate([16, 23]):
        ref = o.layer_output_f32(layer)
        got = be.download_f32(net.head(k))
        assert np.isfinite(got).all()
        worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    print("yolov3-tiny binary16 heads: scale-normalised error %.3e" % worst)
    assert worst <= HEAD_TOL
    # intermediate outputs are binary16 tensors (here: the route + upsample branch)
    mid = be.download_f16(net.layer_output(20))
    ref = o.layer_output_f32(20)
    assert np.abs(mid - ref).max() <= HEAD_TOL * np.abs(ref).max()
    # detections: same records as the f32 path up to the tolerance on the scores
    dets = net.detect(x, 640, 480, 0.25, 0.45, True, 0, 256)
    f32net = ln.GpuExecutableNetwork(be, cfg, 1, ln.LN_F32)
    f32net.load_weights(synth.he_weights(o.layers(), 61, bn_identity=False))
    ref_dets = f32net.detect(x, 640, 480, 0.25, 0.45, True, 0, 256)
    assert abs(len(dets[0]) - len(ref_dets[0])) <= max(2, len(ref_dets[0]) // 50)


def test_yolov4_608_f16_heads(be):
    cfg = zoo.yolov4_cfg(batch=1)
    o = orc.Net(cfg, 1)
    blob = synth.he_weights(o.layers(), 0)
    o.set_weights(blob)
    x = synth.uniform_images(1, 3, 608, 608, 71)
    o.forward_f32(x)
    net = ln.GpuExecutableNetwork(be, cfg, 1, ln.LN_F16)
    net.load_weights(blob)
    net.forward(x)
    yolo = [i for i, l in enumerate(o.layers()) if l["kind"] == "yolo"]
    worst = 0.0
    for k, layer in enumerate(yolo):
        ref, got = o.layer_output_f32(layer), be.download_f32(net.head(k))
        assert np.isfinite(got).all()
        worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    print("YOLOv4-608 binary16 heads: scale-normalised error %.3e" % worst)
    assert worst <= HEAD_TOL
