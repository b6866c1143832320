"""Anchor-free heads ([yolox], [ppyoloe], [yolonas]) on the device: the output activation (lightnet-cuda/src/lib.rs:4884), the
distribution-head box decode (lib.rs:4936) and their candidates through the same device decode + NMS as [yolo] heads
(decode_modern_detections, lightnet-train/src/detect.rs:1035, as decode_network_detections calls it), against the oracle."""
import numpy as np
import pytest

import lightnet_b200 as ln
from oracle import oracle_api as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    return ln.B200Backend(0)


def random_head(rng, batch, channels, g, spread):
    x = rng.normal(0.0, spread, (batch, channels, g, g)).astype(np.float32)
    return x


def test_modern_activation_matches_the_oracle(be):
    rng = np.random.default_rng(1)
    classes = 7
    x = random_head(rng, 3, 4 + 1 + classes, 13, 6.0)
    x[0, 2, 3, 4] = np.nan
    x[1, 5, 0, 0] = np.inf
    x[2, 4, 12, 12] = -np.inf
    x[0, 6, 1, 1] = 80.0
    x[0, 7, 1, 1] = -80.0
    want = orc.modern_activate(x, classes)
    got = be.download_f32(be.modern_yolo_forward_f32(be.upload_f32(x.shape, x), classes))
    assert got.shape == want.shape
    # box entries are copied (sanitised); probabilities: the device's expf is within 2 ulp of libm's
    assert np.array_equal(got[:, :4], want[:, :4])
    assert np.abs(got[:, 4:] - want[:, 4:]).max() <= 2e-7
    assert got[0, 2, 3, 4] == 0.0 and got[1, 5, 0, 0] == 0.5 and got[2, 4, 12, 12] == 0.5


@pytest.mark.parametrize("reg_max,g", [(3, 20), (16, 13), (1, 8)])
def test_modern_predecode_matches_the_oracle(be, reg_max, g):
    rng = np.random.default_rng(reg_max)
    classes, coords = 5, 4 * (reg_max + 1)
    x = random_head(rng, 2, coords + 1 + classes, g, 3.0)
    x[0, 1, 2, 3] = np.nan
    x[1, 0, 0, 0] = 1e30
    act = orc.modern_activate(x, classes)
    want = orc.modern_predecode(act, classes, coords)
    got = be.download_f32(be.modern_yolo_predecode_f32(be.upload_f32(act.shape, act), classes, coords, 1))
    assert got.shape == (2, 5 + classes, g, g)
    assert np.array_equal(got[:, 4:], want[:, 4:])                    # objectness and class planes are copies
    assert np.abs(got[:, :4] - want[:, :4]).max() <= 1e-5             # expectation of a softmax: a few ulp of the f32 sums
    with pytest.raises(ln.BackendError):
        be.modern_yolo_predecode_f32(be.upload_f32(act.shape, act), classes, coords + 4, 1)   # channel count mismatch
    with pytest.raises(ln.BackendError):
        be.modern_yolo_predecode_f32(be.upload_f32(act.shape, act), classes, coords, 0)       # yolox has nothing to predecode


def records_equal(got, want):
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("letterbox", [False, True])
def test_yolox_heads_decode_and_nms_like_the_oracle(be, letterbox):
    rng = np.random.default_rng(5)
    batch, classes = 3, 6
    grids = (20, 10)
    raws = []
    for g in grids:
        x = random_head(rng, batch, 5 + classes, g, 1.0)
        x[:, 0:2] = rng.uniform(-0.5, 1.5, x[:, 0:2].shape)       # centre offsets
        x[:, 2:4] = rng.normal(1.2, 0.6, x[:, 2:4].shape)         # log sizes in cells: boxes that overlap their neighbours
        x[:, 4] = rng.normal(0.0, 2.5, x[:, 4].shape)
        x[:, 5:] = rng.normal(0.0, 2.5, x[:, 5:].shape)
        x[0, 2, 1, 1] = 40.0                                       # clamped to 10 by the decoder
        raws.append(orc.modern_activate(x, classes))
    heads = [dict(raw=be.upload_f32(r.shape, r), classes=classes, anchors=[(1, 1)], kind=1) for r in raws]
    iw, ih = [640, 500, 333], [480, 500, 200]
    got = be.yolo_decode_nms(heads, 320, 320, iw, ih, 0.3, 0.45, letterbox, 0, 2048)
    for b in range(batch):
        spec = [dict(gw=g, gh=g, classes=classes, anchors=[(1, 1)], kind=1) for g in grids]
        want = orc.decode_nms([r[b] for r in raws], spec, 320, 320, iw[b], ih[b], 0.3, 0.45, letterbox, det_exp=True)
        no_pre = orc.decode_nms([r[b] for r in raws], spec, 320, 320, iw[b], ih[b], 0.3, 0.45, letterbox, det_exp=True, skip_pass1=True)
        assert np.array_equal(want, no_pre)          # the IoU > 1.0 pre-pass the device does not run is a no-op on this input
        assert want.shape[0] > 40
        records_equal(got[b], want)
        # decode alone, in emission order
        cand = be.yolo_decode_only(heads, b, 320, 320, iw[b], ih[b], 0.3, letterbox)
        want_c = orc.decode_only([r[b] for r in raws], spec, 320, 320, iw[b], ih[b], 0.3, letterbox, det_exp=True)
        records_equal(cand, want_c)


def test_distribution_heads_decode_and_nms_like_the_oracle(be):
    rng = np.random.default_rng(9)
    batch, classes, reg_max = 2, 4, 7
    coords = 4 * (reg_max + 1)
    grids = (16, 8)
    pre_host, heads = [], []
    for g in grids:
        x = random_head(rng, batch, coords + 1 + classes, g, 2.0)
        x[:, coords] = rng.normal(-1.0, 2.0, x[:, coords].shape)        # a quality logit that is low on most of the map
        act = be.modern_yolo_forward_f32(be.upload_f32(x.shape, x), classes)
        pre = be.modern_yolo_predecode_f32(act, classes, coords, 2)
        heads.append(dict(raw=pre, classes=classes, anchors=[(1, 1)], kind=2))
        pre_host.append(be.download_f32(pre))
    got = be.yolo_decode_nms(heads, 256, 256, [640, 300], [480, 400], 0.6, 0.5, True, 0, 2048)
    for b in range(batch):
        spec = [dict(gw=g, gh=g, classes=classes, anchors=[(1, 1)], kind=2) for g in grids]
        want = orc.decode_nms([p[b] for p in pre_host], spec, 256, 256, [640, 300][b], [480, 400][b], 0.6, 0.5, True, det_exp=True)
        assert want.shape[0] > 20
        # the score is the class score (never below objectness * class), the record keeps the real objectness
        assert np.all(want[:, 1] >= want[:, 2] * want[:, 1] - 1e-7)
        records_equal(got[b], want)


def test_reference_vectors_through_the_device(be):
    # detect.rs:2472-2512: two adjacent cells fire on class 1, NMS merges them; a high threshold keeps nothing
    data = np.zeros((1, 7, 4, 4), np.float32)
    for loc in (0, 1):
        data[0, 2, 0, loc] = np.log(np.float32(4.0))
        data[0, 3, 0, loc] = np.log(np.float32(4.0))
        data[0, 4, 0, loc] = 0.99
        data[0, 6, 0, loc] = 0.98
    head = [dict(raw=be.upload_f32(data.shape, data), classes=2, anchors=[(1, 1)], kind=1)]
    d = be.yolo_decode_nms(head, 16, 16, 16, 16, 0.9, 0.45, False, 0, 16)[0]
    assert d.shape[0] == 1 and d[0, 0] == 1
    assert be.yolo_decode_nms(head, 16, 16, 16, 16, 0.995, 0.45, False, 0, 16)[0].shape[0] == 0
    # detect.rs:2557-2600: every side collapses onto bin 2 around cell (row 2, col 1)
    bins, coords = 4, 16
    x = np.zeros((1, coords + 2, 4, 4), np.float32)
    for side in range(4):
        x[0, side * bins + 2, 2, 1] = 40.0
    x[0, coords, 2, 1] = 40.0
    x[0, coords + 1, 2, 1] = 40.0
    pre = be.modern_yolo_predecode_f32(be.modern_yolo_forward_f32(be.upload_f32(x.shape, x), 1), 1, coords, 1)
    d = be.yolo_decode_nms([dict(raw=pre, classes=1, anchors=[(1, 1)], kind=2)], 16, 16, 16, 16, 0.6, 0.45, False, 0, 16)[0]
    assert d.shape[0] == 1 and np.allclose(d[0, 3:6], [6.0, 10.0, 16.0], atol=1e-2)
    with pytest.raises(ln.BackendError):   # anchor-free heads take one box per cell
        be.yolo_decode_nms([dict(raw=pre, classes=1, anchors=[(1, 1), (2, 2)], kind=2)], 16, 16, 16, 16, 0.6, 0.45, False, 0, 16)


BACKBONE = """
[net]
batch=2
width=64
height=64
channels=3
[convolutional]
batch_normalize=1
filters=32
size=3
stride=2
pad=1
activation=mish
[convolutional]
batch_normalize=1
filters=64
size=3
stride=2
pad=1
activation=mish
[convolutional]
batch_normalize=1
filters=64
size=3
stride=1
pad=1
activation=leaky
"""


def head_cfg(filters, section):
    return BACKBONE + "[convolutional]\nfilters=%d\nsize=1\nstride=1\npad=1\nactivation=linear\n%s" % (filters, section)


@pytest.mark.parametrize("name,classes,reg_max", [("yolox", 3, 0), ("ppyoloe", 4, 3), ("yolonas", 2, 7)])
def test_network_with_an_anchor_free_head(be, name, classes, reg_max):
    """cfg -> layers -> int8 forward -> the head layer's forward (activation, device box decode) -> decode + NMS, against the
    oracle's integer forward of the same backbone (its head section is a one-anchor [yolo] of the same channel count, which
    leaves the convolutions' output untouched) followed by the oracle's modern-head functions."""
    import lightnet_b200.synth as synth
    coords = 4 if name == "yolox" else 4 * (reg_max + 1)
    filters = coords + 1 + classes
    section = "[%s]\nclasses=%d\n%s" % (name, classes, "" if name == "yolox" else "reg_max=%d\n" % reg_max)
    o = orc.Net(head_cfg(filters, "[yolo]\nmask=0\nanchors=1,1\nclasses=%d\nnum=1\n" % (filters - 5)), 2)
    blob = synth.he_weights(o.layers(), 17, bn_identity=False)
    x = synth.uniform_images(2, 3, 64, 64, 18)
    net = ln.GpuExecutableNetwork(be, head_cfg(filters, section), 2, ln.LN_Q8)
    net.load_weights(blob)
    net.calibrate(x)
    o.set_weights(blob)
    o.forward_f32(x, folded=True)
    o.calibrate()
    o.set_scales(net.scales())
    be.set_exact_epilogue(True)
    try:
        dets = net.detect(x, [640, 300], [480, 400], 0.3, 0.45, True, 0, 1024)
        head = be.download_f32(net.head(0))
    finally:
        be.set_exact_epilogue(False)
    o.forward_q8(x)
    raw = o.head_q8(len(o.layers()) - 1)
    assert raw.shape == (2, filters, 16, 16)
    want = orc.modern_activate(raw, classes)
    kind = 1
    if name != "yolox":
        want = orc.modern_predecode(want, classes, coords)
        kind = 2
    assert head.shape == want.shape == (2, 5 + classes, 16, 16)
    assert np.abs(head - want).max() <= 1e-5       # same integer convolutions; expf against libm's exp in the activation
    spec = [dict(gw=16, gh=16, classes=classes, anchors=[(1, 1)], kind=kind)]
    total = 0
    for b in range(2):
        ref = orc.decode_nms([head[b]], spec, 64, 64, [640, 300][b], [480, 400][b], 0.3, 0.45, True, det_exp=True)
        assert np.array_equal(dets[b], ref)
        total += ref.shape[0]
    assert total > 10
