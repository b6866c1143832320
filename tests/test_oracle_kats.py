"""Pins the CPU oracle against the known-answer tests the reference carries for the
detector-inference path.  Each test names the reference test it re-encodes
(paths inside the lightnet project).  CPU only.
"""
import csv
import math
import os

import numpy as np
import pytest

from oracle import oracle_api as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def weights_blob(*arrays):
    return np.concatenate([np.asarray(a, np.float32).ravel() for a in arrays])


# --- lightnet-train/src/detect.rs:1806-1867 new_coords_head_is_decoded_without_sigmoid
def test_decode_new_coords_kat():
    cfg = """
    [net]
    width=32
    height=32
    channels=6
    [maxpool]
    size=32
    stride=32
    [yolo]
    mask=0
    anchors=10,12
    classes=1
    num=1
    scale_x_y=1.2
    new_coords=1
    """
    net = orc.Net(cfg)
    assert net.out_shape(1) == (1, 6, 1, 1)
    head = np.array([0.5, 0.25, 0.5, 0.25, 0.9, 0.8], np.float32).reshape(6, 1, 1)
    spec = dict(gw=1, gh=1, classes=1, anchors=[(10, 12)], scale_x_y=1.2, new_coords=1)
    d = orc.decode_nms([head], [spec], 32, 32, 32, 32, 0.25, 0.45, letterbox=False)
    assert d.shape[0] == 1
    cls, conf, obj, x, y, w, h = d[0]
    assert abs(conf - 0.72) < 1e-5
    assert abs(obj - 0.9) < 1e-6
    assert abs(x - 16.0) < 1e-4 and abs(y - 6.4) < 1e-4
    assert abs(w - 10.0) < 1e-4 and abs(h - 3.0) < 1e-4


# --- lightnet-train/src/detect.rs:1869-1920 decodes_single_yolo_detection
@pytest.mark.parametrize("det_exp", [False, True])
def test_decode_single_kat(det_exp):
    head = np.array([0, 0, 0, 0, 8.0, 8.0], np.float32).reshape(6, 1, 1)
    spec = dict(gw=1, gh=1, classes=1, anchors=[(10, 12)], scale_x_y=1.0, new_coords=0)
    d = orc.decode_nms([head], [spec], 32, 32, 32, 32, 0.25, 0.45, letterbox=False, det_exp=det_exp)
    assert d.shape[0] == 1
    assert d[0, 0] == 0
    assert d[0, 1] > 0.99
    assert abs(d[0, 3] - 16.0) < 0.01
    assert abs(d[0, 5] - 10.0) < 0.01


# --- lightnet-train/src/detect.rs:1922-1965 suppresses_overlapping_boxes_with_nms
def test_nms_suppresses_overlap_kat():
    data = np.zeros(12, np.float32)
    data[4] = 8.0
    data[5] = 8.0
    data[10] = 7.0
    data[11] = 7.0
    spec = dict(gw=1, gh=1, classes=1, anchors=[(10, 12), (10, 12)], scale_x_y=1.0, new_coords=0)
    # DetectionOptions::default(): 0.25 / 0.45 / letterbox
    d = orc.decode_nms([data.reshape(12, 1, 1)], [spec], 32, 32, 32, 32, 0.25, 0.45, letterbox=True)
    assert d.shape[0] == 1
    # without NMS both anchors emit
    d2 = orc.decode_only([data.reshape(12, 1, 1)], [spec], 32, 32, 32, 32, 0.25, letterbox=True)
    assert d2.shape[0] == 2


# --- lightnet-core/src/runtime_tests/tests_03.rs:628-672 runs_single_conv_layer
def test_single_conv_layer_kat():
    cfg = "[net]\nwidth=2\nheight=1\nchannels=1\n[convolutional]\nfilters=1\nsize=1\nstride=1\nactivation=linear\n"
    net = orc.Net(cfg)
    assert net.weight_count() == 2
    net.set_weights(weights_blob([0.5], [2.0]))  # bias, weight (Darknet .weights payload order)
    net.forward_f32(np.array([1.0, 2.0], np.float32))
    assert net.layer_output_f32(0).ravel().tolist() == [2.5, 4.5]


# --- lightnet-core/src/runtime_tests/tests_03.rs:674-728 runs_route_and_upsample_layers
def test_route_and_upsample_kat():
    cfg = ("[net]\nwidth=2\nheight=2\nchannels=1\n[convolutional]\nfilters=1\nsize=1\nstride=1\nactivation=linear\n"
           "[route]\nlayers=-1\n[upsample]\nstride=2\nscale=1\n")
    net = orc.Net(cfg)
    net.set_weights(weights_blob([0.0], [1.0]))
    net.forward_f32(np.array([1, 2, 3, 4], np.float32))
    out = net.layer_output_f32(2)
    assert out.shape == (1, 1, 4, 4)
    assert out[0, 0, 0, 0] == 1.0 and out[0, 0, 3, 3] == 4.0
    assert np.array_equal(out[0, 0], np.kron(np.array([[1, 2], [3, 4]], np.float32), np.ones((2, 2), np.float32)))


def axis_tensor(b, c, h, w):
    # lightnet-model/src/axis_fixture.rs:34 axis_value = n*1000 + c*100 + h*10 + w
    n_, c_, h_, w_ = np.meshgrid(np.arange(b), np.arange(c), np.arange(h), np.arange(w), indexing="ij")
    return (n_ * 1000 + c_ * 100 + h_ * 10 + w_).astype(np.float32)


# --- lightnet-core/src/runtime_tests/tests_01.rs:700-778 convolutional_axis_layout_keeps_nchw_and_group_partitions
def test_conv_axis_layout_kat():
    cfg = "[net]\nwidth=3\nheight=2\nchannels=2\nbatch=2\n[convolutional]\nfilters=2\nsize=1\nstride=1\nbatch_normalize=0\nactivation=linear\n"
    net = orc.Net(cfg)
    net.set_weights(weights_blob([0, 0], [0, 1, 1, 0]))
    x = axis_tensor(2, 2, 2, 3)
    net.forward_f32(x)
    y = net.layer_output_f32(0)
    assert np.array_equal(y[:, 0], x[:, 1]) and np.array_equal(y[:, 1], x[:, 0])

    cfg = "[net]\nwidth=2\nheight=1\nchannels=2\nbatch=2\n[convolutional]\nfilters=2\nsize=1\ngroups=2\nbatch_normalize=0\nactivation=linear\n"
    net = orc.Net(cfg)
    net.set_weights(weights_blob([0, 0], [2, 3]))
    x = axis_tensor(2, 2, 1, 2)
    net.forward_f32(x)
    y = net.layer_output_f32(0)
    assert np.array_equal(y[:, 0], 2 * x[:, 0]) and np.array_equal(y[:, 1], 3 * x[:, 1])


# --- lightnet-core/src/runtime_tests/tests_03.rs:385-420 maxpool spatial axis pin
def test_maxpool_axis_layout_kat():
    cfg = "[net]\nwidth=5\nheight=3\nchannels=2\nbatch=2\n[maxpool]\nsize=3\nstride_x=2\nstride_y=1\npadding=1\n"
    net = orc.Net(cfg)
    assert net.out_shape(0) == (2, 2, 2, 2)
    vals = np.array([(i // 30) * 200 + (i // 15 % 2) * 100 + i % 15 + 1 for i in range(60)], np.float32)
    vals[0] = 13.0
    y = orc.maxpool_f32(vals.reshape(2, 2, 3, 5), 3, 2, 1, 1)
    want = [13, 15, 13, 15, 113, 115, 113, 115, 213, 215, 213, 215, 313, 315, 313, 315]
    assert y.ravel().tolist() == [float(v) for v in want]


# --- lightnet-cuda-oxide/tests/data/conv_shapes.csv (990 conv geometries scanned from the reference cfgs)
def test_conv_shape_rule_table():
    n = 0
    with open(os.path.join(GOLDEN, "conv_shapes.csv")) as f:
        for r in csv.DictReader(f):
            r = {k: int(v) for k, v in r.items()}
            cfg = ("[net]\nwidth=%d\nheight=%d\nchannels=%d\n[convolutional]\nfilters=%d\nsize=%d\nstride_x=%d\nstride_y=%d\n"
                   "dilation=%d\npadding=%d\ngroups=%d\nactivation=linear\n") % (
                r["in_w"], r["in_h"], r["in_c"], r["filters"], r["size"], r["stride_x"], r["stride_y"], r["dilation"],
                r["padding"], r["groups"])
            net = orc.Net(cfg)
            b, c, h, w = net.out_shape(0)
            assert (c, h, w) == (r["filters"], r["out_h"], r["out_w"]), r
            n += 1
    assert n == 990


# --- lightnet-cuda-oxide/tests/data/maxpool_shapes.csv
def test_maxpool_shape_rule_table():
    n = 0
    with open(os.path.join(GOLDEN, "maxpool_shapes.csv")) as f:
        for r in csv.DictReader(f):
            r = {k: int(v) for k, v in r.items()}
            cfg = "[net]\nwidth=%d\nheight=%d\nchannels=%d\n[maxpool]\nsize=%d\nstride_x=%d\nstride_y=%d\npadding=%d\n" % (
                r["in_w"], r["in_h"], r["in_c"], r["size"], r["stride_x"], r["stride_y"], r["padding"])
            net = orc.Net(cfg)
            b, c, h, w = net.out_shape(0)
            assert (c, h, w) == (r["in_c"], r["out_h"], r["out_w"]), r
            n += 1
    assert n == 108


def test_cfg_parse_rules():
    # lightnet-model/src/cfg.rs:109-171: '#'/';' comments (also trailing), case-insensitive keys, last value wins;
    # model.rs:4088-4144: pad=1 -> size/2; model.rs:4165-4183: maxpool size defaults to stride, padding to size-1;
    # model.rs:247-249: batch = batch / subdivisions.
    cfg = """
    [NET]
    Width = 8   # trailing comment
    height=8 ; another
    channels=4
    batch=64
    subdivisions=8
    [Convolutional]
    filters=6
    SIZE=3
    pad=1
    stride=2
    stride=1
    [maxpool]
    stride=2
    [upsample]
    [route]
    layers = -1, 0
    """
    net = orc.Net(cfg)
    assert net.batch == 8
    L = net.layers()
    assert L[0]["padding"] == 1 and L[0]["stride_x"] == 1 and L[0]["act"] == orc.ACT["logistic"]
    assert net.out_shape(0) == (8, 6, 8, 8)
    assert L[1]["size"] == 2 and L[1]["padding"] == 1 and net.out_shape(1) == (8, 6, 4, 4)
    assert net.out_shape(2) == (8, 6, 8, 8)
    assert net.out_shape(3) == (8, 12, 8, 8)
    with pytest.raises(orc.OracleError):
        orc.Net("[net]\nwidth=4\nheight=4\nchannels=1\n[route]\nlayers=0\n")  # forward reference
    with pytest.raises(orc.OracleError):
        orc.Net("width=4\n")


def test_gaussian_yolo_section_is_a_yolo_head():
    # model.rs:4513-4543: [gaussian_yolo] builds the same YoloSpec, with num = max(len(mask), num); exec_forward.rs:908-912: identity at
    # inference; detect.rs:78, :135: decoded by the same function as [yolo]
    body = "mask = 0,1\nanchors = 10,14, 23,27, 37,58\nclasses=3\nscale_x_y=1.05\n"
    cfg = "[net]\nwidth=8\nheight=8\nchannels=3\n[convolutional]\nfilters=16\nsize=1\nactivation=linear\n[%s]\n" + body
    a, b = orc.Net(cfg % "yolo", 1), orc.Net(cfg % "Gaussian_yolo", 1)
    assert a.layers() == b.layers()
    assert b.layers()[1]["kind"] == "yolo"
    from lightnet_b200 import zoo
    assert zoo.head_specs(cfg % "yolo") == zoo.head_specs(cfg % "Gaussian_yolo")
    assert zoo.head_specs(cfg % "yolo")[0]["anchors"] == [(10.0, 14.0), (23.0, 27.0)]


# --- lightnet-cuda-oxide/src/fp8.rs:200-309 (E4M3 grid, round trip, saturation, NaN, ties to even)
def test_fp8_e4m3_codec_kats():
    grid = [(0x00, 0.0), (0x01, 2.0 ** -9), (0x07, 7 * 2.0 ** -9), (0x08, 2.0 ** -6), (0x38, 1.0), (0x39, 1.125), (0x3C, 1.5),
            (0x40, 2.0), (0x7E, 448.0), (0xFE, -448.0)]
    for bits, want in grid:
        assert orc.e4m3_to_f32(bits) == want
    assert math.copysign(1.0, orc.e4m3_to_f32(0x80)) == -1.0
    assert math.isnan(orc.e4m3_to_f32(0x7F))
    for code in range(0x7F):
        v = orc.e4m3_to_f32(code)
        assert orc.f32_to_e4m3(v) == code
        assert orc.f32_to_e4m3(-v) == (code | 0x80)
    assert orc.f32_to_e4m3(1e9) == 0x7E and orc.f32_to_e4m3(-1e9) == 0xFE
    assert orc.f32_to_e4m3(float("inf")) == 0x7E
    assert orc.f32_to_e4m3(float("nan")) == 0x7F
    assert orc.f32_to_e4m3(1.0625) == 0x38
    assert orc.f32_to_e4m3(1.1875) == 0x3A
    assert orc.f32_to_e4m3(1.3125) == 0x3A


# --- lightnet-runtime/src/runtime/layer_ops.rs:1697-1738 activation formulas
def test_activation_formulas():
    for v in [-5.0, -1.0, -0.25, 0.0, 0.3, 2.0, 7.5]:
        f = np.float32(v)
        assert orc.activate("leaky", v) == (f if f > 0 else np.float32(0.1) * f)
        assert abs(orc.activate("logistic", v) - 1 / (1 + math.exp(-v))) < 1e-6
        assert abs(orc.activate("mish", v) - v * math.tanh(math.log1p(math.exp(v)))) < 1e-5
        assert abs(orc.activate("swish", v) - v / (1 + math.exp(-v))) < 1e-5
        assert orc.activate("linear", v) == f


def test_det_exp_tracks_libm():
    xs = np.concatenate([np.linspace(-87, 88, 20001), np.random.default_rng(0).normal(0, 3, 20000)]).astype(np.float32)
    worst = 0.0
    for x in xs:
        got, want = orc.det_expf(float(x)), float(np.exp(np.float64(x)))
        worst = max(worst, abs(got - want) / want)
    assert worst < 4 * 2.0 ** -24, worst  # within a few ulp of the true value
    for act in ("mish", "swish", "logistic"):
        for v in np.linspace(-30, 30, 2001):
            a, b = orc.det_activate(act, float(v)), orc.activate(act, float(v))
            assert abs(a - b) <= 2e-6 * max(1.0, abs(b)), (act, v, a, b)
    assert orc.det_activate("mish", 25.0) == 25.0


# --- lightnet-train/src/detect.rs:1486-1503 bbox_iou
def test_bbox_iou():
    assert orc.bbox_iou([5, 5, 10, 10], [5, 5, 10, 10]) == 1.0
    assert orc.bbox_iou([0, 0, 2, 2], [10, 10, 2, 2]) == 0.0
    assert orc.bbox_iou([0, 0, 2, 2], [2, 0, 2, 2]) == 0.0  # touching edges: inter_area <= 0
    assert abs(orc.bbox_iou([0, 0, 2, 2], [1, 0, 2, 2]) - (2.0 / 6.0)) < 1e-7
    assert orc.bbox_iou([0, 0, -2, 2], [0, 0, 2, 2]) == 0.0  # negative width clamps to zero area


def test_nms_semantics_match_reference_loop():
    """apply_nms (detect.rs:1449-1484) restated in pure Python, run on random same/different-class boxes
    in both unsorted and sorted order; the oracle's C++ must agree record for record."""
    rng = np.random.default_rng(7)

    def py_nms(d, thr):
        n = len(d)
        sup = [False] * n
        for i in range(n):
            if sup[i]:
                continue
            for j in range(i + 1, n):
                if sup[j] or d[i][0] != d[j][0]:
                    continue
                keep, drop = (i, j) if d[i][1] >= d[j][1] else (j, i)
                if orc.bbox_iou(d[keep][3:7], d[drop][3:7]) > thr:
                    sup[drop] = True
        return [r for r, s in zip(d, sup) if not s]

    for trial in range(5):
        n = 120
        recs = np.zeros((n, 7), np.float32)
        recs[:, 0] = rng.integers(0, 3, n)
        recs[:, 1] = rng.choice(np.linspace(0.3, 0.9, 9).astype(np.float32), n)  # many ties
        recs[:, 2] = 0.9
        recs[:, 3:5] = rng.uniform(20, 80, (n, 2))
        recs[:, 5:7] = rng.uniform(10, 40, (n, 2))
        got = orc.nms_records(recs, 0.45)
        d = py_nms([tuple(r) for r in recs], 1.0)
        d.sort(key=lambda r: -r[1])  # Python's sort is stable, like sort_by(total_cmp)
        d = py_nms(d, 0.45)
        d.sort(key=lambda r: -r[1])
        assert got.shape[0] == len(d)
        assert np.array_equal(got, np.asarray(d, np.float32))


def test_nms_class_by_class_equals_the_whole_list_passes():
    """apply_nms never pairs two classes (detect.rs:1461), so running its passes class by class and merging by
    (confidence descending, emission order) gives the records of the whole-list sequence: the form the full-size GPU parity
    tests use on 10^5 tied candidates."""
    rng = np.random.default_rng(17)
    for trial in range(6):
        n = 400
        recs = np.zeros((n, 7), np.float32)
        recs[:, 0] = rng.integers(0, 5, n)
        recs[:, 1] = rng.choice(np.linspace(0.3, 1.0, 6).astype(np.float32), n)  # heavy ties, as with saturated heads
        recs[:, 2] = 0.9
        recs[:, 3:5] = rng.uniform(20, 80, (n, 2))
        recs[:, 5:7] = rng.uniform(10, 40, (n, 2))
        recs[n // 2:n // 2 + 20, 3:7] = recs[:20, 3:7]      # exact duplicates of boxes (some in the same class)
        for skip in (False, True):
            for top_k in (0, 37):
                whole = orc.nms_records(recs, 0.45, top_k=top_k, skip_pass1=skip)
                split = orc.nms_records(recs, 0.45, top_k=top_k, skip_pass1=skip, by_class=True)
                assert np.array_equal(whole, split), (trial, skip, top_k)
    assert np.array_equal(orc.nms_records(recs, 0.0, by_class=True), orc.nms_records(recs, 0.0))  # thr <= 0: nothing suppressed
    # the early-stopping form the CPU arm of the benchmark times: first k records of the pass without the pre-pass
    for k in (1, 25, 10000):
        assert np.array_equal(orc.nms_records_first_k(recs, 0.45, k), orc.nms_records(recs, 0.45, skip_pass1=True)[:k])


def test_bn_fold_matches_unfolded_within_rounding():
    # lightnet-runtime/src/runtime/weights_io.rs:32-92 vs layer_ops.rs:1682-1695
    cfg = "[net]\nwidth=6\nheight=5\nchannels=3\nbatch=2\n[convolutional]\nbatch_normalize=1\nfilters=4\nsize=3\nstride=1\npad=1\nactivation=leaky\n"
    rng = np.random.default_rng(3)
    net = orc.Net(cfg)
    blob = weights_blob(rng.normal(0, 0.1, 4), rng.uniform(0.5, 1.5, 4), rng.normal(0, 0.2, 4), rng.uniform(0.5, 2, 4),
                        rng.normal(0, 0.3, 4 * 3 * 9))
    net.set_weights(blob)
    x = rng.uniform(0, 1, (2, 3, 5, 6)).astype(np.float32)
    net.forward_f32(x, folded=False)
    a = net.layer_output_f32(0)
    net.forward_f32(x, folded=True)
    b = net.layer_output_f32(0)
    assert np.allclose(a, b, rtol=2e-5, atol=2e-5)


def test_conv_against_torch_on_reference_geometries():
    """Geometry cases of lightnet-cuda-oxide/tests/oxide_conv_parity.rs:106-121, checked against an
    independent implementation (torch CPU, float64) at that test's tolerance 1e-3 + 1e-3*|ref|."""
    import torch

    cases = [(2, 5, 7, 9, 6, 1, 1, 1, 0, 1), (2, 3, 9, 11, 5, 3, 1, 1, 1, 1), (1, 2, 8, 8, 3, 3, 1, 1, 0, 1),
             (1, 4, 13, 13, 6, 3, 2, 2, 1, 1), (2, 3, 10, 12, 4, 3, 2, 1, 1, 1), (3, 3, 15, 13, 5, 5, 2, 2, 2, 1), (2, 4, 9, 7, 6, 3, 1, 1, 1, 2),
             (2, 6, 9, 9, 6, 3, 1, 1, 1, 6), (2, 16, 10, 10, 70, 3, 1, 1, 1, 1)]
    rng = np.random.default_rng(11)
    for (b, c, h, w, f, k, sx, sy, pad, g) in cases:
        x = rng.normal(0, 1, (b, c, h, w)).astype(np.float32)
        wt = rng.normal(0, 0.3, (f, c // g, k, k)).astype(np.float32)
        bias = rng.normal(0, 0.1, f).astype(np.float32)
        y = orc.conv_f32(x, wt, bias, stride=sx, stride_y=sy, pad=pad, groups=g)
        ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(wt).double(),
                                         torch.from_numpy(bias).double(), stride=(sy, sx), padding=pad, groups=g).numpy()
        assert y.shape == ref.shape
        assert np.all(np.abs(y - ref) <= 1e-3 + 1e-3 * np.abs(ref))


def test_q8_grouped_conv_accumulators_match_torch():
    """Grouped / depthwise integer accumulators against torch's int64 convolution (forward_layers.rs:646-679 channel rule)."""
    import torch

    rng = np.random.default_rng(6)
    for (c, f, k, stride, pad, groups) in [(8, 12, 3, 1, 1, 4), (8, 8, 3, 2, 1, 8), (6, 9, 1, 1, 0, 3)]:
        x = rng.integers(-127, 128, (2, c, 7, 9), dtype=np.int8)
        w = rng.integers(-127, 128, (f, c // groups, k, k), dtype=np.int8)
        ref = torch.nn.functional.conv2d(torch.from_numpy(x.astype(np.int64)), torch.from_numpy(w.astype(np.int64)), stride=stride, padding=pad, groups=groups).numpy()
        assert np.array_equal(orc.conv_q8_acc(x, w, stride, pad, groups=groups), ref)


def test_q8_conv_accumulators_match_numpy():
    rng = np.random.default_rng(5)
    x = rng.integers(-127, 128, (2, 8, 7, 9), dtype=np.int8)
    w = rng.integers(-127, 128, (5, 8, 3, 3), dtype=np.int8)
    for stride, pad in [(1, 1), (2, 1), (1, 0)]:
        acc = orc.conv_q8_acc(x, w, stride, pad)
        xp = np.pad(x.astype(np.int64), ((0, 0), (0, 0), (pad, pad), (pad, pad)))
        oh, ow = acc.shape[2:]
        ref = np.zeros(acc.shape, np.int64)
        for ky in range(3):
            for kx in range(3):
                patch = xp[:, :, ky:ky + stride * oh:stride, kx:kx + stride * ow:stride]
                ref += np.einsum("bchw,fc->bfhw", patch, w[:, :, ky, kx].astype(np.int64))
        assert np.array_equal(acc, ref)


# ---------------------------------------------------------------------------------------- image pre-processing
# Known answers of lightnet-runtime/src/image.rs:362-441 (fixtures repackaged by tests/golden/make_resize_fixtures.py).

def _resize_fixtures():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resize_fixtures.npz"))


def test_image_from_u8_kat():
    # converts_interleaved_rgb_to_planar (image.rs:415-420)
    out = orc.image_from_u8(np.array([[[255, 128, 0]]], np.uint8))
    assert out.ravel().tolist() == [1.0, np.float32(128.0) / np.float32(255.0), 0.0]


def test_image_resize_linear_exact_matches_opencv_bytes():
    # resize_linear_exact_matches_opencv_bytes (image.rs:365-378): byte for byte
    fx = _resize_fixtures()
    for i in range(3):
        for w, h in ((40, 28), (130, 100)):
            got = orc.image_resize_exact_u8(fx["src%d" % i], w, h)
            assert np.array_equal(got, fx["exact%d_%dx%d" % (i, w, h)]), (i, w, h)


def test_image_resize_matches_darknet_float_resize():
    # resize_matches_darknet_float_resize (image.rs:383-402): max |diff| <= 1e-6
    fx = _resize_fixtures()
    for i in range(3):
        src = orc.image_from_u8(fx["src%d" % i])
        for w, h in ((40, 28), (50, 60)):
            got = orc.image_resize(src, w, h)
            assert np.abs(got - fx["float%d_%dx%d" % (i, w, h)]).max() <= 1e-6, (i, w, h)


def test_image_letterbox_kats():
    fx = _resize_fixtures()
    src = orc.image_from_u8(fx["src0"])
    # letterbox_uses_half_gray_and_integer_offsets (image.rs:404-413): 96x72 into 50x60 -> 50x37 at y offset 11
    assert orc.image_fit_inside(96, 72, 50, 60) == (50, 37)
    boxed, resized = orc.image_letterbox(src, 50, 60), orc.image_resize(src, 50, 37)
    assert boxed[0, 0, 0] == 0.5 and boxed[2, 10, 49] == 0.5 and boxed[2, 48, 0] == 0.5
    assert boxed[1, 11, 7] == resized[1, 0, 7] and boxed[1, 47, 7] == resized[1, 36, 7]
    # resizes_image_bilinearly / letterboxes_image_with_gray_padding (image.rs:422-441)
    two = orc.image_from_u8(np.array([[[0, 0, 0], [255, 0, 0]]], np.uint8))
    assert abs(orc.image_resize(two, 3, 1)[0, 0, 1] - 0.5) < 0.01
    red = orc.image_from_u8(np.array([[[255, 0, 0], [255, 0, 0]]], np.uint8))
    lb = orc.image_letterbox(red, 2, 2)
    assert lb.shape == (3, 2, 2) and abs(lb.ravel()[0] - 1.0) < 0.01 and abs(lb.ravel()[2] - 0.5) < 0.01


# ---- modern anchor-free heads: the reference's own vectors (lightnet-train/src/detect.rs:2422-2600) -------------------------
def _yolox_spec():
    return [dict(gw=4, gh=4, classes=2, anchors=[(1, 1)], kind=1)]


def test_modern_yolox_decodes_a_confident_box():
    # detect.rs:2423-2470 yolox_decodes_a_confident_box: the vector is passed to the decoder as it stands (the decoder clamps
    # objectness and class entries to [0, 1])
    data = np.zeros((7, 4, 4), np.float32)
    data[0, 2, 1] = 1.0
    data[1, 2, 1] = 2.0
    data[2, 2, 1] = np.log(np.float32(4.0))
    data[3, 2, 1] = np.log(np.float32(4.0))
    data[4, 2, 1] = 10.0
    data[5, 2, 1] = 10.0
    for det_exp in (False, True):
        d = orc.decode_nms([data], _yolox_spec(), 16, 16, 16, 16, 0.3, 0.45, False, det_exp=det_exp)
        assert d.shape[0] == 1
        assert d[0, 0] == 0 and d[0, 1] > 0.99
        assert np.allclose(d[0, 3:7], [8.0, 16.0, 16.0, 16.0], atol=1e-3)


def test_modern_threshold_filters_and_nms_deduplicates():
    # detect.rs:2472-2512 the_confidence_threshold_filters_and_nms_deduplicates
    data = np.zeros((7, 4, 4), np.float32)
    for loc in (0, 1):
        data[2, 0, loc] = np.log(np.float32(4.0))
        data[3, 0, loc] = np.log(np.float32(4.0))
        data[4, 0, loc] = 0.99
        data[6, 0, loc] = 0.98
    d = orc.decode_nms([data], _yolox_spec(), 16, 16, 16, 16, 0.9, 0.45, False)
    assert d.shape[0] == 1 and d[0, 0] == 1
    assert orc.decode_nms([data], _yolox_spec(), 16, 16, 16, 16, 0.995, 0.45, False).shape[0] == 0


def test_modern_distribution_head_decodes_through_the_dfl_expectation():
    # detect.rs:2557-2600 the_distribution_heads_decode_through_the_dfl_expectation: 4x4 grid, one class, reg_max = 3
    bins, coords, classes = 4, 16, 1
    data = np.zeros((1, coords + 1 + classes, 4, 4), np.float32)
    row, col = 2, 1
    for side in range(4):
        data[0, side * bins + 2, row, col] = 40.0
    data[0, coords, row, col] = 40.0
    data[0, coords + 1, row, col] = 40.0
    pre = orc.modern_predecode(data, classes, coords)
    assert pre.shape == (1, 5 + classes, 4, 4)
    spec = [dict(gw=4, gh=4, classes=1, anchors=[(1, 1)], kind=2)]
    d = orc.decode_nms([pre[0]], spec, 16, 16, 16, 16, 0.3, 0.45, False)
    assert d.shape[0] == 1
    assert np.allclose(d[0, 3:6], [6.0, 10.0, 16.0], atol=1e-2)
    # the activation of the head's forward (lib.rs:4884) leaves the same detection: sigmoid(40) rounds to 1, and the other
    # cells' class score sigmoid(0) = 0.5 stays under a threshold of 0.6
    act = orc.modern_activate(data, classes)
    assert act[0, coords, row, col] == 1.0 and act[0, coords, 0, 0] == 0.5 and act[0, 2, row, col] == 40.0
    d2 = orc.decode_nms([orc.modern_predecode(act, classes, coords)[0]], spec, 16, 16, 16, 16, 0.6, 0.45, False)
    assert d2.shape[0] == 1 and np.allclose(d2[0, 3:6], [6.0, 10.0, 16.0], atol=1e-2)
