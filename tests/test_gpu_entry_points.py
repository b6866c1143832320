"""Entry points of the C ABI that the network-level tests do not reach on their own: the Darknet .weights file loader, the
device batch-norm fold, and the widen / narrow conversions between f32 and 8-bit tensors.  Needs a B200: run with -m gpu."""
import struct

import numpy as np
import pytest

import lightnet_b200 as ln
from lightnet_b200 import synth
from oracle import oracle_api as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = ln.B200Backend(0)
    yield b
    b.close()


def write_weights(path, payload, major, minor, seen=12345):
    """Darknet .weights layout read by read_header (lightnet-runtime/src/runtime/weights_io.rs:911-928): three i32, then `seen` as
    u64 when major * 10 + minor >= 2 and as u32 otherwise, then the f32 payload."""
    with open(path, "wb") as f:
        f.write(struct.pack("<iii", major, minor, 0))
        f.write(struct.pack("<Q" if major * 10 + minor >= 2 else "<I", seen))
        f.write(np.asarray(payload, np.float32).tobytes())


@pytest.mark.parametrize("major,minor", [(0, 2), (0, 1)])   # 64-bit and 32-bit `seen`
def test_weights_file_single_conv_kat(be, tmp_path, major, minor):
    """lightnet-core/src/runtime_tests/tests_03.rs:628-672 (runs_single_conv_layer) through a real file: a 1x1 convolution with
    bias 0.5 and weight 2.0 maps [1, 2] to [2.5, 4.5]."""
    cfg = "[net]\nwidth=2\nheight=1\nchannels=1\n[convolutional]\nfilters=1\nsize=1\nstride=1\nactivation=linear\n"
    path = str(tmp_path / "one.weights")
    write_weights(path, [0.5, 2.0], major, minor)
    net = ln.GpuExecutableNetwork(be, cfg, 1, ln.LN_F32)
    net.load_weights_file(path)
    net.forward(np.array([1.0, 2.0], np.float32).reshape(1, 1, 1, 2))
    assert be.download_f32(net.layer_output(0)).ravel().tolist() == [2.5, 4.5]


def test_weights_file_equals_blob_and_reports_short_files(be, tmp_path):
    cfg = ("[net]\nwidth=12\nheight=10\nchannels=3\nbatch=2\n[convolutional]\nbatch_normalize=1\nfilters=8\nsize=3\nstride=1\npad=1\nactivation=leaky\n"
           "[convolutional]\nfilters=5\nsize=1\nstride=1\nactivation=linear\n")
    o = orc.Net(cfg, 2)
    blob = synth.he_weights(o.layers(), 5, bn_identity=False)
    x = synth.uniform_images(2, 3, 10, 12, 6)
    outs = []
    for how in ("blob", "file"):
        net = ln.GpuExecutableNetwork(be, cfg, 2, ln.LN_F32)
        if how == "blob":
            net.load_weights(blob)
        else:
            path = str(tmp_path / "net.weights")
            write_weights(path, blob, 0, 2)
            net.load_weights_file(path)
        net.forward(x)
        outs.append(be.download_f32(net.layer_output(1)))
    assert np.array_equal(outs[0], outs[1])
    o.set_weights(blob)
    o.forward_f32(x, folded=True)
    assert np.abs(outs[1] - o.layer_output_f32(1)).max() <= 1e-4 * np.abs(o.layer_output_f32(1)).max()
    short = str(tmp_path / "short.weights")
    write_weights(short, blob[:-3], 0, 2)
    with pytest.raises(ln.BackendError) as e:
        ln.GpuExecutableNetwork(be, cfg, 2, ln.LN_F32).load_weights_file(short)
    assert "expected" in str(e.value)
    with pytest.raises(ln.BackendError):
        ln.GpuExecutableNetwork(be, cfg, 2, ln.LN_F32).load_weights_file(str(tmp_path / "missing.weights"))


def test_batchnorm_fold_matches_the_host_fold(be):
    """batchnorm_fold_f32 (lightnet-cuda/src/lib.rs:6208): scale = gamma / sqrt(var + eps), bias' = bias - mean * scale, the same
    single f32 operations as fold_convolutional_params_for_inference (runtime/weights_io.rs:32-92): equal bit for bit."""
    rng = np.random.default_rng(8)
    n = 300
    gamma = rng.normal(1, 0.3, n).astype(np.float32)
    mean = rng.normal(0, 1, n).astype(np.float32)
    var = rng.uniform(0.01, 4, n).astype(np.float32)
    bias = rng.normal(0, 0.5, n).astype(np.float32)
    eps = np.float32(1e-5)
    up = lambda v: be.upload_f32((1, n, 1, 1), v)
    s, b = be.batchnorm_fold_f32(up(gamma), up(mean), up(var), up(bias), float(eps))
    s_ref = (gamma / np.sqrt(var + eps)).astype(np.float32)
    b_ref = (bias - (mean * s_ref).astype(np.float32)).astype(np.float32)
    assert np.array_equal(be.download_f32(s).ravel(), s_ref)
    assert np.array_equal(be.download_f32(b).ravel(), b_ref)
    with pytest.raises(ln.BackendError):
        be.batchnorm_fold_f32(up(gamma), up(mean), be.upload_f32((1, n - 1, 1, 1), var[:-1]), up(bias), 1e-5)


def test_widen_and_narrow_between_f32_and_8_bit(be):
    """narrow_f32 / widen_f16 analogues (lightnet-cuda/src/lib.rs:6304-6308): narrow quantises on the device exactly like the
    upload of host data does; widen returns code * scale."""
    rng = np.random.default_rng(9)
    x = rng.normal(0, 2, (2, 37, 9, 11)).astype(np.float32)     # 37 channels: padded to 64 in storage
    t = be.upload_f32(x.shape, x)
    # int8: rne(x / s) clamped to +-127
    s = np.float32(np.abs(x).max() / 127.0)
    q = be.narrow_f32(t, float(s), ln.LN_Q8)
    codes, scale = be.download_q(q)
    assert scale == float(s)
    assert np.array_equal(codes, be.download_q(be.upload_q(x.shape, x, float(s), ln.LN_Q8))[0])
    assert np.array_equal(codes, np.clip(np.rint(x * (np.float32(1.0) / s)), -127, 127).astype(np.int8))
    assert np.array_equal(be.download_f32(be.widen_q(q)), codes.astype(np.float32) * s)
    # FP8 E4M3: the oracle codec (pinned by the reference's KATs, lightnet-cuda-oxide/src/fp8.rs:200-309)
    s8 = np.float32(np.abs(x).max() / 448.0)
    q8 = be.narrow_f32(t, float(s8), ln.LN_F8)
    codes8, _ = be.download_q(q8)
    assert np.array_equal(codes8.ravel(), orc.f32_to_e4m3_array((x * (np.float32(1.0) / s8)).ravel()))
    assert np.array_equal(be.download_f32(be.widen_q(q8)), orc.e4m3_table()[codes8] * s8)
    with pytest.raises(ln.BackendError):
        be.narrow_f32(t, 0.0, ln.LN_Q8)
    with pytest.raises(ln.BackendError):
        be.widen_q(t)


def test_region_forward_and_yolo_activate(be):
    """The two classic head activations of the f32 trait: [region] forward (lightnet-cuda/src/lib.rs:5090, host_ops.rs:73-116) and
    yolo_activate_f32 (lib.rs:4951), against numpy restatements of the reference's host loops (libm exp on both sides: 2 ulp)."""
    rng = np.random.default_rng(12)
    anchors, classes = 5, 7
    entries = classes + 5
    x = rng.normal(0, 2, (2, anchors * entries, 6, 7)).astype(np.float32)
    t = be.upload_f32(x.shape, x)
    for softmax in (True, False):
        got = be.download_f32(be.region_forward_f32(t, anchors, entries, classes, softmax)).reshape(2, 42, anchors, entries)
        ref = orc.region_forward(x, anchors, entries, classes, softmax)
        assert np.allclose(got, ref, rtol=3e-6, atol=1e-7)
        assert np.array_equal(got[..., :4], ref[..., :4])          # the box entries are only moved
        if softmax:
            assert np.allclose(got[..., 5:].sum(-1), 1.0, atol=1e-5)
    with pytest.raises(ln.BackendError):
        be.region_forward_f32(t, anchors, entries + 1, classes, True)
    for new_coords, s in ((False, 1.2), (True, 2.0)):
        got = be.download_f32(be.yolo_activate_f32(t, classes, s, new_coords))
        assert np.allclose(got, orc.yolo_activate(x, classes, s, new_coords), rtol=3e-6, atol=1e-7)
