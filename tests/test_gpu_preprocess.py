"""Device image pre-processing against the oracle (which is pinned by the reference's fixtures): bit-identical f32."""
import os

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


def fixtures():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resize_fixtures.npz"))


def test_exact_resize_matches_the_reference_fixtures(be):
    fx = fixtures()
    srcs = [fx["src%d" % i] for i in range(3)]
    for w, h in ((40, 28), (130, 100), (96, 72)):
        got = be.download_f32(be.preprocess_u8(srcs, w, h, ln.LN_PRE_RESIZE_EXACT))
        for i in range(3):
            ref = fx["exact%d_%dx%d" % (i, w, h)] if (w, h) != (96, 72) else srcs[i]
            assert np.array_equal(got[i], orc.image_from_u8(ref)), (i, w, h)


def test_float_resize_and_letterbox_bit_identical_to_the_oracle(be):
    fx = fixtures()
    rng = np.random.default_rng(1)
    images = [fx["src0"], fx["src1"], rng.integers(0, 256, (33, 57, 3), dtype=np.uint8), rng.integers(0, 256, (1, 9, 3), dtype=np.uint8),
              rng.integers(0, 256, (50, 1, 3), dtype=np.uint8), rng.integers(0, 256, (64, 48, 3), dtype=np.uint8)]
    # (a fitted height of 1 from a taller source makes the reference multiply 0 by an infinite scale: NaN pixels on both sides)
    for w, h in ((50, 60), (40, 28), (64, 48), (1, 9), (7, 128)):
        got = be.download_f32(be.preprocess_u8(images, w, h, ln.LN_PRE_RESIZE))
        box = be.download_f32(be.preprocess_u8(images, w, h, ln.LN_PRE_LETTERBOX))
        for i, im in enumerate(images):
            planar = orc.image_from_u8(im)
            assert np.array_equal(got[i], orc.image_resize(planar, w, h), equal_nan=True), ("resize", i, w, h)
            assert np.array_equal(box[i], orc.image_letterbox(planar, w, h), equal_nan=True), ("letterbox", i, w, h)
    # the reference's float fixtures, within its own tolerance
    got = be.download_f32(be.preprocess_u8([fx["src2"]], 50, 60, ln.LN_PRE_RESIZE))
    assert np.abs(got[0] - fx["float2_50x60"]).max() <= 1e-6


def test_preprocess_errors(be):
    im = np.zeros((4, 4, 3), np.uint8)
    with pytest.raises(ln.BackendError):
        be.preprocess_u8([im], 0, 8)
    with pytest.raises(ln.BackendError):
        be.preprocess_u8([im], 8, 8, 7)


@pytest.mark.parametrize("batch", [4, 8])
def test_detect_u8_equals_detect_on_the_oracles_letterbox(be, batch):
    """ln_net_detect_u8 = device letterbox + detect: same records as detect() fed with the oracle's letterboxed f32 batch.
    (detect() itself is run with its host pipeline off, so the reference side is the plain whole-batch path at both sizes.)"""
    from test_gpu_parity import MINI_CFG
    o = orc.Net(MINI_CFG, batch)
    blob = synth.he_weights(o.layers(), 61, bn_identity=False)
    rng = np.random.default_rng(62)
    sizes = [(48, 64), (100, 75), (31, 200), (64, 64), (90, 90), (17, 33), (240, 320), (64, 48)][:batch]   # (h, w)
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for h, w in sizes]
    x = np.stack([orc.image_letterbox(orc.image_from_u8(im), o.width, o.height) for im in images])
    net = ln.GpuExecutableNetwork(be, MINI_CFG, batch, ln.LN_Q8)
    net.load_weights(blob)
    net.calibrate(x)
    net.set_host_pipeline(False)
    ref = net.detect(x, [w for _, w in sizes], [h for h, _ in sizes], 0.2, 0.45, True, 0, 256)
    net.set_host_pipeline(True)
    assert sum(len(r) for r in ref) > 20
    for _ in range(2):
        got = net.detect_u8(images, 0.2, 0.45, True, 0, 256)
        for b in range(batch):
            assert np.array_equal(got[b], ref[b]), b
