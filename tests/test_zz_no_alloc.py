"""The allocation-free decode + NMS entry point (ln_yolo_decode_nms_noalloc) must return exactly what the ordinary one
(ln_yolo_decode_nms) returns.  It exists for hosts that cannot allocate device memory while they serve requests: its
working memory is a fixed array inside the library, which keeps whatever the previous call wrote -- so the check is
made on two different calls in a row, and the second must not be disturbed by the first.  Kept in a file that pytest
collects last: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

import lightnet_b200 as ln

pytestmark = pytest.mark.gpu

ANCH = [(10, 13), (16, 30), (33, 23), (30, 61), (62, 45), (59, 119)]


def heads_for(be, rng, batch, grids, classes, mu):
    dev, raw = [], []
    for i, g in enumerate(grids):
        t = np.empty((batch, 3, 5 + classes, g, g), np.float32)
        t[:, :, 0:2] = rng.normal(0, 1, (batch, 3, 2, g, g))
        t[:, :, 2:4] = rng.normal(0, 0.5, (batch, 3, 2, g, g))
        t[:, :, 4:] = rng.normal(mu, 2, (batch, 3, 1 + classes, g, g))
        t = t.reshape(batch, 3 * (5 + classes), g, g)
        raw.append(t)
        dev.append(dict(raw=be.upload_f32(t.shape, t), classes=classes, anchors=ANCH[3 * i:3 * i + 3], scale_x_y=1.05, new_coords=0))
    return dev


def test_noalloc_entry_point_matches_the_allocating_one():
    be = ln.B200Backend(0)
    rng = np.random.default_rng(42)
    # two different problems back to back: the second runs on working memory the first one dirtied
    calls = [dict(batch=3, grids=[26, 13], classes=20, mu=-2.0, thr=0.05, nms=0.45, top_k=0, maxper=400),
             dict(batch=2, grids=[20, 10], classes=7, mu=-1.0, thr=0.25, nms=0.6, top_k=50, maxper=64)]
    for c in calls:
        dev = heads_for(be, rng, c["batch"], c["grids"], c["classes"], c["mu"])
        want = be.yolo_decode_nms(dev, 320, 320, [640, 500, 320][:c["batch"]], [480, 500, 320][:c["batch"]], c["thr"], c["nms"], True, c["top_k"],
                                  c["maxper"])
        got = be.yolo_decode_nms(dev, 320, 320, [640, 500, 320][:c["batch"]], [480, 500, 320][:c["batch"]], c["thr"], c["nms"], True, c["top_k"],
                                 c["maxper"], noalloc=True)
        assert sum(len(w) for w in want) > 20
        for w, g in zip(want, got):
            assert w.shape == g.shape
            assert np.array_equal(w, g)  # same kernels, same arithmetic: the records are identical, bit for bit
    # a problem whose working set exceeds the fixed array is refused with both sizes in the message, not truncated
    big = np.zeros((64, 3 * 85, 76, 76), np.float32)
    dev = [dict(raw=be.upload_f32(big.shape, big), classes=80, anchors=ANCH[:3], scale_x_y=1.0, new_coords=0)]
    with pytest.raises(ln.BackendError) as e:
        be.yolo_decode_nms(dev, 608, 608, 608, 608, noalloc=True)
    assert e.value.kind == "unsupported" and "67108864" in str(e.value)
    be.close()
