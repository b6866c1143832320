"""The batched callers (lightnet_b200/evaluate.py): mAP known answers of the reference, the validation pass and the
detect-server protocol on a stand-in detector (CPU), and the same callers over a real network on the GPU."""
import io
import json

import numpy as np
import pytest

from lightnet_b200 import evaluate as ev


def truth(c):
    return [c, 0.5, 0.5, 0.4, 0.4]


def pred(c, conf, x):
    return [c, conf, conf, x, 0.5, 0.4, 0.4]


def test_map_precision_envelope_kat():
    # lightnet-train/src/evaluate.rs:1348-1373 ap_precision_envelope_duplicates_background_and_missing_classes
    samples = [(np.array([truth(0)]), np.array([pred(0, 0.9, 0.1), pred(0, 0.8, 0.5), pred(0, 0.7, 0.5)])),
               (np.array([truth(0)]), np.array([pred(0, 0.6, 0.5)])),
               (np.zeros((0, 5)), np.array([pred(1, 0.9, 0.5)]))]
    r = ev.detector_map(samples, 2, 0.5)
    assert r["average_precision"] == [0.5, 0.0]
    assert r["mean_average_precision"] == 0.25
    assert r["ground_truth_counts"] == [2, 0]
    assert r["true_positives"] == [2, 0]
    assert r["false_positives"] == [2, 1]
    assert r["false_negatives"] == [0, 0]
    assert r["detection_counts"] == [4, 1]


def test_map_integrates_all_recall_steps_kat():
    # evaluate.rs:1375-1386 precision_envelope_integrates_all_recall_steps
    samples = [(np.array([truth(0)]), np.array([pred(0, 0.9, 0.5), pred(0, 0.8, 0.1)])), (np.array([truth(0)]), np.array([pred(0, 0.7, 0.5)]))]
    assert abs(ev.detector_map(samples, 1, 0.5)["mean_average_precision"] - 5.0 / 6.0) < 1e-12


def test_map_report_confidence_and_errors():
    # a hit below the report confidence counts for AP but not for the TP / FN columns (evaluate.rs:1093-1102, same matching code)
    r = ev.detector_map([(np.array([truth(0)]), np.array([pred(0, 0.1, 0.5)]))], 1, 0.5)
    assert r["average_precision"] == [1.0] and r["true_positives"] == [0] and r["false_negatives"] == [1] and r["average_iou"] == [0.0]
    with pytest.raises(ValueError):
        ev.detector_map([], 0, 0.5)
    with pytest.raises(ValueError):
        ev.detector_map([(np.array([truth(3)]), np.zeros((0, 7)))], 2, 0.5)
    with pytest.raises(ValueError):
        ev.detector_map([(np.zeros((0, 5)), np.array([pred(0, np.nan, 0.5)]))], 1, 0.5)


class FakeDetector:
    """Stands in for GpuExecutableNetwork.detect_u8: one record per image whose confidence is the image's mean / 255 and
    whose box is the image rectangle; records below the threshold are dropped."""

    def __init__(self, batch):
        self.batch, self.calls = batch, []

    def __call__(self, images, thr, nms, letterbox, top_k, max_per_image, mode=0):
        assert len(images) == self.batch
        self.calls.append((len(images), thr, mode))
        out = []
        for im in images:
            conf = float(im.mean()) / 255.0
            h, w = im.shape[:2]
            rec = np.array([[0, conf, conf, w / 2, h / 2, w, h]], np.float32)
            out.append(rec[rec[:, 1] > thr])
        return out


def test_validation_run_batches_pads_and_normalises():
    images = [np.full((10 + i, 20 + 2 * i, 3), 40 * (i + 1), np.uint8) for i in range(5)]
    labels = [np.array([[0, 0.5, 0.5, 1.0, 1.0]], np.float32)] * 5
    det = FakeDetector(4)
    run = ev.ValidationRun(det, 4, 1)
    dets = run.detections(images, confidence_threshold=0.2, letterbox=False)
    assert [c[0] for c in det.calls] == [4, 4] and det.calls[0][2] == ev.LN_PRE_RESIZE_EXACT
    assert len(dets) == 5
    assert dets[0].shape == (0, 7)                       # 40 / 255 is under the threshold
    for d in dets[1:]:
        assert np.allclose(d[0, 3:], [0.5, 0.5, 1.0, 1.0])   # divided by each image's own size (evaluate.rs:160-166)
    rep = run.evaluate(images, labels, iou_threshold=0.5, confidence_threshold=0.2)
    assert rep["ground_truth_counts"] == [5] and rep["detection_counts"] == [4] and rep["true_positives"] == [4]
    assert abs(rep["average_precision"][0] - 0.8) < 1e-12
    # the report does not depend on the batch size
    rep1 = ev.ValidationRun(FakeDetector(1), 1, 1).evaluate(images, labels, iou_threshold=0.5, confidence_threshold=0.2)
    assert rep1 == rep
    with pytest.raises(ValueError):
        run.detections(images, confidence_threshold=1.5)


class FakeStream:
    """Stands in for the submit_u8 / collect pair of GpuExecutableNetwork on top of a FakeDetector: at most two batches in
    flight, collected in order."""

    def __init__(self, batch):
        self.det, self.queue, self.most = FakeDetector(batch), [], 0

    def submit_u8(self, images, mode=0, packed=None):
        assert images is None and len(self.queue) < 2
        flat, offsets, widths, heights = packed
        self.queue.append(([flat[o:o + 3 * w * h].reshape(h, w, 3) for o, w, h in zip(offsets, widths, heights)], mode))
        self.most = max(self.most, len(self.queue))

    def collect(self, image_w, image_h, thr, nms, letterbox, top_k, max_per_image):
        images, mode = self.queue.pop(0)
        assert list(image_w) == [im.shape[1] for im in images] and list(image_h) == [im.shape[0] for im in images]
        return self.det(images, thr, nms, letterbox, top_k, max_per_image, mode=mode)


def test_validation_run_streamed_gives_the_same_report():
    images = [np.full((10 + i, 20 + 2 * i, 3), 25 * (i + 1), np.uint8) for i in range(9)]
    labels = [np.array([[0, 0.5, 0.5, 1.0, 1.0]], np.float32)] * 9
    plain = ev.ValidationRun(FakeDetector(4), 4, 1)
    fake = FakeStream(4)
    streamed = ev.ValidationRun(None, 4, 1, stream=fake)
    a = plain.detections(images, confidence_threshold=0.2, letterbox=False)
    b = streamed.detections(images, confidence_threshold=0.2, letterbox=False)
    assert len(a) == len(b) == 9 and all(np.array_equal(x, y) for x, y in zip(a, b))
    assert fake.most == 2 and not fake.queue and [c[0] for c in fake.det.calls] == [4, 4, 4]
    assert plain.evaluate(images, labels, confidence_threshold=0.2) == streamed.evaluate(images, labels, confidence_threshold=0.2)
    assert streamed.detections([], confidence_threshold=0.2) == []


def test_detect_server_protocol(tmp_path):
    # lightnet-cli/src/main.rs:558-661: a reply per line, errors as {"error": ...}, default threshold 0.25, normalised boxes
    paths = []
    for i, v in enumerate([200, 100, 30]):
        p = tmp_path / ("im%d.ppm" % i)
        p.write_bytes(b"P6\n# comment\n4 2\n255\n" + bytes([v]) * 24)
        paths.append(str(p))
    assert ev.load_rgb_u8(paths[0]).shape == (2, 4, 3)
    det = FakeDetector(2)
    srv = ev.DetectServer(det, 2)
    lines = [json.dumps({"image": paths[0]}), "not json", json.dumps({"thresh": 0.5}), json.dumps({"image": paths[1], "thresh": 0.5}),
             json.dumps({"image": str(tmp_path / "missing.ppm")}), json.dumps({"image": paths[2], "thresh": 0.05}), "\n"]
    out = io.StringIO()
    srv.serve(iter(l + "\n" for l in lines), out)
    replies = [json.loads(l) for l in out.getvalue().splitlines()]
    assert len(replies) == 6                              # the blank line is skipped
    assert replies[0]["boxes"][0]["class"] == 0 and abs(replies[0]["boxes"][0]["conf"] - 200 / 255) < 1e-6
    assert replies[0]["boxes"][0]["cx"] == 0.5 and replies[0]["boxes"][0]["w"] == 1.0
    assert "invalid request" in replies[1]["error"]
    assert replies[2]["error"] == "request needs an image path"
    assert replies[3] == {"boxes": []}                    # 100 / 255 is under this request's own threshold
    assert "error" in replies[4]
    assert len(replies[5]["boxes"]) == 1
    # requests of one batch are decoded at the lowest threshold among them
    assert all(c[0] == 2 for c in det.calls)


@pytest.mark.gpu
def test_batched_callers_over_a_real_network(tmp_path):
    """A network built for 4 images and one built for 1 give the same normalised records and the same report; the server's
    boxes are the records of the direct call."""
    import lightnet_b200 as ln
    from lightnet_b200 import synth, zoo

    be = ln.B200Backend(0)
    try:
        cfg = zoo.yolov3_tiny_cfg(width=160, height=128, batch=4)
        layers = ln.GpuExecutableNetwork(be, cfg, 1, ln.LN_F32).layers()
        blob = synth.he_weights(layers, 3)
        rng = np.random.default_rng(5)
        images = [rng.integers(0, 256, (90 + 7 * i, 120 + 11 * i, 3), dtype=np.uint8) for i in range(6)]
        labels = [np.array([[int(rng.integers(0, 80)), 0.5, 0.5, 0.3, 0.3]], np.float32) for _ in images]
        reports, dets = [], []
        for batch in (4, 1):
            net = ln.GpuExecutableNetwork(be, cfg, batch, ln.LN_F32)
            net.load_weights(blob)
            run = ev.ValidationRun(net.detect_u8, batch, 80)
            dets.append(run.detections(images, confidence_threshold=0.2, letterbox=True, max_per_image=256))
            reports.append(run.evaluate(images, labels, confidence_threshold=0.2, letterbox=True, max_per_image=256))
            if batch == 4:  # the same pass through the two-slot stream of the network
                streamed = ev.ValidationRun(net.detect_u8, batch, 80, stream=net)
                for a, b in zip(dets[-1], streamed.detections(images, confidence_threshold=0.2, letterbox=True, max_per_image=256)):
                    assert np.array_equal(a, b)
        assert sum(len(d) for d in dets[0]) > 10
        for a, b in zip(*dets):
            assert np.array_equal(a, b)
        assert reports[0] == reports[1]
        net = ln.GpuExecutableNetwork(be, cfg, 4, ln.LN_F32)
        net.load_weights(blob)
        by_name = {"im%d" % i: im for i, im in enumerate(images)}
        srv = ev.DetectServer(net.detect_u8, 4, load=lambda name: by_name[name], max_per_image=256)
        replies = [json.loads(r) for r in srv.handle_lines([json.dumps({"image": "im%d" % i, "thresh": 0.2 + 0.05 * i}) for i in range(6)])]
        for i, rep in enumerate(replies):
            want = dets[0][i][dets[0][i][:, 1] > np.float32(0.2 + 0.05 * i)]
            assert len(rep["boxes"]) == len(want)
            for bx, d in zip(rep["boxes"], want):
                assert bx["class"] == int(d[0]) and bx["conf"] == float(d[1]) and bx["cx"] == float(d[3]) and bx["h"] == float(d[6])
    finally:
        be.close()
