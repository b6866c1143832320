"""Batched callers of the detector path: the two places of the reference that drive detection one image at a time.

* `ValidationRun` stands where `ValidationDataset::evaluate_with_forward` does (lightnet-train/src/evaluate.rs:134-177):
  for every validation image, load -> letterbox (or INTER_LINEAR_EXACT resize when `letterbox` is off, :146-151) ->
  forward -> decode + NMS in the image's own pixel frame -> boxes divided by the image size (:160-166) -> `detector_map`.
  The reference does that with batch 1, sequentially; here the images go through `GpuExecutableNetwork.detect_u8`
  `batch` at a time (device pre-processing, one forward, one decode + NMS per batch), optionally sharded over ranks by
  `sharding.ShardedDetector`.  The per-image records, and therefore the report, do not depend on the batch size.
* `detector_map` is the ranking / matching / integration of evaluate.rs:358-385 and :523-621 (AP per class from the
  precision envelope, counts at the report confidence 0.25).
* `DetectServer` speaks the line protocol of `lightnet-rs detect-server` (lightnet-cli/src/main.rs:558-661): one JSON
  request `{"image": path, "thresh": t}` per line, one reply `{"boxes": [{"class","conf","cx","cy","w","h"}]}` or
  `{"error": message}` per line, letterbox, NMS 0.45.  Requests are collected into batches; a request's own threshold is
  applied to the records of a batch that was decoded at the lowest threshold in it (greedy NMS never lets a lower-scoring
  box suppress a higher-scoring one, so the records above a threshold are those of a run at that threshold).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Iterable, List, Sequence

import numpy as np

from . import LN_PRE_LETTERBOX, LN_PRE_RESIZE_EXACT

REPORT_CONFIDENCE = 0.25  # evaluate.rs:28


def load_rgb_u8(path: str) -> np.ndarray:
    """An image file as an interleaved 8-bit RGB array [h, w, 3] (PlanarRgbImage::load keeps 8-bit RGB, image.rs:57).
    Binary PPM (P6, maxval 255) is read here; other formats go through Pillow when it is installed."""
    with open(path, "rb") as f:
        data = f.read()
    if data[:2] == b"P6":
        fields, pos = [], 2
        while len(fields) < 3:
            while data[pos:pos + 1].isspace():
                pos += 1
            if data[pos:pos + 1] == b"#":
                pos = data.index(b"\n", pos) + 1
                continue
            end = pos
            while not data[end:end + 1].isspace():
                end += 1
            fields.append(int(data[pos:end]))
            pos = end
        w, h, maxval = fields
        if maxval != 255:
            raise ValueError("%s: only 8-bit PPM is supported" % path)
        pix = np.frombuffer(data, np.uint8, count=w * h * 3, offset=pos + 1)
        return pix.reshape(h, w, 3).copy()
    try:
        from PIL import Image
    except ImportError as e:  # pragma: no cover
        raise ValueError("%s: not a binary PPM and Pillow is not installed" % path) from e
    with Image.open(path) as im:
        return np.asarray(im.convert("RGB"), np.uint8).copy()


def _iou(d, t) -> np.float32:
    """evaluate.rs:622-632 on centre/size boxes, f32 arithmetic."""
    f = np.float32
    dx, dy, dw, dh = (f(v) for v in d)
    tx, ty, tw, th = (f(v) for v in t)
    half = f(0.5)
    iw = max(min(dx + dw * half, tx + tw * half) - max(dx - dw * half, tx - tw * half), f(0))
    ih = max(min(dy + dh * half, ty + th * half) - max(dy - dh * half, ty - th * half), f(0))
    inter = f(iw * ih)
    union = f(max(dw, f(0)) * max(dh, f(0)) + max(tw, f(0)) * max(th, f(0)) - inter)
    return f(inter / union) if union > 0 else f(0)


def detector_map(samples, classes: int, iou_threshold: float) -> dict:
    """samples: per image (labels [n, 5] {class, x, y, w, h}, detections [m, 7] {class, conf, obj, x, y, w, h}), boxes of both
    in the same normalised frame.  Returns the fields of MapReport (evaluate.rs:12-27)."""
    if classes <= 0 or not np.isfinite(iou_threshold) or not (0.0 <= iou_threshold <= 1.0):
        raise ValueError("invalid mAP class count or IoU threshold")
    counts = [0] * classes
    preds: List[list] = [[] for _ in range(classes)]
    for image, (truth, dets) in enumerate(samples):
        for lab in np.asarray(truth, np.float32).reshape(-1, 5):
            c = int(lab[0])
            if not 0 <= c < classes:
                raise ValueError("validation truth class out of range")
            counts[c] += 1
        for det in np.asarray(dets, np.float32).reshape(-1, 7):
            c = int(det[0])
            if not 0 <= c < classes or not np.isfinite(det[1]):
                raise ValueError("invalid validation detection class/score")
            preds[c].append((image, det))
    thr = np.float32(iou_threshold)
    report = dict(average_precision=[0.0] * classes, ground_truth_counts=counts, detection_counts=[len(p) for p in preds],
                  true_positives=[0] * classes, false_positives=[0] * classes, false_negatives=[0] * classes, average_iou=[0.0] * classes)
    for c, ranked in enumerate(preds):
        ranked.sort(key=lambda e: -float(e[1][1]))  # stable, like sort_by(total_cmp) on finite scores
        used = [np.zeros(len(np.asarray(s[0]).reshape(-1, 5)), bool) for s in samples]
        points = []
        tp = fp = rtp = rfp = 0
        iou_sum = 0.0
        for image, det in ranked:
            labels = np.asarray(samples[image][0], np.float32).reshape(-1, 5)
            best, best_iou = -1, thr
            for index, lab in enumerate(labels):
                if int(lab[0]) != c:
                    continue
                v = _iou(det[3:7], lab[1:5])
                if v > best_iou:
                    best, best_iou = index, v
            counted = det[1] >= np.float32(REPORT_CONFIDENCE)
            if best >= 0 and not used[image][best]:
                used[image][best] = True
                tp += 1
                if counted:
                    rtp += 1
                    iou_sum += float(best_iou)
            else:
                fp += 1
                rfp += int(counted)
            points.append((tp / max(counts[c], 1), tp / (tp + fp)))
        envelope = area = 0.0
        for i in range(len(points) - 1, -1, -1):
            envelope = max(envelope, points[i][1])
            prev = points[i - 1][0] if i else 0.0
            area += (points[i][0] - prev) * envelope
        report["average_precision"][c] = area
        report["true_positives"][c] = rtp
        report["false_positives"][c] = rfp
        report["false_negatives"][c] = max(counts[c] - rtp, 0)
        report["average_iou"][c] = iou_sum / rtp if rtp else 0.0
    report["mean_average_precision"] = sum(report["average_precision"]) / classes
    return report


def normalise(records: np.ndarray, width: int, height: int) -> np.ndarray:
    """evaluate.rs:160-166: x, w by the image width and y, h by its height, single f32 divisions."""
    out = np.array(records, np.float32, copy=True).reshape(-1, 7)
    out[:, 3] /= np.float32(width)
    out[:, 5] /= np.float32(width)
    out[:, 4] /= np.float32(height)
    out[:, 6] /= np.float32(height)
    return out


class ValidationRun:
    """Batched `detector map` pass.  `detect_u8(images, ...)` is `GpuExecutableNetwork.detect_u8` of a network built for `batch`
    images (or a `sharding.ShardedDetector` around it); images are interleaved 8-bit RGB arrays of any sizes.  With `stream` =
    that network (anything with its `submit_u8` / `collect`), the batches go through the two-slot stream instead: packing, upload
    and resize of the next batch run while the current one is in the layers; the records are the same."""

    def __init__(self, detect_u8: Callable[..., list], batch: int, classes: int, stream=None):
        if batch < 1 or classes < 1:
            raise ValueError("batch and classes must be positive")
        self.detect_u8, self.batch, self.classes, self.stream = detect_u8, batch, classes, stream

    def detections(self, images: Sequence[np.ndarray], confidence_threshold=0.25, nms_threshold=0.45, letterbox=True, max_per_image=1024):
        """Per image, in order: normalised records.  A short last batch is filled by repeating its last image; the results of the
        fill-ins are dropped."""
        if not (np.isfinite(confidence_threshold) and 0.0 <= confidence_threshold <= 1.0 and np.isfinite(nms_threshold) and 0.0 <= nms_threshold <= 1.0):
            raise ValueError("invalid validation confidence/NMS threshold")  # evaluate.rs:337-345
        mode = LN_PRE_LETTERBOX if letterbox else LN_PRE_RESIZE_EXACT
        out = []
        parts = []
        for start in range(0, len(images), self.batch):
            part = list(images[start:start + self.batch])
            real = len(part)
            parts.append((part + [part[-1]] * (self.batch - real), real))
        if self.stream is not None and parts:
            from . import pack_u8_images

            def submit(k):
                packed = pack_u8_images(parts[k][0])
                self.stream.submit_u8(None, mode=mode, packed=packed)
                return packed

            current = submit(0)
            for k, (part, real) in enumerate(parts):
                following = submit(k + 1) if k + 1 < len(parts) else None
                recs = self.stream.collect(current[2], current[3], confidence_threshold, nms_threshold, letterbox, 0, max_per_image)
                for im, r in zip(part[:real], recs[:real]):
                    out.append(normalise(r, im.shape[1], im.shape[0]))
                current = following
            return out
        for part, real in parts:
            recs = self.detect_u8(part, confidence_threshold, nms_threshold, letterbox, 0, max_per_image, mode=mode)
            for im, r in zip(part[:real], recs[:real]):
                out.append(normalise(r, im.shape[1], im.shape[0]))
        return out

    def evaluate(self, images: Sequence[np.ndarray], labels: Sequence[np.ndarray], iou_threshold=0.5, **options) -> dict:
        if len(images) != len(labels):
            raise ValueError("one label array per image")
        dets = self.detections(images, **options)
        return detector_map(list(zip(labels, dets)), self.classes, iou_threshold)


class DetectServer:
    """`lightnet-rs detect-server` over a batched detector: `handle_lines` answers a group of request lines, `serve` runs the
    stdin / stdout loop, answering in request order and flushing whenever `batch` requests are pending or the input ends."""

    def __init__(self, detect_u8: Callable[..., list], batch: int, load: Callable[[str], np.ndarray] = load_rgb_u8, max_per_image=1024):
        self.detect_u8, self.batch, self.load, self.max_per_image = detect_u8, batch, load, max_per_image

    def handle_lines(self, lines: Sequence[str]) -> List[str]:
        replies: List = [None] * len(lines)
        work = []  # (position, image, threshold)
        for pos, line in enumerate(lines):
            try:
                req = json.loads(line)
            except ValueError as e:
                replies[pos] = {"error": "invalid request: %s" % e}
                continue
            image = req.get("image") if isinstance(req, dict) else None
            if not isinstance(image, str):
                replies[pos] = {"error": "request needs an image path"}
                continue
            t = req.get("thresh", 0.25)
            t = float(t) if isinstance(t, (int, float)) and not isinstance(t, bool) else 0.25
            try:
                work.append((pos, self.load(image), min(max(np.float32(t), np.float32(0)), np.float32(1))))
            except Exception as e:  # a bad image never terminates the server
                replies[pos] = {"error": str(e)}
        for start in range(0, len(work), self.batch):
            part = work[start:start + self.batch]
            images = [w[1] for w in part]
            images += [images[-1]] * (self.batch - len(part))
            low = min(w[2] for w in part)
            try:
                recs = self.detect_u8(images, float(low), 0.45, True, 0, self.max_per_image, mode=LN_PRE_LETTERBOX)
            except Exception as e:
                for pos, _, _ in part:
                    replies[pos] = {"error": str(e)}
                continue
            for (pos, im, t), r in zip(part, recs):
                h, w = im.shape[:2]
                r = r[r[:, 1] > t]  # the decode keeps confidence > threshold (detect.rs:1005)
                wn, hn = np.float32(max(w, 1)), np.float32(max(h, 1))
                replies[pos] = {"boxes": [{"class": int(d[0]), "conf": float(d[1]), "cx": float(d[3] / wn), "cy": float(d[4] / hn),
                                           "w": float(d[5] / wn), "h": float(d[6] / hn)} for d in r]}
        return [json.dumps(r) for r in replies]

    def serve(self, stdin: Iterable[str], stdout) -> None:
        pending: List[str] = []

        def flush():
            for reply in self.handle_lines(pending):
                stdout.write(reply + "\n")
            stdout.flush()
            pending.clear()

        for line in stdin:
            if not line.strip():
                continue
            pending.append(line)
            if len(pending) >= self.batch:
                flush()
        if pending:
            flush()


def read_yolo_labels(path: str, classes: int) -> np.ndarray:
    """A Darknet label file: `class x y w h` per line, normalised centre / size (load_yolo_labels; evaluate.rs:111)."""
    rows = []
    if os.path.exists(path):
        for line in open(path):
            f = line.split()
            if len(f) < 5:
                continue
            c = int(f[0])
            if not 0 <= c < classes:
                raise ValueError("%s: class %d out of range" % (path, c))
            rows.append([c] + [float(v) for v in f[1:5]])
    return np.asarray(rows, np.float32).reshape(-1, 5)
