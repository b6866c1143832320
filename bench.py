"""Benchmark of the detector-inference hot path: YOLOv4-608 int8, conv stack + [yolo] decode + NMS.

    python bench.py --gpus N --steps K --warmup W            (this library, one process per GPU)
    python bench.py --impl reference --gpus N --steps K --warmup W   (the CPU restatement of the reference path)

(`--workload` selects one of the baseline's other GPU configurations; the default is the headline one described here.)

A step is one pass over one batch of `--batch` synthetic images per GPU (uniform [0,1) f32, 608x608x3, larger than
L2) through the network built from the generated yolov4 cfg with He-normal random weights: forward, device decode
(threshold 0.25) and per-class NMS (IoU 0.45); the detections land in host memory.  `value` times that with the
input batch already resident in HBM; `e2e` times the same K batches given as HOST buffers (pinned) through
`submit`/`collect`, which keep two batches in flight so the host->device copy of one batch runs under the layers of
the previous one; every step's upload and the device->host read of its detections are inside the timed region.
`e2e_sync` is the same through the one-call-per-batch `detect` (upload, layers and read-back in series), `e2e_u8` /
`e2e_u8_sync` the two forms fed with 8-bit camera images (letterboxed on the device).  Batches are independent, so N
GPUs each run their own batch with no collective on the path (weak scaling); timing is CUDA events on the launching
stream, max over ranks.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "images/sec YOLOv4-608 int8 (conv stack + yolo decode + NMS)"
CONF_THR, NMS_THR, MAX_PER_IMAGE = 0.25, 0.45, 1024

# The default is the headline workload.  The other two are the remaining GPU configurations of the baseline, kept here so
# that their numbers come from the same timing code: `--workload yolov7-640-fp8` (batch 32) and `--workload nms-stress`
# (decode + NMS alone: 256 images x 25200 candidates x 80 classes, threshold 0.001, IoU 0.65, top-k 300).
WORKLOADS = {
    "yolov4-608-int8": dict(model="yolov4", size=608, batch=64, precision="int8", metric=METRIC),
    "yolov7-640-fp8": dict(model="yolov7", size=640, batch=32, precision="fp8",
                           metric="images/sec YOLOv7-640 FP8 E4M3 (conv stack + yolo decode + NMS)"),
    "nms-stress": dict(model=None, size=640, batch=256, precision="f32", metric="decode + NMS GB/s (25200 candidates x 80 classes per image)"),
    "preprocess": dict(model=None, size=608, batch=64, precision="f32", metric="images/sec letterbox pre-processing (640x480 8-bit RGB -> 608x608 f32 NCHW)"),
    "conv-sweep": dict(model=None, size=0, batch=16, precision="int8+fp8", metric="TOP/s single-layer implicit-GEMM convolution (bias + leaky epilogue)"),
    "mma-peak": dict(model=None, size=0, batch=1, precision="int8", metric="TOP/s of a tcgen05.mma-only loop (M=128, N=256, operands resident in shared memory)"),
}
# (channels, height, width, filters, kernel, stride, pad) of the single-layer sweep
SWEEP_LAYERS = [(256, 52, 52, 512, 3, 1, 1), (512, 52, 52, 256, 1, 1, 0), (128, 104, 104, 256, 3, 2, 1)]
STRESS_THR, STRESS_NMS, STRESS_TOPK = 0.001, 0.65, 300


# ncu summaries under profiles/ that hold the tensor-pipe counters of a layer class, keyed by (kernel size, stride, in_c, out_c)
LAYER_CLASS_PROFILES = {
    (3, 1, 128, 128): "profiles/conv_umma_3x3_c128_k128_int8_n64.md",
    (1, 1, 64, 64): "profiles/conv_umma_1x1_c64_k64_mish_int8_n16_global_table.md",
    (3, 1, 256, 512): "profiles/conv_umma_3x3_c256_k512_int8_n128.md",
    (3, 1, 3, 32): "profiles/conv_stem_k3c3_i8_608_n16.md",
    (1, 1, 128, 128): "profiles/conv_umma_1x1_c128_k128_mish_int8_n64.md",
    (3, 1, 32, 64): "profiles/conv_umma_layer_classes_int8.md",
    (3, 1, 256, 256): "profiles/conv_umma_layer_classes_int8.md",
    (1, 1, 128, 64): "profiles/conv_umma_layer_classes_int8.md",
    (3, 1, 512, 1024): "profiles/conv_umma_layer_classes_int8.md",
    (1, 1, 256, 256): "profiles/conv_umma_layer_classes_int8.md",
}


def layer_bytes(layers, i, batch):
    """Algorithmic bytes of convolution i: input, weights and output once at storage width (f32 output for a head), and the
    residual read where the shortcut behind it runs in its epilogue."""
    l = layers[i]
    head = i + 1 < len(layers) and layers[i + 1]["kind"] == "yolo"
    fused = i + 1 < len(layers) and layers[i + 1]["kind"] == "shortcut"
    return (batch * l["in_w"] * l["in_h"] * l["in_c"] * (4 if i == 0 else 1) + l["out_c"] * l["in_c"] * l["size"] ** 2  # (the first layer reads the f32 image)
            + batch * l["out_w"] * l["out_h"] * l["out_c"] * (4 if head else 2 if fused else 1))


def layer_classes(layers, per_layer_ms, batch, peak_tops, hbm_gbs, top=10):
    """Per layer class (kernel, stride, channels -> filters): launches, total ms, TOP/s over the class, its arithmetic intensity
    (operations per algorithmic byte), the roofline that intensity allows (peak x min(1, intensity / ridge), ridge = peak /
    HBM bandwidth) with the fraction of it reached, and the ncu summary that holds its counters where one is committed.
    Sorted by time, the `top` slowest classes; the second value is the whole stack against the sum of its layers' bounds."""
    acc = {}
    t_bound = t_all = 0.0
    for i, (l, ms) in enumerate(zip(layers, per_layer_ms)):
        if l["kind"] != "conv" or ms <= 0:
            continue
        key = (l["size"], l["stride_x"], l["in_c"], l["out_c"])
        ops = 2.0 * l["out_w"] * l["out_h"] * l["out_c"] * l["in_c"] * l["size"] ** 2 * batch
        nbytes = float(layer_bytes(layers, i, batch))
        a = acc.setdefault(key, [0, 0.0, 0.0, 0.0])
        a[0] += 1
        a[1] += float(ms)
        a[2] += ops
        a[3] += nbytes
        if i > 0:  # (the first layer is not a launch of the tensor-core kernel)
            t_bound += max(ops / (peak_tops * 1e12), nbytes / (hbm_gbs * 1e9)) * 1e3
            t_all += float(ms)
    ridge = peak_tops * 1e12 / (hbm_gbs * 1e9)
    rows = []
    for key, (n, ms, ops, nbytes) in sorted(acc.items(), key=lambda kv: -kv[1][1])[:top]:
        ai = ops / nbytes
        bound = peak_tops * min(1.0, ai / ridge)
        rows.append({"layer": "%dx%d s%d C%d->K%d" % (key[0], key[0], key[1], key[2], key[3]), "launches": n, "ms": round(ms, 4),
                     "tops": round(ops / ms / 1e9, 1), "ops_per_byte": round(ai, 1), "bound_tops": round(bound, 1),
                     "frac_of_bound": round(ops / ms / 1e9 / bound, 3), "profile": LAYER_CLASS_PROFILES.get(key)})
    return rows, {"ridge_ops_per_byte": round(ridge, 1), "bound_ms": round(t_bound, 4), "measured_ms": round(t_all, 4),
                  "frac": round(t_bound / t_all, 4) if t_all > 0 else None,
                  "basis": "sum over the tensor-core layers of max(operations / peak, algorithmic bytes / measured HBM bandwidth) against the sum of their measured times (profiled forward)"}


def conv_bytes_per_image(layers):
    """Algorithmic bytes of the tensor-core convolutions: every input and output tensor once (int8; f32 for the heads)."""
    total = 0
    for i, l in enumerate(layers):
        if l["kind"] != "conv" or i == 0:
            continue
        head = i + 1 < len(layers) and layers[i + 1]["kind"] == "yolo"
        total += l["in_w"] * l["in_h"] * l["in_c"] + l["out_w"] * l["out_h"] * l["out_c"] * (4 if head else 1)
    return total


def head_bytes(layers, batch):
    """Algorithmic bytes of decode + NMS: every f32 head value once."""
    return sum(4 * batch * layers[i - 1]["out_w"] * layers[i - 1]["out_h"] * layers[i - 1]["out_c"] for i, l in enumerate(layers) if l["kind"] == "yolo")


def conv_ops_per_image(layers):
    return sum(2 * l["out_w"] * l["out_h"] * l["out_c"] * l["in_c"] * l["size"] ** 2 for l in layers if l["kind"] == "conv")


class ClockSampler(threading.Thread):
    """nvidia-smi clocks / throttle reasons of one GPU every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([v.strip() for v in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(self.samples)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d.get("bf16_tflops_sustained", 1389.8), d.get("hbm_gbs", 6543.7), "measured"
    return 1400.0, 6650.0, "fallback"


def cpu_reference_sample(batch, threads, model="yolov4", size=608, with_unbounded_estimate=True):
    """Times the reference's CPU path (oracle restatement: f32 direct convolution with unfolded batch norm, libm
    activations, decode, confidence sort, apply_nms) on ONE image of the workload.  Returns a dict of seconds.

    Everything in `measured_s` is timed in full on that image, doing the work the GPU arm does: the whole conv stack,
    the decode of every head, and the sorted-list apply_nms pass (lightnet-train/src/detect.rs:1449-1484) stopped once
    MAX_PER_IMAGE rows are kept -- exact for those records, and the GPU arm's own stopping rule.  Like the device path it
    leaves out the thr = 1.0 pre-pass of detect.rs:127-128.

    `unbounded_nms_estimate_s` is NOT part of any reported rate: the reference itself runs apply_nms to the end over all
    ~10^6 candidates of such an image (random weights saturate the heads), a pair loop of minutes to hours; it is timed on
    1/16 of the grid cells and scaled by 16^2, and reported separately, flagged as an extrapolation."""
    from lightnet_b200 import synth, zoo
    from oracle import oracle_api as orc

    cfg = (zoo.yolov4_cfg if model == "yolov4" else zoo.yolov7_cfg)(size, size, batch=1)
    o = orc.Net(cfg, 1)
    o.set_weights(synth.he_weights(o.layers(), 0))
    x = synth.uniform_images(1, 3, size, size, 1)
    orc.set_threads(threads)
    t0 = time.perf_counter()
    o.forward_f32(x)
    t_conv = time.perf_counter() - t0
    specs = zoo.head_specs(cfg)
    yolo_layers = [i for i, l in enumerate(o.layers()) if l["kind"] == "yolo"]
    heads = [np.ascontiguousarray(o.layer_output_f32(li)[0]) for li in yolo_layers]
    full = [dict(sp, gw=h.shape[2], gh=h.shape[1]) for sp, h in zip(specs, heads)]
    t0 = time.perf_counter()
    cands = orc.decode_only(heads, full, size, size, size, size, CONF_THR, letterbox=True)
    t_decode = time.perf_counter() - t0
    t0 = time.perf_counter()
    kept = orc.nms_records_first_k(cands, NMS_THR, MAX_PER_IMAGE)
    t_nms = time.perf_counter() - t0
    out = {"conv_s": t_conv, "decode_s": t_decode, "nms_s": t_nms, "measured_s": t_conv + t_decode + t_nms, "candidates": int(len(cands)),
           "kept": int(len(kept)), "threads": threads}
    if with_unbounded_estimate:
        sub_heads = [np.ascontiguousarray(h[:, ::4, ::4]) for h in heads]
        sub = [dict(sp, gw=h.shape[2], gh=h.shape[1]) for sp, h in zip(specs, sub_heads)]
        t0 = time.perf_counter()
        orc.decode_nms(sub_heads, sub, size, size, size, size, CONF_THR, NMS_THR, letterbox=True)
        out["unbounded_nms_estimate_s"] = (time.perf_counter() - t0) * 256.0
    out["note"] = ("1 image of the batch of %d, all measured: f32 conv stack %.1f s on %d threads (OpenMP over (image, filter)), decode of %d candidates %.2f s, "
                   "confidence sort + apply_nms stopped at %d kept rows %.2f s (one thread, like the reference); no thr=1.0 pre-pass, as on the device"
                   % (batch, t_conv, threads, len(cands), t_decode, MAX_PER_IMAGE, t_nms))
    return out


def cpu_stress_sample(threads):
    """decode + NMS of the reference (oracle restatement, one thread: the reference's decode and apply_nms are serial) on
    ONE full image of the stress workload, all measured: decode of every candidate, confidence sort, and the sorted-list
    apply_nms pass stopped at top-k kept rows (exact for those records; the device path's stopping rule); no thr = 1.0
    pre-pass, as on the device.  Returns (seconds per image, note)."""
    from lightnet_b200 import synth
    from oracle import oracle_api as orc

    heads = [np.ascontiguousarray(h[0]) for h in synth.stress_heads(1)]
    specs = synth.stress_head_specs()
    for sp, h in zip(specs, heads):
        sp["gw"], sp["gh"] = h.shape[2], h.shape[1]
    t0 = time.perf_counter()
    cands = orc.decode_only(heads, specs, 640, 640, 640, 640, STRESS_THR, letterbox=True)
    t_dec = time.perf_counter() - t0
    kept = orc.nms_records_first_k(cands, STRESS_NMS, STRESS_TOPK)
    dt = time.perf_counter() - t0
    note = ("1 image of 256 in full, all measured, one thread: decode of %d candidates %.2f s, confidence sort + apply_nms stopped at %d kept rows %.2f s"
            % (len(cands), t_dec, len(kept), dt - t_dec))
    return dt, note


def run_reference(args, rank):
    """`--impl reference`: the reference's own CPU implementation of the path (restated in the oracle; the Rust crate cannot
    be built in this image), all host threads, a bounded sample per step."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    wl = WORKLOADS[args.workload]
    steps = max(1, min(args.steps, 2))
    total, note = 0.0, ""
    if args.workload in ("conv-sweep", "mma-peak"):
        emit_line(({"impl": "reference", "unavailable": "the reference has no int8 / FP8 convolution; this workload has no CPU arm"}))
        return
    if args.workload == "preprocess":
        from oracle import oracle_api as orc
        rng = np.random.default_rng(300)
        ims = [rng.integers(0, 256, (480, 640, 3), dtype=np.uint8) for _ in range(8)]
        t0 = time.perf_counter()
        for im in ims:
            orc.image_letterbox(orc.image_from_u8(im), 608, 608)
        v = 8.0 / (time.perf_counter() - t0)
        emit_line(({"impl": "reference", "metric": WORKLOADS["preprocess"]["metric"], "value": v, "unit": "images/s", "n_gpus": args.gpus, "steps": 1,
                          "warmup": 0, "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic", "config": {"workload": "letterbox of random 640x480 8-bit RGB images to 608x608 f32 NCHW"},
                          "cpu_baseline": {"value": v, "unit": "images/s", "cores": 1, "kind": "port", "sample": "8 images, one thread"},
                          "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    parts, unbounded = None, None
    for _ in range(steps):
        if wl["model"] is None:
            dt, note = cpu_stress_sample(1)
        else:
            parts = cpu_reference_sample(args.batch, cores, wl["model"], wl["size"], with_unbounded_estimate=unbounded is None)
            unbounded = parts.get("unbounded_nms_estimate_s", unbounded)
            dt, note = parts["measured_s"], parts["note"]
        total += dt
    dt = total / steps
    if wl["model"] is None:
        v, unit, cores = stress_bytes(1) / dt / 1e9, "GB/s", 1
    else:
        v, unit = 1.0 / dt, "images/s"
    line = {"impl": "reference", "metric": wl["metric"], "value": v, "unit": unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": 0, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_text(args.workload), "batch_per_gpu": args.batch,
                       "step": "one image of the batch per step (a bounded sample); steps capped at 2"},
            "cpu_baseline": {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": note},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    line["extrapolated"] = False
    if wl["model"] is not None:
        line["measured_s"] = {k: parts[k] for k in ("conv_s", "decode_s", "nms_s", "measured_s")}
        line["conv_stack_images_per_s"] = 1.0 / parts["conv_s"]
        line["extrapolated_s"] = {"unbounded_nms_estimate_s": unbounded,
                                  "note": "not in value: what apply_nms run to the end (the reference's own behaviour) would add, from 1/16 of the cells x 16^2"}
    emit_line(line)


def workload_text(name):
    wl = WORKLOADS[name]
    if wl["model"] is None:
        return ("decode + NMS stress: 25200 candidates (3 anchors x (80^2+40^2+20^2)) x 80 classes per image, logits xy N(0,1), wh N(0,0.5), "
                "obj/class N(-4,2); threshold %.3f, NMS IoU %.2f, top-k %d" % (STRESS_THR, STRESS_NMS, STRESS_TOPK))
    return "%s-%d %s conv stack + decode(%.2f) + NMS(%.2f), He-normal random weights, uniform[0,1) images" % (
        wl["model"], wl["size"], wl["precision"], CONF_THR, NMS_THR)


def stress_bytes(batch):
    """Algorithmic bytes of decode + NMS: every raw head value is read once (f32)."""
    return batch * 25200 * 85 * 4


def cpu_baseline(batch, model="yolov4", size=608):
    cores = os.cpu_count() or 1
    parts = cpu_reference_sample(batch, cores, model, size, with_unbounded_estimate=False)
    return {"value": 1.0 / parts["measured_s"], "unit": "images/s", "cores": cores, "kind": "port", "sample": parts["note"],
            "measured_s": {k: parts[k] for k in ("conv_s", "decode_s", "nms_s", "measured_s")}, "extrapolated": False}


def make_timer(stream, world):
    """timed(fn, steps): milliseconds of `steps` calls, CUDA events on the launching stream, barrier + device synchronize on
    both sides, maximum over ranks."""
    import torch
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        e1.synchronize()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    return timed


def run_conv_sweep(args, be, rank, world, local_rank):
    """Single layers through the operator-level entry point (ln_conv2d_bias_act_q): weights N(0, 0.02), activations
    leaky(N(0, 1)), bias + leaky epilogue, int8 and FP8.  The operands of one layer fit in L2, so a 512 MB buffer is
    rewritten between timed launches; each launch is timed on its own with CUDA events on the ctx stream."""
    import torch

    import lightnet_b200 as ln

    N = args.batch
    flush = be.zeros_f32((1, 1, 8192, 16384))     # 512 MB
    rng = np.random.default_rng(3)
    bf16_tf, _, basis = measured_peaks()
    peak = 2.0 * bf16_tf
    rows = []
    layers = SWEEP_LAYERS if args.layer < 0 else [SWEEP_LAYERS[args.layer]]
    if args.shape:
        layers = [tuple(int(v) for v in args.shape.split(","))]
    kinds = [("int8", ln.LN_Q8, 127.0), ("fp8", ln.LN_F8, 448.0)]
    if args.precision:
        kinds = [k for k in kinds if k[0] == args.precision]
    launches0 = be.launch_count
    for (c, h, w, f, k, st, p) in layers:
        wt = rng.normal(0, 0.02, (f, c, k, k)).astype(np.float32)
        act = rng.normal(0, 1, (N, c, h, w)).astype(np.float32)
        act = np.where(act > 0, act, np.float32(0.1) * act).astype(np.float32)
        bias = rng.normal(0, 0.05, f).astype(np.float32)
        oh, ow = (h + 2 * p - k) // st + 1, (w + 2 * p - k) // st + 1
        for name, dt, qmax in kinds:
            tw = be.upload_f32(wt.shape, wt)
            wq = be.conv_weights_q(tw, f, c, k, dt)
            tx = be.upload_q(act.shape, act, float(np.abs(act).max() / qmax), dt)
            tb = be.upload_f32((1, f, 1, 1), bias)
            run = lambda: be.conv2d_bias_act_q(tx, wq, tb, (N, f, oh, ow), c, h, w, f, k, st, st, 1, p, 1, args.activation, 4.0 / qmax, ln.LN_OUT_Q)
            for _ in range(max(args.warmup, 3)):
                run()
            ms = []
            be.set_kernel_timing(True)
            for _ in range(args.steps):
                be.activation_f32(flush, "linear")      # rewrites 512 MB: nothing of the layer is left in L2
                run()
                ms.append(be.last_kernel_ms())           # CUDA events around the convolution kernel, on the ctx stream
            be.set_kernel_timing(False)
            t = float(np.median(ms))
            ops = 2.0 * N * oh * ow * f * c * k * k
            rows.append({"layer": "%dx%d s%d C%d->K%d at %dx%d" % (k, k, st, c, f, h, w), "precision": name, "ms": t,
                         "tops": ops / t / 1e9, "frac_of_peak": ops / t / 1e9 / peak})
    launches = be.launch_count - launches0
    if rank == 0:
        best = max(rows, key=lambda r: r["tops"])
        emit_line(({
            "metric": WORKLOADS["conv-sweep"]["metric"], "value": best["tops"], "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": best["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8+fp8", "data": "synthetic",
            "config": {"workload": "single-layer conv sweep, N=%d, weights N(0,0.02), activations leaky(N(0,1)), bias + %s epilogue" % (N, args.activation),
                       "l2": "512 MB rewritten between timed launches", "timing": "median of per-launch CUDA-event times of the convolution kernel (ln_ctx_set_kernel_timing)"},
            "layers": rows, "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "conv_umma_kernel", "achieved": best["tops"], "peak": peak, "unit": "TOP/s",
                         "frac": best["tops"] / peak, "traffic": None, "peak_basis": "2 x %s bf16 sustained (%.1f TFLOP/s)" % (basis, bf16_tf)}}))


def run_mma_peak(args, be, rank, world, local_rank):
    """The tensor-pipe denominators: tcgen05.mma issued back to back on every SM with nothing else in the way (ln_debug_mma_peak),
    for the three operand types, timed with CUDA events inside the library."""
    import lightnet_b200 as ln

    iters = 8192
    launches0 = be.launch_count
    vals = {name: max(be.mma_peak(dt, iters) for _ in range(max(args.steps, 3))) for name, dt in (("int8", ln.LN_Q8), ("fp8", ln.LN_F8), ("f16", ln.LN_F16))}
    bf16_tf, hbm_file, basis = measured_peaks()
    # the other denominator measured here as well: a large device-to-device copy (1 GiB read + 1 GiB written per pass, so far
    # beyond L2), best of a few passes, CUDA events on the copying stream
    import torch
    dev = torch.device("cuda", local_rank)
    src = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    dst = torch.empty_like(src)
    best = 0.0
    for i in range(8):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dst.copy_(src)
        e1.record()
        e1.synchronize()
        if i >= 3:
            best = max(best, 2.0 * src.numel() / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    del src, dst
    if rank == 0:
        emit_line({"metric": WORKLOADS["mma-peak"]["metric"], "value": vals["int8"], "unit": "TOP/s", "n_gpus": world, "steps": max(args.steps, 3), "warmup": 1,
                   "ms_per_step": 2.0 * 128 * 256 * 32 * 4 * iters * be_sm_count(be) / (vals["int8"] * 1e12) * 1e3, "higher_is_better": True, "scaling": "weak",
                   "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                   "config": {"workload": "tcgen05.mma kind::i8 / f8f6f4 / f16, %d x 4 instructions per SM, best of %d launches" % (iters, max(args.steps, 3)),
                              "l2": "no memory traffic: operands stay in shared memory"},
                   "peaks_tops": vals, "copy_gbs": {"value": best, "basis": "device-to-device copy of 1 GiB (read + write bytes), best of 5 after 3 warm-ups", "measured_peaks_file": hbm_file},
                   "gpu_launches": int(be.launch_count - launches0),
                   "roofline": {"bound": "tensor", "kernel": "mma_peak_kernel", "achieved": vals["int8"], "peak": 2.0 * bf16_tf, "unit": "TOP/s",
                                "frac": vals["int8"] / (2.0 * bf16_tf), "traffic": None, "peak_basis": "2 x %s bf16 sustained (%.1f TFLOP/s)" % (basis, bf16_tf)}})


def be_sm_count(be):
    import torch
    return torch.cuda.get_device_properties(be.device).multi_processor_count


def run_preprocess(args, be, rank, world, local_rank):
    """ln_image_preprocess_u8 on a batch of synthetic 640x480 8-bit images in pinned host memory (the upload is inside the call);
    CPU arm: the oracle's restatement of PlanarRgbImage::from_interleaved_rgb_u8 + letterbox on one image, one thread."""
    import torch

    import lightnet_b200 as ln

    B = args.batch
    rng = np.random.default_rng(300 + rank)
    images = [rng.integers(0, 256, (480, 640, 3), dtype=np.uint8) for _ in range(B)]
    flat, off, w, h = ln.pack_u8_images(images)
    flat = torch.from_numpy(flat).pin_memory().numpy()
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local_rank))
    timed = make_timer(stream, world)
    size = WORKLOADS["preprocess"]["size"]

    def call():
        return be._out(be.lib.ln_image_preprocess_u8, ln._ptr(flat), ln._ptr(off), ln._ptr(w), ln._ptr(h), B, ln.LN_PRE_LETTERBOX, size, size)

    for _ in range(max(args.warmup, 3)):
        call()
    launches0 = be.launch_count
    ms = timed(call, args.steps)
    launches = be.launch_count - launches0
    out_bytes = B * 3 * size * size * 4
    _, hbm_gbs, basis = measured_peaks()
    if rank == 0:
        line = {"metric": WORKLOADS["preprocess"]["metric"], "value": B * world * args.steps / (ms * 1e-3), "unit": "images/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "letterbox of %d random 640x480 8-bit RGB images to %dx%d f32 NCHW" % (B, size, size), "batch_per_gpu": B,
                           "l2": "output larger than L2 (%.0f MB)" % (out_bytes / 1e6)},
                "e2e": {"value": B * world * args.steps / (ms * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(flat.nbytes), "d2h_bytes_per_step": 0,
                        "api": "ln_image_preprocess_u8 (the timed call takes host pixels: value and e2e are the same measurement)"},
                "gpu_launches": int(launches),
                "roofline": {"bound": "hbm", "kernel": "image_float_resize_kernel + the upload of the pixels", "achieved": (flat.nbytes + out_bytes) * args.steps / (ms * 1e-3) / 1e9,
                             "peak": hbm_gbs, "unit": "GB/s", "frac": (flat.nbytes + out_bytes) * args.steps / (ms * 1e-3) / 1e9 / hbm_gbs, "traffic": None,
                             "peak_basis": "%s copy bandwidth; the call is bound by the 59 MB upload over PCIe, not by HBM" % basis}}
        if not args.no_cpu_baseline:
            from oracle import oracle_api as orc
            t0 = time.perf_counter()
            for im in images[:8]:
                orc.image_letterbox(orc.image_from_u8(im), size, size)
            dt = (time.perf_counter() - t0) / 8
            line["cpu_baseline"] = {"value": 1.0 / dt, "unit": "images/s", "cores": 1, "kind": "port", "sample": "8 of the %d images, one thread (the reference's resize is serial)" % B}
        emit_line((line))


def run_nms_stress(args, be, rank, world, local_rank):
    """decode + NMS alone on synthetic heads (resident in HBM for `value`; uploaded from pinned host memory inside the timed
    region for `e2e`).  The heads of 256 images are 2.19 GB, far larger than L2."""
    import torch

    from lightnet_b200 import synth

    B = args.batch
    heads_np = synth.stress_heads(B, seed=2 + rank)
    specs = synth.stress_head_specs()
    pinned = [torch.from_numpy(h).pin_memory() for h in heads_np]
    heads_np = [p.numpy() for p in pinned]
    dev = [dict(raw=be.upload_f32(h.shape, h), classes=s["classes"], anchors=s["anchors"], scale_x_y=1.0, new_coords=0)
           for h, s in zip(heads_np, specs)]
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local_rank))
    timed = make_timer(stream, world)
    call = lambda hs: be.yolo_decode_nms(hs, 640, 640, 640, 640, STRESS_THR, STRESS_NMS, True, STRESS_TOPK, STRESS_TOPK)

    def e2e_call():
        hs = [dict(d, raw=be.upload_f32(h.shape, h)) for d, h in zip(dev, heads_np)]
        return call(hs)

    dets = None
    for _ in range(args.warmup):
        dets = call(dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = be.launch_count
    ms = timed(lambda: call(dev), args.steps)
    launches = be.launch_count - launches0
    e2e_call()
    ms_e2e = timed(e2e_call, args.steps)
    clocks = sampler.summary()
    nbytes = stress_bytes(B)
    _, hbm_gbs, basis = measured_peaks()
    gbs = nbytes * args.steps / (ms * 1e-3) / 1e9
    if rank == 0:
        line = {
            "metric": WORKLOADS["nms-stress"]["metric"], "value": gbs * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_text("nms-stress"), "batch_per_gpu": B, "l2": "inputs larger than L2 (%.2f GB of heads)" % (nbytes / 1e9),
                       "parallelism": "batch-sharded, no collective"},
            "images_per_s": B * world * args.steps / (ms * 1e-3),
            "e2e": {"value": nbytes * world * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(nbytes),
                    "d2h_bytes_per_step": int(B * STRESS_TOPK * 28 + B * 4), "api": "ln_tensor_upload_f32 x3 + ln_yolo_decode_nms"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "whole decode + NMS call (scan, selection, sort, suppression kernels)", "achieved": gbs,
                         "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs, "traffic": None, "peak_basis": "%s copy bandwidth" % basis},
            "clocks": clocks,
            "detections_first_image": int(len(dets[0])) if dets is not None else None,
        }
        if world == 1 and not args.no_cpu_baseline:
            dt, note = cpu_stress_sample(1)
            line["cpu_baseline"] = {"value": stress_bytes(1) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port", "sample": note}
        emit_line((line))


def bind_to_gpu_cpus(device_index):
    """One rank per GPU: run this process (and so first-touch its pinned upload buffers) on the host cores next to its GPU,
    as the driver reports them (read-only NVML query; only this process's own CPU affinity changes).  Best effort."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:  # the CUDA index need not be the NVML index: go through the PCI address
            import torch
            pr = torch.cuda.get_device_properties(device_index)
            h = pynvml.nvmlDeviceGetHandleByPciBusId(("%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)).encode())
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus = near & os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception as e:  # no NVML, a restricted container, ...: keep the affinity as it is
        print("cpu binding skipped: %s" % e, file=sys.stderr)


_RESULT_OUT = None


def claim_stdout():
    """Keeps the process's real stdout for the one JSON line and points file descriptor 1 at stderr, so that whatever a
    library prints on stdout (NCCL's version banner under torchrun) cannot land beside the line."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit_line(obj):
    out = _RESULT_OUT or sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="yolov4-608-int8", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="images per GPU per step (0 = the workload's own: 64 / 32 / 256)")
    ap.add_argument("--micro-batch", type=int, default=0, help="images per pass through the layers; 0 (default, fastest) = the whole batch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layer", type=int, default=-1, help="conv-sweep: index of the one layer to run (default all)")
    ap.add_argument("--precision", default="", choices=["", "int8", "fp8"], help="conv-sweep: one precision only")
    ap.add_argument("--shape", default="", help="conv-sweep: one layer C,H,W,K,k,stride,pad instead of the three of the sweep")
    ap.add_argument("--activation", default="leaky", help="conv-sweep: epilogue activation (leaky, mish, swish, relu, linear, logistic)")
    ap.add_argument("--width", type=int, default=0)
    ap.add_argument("--height", type=int, default=0)
    args = ap.parse_args()
    claim_stdout()
    wl = WORKLOADS[args.workload]
    args.batch = args.batch or wl["batch"]
    args.width = args.width or wl["size"]
    args.height = args.height or wl["size"]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    import lightnet_b200 as ln
    from lightnet_b200 import synth, zoo

    torch.cuda.set_device(local_rank)
    if world > 1:
        bind_to_gpu_cpus(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B = args.batch
    be = ln.B200Backend(local_rank)
    if wl["model"] is None:
        {"conv-sweep": run_conv_sweep, "preprocess": run_preprocess, "mma-peak": run_mma_peak}.get(args.workload, run_nms_stress)(args, be, rank, world, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return
    make_cfg = zoo.yolov4_cfg if wl["model"] == "yolov4" else zoo.yolov7_cfg
    prec = ln.LN_Q8 if wl["precision"] == "int8" else ln.LN_F8
    cfg = make_cfg(args.width, args.height, batch=B)
    layers = ln.GpuExecutableNetwork(be, make_cfg(args.width, args.height, batch=1), 1, ln.LN_F32).layers()
    blob = synth.he_weights(layers, 0)
    # calibration: a small f32 batch on the device gives the per-tensor scales
    calib = ln.GpuExecutableNetwork(be, make_cfg(args.width, args.height, batch=2), 2, prec)
    calib.load_weights(blob)
    calib.calibrate(synth.uniform_images(2, 3, args.height, args.width, 7))
    scales = calib.scales()
    del calib
    net = ln.GpuExecutableNetwork(be, cfg, B, prec)
    net.load_weights(blob)
    net.set_scales(scales)
    net.set_micro_batch(args.micro_batch if args.micro_batch < B else 0)

    x_host = torch.from_numpy(synth.uniform_images(B, 3, args.height, args.width, 100 + rank)).pin_memory()
    x_np = x_host.numpy()
    x_dev = be.upload_f32(x_np.shape, x_np)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local_rank))
    # the records come back into page-locked host buffers (by DMA, no staging copy), reused from step to step
    rec_pinned = torch.empty((B, MAX_PER_IMAGE, 7), dtype=torch.float32).pin_memory()
    cnt_pinned = torch.zeros((B,), dtype=torch.int32).pin_memory()
    det_args = (args.width, args.height, CONF_THR, NMS_THR, True, 0, MAX_PER_IMAGE, (rec_pinned.numpy(), cnt_pinned.numpy()))

    timed = make_timer(stream, world)

    dets = None
    for _ in range(args.warmup):
        dets = net.detect_device(x_dev, *det_args)
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = be.launch_count
    ms = timed(lambda: net.detect_device(x_dev, *det_args), args.steps)
    launches = be.launch_count - launches0
    fwd_ms, nms_ms = net.last_times_ms()
    for _ in range(args.warmup):   # the host-input path has its own plans and graphs to warm
        net.detect(x_np, *det_args)
    ms_sync = timed(lambda: net.detect(x_np, *det_args), args.steps)
    # A stream of batches through ln_net_submit / ln_net_collect: the upload of batch i + 1 (from its own pinned buffer) runs
    # while batch i goes through the layers.  Every step's upload and every step's read-back are inside the timed region.
    x2_host = torch.from_numpy(synth.uniform_images(B, 3, args.height, args.width, 300 + rank)).pin_memory()
    xs = (x_np, x2_host.numpy())

    def stream_of_batches(steps):
        net.submit(xs[0])
        for i in range(steps):
            if i + 1 < steps:
                net.submit(xs[(i + 1) & 1])
            net.collect(*det_args)

    stream_of_batches(max(args.warmup, 2))
    ms_e2e = timed(lambda: stream_of_batches(args.steps), 1)
    # what the PCIe link gives this rank while all ranks copy at once: one plain pinned -> device copy of the batch per step
    tstream = torch.cuda.Stream(device=torch.device("cuda", local_rank))
    with torch.cuda.stream(tstream):
        scratch_dev = torch.empty(x_host.shape, dtype=torch.float32, device=torch.device("cuda", local_rank))
        scratch_dev.copy_(x_host, non_blocking=True)
    tstream.synchronize()
    timed_copy = make_timer(tstream, world)

    def plain_copy():
        with torch.cuda.stream(tstream):
            scratch_dev.copy_(x_host, non_blocking=True)

    ms_copy = timed_copy(plain_copy, args.steps)
    del scratch_dev
    # the same call fed with 8-bit camera-sized images (640 x 480, letterboxed on the device): what a caller that does not
    # pre-process on the host pays end to end
    rng8 = np.random.default_rng(200 + rank)
    images8 = [rng8.integers(0, 256, (480, 640, 3), dtype=np.uint8) for _ in range(B)]
    flat8, off8, w8, h8 = ln.pack_u8_images(images8)
    flat8_pinned = torch.from_numpy(flat8).pin_memory()
    packed8 = (flat8_pinned.numpy(), off8, w8, h8)
    u8_call = lambda: net.detect_u8(None, CONF_THR, NMS_THR, True, 0, MAX_PER_IMAGE, packed=packed8, out=det_args[-1])
    for _ in range(args.warmup):
        u8_call()
    ms_u8_sync = timed(u8_call, args.steps)
    # the stream of batches again, fed with the 8-bit images (two pinned pixel buffers; upload + letterbox of batch i + 1 run
    # on the copy stream while batch i goes through the layers)
    images8b = [rng8.integers(0, 256, (480, 640, 3), dtype=np.uint8) for _ in range(B)]
    flat8b, off8b, w8b, h8b = ln.pack_u8_images(images8b)
    flat8b_pinned = torch.from_numpy(flat8b).pin_memory()
    packs8 = (packed8, (flat8b_pinned.numpy(), off8b, w8b, h8b))
    u8_args = (CONF_THR, NMS_THR, True, 0, MAX_PER_IMAGE, det_args[-1])

    def stream_of_u8_batches(steps):
        net.submit_u8(None, packed=packs8[0])
        for i in range(steps):
            if i + 1 < steps:
                net.submit_u8(None, packed=packs8[(i + 1) & 1])
            pk = packs8[i & 1]
            net.collect(pk[2], pk[3], *u8_args)

    stream_of_u8_batches(max(args.warmup, 2))
    ms_u8 = timed(lambda: stream_of_u8_batches(args.steps), 1)
    clocks = sampler.summary()

    # roofline of the dominant kernel (tensor-core convolution), from a profiled forward
    net.set_profile(True)
    net.forward_device(x_dev)
    per_layer, per_op = net.profile()
    net.set_profile(False)
    umma_ms, umma_launches = per_op["conv_umma"]
    ops_img = conv_ops_per_image(layers) - 2 * layers[0]["out_w"] * layers[0]["out_h"] * layers[0]["out_c"] * layers[0]["in_c"] * layers[0]["size"] ** 2
    bf16_tf, hbm_gbs, basis = measured_peaks()
    peak = 2.0 * bf16_tf  # dense int8 / FP8 tensor throughput is twice bf16 on this part
    mma_peak = max(be.mma_peak(prec, 4096) for _ in range(3))  # the same denominator measured: a tcgen05.mma-only loop on every SM
    achieved = ops_img * B / (umma_ms * 1e-3) / 1e12 if umma_ms > 0 else 0.0

    classes, adjusted = layer_classes(layers, per_layer, B, peak, hbm_gbs)
    if rank == 0:
        line = {
            "metric": wl["metric"], "value": B * world * args.steps / (ms * 1e-3), "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": wl["precision"], "data": "synthetic",
            "config": {"workload": workload_text(args.workload),
                       "batch_per_gpu": B, "micro_batch": args.micro_batch, "max_detections_per_image": MAX_PER_IMAGE,
                       "l2": "inputs larger than L2 (%.0f MB f32 batch)" % (x_np.nbytes / 1e6), "parallelism": "batch-sharded, no collective"},
            "e2e": {"value": B * world * args.steps / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(x_np.nbytes),
                    "d2h_bytes_per_step": int(B * MAX_PER_IMAGE * 28 + B * 4),
                    "api": "ln_net_submit + ln_net_collect on a stream of host f32 NCHW batches (two pinned buffers, the upload of the next batch overlaps the layers of the current one; %d uploads and %d read-backs inside the timed region)" % (args.steps, args.steps)},
            "h2d": {"gbs_per_rank": x_np.nbytes * args.steps / (ms_copy * 1e-3) / 1e9, "ms_per_batch": ms_copy / args.steps,
                    "basis": "a plain cudaMemcpyAsync of the pinned f32 batch on every rank at once, slowest rank"},
            "e2e_sync": {"value": B * world * args.steps / (ms_sync * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(x_np.nbytes),
                         "api": "ln_net_detect, one synchronous call per batch (the batch is uploaded and run in two parts, %d + %d images, as a two-stage pipeline)" % ((B // 4, B - B // 4) if B >= 16 else (B // 2, B - B // 2))},
            "e2e_u8": {"value": B * world * args.steps / (ms_u8 * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(flat8.nbytes),
                       "api": "ln_net_submit_u8 + ln_net_collect on a stream of batches of host 8-bit 640x480 RGB images (device letterbox on the copy stream under the layers of the previous batch)"},
            "e2e_u8_sync": {"value": B * world * args.steps / (ms_u8_sync * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(flat8.nbytes),
                            "api": "ln_net_detect_u8, one synchronous call per batch (upload -> device letterbox -> detections)"},
            "gpu_launches": int(launches),
            "phases_ms": {"layers": fwd_ms, "decode_nms": nms_ms},
            "roofline": {"bound": "tensor", "kernel": "conv_umma_kernel (%s implicit GEMM, all layers but the first)" % wl["precision"], "achieved": achieved,
                         "peak": peak, "unit": "TOP/s", "frac": achieved / peak,
                         "traffic": None,
                         "traffic_basis": "not measured at this batch: an ncu capture of all launches of a 64-image step is beyond the size a capture may have; per-launch DRAM bytes of eleven layer classes are in profiles/conv_umma_layer_classes_int8.md: reads equal the algorithmic input bytes in every class (taps and filter tiles re-read L2, not DRAM), writes stay below the output bytes while an output fits in L2",
                         "algorithmic_bytes": conv_bytes_per_image(layers) * B,
                         "peak_basis": "2 x %s bf16 sustained (%.1f TFLOP/s)" % (basis, bf16_tf), "launches_per_step": umma_launches,
                         "peak_mma_loop": mma_peak, "frac_of_mma_loop": achieved / mma_peak if mma_peak > 0 else None,
                         "peak_mma_loop_basis": "tcgen05.mma-only loop of this library on this GPU (ln_debug_mma_peak), burst clocks",
                         "ms_per_step": umma_ms, "intensity_adjusted": adjusted},
            "kernel_classes_ms": {k: v[0] for k, v in per_op.items()},
            "layer_classes": classes,
            "nms_gbs": {"value": head_bytes(layers, B) / (nms_ms * 1e-3) / 1e9 if nms_ms > 0 else None, "unit": "GB/s",
                        "basis": "f32 head tensors read once (%d bytes) / phases_ms.decode_nms" % head_bytes(layers, B),
                        "frac_of_hbm": head_bytes(layers, B) / (nms_ms * 1e-3) / 1e9 / hbm_gbs if nms_ms > 0 else None},
            "clocks": clocks,
            "detections_first_image": int(len(dets[0])) if dets is not None else None,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(B, wl["model"], wl["size"])
        emit_line((line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
