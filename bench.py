"""Benchmark of the detector-inference hot path: YOLOv4-608 int8, conv stack + [yolo] decode + NMS.

    python bench.py --gpus N --steps K --warmup W            (this library, one process per GPU)
    python bench.py --impl reference --gpus N --steps K --warmup W   (the CPU restatement of the reference path)

A step is one pass over one batch of `--batch` synthetic images per GPU (uniform [0,1) f32, 608x608x3, larger than
L2) through the network built from the generated yolov4 cfg with He-normal random weights: forward, device decode
(threshold 0.25) and per-class NMS (IoU 0.45); the detections land in host memory.  `value` times that with the
input batch already resident in HBM; `e2e` times the same call given HOST buffers (pinned), so the host->device copy
of the batch and the device->host read of the detections are inside the timed region.  Batches are independent, so N
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


def cpu_reference_sample(batch, threads):
    """Times the reference's CPU path (oracle restatement: f32 direct convolution with unfolded batch norm, libm
    activations, decode, the two apply_nms passes) on ONE image of the workload and returns (seconds per image, note).

    The conv stack of the image is timed in full.  decode + NMS is timed on a sample: apply_nms
    (lightnet-train/src/detect.rs:1449-1484) visits every pair of candidates, and this workload (random weights,
    saturated heads) yields about 10^6 candidates per image, i.e. minutes of single-threaded pair visits.  The sample
    keeps every 4th row and every 4th column of each head (1/16 of the cells, hence of the candidates); its time is
    multiplied by 16^2, the growth of the pair count."""
    from lightnet_b200 import synth, zoo
    from oracle import oracle_api as orc

    cfg = zoo.yolov4_cfg(batch=1)
    o = orc.Net(cfg, 1)
    o.set_weights(synth.he_weights(o.layers(), 0))
    x = synth.uniform_images(1, 3, 608, 608, 1)
    orc.set_threads(threads)
    t0 = time.perf_counter()
    o.forward_f32(x)
    t_conv = time.perf_counter() - t0
    specs = zoo.head_specs(cfg)
    heads, sub = [], []
    yolo_layers = [i for i, l in enumerate(o.layers()) if l["kind"] == "yolo"]
    for li, sp in zip(yolo_layers, specs):
        h = o.layer_output_f32(li)[0]                      # [255, g, g]
        hs = np.ascontiguousarray(h[:, ::4, ::4])
        heads.append(hs)
        sub.append(dict(gw=hs.shape[2], gh=hs.shape[1], classes=sp["classes"], anchors=sp["anchors"], scale_x_y=sp["scale_x_y"],
                        new_coords=sp["new_coords"]))
    t0 = time.perf_counter()
    d = orc.decode_nms(heads, sub, 608, 608, 608, 608, CONF_THR, NMS_THR, letterbox=True)
    t_nms_sample = time.perf_counter() - t0
    t_nms = t_nms_sample * 256.0
    note = ("1 image of the batch of %d: f32 conv stack in full (%.1f s on %d threads, OpenMP over (image, filter)); decode + NMS timed on "
            "1/16 of the grid cells (%.2f s, %d boxes kept) and scaled by 16^2 = %.0f s, apply_nms being quadratic in the candidate count"
            % (batch, t_conv, threads, t_nms_sample, len(d), t_nms))
    return t_conv + t_nms, note


def run_reference(args, rank):
    """`--impl reference`: the reference's own CPU implementation of the path (restated in the oracle; the Rust crate cannot
    be built in this image), all host threads, a bounded sample per step."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    steps = max(1, min(args.steps, 2))
    total, note = 0.0, ""
    for _ in range(steps):
        dt, note = cpu_reference_sample(args.batch, cores)
        total += dt
    dt = total / steps
    v = 1.0 / dt
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": args.gpus, "steps": steps,
                      "warmup": 0, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "yolov4-608 conv stack + decode(0.25) + NMS(0.45), He-normal random weights, uniform[0,1) images",
                                 "batch_per_gpu": args.batch},
                      "cpu_baseline": {"value": v, "unit": "images/s", "cores": cores, "kind": "port", "sample": note},
                      "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def cpu_baseline(batch):
    cores = os.cpu_count() or 1
    dt, note = cpu_reference_sample(batch, cores)
    return {"value": 1.0 / dt, "unit": "images/s", "cores": cores, "kind": "port", "sample": note}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64, help="images per GPU per step")
    ap.add_argument("--micro-batch", type=int, default=0, help="images per pass through the layers (activations stay in L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--width", type=int, default=608)
    ap.add_argument("--height", type=int, default=608)
    args = ap.parse_args()
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B = args.batch
    be = ln.B200Backend(local_rank)
    cfg = zoo.yolov4_cfg(args.width, args.height, batch=B)
    layers = ln.GpuExecutableNetwork(be, zoo.yolov4_cfg(args.width, args.height, batch=1), 1, ln.LN_F32).layers()
    blob = synth.he_weights(layers, 0)
    # calibration: a small f32 batch on the device gives the per-tensor scales
    calib = ln.GpuExecutableNetwork(be, zoo.yolov4_cfg(args.width, args.height, batch=2), 2, ln.LN_Q8)
    calib.load_weights(blob)
    calib.calibrate(synth.uniform_images(2, 3, args.height, args.width, 7))
    scales = calib.scales()
    del calib
    net = ln.GpuExecutableNetwork(be, cfg, B, ln.LN_Q8)
    net.load_weights(blob)
    net.set_scales(scales)
    net.set_micro_batch(args.micro_batch if args.micro_batch < B else 0)

    x_host = torch.from_numpy(synth.uniform_images(B, 3, args.height, args.width, 100 + rank)).pin_memory()
    x_np = x_host.numpy()
    x_dev = be.upload_f32(x_np.shape, x_np)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local_rank))
    det_args = (args.width, args.height, CONF_THR, NMS_THR, True, 0, MAX_PER_IMAGE)

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

    dets = None
    for _ in range(args.warmup):
        dets = net.detect_device(x_dev, *det_args)
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = be.launch_count
    ms = timed(lambda: net.detect_device(x_dev, *det_args), args.steps)
    launches = be.launch_count - launches0
    fwd_ms, nms_ms = net.last_times_ms()
    ms_e2e = timed(lambda: net.detect(x_np, *det_args), args.steps)
    clocks = sampler.summary()

    # roofline of the dominant kernel (tensor-core convolution), from a profiled forward
    net.set_profile(True)
    net.forward_device(x_dev)
    per_layer, per_op = net.profile()
    net.set_profile(False)
    umma_ms, umma_launches = per_op["conv_umma"]
    ops_img = conv_ops_per_image(layers) - 2 * layers[0]["out_w"] * layers[0]["out_h"] * layers[0]["out_c"] * layers[0]["in_c"] * layers[0]["size"] ** 2
    bf16_tf, hbm_gbs, basis = measured_peaks()
    peak = 2.0 * bf16_tf  # dense int8 tensor throughput is twice bf16 on this part
    achieved = ops_img * B / (umma_ms * 1e-3) / 1e12 if umma_ms > 0 else 0.0

    if rank == 0:
        line = {
            "metric": METRIC, "value": B * world * args.steps / (ms * 1e-3), "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": "yolov4-%d conv stack + decode(%.2f) + NMS(%.2f), He-normal random weights, uniform[0,1) images" % (args.width, CONF_THR, NMS_THR),
                       "batch_per_gpu": B, "micro_batch": args.micro_batch, "max_detections_per_image": MAX_PER_IMAGE,
                       "l2": "inputs larger than L2 (%.0f MB f32 batch)" % (x_np.nbytes / 1e6), "parallelism": "batch-sharded, no collective"},
            "e2e": {"value": B * world * args.steps / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(x_np.nbytes),
                    "d2h_bytes_per_step": int(B * MAX_PER_IMAGE * 28 + B * 4), "api": "ln_net_detect (host f32 NCHW batch -> detections)"},
            "gpu_launches": int(launches),
            "phases_ms": {"layers": fwd_ms, "decode_nms": nms_ms},
            "roofline": {"bound": "tensor", "kernel": "conv_umma_kernel (int8 implicit GEMM, all layers but the first)", "achieved": achieved,
                         "peak": peak, "unit": "TOP/s", "frac": achieved / peak, "traffic": None,
                         "peak_basis": "2 x %s bf16 sustained (%.1f TFLOP/s)" % (basis, bf16_tf), "launches_per_step": umma_launches,
                         "ms_per_step": umma_ms},
            "kernel_classes_ms": {k: v[0] for k, v in per_op.items()},
            "clocks": clocks,
            "detections_first_image": int(len(dets[0])) if dets is not None else None,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(B)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
