"""bench.py prints exactly one JSON line on stdout, whatever else the run writes (checked on the arm that needs no GPU)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_of_the_conv_sweep_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "conv-sweep"],
                       capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and "unavailable" in line


def test_library_output_on_stdout_is_kept_away_from_the_json_line():
    code = ("import os, sys; sys.path.insert(0, %r); import bench; bench.claim_stdout(); "
            "os.write(1, b'banner from a library\\n'); print('python print'); bench.emit_line({'ok': 1})") % ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == json.dumps({"ok": 1})
    assert "banner from a library" in r.stderr and "python print" in r.stderr


def test_layer_classes_put_each_layer_against_the_roofline_its_intensity_allows():
    """`layer_classes`: operations per algorithmic byte, the bound peak * min(1, intensity / ridge) and the fraction reached, on
    the real YOLOv4-608 layer list with made-up times; the stack figure is the sum of the per-layer bounds over the sum of times."""
    sys.path.insert(0, ROOT)
    import bench
    from lightnet_b200 import zoo
    from oracle import oracle_api as orc

    layers = orc.Net(zoo.yolov4_cfg(608, 608, batch=1), 1).layers()
    times = [0.05 if l["kind"] == "conv" else 0.0 for l in layers]
    peak, hbm, batch = 2779.6, 6543.7, 64
    rows, stack = bench.layer_classes(layers, times, batch, peak, hbm)
    assert abs(stack["ridge_ops_per_byte"] - peak * 1e12 / (hbm * 1e9)) < 0.1
    by_name = {r["layer"]: r for r in rows}
    r = by_name["1x1 s1 C64->K64"]
    # 2 * 64 * 64 operations per pixel over 64 bytes in + 64 bytes out (+ the weights, negligible): left of the ridge
    assert abs(r["ops_per_byte"] - 64.0) < 0.1 and abs(r["bound_tops"] - peak * 64.0 / stack["ridge_ops_per_byte"]) < 2.0
    assert abs(r["frac_of_bound"] - r["tops"] / r["bound_tops"]) < 2e-3
    dense = [x for x in rows if x["layer"].startswith("3x3 s1 C512->K1024")]
    assert dense and dense[0]["bound_tops"] == peak  # right of the ridge: the tensor roof
    # a convolution whose shortcut runs in its epilogue also reads the residual; a head writes f32
    i_fused = next(i for i, l in enumerate(layers) if l["kind"] == "conv" and layers[i + 1]["kind"] == "shortcut")
    i_head = next(i for i, l in enumerate(layers) if l["kind"] == "conv" and layers[i + 1]["kind"] == "yolo")
    lf, lh = layers[i_fused], layers[i_head]
    px = lambda l: batch * l["out_w"] * l["out_h"] * l["out_c"]
    assert bench.layer_bytes(layers, i_fused, batch) == batch * lf["in_w"] * lf["in_h"] * lf["in_c"] + lf["out_c"] * lf["in_c"] * lf["size"] ** 2 + 2 * px(lf)
    assert bench.layer_bytes(layers, i_head, batch) == batch * lh["in_w"] * lh["in_h"] * lh["in_c"] + lh["out_c"] * lh["in_c"] * lh["size"] ** 2 + 4 * px(lh)
    assert 0.0 < stack["frac"] < 1.0 and abs(stack["frac"] - stack["bound_ms"] / stack["measured_ms"]) < 1e-3
