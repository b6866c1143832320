"""Writes tests/golden/reference_cfg_layers.json: the layer lists and head parameters the oracle's parser reads from the
reference's own cfg files (cfg/yolov3-tiny.cfg, cfg/yolov4.cfg, cfg/yolov7.cfg), so that the generated architectures of
lightnet_b200.zoo can be checked against them where no reference checkout is mounted.

    LIGHTNET_REFERENCE=<checkout> python tests/golden/make_cfg_layers.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from lightnet_b200 import zoo  # noqa: E402
from oracle import oracle_api as orc  # noqa: E402

ref = os.environ["LIGHTNET_REFERENCE"]
out = {}
for name in ("yolov3-tiny.cfg", "yolov4.cfg", "yolov7.cfg"):
    text = open(os.path.join(ref, "cfg", name)).read()
    net = orc.Net(text, 1)
    out[name] = {"input": [net.width, net.height, net.channels], "layers": net.layers(), "heads": zoo.head_specs(text)}
with open(os.path.join(HERE, "reference_cfg_layers.json"), "w") as f:
    json.dump(out, f, separators=(",", ":"))
print("wrote", {k: len(v["layers"]) for k, v in out.items()})
