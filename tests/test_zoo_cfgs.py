"""The generated architectures must be layer-for-layer the reference's cfg files and carry the MAC counts computed from
those files.  The reference's files are represented by tests/golden/reference_cfg_layers.json (what the oracle's parser
reads from them; written by tests/golden/make_cfg_layers.py); when the environment variable LIGHTNET_REFERENCE names a
checkout, the files themselves are parsed as well."""
import json
import os

import pytest

from lightnet_b200 import zoo
from oracle import oracle_api as orc

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "reference_cfg_layers.json")))
CASES = [("yolov3-tiny.cfg", zoo.yolov3_tiny_cfg, 2.782), ("yolov4.cfg", zoo.yolov4_cfg, 64.195), ("yolov7.cfg", zoo.yolov7_cfg, 52.256)]


def _macs(net):
    return sum(l["out_w"] * l["out_h"] * l["out_c"] * l["in_c"] * l["size"] ** 2 for l in net.layers() if l["kind"] == "conv")


@pytest.mark.parametrize("name,gen,gmac", CASES)
def test_generated_cfg_matches_reference(name, gen, gmac):
    mine = orc.Net(gen(), 1)
    assert abs(_macs(mine) / 1e9 - gmac) < 5e-4
    ref = GOLDEN[name]
    assert [mine.width, mine.height, mine.channels] == ref["input"]
    assert mine.num_layers == len(ref["layers"])
    for a, b in zip(mine.layers(), ref["layers"]):
        assert a == b
    heads = json.loads(json.dumps(zoo.head_specs(gen())))   # tuples -> lists, as in the fixture
    assert heads == ref["heads"]


@pytest.mark.parametrize("name,gen,gmac", CASES)
def test_golden_layers_are_what_the_reference_files_parse_to(name, gen, gmac):
    if not os.environ.get("LIGHTNET_REFERENCE"):
        pytest.skip("LIGHTNET_REFERENCE does not name a reference checkout")
    text = open(os.path.join(os.environ["LIGHTNET_REFERENCE"], "cfg", name)).read()
    ref = orc.Net(text, 1)
    assert ref.layers() == GOLDEN[name]["layers"]
    assert json.loads(json.dumps(zoo.head_specs(text))) == GOLDEN[name]["heads"]
