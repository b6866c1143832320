"""The generated architectures must be layer-for-layer the reference's cfg files (checked with the oracle's
parser when the reference checkout is present) and carry the MAC counts computed from those files."""
import os

import pytest

from lightnet_b200 import zoo
from oracle import oracle_api as orc

# cfg directory of a reference checkout, when one is mounted (LIGHTNET_REFERENCE names the checkout)
REF_CFG = os.path.join(os.environ.get("LIGHTNET_REFERENCE", os.path.join(os.sep, "root", "reference")), "cfg")


def _macs(net):
    return sum(l["out_w"] * l["out_h"] * l["out_c"] * l["in_c"] * l["size"] ** 2 for l in net.layers() if l["kind"] == "conv")


@pytest.mark.parametrize("name,gen,gmac", [("yolov3-tiny.cfg", zoo.yolov3_tiny_cfg, 2.782), ("yolov4.cfg", zoo.yolov4_cfg, 64.195),
                                           ("yolov7.cfg", zoo.yolov7_cfg, 52.256)])
def test_generated_cfg_matches_reference(name, gen, gmac):
    mine = orc.Net(gen(), 1)
    assert abs(_macs(mine) / 1e9 - gmac) < 5e-4
    path = os.path.join(REF_CFG, name)
    if not os.path.exists(path):
        pytest.skip("reference checkout not mounted")
    ref = orc.Net(open(path).read(), 1)
    assert mine.num_layers == ref.num_layers
    assert (mine.width, mine.height, mine.channels) == (ref.width, ref.height, ref.channels)
    for a, b in zip(mine.layers(), ref.layers()):
        assert a == b
    assert zoo.head_specs(gen()) == zoo.head_specs(open(path).read())
