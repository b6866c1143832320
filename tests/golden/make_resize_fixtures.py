"""Repackages the reference's resize fixtures into one compressed archive.

Source: src/lightnet-core/tests/fixtures/resize{0,1,2}_{src_96x72.rgb, exact_40x28.rgb, exact_130x100.rgb,
float_40x28.f32, float_50x60.f32} of the reference checkout (crops of video frames and the outputs of OpenCV's
INTER_LINEAR_EXACT and of a float32 replica of Darknet's resize_image, used by the tests at
lightnet-runtime/src/image.rs:362-402).  Run from the repository root with the reference checkout's path as argument:

    python tests/golden/make_resize_fixtures.py /path/to/reference
"""
import os
import sys

import numpy as np


def main(ref):
    d = os.path.join(ref, "src", "lightnet-core", "tests", "fixtures")
    out = {}
    for i in range(3):
        out["src%d" % i] = np.fromfile(os.path.join(d, "resize%d_src_96x72.rgb" % i), np.uint8).reshape(72, 96, 3)
        for w, h in ((40, 28), (130, 100)):
            out["exact%d_%dx%d" % (i, w, h)] = np.fromfile(os.path.join(d, "resize%d_exact_%dx%d.rgb" % (i, w, h)), np.uint8).reshape(h, w, 3)
        for w, h in ((40, 28), (50, 60)):
            out["float%d_%dx%d" % (i, w, h)] = np.fromfile(os.path.join(d, "resize%d_float_%dx%d.f32" % (i, w, h)), "<f4").reshape(3, h, w)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "resize_fixtures.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
