"""Regenerates tests/golden/*_shapes.csv from the reference's own geometry tables.

Run where the reference checkout is mounted:
    python tests/golden/make_shape_tables.py /path/to/reference
The reference keeps, for its real-GPU parity tests, tables of every conv / maxpool
geometry found in its 101 cfg files together with the output extents its shape rules
give (src/lightnet-cuda-oxide/tests/data/{conv,maxpool}_shapes.csv).  Only the numeric
geometry columns are kept here; they pin conv_dim / pool_dim.
"""
import csv
import os
import sys


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    data = os.path.join(ref, "src", "lightnet-cuda-oxide", "tests", "data")
    with open(os.path.join(data, "conv_shapes.csv")) as f, open(os.path.join(here, "conv_shapes.csv"), "w") as o:
        o.write("in_c,in_h,in_w,filters,size,stride_x,stride_y,dilation,padding,groups,out_h,out_w\n")
        for r in csv.DictReader(f):
            o.write(",".join(r[k] for k in ("in_c", "in_h", "in_w", "filters", "size", "stride_x", "stride_y", "dilation",
                                            "padding", "groups", "out_h", "out_w")) + "\n")
    with open(os.path.join(data, "maxpool_shapes.csv")) as f, open(os.path.join(here, "maxpool_shapes.csv"), "w") as o:
        o.write("size,stride_x,stride_y,padding,in_c,in_h,in_w,out_h,out_w\n")
        for r in csv.DictReader(f):
            o.write(",".join(r[k] for k in ("size", "stride_x", "stride_y", "padding", "in_c", "in_h", "in_w", "out_h",
                                            "out_w")) + "\n")


if __name__ == "__main__":
    main(sys.argv[1])
