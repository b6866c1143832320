"""Host-side planner helpers of the convolution kernel, compiled with g++ from the header they live in (no GPU)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INCLUDE = "/usr/local/cuda/include"

PROGRAM = r"""
#include <cstdio>
#include <cstdlib>
#include "ln_conv_plan.h"
int main(int argc, char** argv) {
    for (int i = 1; i + 3 < argc; i += 4)
        printf("%d\n", ln_acc_shift((float)atof(argv[i]), (float)atof(argv[i + 1]), (float)atof(argv[i + 2]), (float)atof(argv[i + 3])));
    return 0;
}
"""


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INCLUDE), reason="needs g++ and the CUDA headers")
def test_acc_shift_rule(tmp_path):
    """ln_acc_shift: 0 while 127 * max_l1 stays below 2^22; otherwise the smallest shift that brings the bound under 2^22, allowed
    only while half of what is dropped (2^(shift-1) accumulator units) times the largest multiplier s_x * s_w / s_y stays at or
    under 0.02 of a code; -1 when that fails or more than 8 bits would be needed."""
    src = tmp_path / "acc_shift.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "acc_shift"
    subprocess.run(["g++", "-std=c++17", "-I" + CUDA_INCLUDE, "-I" + os.path.join(ROOT, "include"),
                    "-I" + os.path.join(ROOT, "lightnet_b200", "csrc"), str(src), "-o", str(exe)], check=True)
    cases = [
        # max_l1, s_x, max s_w, 1 / s_y  ->  expected
        ((1000.0, 0.01, 0.001, 10.0), 0),          # 127 k < 2^22
        ((33025.0, 0.01, 0.001, 10.0), 0),         # 4 194 175 < 2^22: still none
        ((33027.0, 0.01, 0.001, 10.0), 1),         # just above: one bit, costs 1 * 1e-4 codes
        ((33027.0, 1.0, 0.5, 1.0), -1),            # one bit would cost half a code
        ((143000.0, 0.02, 0.002, 8.0), 3),         # 18.2 M < 2^25: three bits, 4 * 3.2e-4 codes
        ((143000.0, 0.02, 0.002, 20.0), 3),        # 4 * 8e-4 = 0.0032
        ((143000.0, 0.2, 0.01, 10.0), -1),         # 4 * 0.02 = 0.08 of a code: refused
        ((8.0e6, 1e-4, 1e-4, 1.0), 8),             # 1.016e9 < 2^30
        ((2.0e7, 1e-4, 1e-4, 1.0), -1),            # beyond 2^30: nothing up to eight bits is enough
    ]
    args = [repr(float(v)) for c, _ in cases for v in c]
    out = subprocess.run([str(exe)] + args, check=True, capture_output=True, text=True).stdout.split()
    assert [int(v) for v in out] == [want for _, want in cases]
