"""Builds liblightnet_b200.so in-tree with nvcc for sm_100a.

    python -m lightnet_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and resolves the one driver entry point it
needs at run time, so it loads (and exports its symbols) on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "liblightnet_b200.so")
SOURCES = ["ln_runtime.cu", "ln_f32_ops.cu", "ln_q8_ops.cu", "ln_f16_ops.cu", "ln_conv_umma.cu", "ln_yolo.cu", "ln_image.cu", "ln_net.cu"]
HEADERS = ["ln_common.h", "ln_conv_plan.h", "ln_conv_layout.inc", os.path.join("..", "..", "include", "lightnet_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
]


# extra compiler flags from the environment, e.g. LN_NVCC_EXTRA=-DLN_CONV_ROLE_TIMING to compile the role clocks of the
# tensor-core convolution in (read back with ln_ctx_debug_cycles when LN_DEBUG_CYCLES is set)
NVCC_FLAGS += os.environ.get("LN_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write("---- %s ----\n%s\n" % (src, out))
        elif verbose or out.strip():
            sys.stderr.write("---- %s ----\n%s\n" % (src, out))
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
