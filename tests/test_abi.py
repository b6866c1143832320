"""CPU-only checks of the drop-in boundary: the library builds for sm_100a, loads without a GPU, exports every
symbol include/lightnet_b200.h declares, and refuses to run without a device (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

import lightnet_b200 as ln
from lightnet_b200 import build as ln_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(ln.LIB_PATH):
        ln_build.build()
    return ln.load_library()


def header_functions():
    text = open(os.path.join(ROOT, "include", "lightnet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ln_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = header_functions()
    assert len(names) > 50
    for n in names:
        assert hasattr(lib, n), n
    # the binding table and the header agree
    assert sorted(ln.SYMBOLS) == names


def test_header_cites_reference_interfaces():
    text = open(os.path.join(ROOT, "include", "lightnet_b200.h")).read()
    for cite in ("lib.rs:460", "lib.rs:6295", "lib.rs:1776", "lib.rs:937", "lib.rs:2036", "lib.rs:3963", "detect.rs:113-244",
                 "gpu_forward_compact.rs:8"):
        assert cite in text, cite


def test_no_cpu_fallback(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(ln.BackendError) as e:
        ln.B200Backend(0)
    assert e.value.kind == "cuda"
    assert "no CPU fallback" in str(e.value)


def test_product_does_not_touch_the_oracle():
    """Nothing under lightnet_b200/ or include/ may import, link or name the oracle."""
    for base in ("lightnet_b200", "include"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, base)):
            if "build" in dirpath.split(os.sep):
                continue
            for f in files:
                if f.endswith((".py", ".cu", ".h", ".cpp", ".cuh")):
                    text = open(os.path.join(dirpath, f)).read()
                    assert "oracle" not in text.lower(), os.path.join(dirpath, f)
