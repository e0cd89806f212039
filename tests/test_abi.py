"""CPU-only: the C-ABI library loads and exports every symbol the header declares."""
import os
import re

from tcbnn_b200 import build, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tcbnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tcbnn_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    build.build()
    L = lib.load()
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), n
    assert sorted(lib.SIGNATURES) == names
    assert L.tcbnn_version() >= 100


def test_conv_shape_is_host_only():
    import ctypes as C
    d = lib.ConvDesc(B=1, H=224, W=224, C=3, O=64, R=7, S=7, stride_h=4, stride_w=4, padding=1, pool=1)
    lib.call("tcbnn_conv_shape", C.byref(d))
    assert (d.pad_h, d.pad_w, d.OH, d.OW) == (3, 3, 56, 56)
