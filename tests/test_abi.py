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


def test_specialised_first_layer_source_compiles_without_a_gpu():
    """tcbnn_inconv_specialize's generator + NVRTC for sm_100a; loading the result needs a GPU
    and is covered by the GPU tests."""
    import ctypes as C
    import pytest
    try:
        C.CDLL("libnvrtc.so.12")
    except OSError:
        pytest.skip("no libnvrtc on this machine")
    for (O, R, stride, pool) in [(64, 7, 4, 1), (24, 3, 1, 2), (128, 3, 1, 1)]:
        d = lib.ConvDesc(B=2, H=32, W=32, C=3, O=O, R=R, S=R, stride_h=stride, stride_w=stride, padding=1, pool=pool)
        lib.call("tcbnn_conv_shape", C.byref(d))
        n = C.c_longlong(0)
        lib.call("tcbnn_inconv_specialize_selftest", C.byref(d), 3, C.byref(n))
        assert n.value > 20 * R * R * O
    d = lib.ConvDesc(B=2, H=32, W=32, C=3, O=160, R=3, S=3, stride_h=1, stride_w=1, padding=1, pool=1)
    lib.call("tcbnn_conv_shape", C.byref(d))
    with pytest.raises(lib.TcbnnError):
        lib.call("tcbnn_inconv_specialize_selftest", C.byref(d), 3, None)
