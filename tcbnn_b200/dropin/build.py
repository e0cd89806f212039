"""Build the C++ side of the drop-in header API.

    python -m tcbnn_b200.dropin.build [--ref-root /path/to/TCBNN]

build/dropin/net_runner        : tcbnn_b200/dropin/net_runner.cu (generic cooperative-kernel driver)
build/dropin/<driver>          : the reference's own, UNCHANGED driver sources (mnist_mlp.cu,
    cifar10_vgg.cu, cifar10_resnet.cu, imagenet_resnet.cu, alexnet.cu, imagenet_vgg.cu and the
    OpenMP-thread-per-GPU benn_scaleup.cu) compiled against the drop-in utility.h / param.h /
    kernel.cuh and linked with libtcbnn_b200.so (the drop-in routes the drivers' network launch
    to the library's kernels, see param.h).  With shim=<header> the binaries are named
    <driver>_shim and are built with that header force-included (the tests pass one that makes a
    driver print the time it measures and dump the logits it downloads).  The sources are copied at build time into the git-ignored
    build/ folder (a driver's `#include "param.h"` looks in its own folder first, so it must not
    sit next to the reference headers), together with the reference's data.h; the dataset readers
    are replaced by synthetic_data.cpp and libjpeg by empty stub headers.  Skipped when the
    reference tree is absent.
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(ROOT, "build", "dropin")
# -maxrregcount=64 as in the reference Makefile (Makefile:15): the drivers launch 1024-thread blocks
NVCC = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-rdc=true",
        "-maxrregcount=64", "-w"]
DRIVERS = ["mnist_mlp", "cifar10_vgg", "cifar10_resnet", "imagenet_resnet", "alexnet", "imagenet_vgg", "benn_scaleup"]
PKG = os.path.dirname(HERE)
# the drivers call into libtcbnn_b200.so; found at run time relative to the binary (build/dropin/)
LINK = ["-L", PKG, "-ltcbnn_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../tcbnn_b200"]
EXTRA = {"benn_scaleup": ["-Xcompiler", "-fopenmp", "-lnccl"]}


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build failed")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    csrc = os.path.join(os.path.dirname(HERE), "csrc")
    return [os.path.join(HERE, f) for f in ("utility.h", "param.h", "kernel.cuh")] + \
           [os.path.join(csrc, f) for f in ("bnn_layers.cuh", "bnn_warp.cuh")] + \
           [os.path.join(ROOT, "include", "tcbnn_b200.h")]


def build_runner():
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "net_runner.cu")
    out = os.path.join(OUT, "net_runner")
    if _stale(out, [src] + _headers()):
        _run(NVCC + ["-I", HERE, "-o", out, src] + LINK)
    return out


def default_ref_root():
    """$TCBNN_REF_ROOT, else a folder named `reference` beside this repository."""
    return os.environ.get("TCBNN_REF_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


def build_reference_drivers(ref_root=None, shim=None):
    ref_root = ref_root or default_ref_root()
    shim_h = shim
    if not os.path.exists(os.path.join(ref_root, "data.h")):
        return []
    os.makedirs(OUT, exist_ok=True)
    shutil.copyfile(os.path.join(ref_root, "data.h"), os.path.join(OUT, "data.h"))
    data_src = os.path.join(HERE, "synthetic_data.cpp")
    from concurrent.futures import ThreadPoolExecutor

    def one(name):
        src = os.path.join(ref_root, name + ".cu")
        if not os.path.exists(src):
            return None
        staged = os.path.join(OUT, name + ".cu")
        out = os.path.join(OUT, name + ("_shim" if shim else ""))
        if _stale(out, [src, data_src] + _headers() + ([shim_h] if shim else [])):
            shutil.copyfile(src, staged)
            try:
                _run(NVCC + (["-include", shim_h] if shim else []) +
                     ["-I", OUT, "-I", HERE, "-I", os.path.join(HERE, "stubs"), "-o", out, staged, data_src] +
                     LINK + EXTRA.get(name, []))
            except RuntimeError:
                if name in EXTRA:          # needs OpenMP and the NCCL headers: optional
                    return None
                raise
        return out

    with ThreadPoolExecutor(max_workers=len(DRIVERS)) as pool:      # the compiles are independent
        return [b for b in pool.map(one, DRIVERS) if b]


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=None)
    ap.add_argument("--shim", default=None, help="header to force-include (builds <driver>_shim)")
    a = ap.parse_args()
    print(build_runner())
    for b in build_reference_drivers(a.ref_root, a.shim):
        print(b)
