"""Build the CPU oracle (test infrastructure) and, when the reference tree is present,
the reference's own host popcount functions into oracle/_ref/.

    python oracle/build.py [--native] [--ref-root /path/to/TCBNN]

liboracle.so        : oracle/tcbnn_oracle.cpp, x86-64-v3 so the file also runs on other hosts
liboracle_native.so : same source with -march=native (built on the machine that times it)
_ref/libref_bmm.so  : BMMAcpu / WMMABOOLCPU compiled from the reference's source files where
                      they lie (never copied); skipped when the tree is absent.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def default_ref_root():
    """Where the reference tree (pnnl/TCBNN) is looked for when no --ref-root is given: the
    TCBNN_REF_ROOT environment variable, else a folder named `reference` beside this repository.
    Nothing is built from it when it does not exist."""
    env = os.environ.get("TCBNN_REF_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build failed: " + cmd[0])


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(native=False):
    src = os.path.join(HERE, "tcbnn_oracle.cpp")
    out = os.path.join(HERE, "liboracle_native.so" if native else "liboracle.so")
    if _stale(out, [src]):
        march = "-march=native" if native else "-march=x86-64-v3"
        _run(["g++", "-O3", march, "-fopenmp", "-shared", "-fPIC", "-std=c++17", "-o", out, src])
    return out


def build_ref(ref_root=None):
    ref_root = ref_root or default_ref_root()
    tc = os.path.join(ref_root, "bmm", "tensorcore_kernel.cu")
    mt = os.path.join(ref_root, "bmm", "bmma_op_test", "main_test.cu")
    bc = os.path.join(ref_root, "bconv", "bmma_kernel.cu")
    if not (os.path.exists(tc) and os.path.exists(mt) and os.path.exists(bc)):
        return None
    outdir = os.path.join(HERE, "_ref")
    os.makedirs(outdir, exist_ok=True)
    out = os.path.join(outdir, "libref_bmm.so")
    wrap = os.path.join(HERE, "ref_wrap.cu")
    if _stale(out, [wrap, tc, mt, bc]):
        objs = []
        for which, src in ((1, tc), (2, mt), (3, bc)):
            obj = os.path.join(outdir, "ref_wrap_%d.o" % which)
            _run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-w",
                  "-Xcompiler", "-fPIC", "-DWHICH=%d" % which, '-DREF_SRC="%s"' % src,
                  "-c", "-o", obj, wrap])
            objs.append(obj)
        _run(["nvcc", "-shared", "-o", out] + objs)
    return out


REF_DRIVERS = ["mnist_mlp", "cifar10_vgg", "cifar10_resnet", "imagenet_resnet", "alexnet", "imagenet_vgg"]


def build_ref_drivers(ref_root=None):
    """The reference's unchanged drivers with the reference's own headers (WMMA b1 kernels) for
    sm_100a: _ref/ref_<driver>.  Compiled from the sources where they lie (nothing is copied);
    only the dataset readers are replaced (seeded synthetic images, the drop-in's
    synthetic_data.cpp, libjpeg stubbed) and ref_driver_shim.h is force-included so that the
    drivers print the time they measure.  Flags as the reference Makefile (:15)."""
    ref_root = ref_root or default_ref_root()
    if not os.path.exists(os.path.join(ref_root, "kernel.cuh")):
        return []
    outdir = os.path.join(HERE, "_ref")
    os.makedirs(outdir, exist_ok=True)
    dropin = os.path.join(os.path.dirname(HERE), "tcbnn_b200", "dropin")
    data_src = os.path.join(dropin, "synthetic_data.cpp")
    shim = os.path.join(HERE, "ref_driver_shim.h")
    from concurrent.futures import ThreadPoolExecutor

    def one(name):
        src = os.path.join(ref_root, name + ".cu")
        if not os.path.exists(src):
            return None
        out = os.path.join(outdir, "ref_" + name)
        if _stale(out, [src, data_src, shim, os.path.join(ref_root, "kernel.cuh"), os.path.join(ref_root, "param.h")]):
            _run(["nvcc", "-std=c++14", "-O3", "-w", "-gencode", "arch=compute_100a,code=sm_100a",
                  "-maxrregcount=64", "-rdc=true", "-include", shim, "-I", ref_root,
                  "-I", os.path.join(dropin, "stubs"), "-o", out, src, data_src])
        return out

    with ThreadPoolExecutor(max_workers=len(REF_DRIVERS)) as pool:
        return [b for b in pool.map(one, REF_DRIVERS) if b]


def build_ref_runner(ref_root=None):
    """tcbnn_b200/dropin/net_runner.cu (this repository's generic driver on the reference's public
    API: network from a text description, one cooperative kernel, logits and every layer's
    download_full_output() to files) compiled against the REFERENCE's own utility.h / param.h /
    kernel.cuh: _ref/ref_net_runner, the layer-by-layer pin of the oracle.  The runner source is
    staged next to the binary so that its quote-includes resolve to the reference's headers."""
    ref_root = ref_root or default_ref_root()
    if not os.path.exists(os.path.join(ref_root, "kernel.cuh")):
        return None
    import shutil
    outdir = os.path.join(HERE, "_ref")
    os.makedirs(outdir, exist_ok=True)
    src = os.path.join(os.path.dirname(HERE), "tcbnn_b200", "dropin", "net_runner.cu")
    staged = os.path.join(outdir, "ref_net_runner.cu")
    out = os.path.join(outdir, "ref_net_runner")
    if _stale(out, [src, os.path.join(ref_root, "kernel.cuh"), os.path.join(ref_root, "param.h"),
                    os.path.join(HERE, "ref_driver_shim.h")]):
        shutil.copyfile(src, staged)
        _run(["nvcc", "-std=c++14", "-O3", "-w", "-gencode", "arch=compute_100a,code=sm_100a",
              "-maxrregcount=64", "-rdc=true", "-include", os.path.join(HERE, "ref_driver_shim.h"),
              "-I", ref_root, "-o", out, staged])
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--native", action="store_true")
    ap.add_argument("--ref-root", default=None, help="reference tree (default: $TCBNN_REF_ROOT, else ../reference)")
    a = ap.parse_args()
    print(build_oracle(False))
    if a.native:
        print(build_oracle(True))
    print(build_ref(a.ref_root))
    for b in build_ref_drivers(a.ref_root):
        print(b)
    print(build_ref_runner(a.ref_root))
