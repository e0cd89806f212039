"""Build build/host/fast_runner: the generic C++ driver on tcbnn_host.hpp, linked against
libtcbnn_b200.so (in-tree, found again at run time through an rpath)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT = os.path.join(ROOT, "build", "host")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_fast_runner():
    from .. import build as libbuild
    libbuild.build()
    os.makedirs(OUT, exist_ok=True)
    out = os.path.join(OUT, "fast_runner")
    src = os.path.join(HERE, "fast_runner.cpp")
    hdr = os.path.join(HERE, "tcbnn_host.hpp")
    api = os.path.join(ROOT, "include", "tcbnn_b200.h")
    lib = os.path.join(PKG, "libtcbnn_b200.so")
    if _stale(out, [src, hdr, api, lib]):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        cmd = ["g++", "-std=c++14", "-O2", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", HERE,
               "-I", os.path.join(cuda, "include"), "-o", out, src,
               "-L", PKG, "-ltcbnn_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
               "-Wl,-rpath," + PKG, "-Wl,-rpath," + os.path.join(cuda, "lib64")]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed building fast_runner:\n" + r.stdout + r.stderr)
    return out


if __name__ == "__main__":
    print(build_fast_runner())
