"""GPU parity of the C++ header-level drop-in (tcbnn_b200/dropin: utility.h, param.h, kernel.cuh).

build/dropin/net_runner builds a network with the reference's class names and runs it as one
cooperative kernel with grid.sync() between layers, the way the reference drivers do.  Its
logits and every layer's unpacked +-1 activations are compared with the CPU oracle."""
import json
import os
import subprocess

import numpy as np
import pytest

import networks as onet
from tcbnn_b200 import dropin, models
from tcbnn_b200.dropin import build as dbuild

pytestmark = pytest.mark.gpu


def _unpacked(act, layer):
    """oracle bit words -> +-1 floats in the order download_full_output() returns them."""
    import oracle as orc
    t = layer["type"]
    B = act.shape[0]
    if t in ("in", "fc"):
        n = layer["K"] if t == "in" else layer["N"]
        return orc.unpack_rows(act.reshape(B, -1), n)
    O, Ow = layer["O"], (layer["O"] + 31) // 32
    words = layer["OH"] * layer["OW"] * Ow
    bits = act.reshape(B, -1)[:, :words].reshape(B * layer["OH"] * layer["OW"], Ow)
    return orc.unpack_rows(np.ascontiguousarray(bits), O)


def _run(spec, seed, tmp_path, cuda, runner=None, weights="text", runs=1):
    """runner: the binary to run; default the generic driver built on the drop-in headers (the
    reference-header build of the same driver is tests/test_gpu_reference_kernels.py's).
    weights: "text" (the reference's file format), "binary" (raw fp32 file) or "memory" (host
    array); runs: forward launches on the same layer objects."""
    runner = runner or dbuild.build_runner()
    w = models.synthetic_weights(spec, seed)
    x = models.synthetic_input(spec, seed + 1)
    d = str(tmp_path)
    dropin.write_spec(spec, os.path.join(d, "spec.txt"))
    wname = "weights.txt" if weights == "text" else "weights.bin"
    if weights == "text":
        dropin.write_weights(w, os.path.join(d, wname))
    else:
        dropin.write_weights_binary(w, os.path.join(d, wname))
    np.ascontiguousarray(x, dtype=np.float32).tofile(os.path.join(d, "input.bin"))
    env = dict(os.environ, TCBNN_DUMP_DIR=d, TCBNN_RUNS=str(runs))
    if weights == "memory":
        env["TCBNN_WEIGHTS_IN_MEMORY"] = "1"
    r = subprocess.run([runner, os.path.join(d, "spec.txt"), os.path.join(d, wname),
                        os.path.join(d, "input.bin"), os.path.join(d, "logits.bin")],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    info = json.loads(r.stdout.strip().splitlines()[-1])
    assert info["batch"] == spec["batch"] and info["layers"] == len(spec["layers"])
    acts, _ = onet.run(spec, w, x)
    shapes = models.layer_shapes(spec)
    for i, (layer, act) in enumerate(zip(shapes[:-1], acts[:-1])):
        got = np.fromfile(os.path.join(d, "layer%02d.bin" % i), dtype=np.float32)
        exp = _unpacked(act, layer).ravel()
        assert got.size == exp.size, (i, layer["name"])
        assert np.array_equal(got, exp), "layer %d %s" % (i, layer["name"])
    logits = np.fromfile(os.path.join(d, "logits.bin"), dtype=np.float32).reshape(acts[-1].shape)
    np.testing.assert_allclose(logits, acts[-1], rtol=1e-5, atol=1e-5)


def test_dropin_mlp(cuda, tmp_path):
    _run(models.mlp_spec(256), 40, tmp_path, cuda)


def test_dropin_vgg_cifar(cuda, tmp_path):
    _run(models.vgg_cifar_spec(8), 41, tmp_path, cuda)


def test_dropin_resnet18_small_image(cuda, tmp_path):
    _run(models.resnet18_spec(8, image=64, classes=100), 42, tmp_path, cuda)


def test_dropin_resnet_cifar(cuda, tmp_path):
    _run(models.resnet_cifar_spec(4), 43, tmp_path, cuda)


def test_dropin_binary_weights_and_repeated_runs(cuda, tmp_path):
    """initialize() from a raw fp32 file and from a host array (tcbnn_dropin::Weights), and three
    forward launches on the same layer objects: same activations and logits as the oracle."""
    _run(models.resnet_cifar_spec(4), 44, tmp_path, cuda, weights="binary", runs=3)
    _run(models.vgg_cifar_spec(8), 45, tmp_path, cuda, weights="memory", runs=2)


def test_reference_drivers_built_against_dropin_run(cuda, tmp_path):
    """The reference's unchanged mnist_mlp.cu / cifar10_vgg.cu / cifar10_resnet.cu, compiled
    against the drop-in headers, run to completion on synthetic weight files (they print no
    result; parity of the same code path is what the tests above check)."""
    out = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "build", "dropin")
    cases = [("mnist_mlp", "mlp_mnist.csv", models.mlp_spec(32768)),
             ("cifar10_vgg", "vgg_cifar10.csv", models.vgg_cifar_spec(512)),
             ("cifar10_resnet", "resnet_cifar10.csv", models.resnet_cifar_spec(512))]
    ran = 0
    for exe, csv, spec in cases:
        path = os.path.join(out, exe)
        if not os.path.exists(path):
            continue
        dropin.write_weights(models.synthetic_weights(spec, 5), os.path.join(str(tmp_path), csv))
        r = subprocess.run([path], cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, exe + ": " + r.stdout[-2000:] + r.stderr[-2000:]
        assert "failed" not in r.stderr and "NULL pointer" not in r.stderr, exe + r.stderr[-2000:]
        ran += 1
    if ran == 0:
        pytest.skip("reference drivers were not built (reference tree absent at build time)")
