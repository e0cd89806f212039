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


def _run(spec, seed, tmp_path, cuda, runner=None, weights="text", runs=1, fast=False, live=None, extra_env=None):
    """runner: the binary to run; default the generic driver built on the drop-in headers (the
    reference-header build of the same driver is tests/test_gpu_reference_kernels.py's).
    weights: "text" (the reference's file format), "binary" (raw fp32 file) or "memory" (host
    array); runs: forward launches on the same layer objects; fast: the layers are queued through
    the C ABI (what the drop-in does for the reference's drivers) instead of the cooperative kernel;
    live: after the first runs the objects are switched to the first `live` images (set_batch) and
    the last run, the dumps and the logits are compared with the oracle on exactly those images."""
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
    if fast:
        env["TCBNN_RUNNER_FAST"] = "1"
    if live is not None:
        env["TCBNN_LIVE_BATCH"] = str(live)
    env.update(extra_env or {})
    r = subprocess.run([runner, os.path.join(d, "spec.txt"), os.path.join(d, wname),
                        os.path.join(d, "input.bin"), os.path.join(d, "logits.bin")],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    info = json.loads(r.stdout.strip().splitlines()[-1])
    assert info["batch"] == spec["batch"] and info["layers"] == len(spec["layers"])
    assert info.get("fast", 0) == int(fast)
    if live is not None:
        spec, x = dict(spec, batch=live), x[:live]
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


@pytest.mark.parametrize("which", ["mlp", "vgg_cifar", "resnet18_small", "resnet_cifar", "resnet18_64"])
def test_dropin_fast_path_layer_by_layer(cuda, tmp_path, which):
    """The drop-in classes' C-ABI path (tcgen05 kernels, int16 residual rows, hand-over of the
    pre-expanded input between layers): every layer's activations and the logits against the
    oracle, and a second pass on the same objects."""
    spec = {"mlp": models.mlp_spec(256), "vgg_cifar": models.vgg_cifar_spec(8),
            "resnet18_small": models.resnet18_spec(8, image=64, classes=100),
            "resnet_cifar": models.resnet_cifar_spec(4),
            "resnet18_64": models.resnet18_spec(64, image=96, classes=40)}[which]
    _run(spec, 70, tmp_path, cuda, fast=True, runs=2)


@pytest.mark.parametrize("fast", [False, True])
def test_dropin_set_batch_ragged_last_batch(cuda, tmp_path, fast):
    """Objects built for 8 images run the full batch twice and then the first 3 images
    (set_batch) on both of the drop-in's paths."""
    _run(models.resnet18_spec(8, image=64, classes=100), 46, tmp_path, cuda, runs=3, fast=fast, live=3)
    _run(models.mlp_spec(64), 47, tmp_path, cuda, runs=2, fast=fast, live=5)


def test_dropin_binary_weights_and_repeated_runs(cuda, tmp_path):
    """initialize() from a raw fp32 file and from a host array (tcbnn_dropin::Weights), and three
    forward launches on the same layer objects: same activations and logits as the oracle."""
    _run(models.resnet_cifar_spec(4), 44, tmp_path, cuda, weights="binary", runs=3)
    _run(models.vgg_cifar_spec(8), 45, tmp_path, cuda, weights="memory", runs=2)


DRIVER_CASES = [("mnist_mlp", "mlp_mnist.csv", lambda: models.mlp_spec(32768), "mnist"),
                ("cifar10_vgg", "vgg_cifar10.csv", lambda: models.vgg_cifar_spec(512), "cifar"),
                ("cifar10_resnet", "resnet_cifar10.csv", lambda: models.resnet_cifar_spec(512), "cifar"),
                ("imagenet_resnet", "resnet_imagenet.csv", lambda: models.resnet18_spec(512), "imagenet"),
                ("alexnet", "alexnet_imagenet.csv", lambda: models.alexnet_spec(512), "imagenet"),
                ("imagenet_vgg", "vgg_imagenet.csv", lambda: models.vgg16_imagenet_spec(512), "imagenet")]


def run_driver(path, cwd, extra_env=None):
    """Runs a driver built with the test shim (oracle/ref_driver_shim.h): returns (logits as a flat
    fp32 array -- the last device-to-host copy, i.e. the output layer's download_output() -- and
    the time the driver measured around its network launch)."""
    import re
    dump = os.path.join(cwd, os.path.basename(path) + "_logits.bin")
    env = dict(os.environ, TCBNN_REF_DUMP=dump)
    env.update(extra_env or {})
    r = subprocess.run([path], cwd=cwd, capture_output=True, text=True, timeout=1800, env=env)
    assert r.returncode == 0, path + ": " + r.stdout[-1500:] + r.stderr[-1500:]
    m = re.search(r"TCBNN_REF_INFERENCE_MS ([0-9.]+) (.*)", r.stdout)
    assert m and m.group(2).strip() == "no error", path + ": " + r.stdout[-1500:]
    return np.fromfile(dump, dtype=np.float32), float(m.group(1))


@pytest.mark.parametrize("exe,csv,mkspec,kind", DRIVER_CASES, ids=[c[0] for c in DRIVER_CASES])
def test_unchanged_reference_driver_on_dropin(cuda, tmp_path, exe, csv, mkspec, kind):
    """The reference's UNCHANGED driver source compiled against the drop-in headers and linked with
    libtcbnn_b200.so (build/dropin/<driver>_shim): its one network launch is routed to the
    library's kernels.  The logits it downloads must equal this library's Python path on the same
    weights and the stand-in readers' images (which tests/test_gpu_reference_kernels.py shows
    equal to the reference's own build), and the CPU oracle on the first images.  Prints the time
    the driver measures around its launch (run with -s)."""
    import torch
    import util
    out = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "build", "dropin")
    path = os.path.join(out, exe + "_shim")
    if not os.path.exists(path):
        pytest.skip("build/dropin/%s_shim not built (reference tree absent at build time)" % exe)
    spec = mkspec()
    w = models.synthetic_weights(spec, 5)
    dropin.write_weights(w, os.path.join(str(tmp_path), csv))
    logits, ms = run_driver(path, str(tmp_path))
    B, classes = spec["batch"], spec["layers"][-1]["N"]
    logits = logits[:B * classes].reshape(B, classes)
    x = util.reader_images(kind, B)
    bound = float(np.abs(x).max()) if "resnet" in exe else None
    net = models.Network(spec, w, torch.from_numpy(np.ascontiguousarray(x)).to(cuda), input_abs_bound=bound)
    ours = net.forward().cpu().numpy()[:, :classes]
    del net
    np.testing.assert_allclose(logits, ours, rtol=1e-5, atol=1e-4, err_msg=exe)
    sub = 8
    acts, _ = onet.run(dict(spec, batch=sub), w, x[:sub])
    np.testing.assert_allclose(logits[:sub], acts[-1][:, :classes], rtol=1e-5, atol=1e-4, err_msg=exe + " (oracle)")
    res = {"driver": exe, "batch": B, "dropin_ms": ms, "images_per_s": B / (ms * 1e-3)}
    if exe == "imagenet_resnet":
        # the same binary on its own cooperative kernel (warp-level b1 layer loops)
        l2, ms2 = run_driver(path, str(tmp_path), {"TCBNN_DROPIN_COOPERATIVE": "1"})
        np.testing.assert_allclose(l2[:B * classes].reshape(B, classes), ours, rtol=1e-5, atol=1e-4, err_msg=exe + " (cooperative)")
        res["cooperative_ms"] = ms2
    print("\nDROPIN_DRIVER " + json.dumps(res))


def test_benn_scaleup_driver_on_dropin_two_gpus(cuda, tmp_path):
    """benn_scaleup.cu, unchanged: one OpenMP thread per GPU builds its own network and launches
    it, then ncclReduce(max) of the logits (benn_scaleup.cu:231-403).  Needs two GPUs."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "build", "dropin")
    path = os.path.join(out, "benn_scaleup")
    if not os.path.exists(path):
        pytest.skip("build/dropin/benn_scaleup not built")
    spec = models.resnet18_spec(8)
    dropin.write_weights(models.synthetic_weights(spec, 5), os.path.join(str(tmp_path), "resnet_imagenet.csv"))
    r = subprocess.run([path], cwd=str(tmp_path), capture_output=True, text=True, timeout=1800,
                       env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "failed" not in r.stderr and "NCCL error" not in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    print("\nBENN_SCALEUP " + r.stdout[-600:])
