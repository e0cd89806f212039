"""Same-box baseline: the reference's own sm_75-era WMMA bit-GEMM kernels
(bmm/tensorcore_kernel.cu BMMA / BMMApipe / BMMAS), compiled for sm_100a from the reference
sources into oracle/_ref/libref_bmm.so, run on the standalone bit-GEMM configuration next to
tcbnn_bgemm.  All must equal the CPU oracle; the timings are printed (run with -s)."""
import ctypes as C
import json

import numpy as np
import pytest
import torch

import oracle as orc
import util
from tcbnn_b200 import ops

pytestmark = pytest.mark.gpu


def test_reference_bitgemm_kernels_match_and_time(cuda):
    R = orc.ref_lib()
    if R is None or not hasattr(R, "ref_gpu_bmm"):
        pytest.skip("oracle/_ref/libref_bmm.so not built (reference tree absent at build time)")
    M = N = 1024
    K = 4096
    g = util.rng(1)
    A, B = util.rand_words(g, (M, K // 32)), util.rand_words(g, (N, K // 32))
    expect = orc.bgemm(A, B, K)
    dA = torch.from_numpy(A.view(np.int32)).to(cuda)
    dB = torch.from_numpy(B.view(np.int32)).to(cuda)
    out = torch.zeros((M, N), dtype=torch.int32, device=cuda)
    res = {}
    for which, name in ((0, "BMMA<4,4>"), (1, "BMMApipe<4,4>"), (2, "BMMAS<4>")):
        out.zero_()
        ms = C.c_float(0)
        torch.cuda.synchronize()
        rc = R.ref_gpu_bmm(C.c_void_p(dA.data_ptr()), C.c_void_p(dB.data_ptr()), C.c_void_p(out.data_ptr()),
                           M, N, K, which, 20, C.byref(ms))
        assert rc == 0, name
        assert np.array_equal(out.cpu().numpy(), expect), name
        res[name] = {"ms": ms.value, "tops": 2.0 * M * N * K / (ms.value * 1e-3) / 1e12}
    ws = ops.gemm_workspace(M, N, K, cuda)
    ours = ops.bgemm(dA, dB, K, workspace=ws)
    assert np.array_equal(ours.cpu().numpy(), expect)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        ops.bgemm(dA, dB, K, out=ours, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    res["tcbnn_bgemm"] = {"ms": ms, "tops": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    print("\nSAME_BOX_BITGEMM " + json.dumps(res))


def test_reference_network_drivers_same_box(cuda, tmp_path):
    """The reference's unchanged drivers built with the reference's OWN headers (its WMMA b1
    kernels in one cooperative launch) for sm_100a into oracle/_ref/ref_<driver>, run once each on
    synthetic weight files and images.  They must finish without a CUDA error; the time each
    driver measures around its forward launch (one cold launch, utility.h:161-173) is printed next
    to this repository's time for the same topology and batch (run with -s)."""
    import os
    import re
    import subprocess
    from tcbnn_b200 import dropin, models
    ref = os.path.join(os.path.dirname(os.path.abspath(orc.__file__)), "_ref")
    cases = [("mnist_mlp", "mlp_mnist.csv", models.mlp_spec(32768)),
             ("cifar10_vgg", "vgg_cifar10.csv", models.vgg_cifar_spec(512)),
             ("cifar10_resnet", "resnet_cifar10.csv", models.resnet_cifar_spec(512)),
             ("imagenet_resnet", "resnet_imagenet.csv", models.resnet18_spec(512))]
    res = {}
    for exe, csv, spec in cases:
        path = os.path.join(ref, "ref_" + exe)
        if not os.path.exists(path):
            continue
        w = models.synthetic_weights(spec, 5)
        dropin.write_weights(w, os.path.join(str(tmp_path), csv))
        r = subprocess.run([path], cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, exe + ": " + r.stdout[-1500:] + r.stderr[-1500:]
        m = re.search(r"TCBNN_REF_INFERENCE_MS ([0-9.]+) (.*)", r.stdout)
        assert m, exe + ": no timing line\n" + r.stdout[-1500:]
        assert m.group(2).strip() == "no error", exe + ": " + m.group(2)
        ref_ms = float(m.group(1))
        x = models.synthetic_input(spec, 6)
        net = models.Network(spec, w, torch.from_numpy(np.ascontiguousarray(x)),
                             input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND if "resnet" in exe else None)
        for _ in range(3):
            net.forward()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            net.forward()
        e1.record()
        torch.cuda.synchronize()
        ours = e0.elapsed_time(e1) / 5
        B = spec["batch"]
        res[exe] = {"batch": B, "reference_ms": ref_ms, "reference_images_per_s": B / (ref_ms * 1e-3),
                    "tcbnn_b200_ms": ours, "tcbnn_b200_images_per_s": B / (ours * 1e-3), "ratio": ref_ms / ours}
        del net
    if not res:
        pytest.skip("oracle/_ref/ref_<driver> not built (reference tree absent at build time)")
    print("\nSAME_BOX_NETWORKS " + json.dumps(res))
