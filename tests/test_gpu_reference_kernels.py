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


def test_reference_bitconv_kernel_matches_and_times(cuda):
    """The reference's standalone bit convolution (bconv/bmma_kernel.cu BTC_bin_*_128 +
    BTC_Conv2d_balance_128, launched as bconv/benchmark-bconv.cu:516-540 does) on the standalone
    conv configuration, 256 x 56 x 56 x 128 -> 128, 3x3, stride 1, SAME padding: its int32 sums
    must equal tcbnn_conv_layer's accumulators everywhere and the CPU oracle's on the first
    images; both timings are printed (run with -s)."""
    R = orc.ref_lib()
    if R is None or not hasattr(R, "ref_gpu_bconv128"):
        pytest.skip("oracle/_ref/libref_bmm.so not built (reference tree absent at build time)")
    N, H, Cc, O = 256, 56, 128, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(11)
    x = torch.randint(0, 2, (N, H, H, Cc), device=cuda, generator=g, dtype=torch.int8).float() * 2 - 1
    F = torch.randint(0, 2, (9, Cc, O), device=cuda, generator=g, dtype=torch.int8).float() * 2 - 1
    ref_out = torch.zeros((H, H, N, O), dtype=torch.int32, device=cuda)
    ms = C.c_float(0)
    torch.cuda.synchronize()
    rc = R.ref_gpu_bconv128(C.c_void_p(x.data_ptr()), C.c_void_p(F.data_ptr()), C.c_void_p(ref_out.data_ptr()),
                            N, H, H, Cc, O, 3, 3, 1, 1, H, H, 5, C.byref(ms))
    assert rc == 0
    ref_nhwo = ref_out.permute(2, 0, 1, 3).contiguous()
    d = ops.conv_desc(N, H, H, Cc, O, 3, 3)
    xb = ops.pack_rows(x.reshape(N * H * H, Cc)).reshape(N, H, H, Cc // 32)
    fb = ops.pack_conv_filter(F)
    prep = ops.conv_prepare(d, fb)
    thr = torch.zeros((O,), device=cuda)
    out, _, acc = ops.conv_layer(d, xb, prep, thr, want_acc=True)
    assert torch.equal(acc, ref_nhwo)
    sub = 4
    _, _, ea = orc.conv_layer(xb[:sub].cpu().numpy(), fb.cpu().numpy(), thr.cpu().numpy(), Cc, 3, 3, want_acc=True)
    assert np.array_equal(ref_nhwo[:sub].cpu().numpy(), ea)
    del acc, ref_out
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        ops.conv_layer(d, xb, prep, thr, out=out)
    e0.record()
    for _ in range(20):
        ops.conv_layer(d, xb, prep, thr, out=out)
    e1.record()
    torch.cuda.synchronize()
    t = e0.elapsed_time(e1) / 20
    work = 2.0 * N * H * H * O * 9 * Cc
    print("\nSAME_BOX_BITCONV " + json.dumps({
        "BTC_Conv2d_balance_128": {"ms": ms.value, "tops": work / (ms.value * 1e-3) / 1e12},
        "tcbnn_conv_layer": {"ms": t, "tops": work / (t * 1e-3) / 1e12}, "ratio": ms.value / t}))


def test_reference_network_drivers_same_box(cuda, tmp_path):
    """The reference's unchanged drivers built with the reference's OWN headers (its WMMA b1
    kernels in one cooperative launch) for sm_100a into oracle/_ref/ref_<driver>, run once each on
    synthetic weight files and the stand-in readers' images.

    Parity: the logits the reference computes (its output layer's download_output(), captured by
    oracle/ref_driver_shim.h) against this library's on the same weights and the same images --
    the network-level pin of every layer epilogue on the way (threshold, OR-pool, residual add /
    2x2 max, first-layer sums, FC, scale + bias).  A subset of images also goes through the CPU
    oracle.  Timing: what each driver measures around its forward launch (one cold launch,
    utility.h:161-173) next to this library's time (run with -s)."""
    import os
    import re
    import subprocess
    import networks as onet
    from tcbnn_b200 import dropin, models
    ref = os.path.join(os.path.dirname(os.path.abspath(orc.__file__)), "_ref")
    cases = [("mnist_mlp", "mlp_mnist.csv", models.mlp_spec(32768), "mnist"),
             ("cifar10_vgg", "vgg_cifar10.csv", models.vgg_cifar_spec(512), "cifar"),
             ("cifar10_resnet", "resnet_cifar10.csv", models.resnet_cifar_spec(512), "cifar"),
             ("imagenet_resnet", "resnet_imagenet.csv", models.resnet18_spec(512), "imagenet")]
    res = {}
    for exe, csv, spec, kind in cases:
        path = os.path.join(ref, "ref_" + exe)
        if not os.path.exists(path):
            continue
        w = models.synthetic_weights(spec, 5)
        dropin.write_weights(w, os.path.join(str(tmp_path), csv))
        dump = os.path.join(str(tmp_path), exe + "_logits.bin")
        r = subprocess.run([path], cwd=str(tmp_path), capture_output=True, text=True, timeout=600,
                           env=dict(os.environ, TCBNN_REF_DUMP=dump))
        assert r.returncode == 0, exe + ": " + r.stdout[-1500:] + r.stderr[-1500:]
        m = re.search(r"TCBNN_REF_INFERENCE_MS ([0-9.]+) (.*)", r.stdout)
        assert m, exe + ": no timing line\n" + r.stdout[-1500:]
        assert m.group(2).strip() == "no error", exe + ": " + m.group(2)
        ref_ms = float(m.group(1))
        B = spec["batch"]
        classes = spec["layers"][-1]["N"]
        ref_logits = np.fromfile(dump, dtype=np.float32)
        assert ref_logits.size >= B * classes, (exe, ref_logits.size)
        ref_logits = ref_logits[:B * classes].reshape(B, classes)
        x = util.reader_images(kind, B)
        bound = float(np.abs(x).max()) if "resnet" in exe else None   # int16 residual rows when it fits
        net = models.Network(spec, w, torch.from_numpy(np.ascontiguousarray(x)).to(cuda), input_abs_bound=bound)
        ours = net.forward().cpu().numpy()[:, :classes]
        np.testing.assert_allclose(ours, ref_logits, rtol=1e-5, atol=1e-4, err_msg=exe)
        sub = 16                                        # the CPU oracle on the first images
        sspec = dict(spec, batch=sub)
        acts, _ = onet.run(sspec, w, x[:sub])
        np.testing.assert_allclose(acts[-1][:, :classes], ref_logits[:sub], rtol=1e-5, atol=1e-4, err_msg=exe + " (oracle)")
        for _ in range(3):
            net.forward()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            net.forward()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / 5
        res[exe] = {"batch": B, "reference_ms": ref_ms, "reference_images_per_s": B / (ref_ms * 1e-3),
                    "tcbnn_b200_ms": t, "tcbnn_b200_images_per_s": B / (t * 1e-3), "ratio": ref_ms / t,
                    "max_abs_logit_diff": float(np.max(np.abs(ours - ref_logits)))}
        del net
    if not res:
        pytest.skip("oracle/_ref/ref_<driver> not built (reference tree absent at build time)")
    print("\nSAME_BOX_NETWORKS " + json.dumps(res))


def _ref_runner():
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(orc.__file__)), "_ref", "ref_net_runner")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/ref_net_runner not built (reference tree absent at build time)")
    return path


@pytest.mark.parametrize("which", ["mlp", "vgg_cifar", "resnet18_small", "resnet_cifar"])
def test_oracle_matches_reference_implementation_layer_by_layer(cuda, tmp_path, which):
    """The layer-level pin: the generic driver (tcbnn_b200/dropin/net_runner.cu) compiled against
    the REFERENCE's own headers runs the reference's In128 / Fc128 / Out128 / InConv128 / Conv128
    kernels on the GPU; every layer's unpacked +-1 activations (download_full_output()) and the
    logits must equal the CPU oracle's on the same weights and inputs."""
    from tcbnn_b200 import models
    from test_gpu_dropin import _run
    spec = {"mlp": models.mlp_spec(256), "vgg_cifar": models.vgg_cifar_spec(8),
            "resnet18_small": models.resnet18_spec(8, image=64, classes=100),
            "resnet_cifar": models.resnet_cifar_spec(8)}[which]
    _run(spec, 60, tmp_path, cuda, runner=_ref_runner())


def test_standalone_conv_full_size_with_thresholds(cuda):
    """The standalone conv configuration at full size with its thresholds: 256 x 56 x 56 x 128 ->
    128, 3x3, stride 1, SAME padding, per-channel fp32 thresholds N(0, 8) (8 is the standard
    deviation).  Packed output bits and int32 accumulators against the CPU oracle on the first and
    last 8 images, the accumulators of ALL images against the reference's own kernel where it was
    built, and the packed bits of all images against the accumulators thresholded in torch."""
    N, H, Cc, O = 256, 56, 128, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(2)
    x = torch.randint(0, 2, (N, H, H, Cc), device=cuda, generator=g, dtype=torch.int8).float() * 2 - 1
    g.manual_seed(3)
    F = torch.randint(0, 2, (9, Cc, O), device=cuda, generator=g, dtype=torch.int8).float() * 2 - 1
    g.manual_seed(4)
    thr = torch.randn((O,), device=cuda, generator=g) * 8.0
    d = ops.conv_desc(N, H, H, Cc, O, 3, 3)
    xb = ops.pack_rows(x.reshape(N * H * H, Cc)).reshape(N, H, H, Cc // 32)
    fb = ops.pack_conv_filter(F)
    prep = ops.conv_prepare(d, fb)
    out, _, acc = ops.conv_layer(d, xb, prep, thr, want_acc=True)
    assert ops.conv_status(d, prep) == 0
    sub = 8
    for sl in (slice(0, sub), slice(N - sub, N)):
        eb, _, ea = orc.conv_layer(xb[sl].cpu().numpy(), fb.cpu().numpy(), thr.cpu().numpy(), Cc, 3, 3, want_acc=True)
        assert np.array_equal(acc[sl].cpu().numpy(), ea)
        assert np.array_equal(out[sl].cpu().numpy().view(np.uint32).reshape(eb.shape), eb)
    # all images: bit o of a pixel is !((float)acc < thr[o]) (kernel.cuh:795-796)
    bits = ~(acc.float() < thr.view(1, 1, 1, O))
    weights = (2 ** torch.arange(31, -1, -1, device=cuda, dtype=torch.int64)).view(1, 1, 1, 1, 32)
    words = (bits.view(N, H, H, O // 32, 32).to(torch.int64) * weights).sum(-1)
    got = out.view(N, H, H, O // 32).to(torch.int64) & 0xFFFFFFFF
    assert torch.equal(got, words)
    R = orc.ref_lib()
    if R is not None and hasattr(R, "ref_gpu_bconv128"):
        ref_out = torch.zeros((H, H, N, O), dtype=torch.int32, device=cuda)
        ms = C.c_float(0)
        torch.cuda.synchronize()
        rc = R.ref_gpu_bconv128(C.c_void_p(x.data_ptr()), C.c_void_p(F.data_ptr()), C.c_void_p(ref_out.data_ptr()),
                                N, H, H, Cc, O, 3, 3, 1, 1, H, H, 1, C.byref(ms))
        assert rc == 0
        assert torch.equal(acc, ref_out.permute(2, 0, 1, 3).contiguous())
