"""GPU parity of whole networks, layer by layer, against the CPU oracle."""
import numpy as np
import pytest
import torch

import networks as onet
from tcbnn_b200 import models

pytestmark = pytest.mark.gpu


def _compare(spec, seed, cuda, input_abs_bound=None):
    w = models.synthetic_weights(spec, seed)
    x = models.synthetic_input(spec, seed + 1)
    acts, ress = onet.run(spec, w, x)
    net = models.Network(spec, w, x, input_abs_bound=input_abs_bound)
    logits = net.forward()
    torch.cuda.synchronize()
    for i, (layer, a, r) in enumerate(zip(net.layers, acts, ress)):
        got = layer.get_output_gpu().cpu().numpy()
        if got.dtype == np.int32:
            got = got.view(np.uint32)
            assert np.array_equal(got.reshape(a.shape), a), "layer %d %s bits" % (i, layer.name)
        if r is not None:
            if input_abs_bound is not None:
                assert layer.get_output_residual_gpu().dtype == torch.int16
            gr = layer.download_output_residual()          # int32 NHWC whatever the device layout
            assert np.array_equal(gr, r), "layer %d %s residual" % (i, layer.name)
    ref = acts[-1]
    got = logits.cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5)
    # a second pass over the same objects gives the same logits (layers store, never OR)
    again = net.forward().cpu().numpy()
    assert np.array_equal(again, got)


def test_mlp(cuda):
    _compare(models.mlp_spec(256), 5, cuda)


def test_vgg_cifar(cuda):
    _compare(models.vgg_cifar_spec(8), 10, cuda)


def test_alexnet_small_image(cuda):
    # alexnet.cu topology (11x11/4 + pool, 5x5 + pool, 192 / 384 channels) on 96x96 images
    _compare(models.alexnet_spec(4, image=96, hidden=256, classes=100), 40, cuda)


def test_vgg16_imagenet_small_image(cuda):
    # imagenet_vgg.cu topology (13 conv layers, five of them pooled) on 32x32 images
    _compare(models.vgg16_imagenet_spec(3, image=32, hidden=256, classes=100), 50, cuda)


def test_resnet18_small_image(cuda):
    # same topology, 64x64 input -> 16x16 ... 2x2 feature maps
    _compare(models.resnet18_spec(8, image=64, classes=100), 20, cuda)


def test_resnet18_224(cuda):
    _compare(models.resnet18_spec(2), 30, cuda)


def test_resnet18_224_int16_residuals(cuda):
    # same network with the stated input bound: residual chain stored as int16, values identical
    _compare(models.resnet18_spec(3), 31, cuda, input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND)


def test_resnet18_chunked_residual_layout_is_wired_where_it_pays(cuda):
    """With int16 residuals every residual tensor of the network (first layer -> ... -> L4B1C2; the
    last block saves none) is kept in the chunk-major layout: all its producers and consumers run
    the loader-fed kernel, whose tile-per-group epilogue takes that layout only; pooled ones are
    then read in place, so no layer launches a pooling pass."""
    spec = models.resnet18_spec(2)
    net = models.Network(spec, models.synthetic_weights(spec, 32), models.synthetic_input(spec, 33),
                         input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND)
    by = {l.name: l for l in net.layers}
    assert by["Conv1"].residual_chunked
    for stage in "1234":
        for block in "12":
            l = by["L%sB%sC2" % (stage, block)]
            assert l.input_residual_chunked, l.name
            if l.output_residual_gpu is not None:
                assert l.residual_chunked, l.name
            assert l.kernel_launches() == 1, l.name


def test_resnet18_both_conv_kernels(cuda):
    from tcbnn_b200 import ops
    try:
        ops.set_conv_path(1)                 # warp-level b1 MMA everywhere
        _compare(models.resnet18_spec(2, image=64, classes=100), 21, cuda)
    finally:
        ops.set_conv_path(0)


def test_resnet18_uint8_images_give_identical_results(cuda):
    """Byte images + per-channel value table through tcbnn_inconv_layer_u8: every tensor equal
    to the fp32-image run of the same network."""
    spec = models.resnet18_spec(3)
    w = models.synthetic_weights(spec, 50)
    x = models.synthetic_input(spec, 51)
    u8, lut = models.synthetic_input_u8(spec, 51)
    assert np.array_equal(lut[np.arange(3)[None, :, None, None], u8], x)       # same pixels
    ref = models.Network(spec, w, x)
    got = models.Network(spec, w, torch.from_numpy(u8), input_lut=lut)
    a, b = ref.forward().cpu().numpy(), got.forward().cpu().numpy()
    for la, lb in zip(ref.layers, got.layers):
        assert torch.equal(la.get_output_gpu(), lb.get_output_gpu()), la.name
    assert np.array_equal(a, b)
    acts, _ = onet.run(spec, w, x)
    np.testing.assert_allclose(b, acts[-1], rtol=1e-5, atol=1e-5)


def test_forward_graph_replay_equals_eager_forward(cuda):
    """Network.forward_graph: the same launches captured into a CUDA graph; replays follow the
    contents of the input buffer and give the eager results bit for bit."""
    spec = models.resnet18_spec(4, image=64, classes=100)
    w = models.synthetic_weights(spec, 60)
    x0 = models.synthetic_input(spec, 61)
    x1 = models.synthetic_input(spec, 62)
    net = models.Network(spec, w, x0, input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND)
    eager0 = net.forward().clone()
    g0 = net.forward_graph().clone()            # captures
    assert torch.equal(g0, eager0)
    net.layers[0].input_gpu.copy_(torch.from_numpy(x1).to(cuda).reshape(net.layers[0].input_gpu.shape))
    g1 = net.forward_graph().clone()            # replays on the new images
    eager1 = net.forward().clone()
    assert torch.equal(g1, eager1) and not torch.equal(g1, g0)
    acts, _ = onet.run(spec, w, x1)
    np.testing.assert_allclose(g1.cpu().numpy(), acts[-1], rtol=1e-5, atol=1e-5)


def test_host_feeder_overlapped_copies_give_each_batch_its_own_logits(cuda):
    """models.HostFeeder: pinned host batches in, input copy of batch i+1 and logits read of
    batch i beside the compute of the batch between them; every batch's logits equal those of
    a plain forward pass on that batch, with and without graph replay."""
    spec = models.resnet18_spec(4, image=64, classes=100)
    w = models.synthetic_weights(spec, 70)
    xs = [models.synthetic_input(spec, 71 + i) for i in range(4)]
    expect = []
    for x in xs:
        expect.append(models.Network(spec, w, x, input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND).forward().cpu().numpy())
    for graph in (False, True):
        net = models.Network(spec, w, xs[0], input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND)
        feeder = models.HostFeeder(net, graph=graph)
        host = [torch.from_numpy(np.ascontiguousarray(x)).pin_memory() for x in xs]
        last = torch.empty((4, 100), dtype=torch.float32).pin_memory()
        got = []
        feeder.run(host, lambda out: got.append(out.clone()), last)
        torch.cuda.synchronize()
        assert len(got) == len(xs)
        for g, e in zip(got, expect):
            assert np.array_equal(g.cpu().numpy(), e)
        assert np.array_equal(last.numpy(), expect[-1])


@pytest.mark.parametrize("which", ["resnet18", "vgg_cifar", "mlp"])
def test_set_batch_runs_ragged_batches_on_the_same_objects(cuda, which):
    """Layer objects built for 8 images process 5, then 8, then 3 images (Network.set_batch)
    without being rebuilt: every layer's bits and the logits of the live images equal the oracle's
    on exactly those images (the reference fixes the batch at construction, param.h:875-881)."""
    spec = {"resnet18": models.resnet18_spec(8, image=64, classes=100), "vgg_cifar": models.vgg_cifar_spec(8),
            "mlp": models.mlp_spec(8)}[which]
    w = models.synthetic_weights(spec, 80)
    bound = models.SYNTHETIC_IMAGE_ABS_BOUND if which == "resnet18" else None
    net = models.Network(spec, w, models.synthetic_input(spec, 81), input_abs_bound=bound)
    net.forward()
    for step, n in enumerate((5, 8, 3)):
        x = models.synthetic_input(spec, 90 + step, batch=n)
        net.set_batch(n)
        net.set_input(x)
        logits = (net.forward_graph() if step else net.forward())[:n].cpu().numpy()
        acts, ress = onet.run(dict(spec, batch=n), w, x)
        for i, (layer, a, r) in enumerate(zip(net.layers[:-1], acts[:-1], ress[:-1])):
            got = layer.get_output_gpu()[:n].cpu().numpy().view(np.uint32)
            assert np.array_equal(got.reshape(a.shape), a), "batch %d layer %d %s bits" % (n, i, layer.name)
            if r is not None:
                gr = layer.download_output_residual()
                assert np.array_equal(gr, r), "batch %d layer %d %s residual" % (n, i, layer.name)
        np.testing.assert_allclose(logits, acts[-1], rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        net.set_batch(9)


@pytest.mark.parametrize("which,sub", [("mlp", 512), ("vgg_cifar", 32)])
def test_baseline_batch_logits_against_oracle_slice(cuda, which, sub):
    """The MLP at batch 8192 and the CIFAR VGG at batch 1024 (the standalone network
    configurations at their full batch): the logits of the first images must equal the CPU
    oracle's on exactly those images (every image is processed independently), and all logits
    must be finite.  1e-5 relative."""
    spec = models.mlp_spec(8192) if which == "mlp" else models.vgg_cifar_spec(1024)
    w = models.synthetic_weights(spec, 110)
    x = models.synthetic_input(spec, 111)
    net = models.Network(spec, w, x)
    logits = net.forward_graph().cpu().numpy()
    assert np.all(np.isfinite(logits))
    acts, _ = onet.run(dict(spec, batch=sub), w, x[:sub])
    np.testing.assert_allclose(logits[:sub], acts[-1], rtol=1e-5, atol=1e-5)
    # and the last images, which sit in the last tiles of every layer
    acts, _ = onet.run(dict(spec, batch=sub), w, x[-sub:])
    np.testing.assert_allclose(logits[-sub:], acts[-1], rtol=1e-5, atol=1e-5)
