"""GPU parity of the C++ host classes on the C ABI (tcbnn_b200/host/tcbnn_host.hpp): the generic
driver build/host/fast_runner builds each network with the reference's class names and
constructor arguments and runs it through libtcbnn_b200.so layer by layer (tcgen05 kernels, the
first layer compiled for its filter, hand-over between conv layers).  Logits and every layer's
unpacked +-1 activations are compared with the CPU oracle."""
import pytest

from tcbnn_b200 import models
from tcbnn_b200.host import build as hbuild
from test_gpu_dropin import _run

pytestmark = pytest.mark.gpu


def test_host_cpp_mlp(cuda, tmp_path):
    _run(models.mlp_spec(256), 80, tmp_path, cuda, runner=hbuild.build_fast_runner())


def test_host_cpp_vgg_cifar_binary_weights(cuda, tmp_path):
    _run(models.vgg_cifar_spec(8), 81, tmp_path, cuda, runner=hbuild.build_fast_runner(), weights="binary")


def test_host_cpp_resnet18_small_image_repeated_runs(cuda, tmp_path):
    _run(models.resnet18_spec(8, image=64, classes=100), 82, tmp_path, cuda, runner=hbuild.build_fast_runner(), runs=3)


def test_host_cpp_resnet_cifar(cuda, tmp_path):
    _run(models.resnet_cifar_spec(4), 83, tmp_path, cuda, runner=hbuild.build_fast_runner())


def test_host_cpp_without_handover(cuda, tmp_path, monkeypatch):
    monkeypatch.setenv("TCBNN_NO_HANDOVER", "1")
    _run(models.resnet18_spec(4, image=64, classes=100), 84, tmp_path, cuda, runner=hbuild.build_fast_runner())


def test_host_cpp_int16_residuals(cuda, tmp_path, monkeypatch):
    """set_residual_bytes(2) on every layer: same activations and logits (the synthetic images
    keep the running sums far inside int16)."""
    monkeypatch.setenv("TCBNN_RESIDUAL16", "1")
    _run(models.resnet18_spec(4, image=64, classes=100), 85, tmp_path, cuda, runner=hbuild.build_fast_runner())


def test_host_cpp_chunked_int16_residuals(cuda, tmp_path, monkeypatch):
    """set_residual_bytes(TCBNN_RES_INT16_CHUNKED) on every layer: the conv layers run the
    tile-per-group epilogue on chunk-major residual tensors; same activations and logits."""
    monkeypatch.setenv("TCBNN_RESIDUAL16", "chunked")
    _run(models.resnet18_spec(4, image=64, classes=100), 89, tmp_path, cuda, runner=hbuild.build_fast_runner())
    _run(models.resnet18_spec(3), 90, tmp_path, cuda, runner=hbuild.build_fast_runner(), runs=2)


def test_host_cpp_reference_signatures_and_ragged_batch(cuda, tmp_path):
    """The layer lines of a reference driver compile against the host classes as they are:
    initialize(FILE*, prev [, residual]) with the residual's channel count and element size looked
    up from its producer.  The same objects then run the first 5 of their 8 images (set_batch)."""
    _run(models.resnet18_spec(8, image=64, classes=100), 86, tmp_path, cuda, runner=hbuild.build_fast_runner(),
         extra_env={"TCBNN_TEXT_SIGNATURES": "1"})
    _run(models.resnet18_spec(8, image=64, classes=100), 87, tmp_path, cuda, runner=hbuild.build_fast_runner(),
         runs=2, live=5, extra_env={"TCBNN_TEXT_SIGNATURES": "1", "TCBNN_RESIDUAL16": "1"})
    _run(models.vgg_cifar_spec(8), 88, tmp_path, cuda, runner=hbuild.build_fast_runner(), runs=2, live=3)
