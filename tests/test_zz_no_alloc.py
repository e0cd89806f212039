"""The allocation-free FC entry point (tcbnn_fc_layer_noalloc) against tcbnn_fc_layer.

Some callers cannot allocate device memory around a layer call: their own arena already owns
the GPU's memory, or they sit in a serving loop where an allocation's device-wide
synchronisation is not acceptable.  For them the library keeps the split-K scratch in a fixed
array of its own.  This file checks, through the C ABI, that the entry point gives exactly the
bits of the workspace-taking one on two calls in a row (the second with different inputs, so
stale scratch contents from the first call would show), and that a shape whose partial sums do
not fit the array is refused with a clear message.  It is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import util
from tcbnn_b200 import lib, ops

pytestmark = pytest.mark.gpu


def _case(g, M, N, K, cuda):
    ld = ops.step128_words(K)
    A = util.mask_row_pad(util.rand_words(g, (M, ld)), K)
    W = util.mask_row_pad(util.rand_words(g, (N, ld)), K)
    thr = (g.standard_normal(N) * np.sqrt(K)).astype(np.float32)
    to = lambda a: torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(cuda)
    return to(A), to(W), to(thr)


def _noalloc(A, W, thr, K):
    M, lda = A.shape
    N, ldw = W.shape
    out = torch.zeros((M, ops.step128_words(N)), dtype=torch.int32, device=A.device)
    lib.call("tcbnn_fc_layer_noalloc", ops._ptr(A), ops._ptr(W), ops._ptr(thr), M, K, N, lda, ldw,
             ops._ptr(out), out.shape[1], ops._stream())
    return out


def test_noalloc_matches_workspace_variant_twice(cuda):
    g = util.rng(2024)
    M, N, K = 256, 128, 8192                      # few tiles, long K: the split-K path
    need = lib.load().tcbnn_gemm_workspace_bytes(M, N, K)
    assert 0 < need <= lib.load().tcbnn_noalloc_scratch_bytes()
    for _ in range(2):
        A, W, thr = _case(g, M, N, K, cuda)
        ws = ops.gemm_workspace(M, N, K, cuda)
        ref = ops.fc_layer(A, W, thr, K, workspace=ws)
        got = _noalloc(A, W, thr, K)
        torch.cuda.synchronize()
        assert torch.equal(got, ref)              # packed bits: exact


def test_noalloc_small_shape_without_split(cuda):
    g = util.rng(7)
    A, W, thr = _case(g, 64, 40, 200, cuda)
    assert torch.equal(_noalloc(A, W, thr, 200), ops.fc_layer(A, W, thr, 200))


def test_noalloc_rejects_oversized_shape(cuda):
    L = lib.load()
    M, N, K = 1024, 512, 25088                    # 5 splits x 2 MiB of partials > 8 MiB
    assert L.tcbnn_gemm_workspace_bytes(M, N, K) > L.tcbnn_noalloc_scratch_bytes()
    dummy = torch.zeros((8,), dtype=torch.int32, device=cuda)
    rc = L.tcbnn_fc_layer_noalloc(ops._ptr(dummy), ops._ptr(dummy), ops._ptr(dummy), M, K, N,
                                  K // 32, K // 32, ops._ptr(dummy), N // 32, C.c_void_p(0))
    assert rc != 0
    assert b"scratch" in L.tcbnn_last_error()
