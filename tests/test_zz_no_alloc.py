"""The allocation-free FC entry point (tcbnn_fc_layer_noalloc) against tcbnn_fc_layer.

Some callers cannot allocate device memory around a layer call: their own arena already owns
the GPU's memory, or they sit in a serving loop where an allocation's device-wide
synchronisation is not acceptable.  For them the library keeps the split-K scratch in a fixed
array of its own.  This file checks, through the C ABI, that the entry point gives exactly the
bits of the workspace-taking one on two calls in a row (the second with different inputs, so
stale scratch contents from the first call would show), and that a shape whose partial sums do
not fit the array is refused with a clear message.  The bits are also compared with the CPU
oracle, and the free device memory is read before and after a call that follows the first one:
a call that allocated anything would show there.  It is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as orc
import util
from tcbnn_b200 import lib, ops

pytestmark = pytest.mark.gpu


def _case(g, M, N, K, cuda):
    ld = ops.step128_words(K)
    A = util.mask_row_pad(util.rand_words(g, (M, ld)), K)
    W = util.mask_row_pad(util.rand_words(g, (N, ld)), K)
    thr = (g.standard_normal(N) * np.sqrt(K)).astype(np.float32)
    to = lambda a: torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(cuda)
    return to(A), to(W), to(thr), orc.fc_layer(A, W, thr, K)


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
    for call in range(2):
        A, W, thr, expect = _case(g, M, N, K, cuda)
        ws = ops.gemm_workspace(M, N, K, cuda)
        ref = ops.fc_layer(A, W, thr, K, workspace=ws)
        got = _noalloc(A, W, thr, K)
        torch.cuda.synchronize()
        assert torch.equal(got, ref)              # packed bits: exact
        assert np.array_equal(got.cpu().numpy().view(np.uint32), expect)      # and the CPU oracle's
        if call == 1:
            # the array's address is known by now: a further call must leave the device's free
            # memory exactly as it found it (the output buffer is allocated before the reading)
            out = torch.zeros((M, ops.step128_words(N)), dtype=torch.int32, device=cuda)
            torch.cuda.synchronize()
            free0, _ = torch.cuda.mem_get_info()
            lib.call("tcbnn_fc_layer_noalloc", ops._ptr(A), ops._ptr(W), ops._ptr(thr), M, K, N, A.shape[1],
                     W.shape[1], ops._ptr(out), out.shape[1], ops._stream())
            torch.cuda.synchronize()
            free1, _ = torch.cuda.mem_get_info()
            assert free1 == free0
            assert torch.equal(out, ref)


def test_noalloc_small_shape_without_split(cuda):
    g = util.rng(7)
    A, W, thr, expect = _case(g, 64, 40, 200, cuda)
    got = _noalloc(A, W, thr, 200)
    assert torch.equal(got, ops.fc_layer(A, W, thr, 200))
    assert np.array_equal(got.cpu().numpy().view(np.uint32), expect)


def test_noalloc_rejects_oversized_shape(cuda):
    L = lib.load()
    M, N, K = 1024, 512, 25088                    # 5 splits x 2 MiB of partials > 8 MiB
    assert L.tcbnn_gemm_workspace_bytes(M, N, K) > L.tcbnn_noalloc_scratch_bytes()
    dummy = torch.zeros((8,), dtype=torch.int32, device=cuda)
    rc = L.tcbnn_fc_layer_noalloc(ops._ptr(dummy), ops._ptr(dummy), ops._ptr(dummy), M, K, N,
                                  K // 32, K // 32, ops._ptr(dummy), N // 32, C.c_void_p(0))
    assert rc != 0
    assert b"scratch" in L.tcbnn_last_error()
