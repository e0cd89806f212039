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
