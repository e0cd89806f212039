"""Regenerates the golden vectors in this folder.  Needs the reference tree (for
oracle/_ref/libref_bmm.so, built from the reference's own source files) and glibc.

    python tests/golden/make_golden.py

wmma_kat_srand4.npz : the reference's one seeded known-answer recipe -- srand(4); A, B, C
    filled word by word with rand() (bmm/bmma_op_test/main_test.cu:293-298); expected
    D = WMMABOOLCPU(A, B, C) computed by the reference's host function (:232-254).
    Shapes (m, n, k): the reference's own 8x8x128 plus three larger ones.
bmma_cpu_ref.npz    : BMMAcpu (bmm/tensorcore_kernel.cu:38-57) outputs on words drawn from
    numpy's PCG64 with the seeds stored in the file.
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import oracle as orc  # noqa: E402


def main():
    libc = ctypes.CDLL("libc.so.6")
    libc.rand.restype = ctypes.c_int
    kat = {}
    for (m, n, k) in [(8, 8, 128), (16, 8, 256), (24, 40, 384), (64, 32, 1024)]:
        libc.srand(4)
        A = np.array([libc.rand() for _ in range(m * k // 32)], dtype=np.uint32).reshape(m, k // 32)
        B = np.array([libc.rand() for _ in range(k * n // 32)], dtype=np.uint32).reshape(n, k // 32)
        Cc = np.array([libc.rand() for _ in range(m * n)], dtype=np.int64).astype(np.int32).reshape(m, n)
        D = orc.ref_wmma_bool_cpu(A, B, Cc, k)
        tag = "%dx%dx%d" % (m, n, k)
        kat["A_" + tag], kat["B_" + tag], kat["C_" + tag], kat["D_" + tag] = A, B, Cc, D
    np.savez_compressed(os.path.join(HERE, "wmma_kat_srand4.npz"), **kat)

    ref = {}
    for seed, (m, n, k) in enumerate([(32, 32, 128), (40, 24, 640), (64, 48, 4096)], start=11):
        rng = np.random.Generator(np.random.PCG64(seed))
        A = rng.integers(0, 2**32, size=(m, k // 32), dtype=np.uint64).astype(np.uint32)
        B = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
        tag = "%dx%dx%d" % (m, n, k)
        ref["seed_" + tag] = np.array([seed])
        ref["A_" + tag], ref["B_" + tag] = A, B
        ref["popc_" + tag] = orc.ref_bmma_cpu(A, B, k)
    np.savez_compressed(os.path.join(HERE, "bmma_cpu_ref.npz"), **ref)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
