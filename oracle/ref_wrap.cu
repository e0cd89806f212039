// Build-time wrapper that exposes the reference's own host popcount loops through a C ABI.
// It contains no reference code: the reference source file is #included from where it lies
// (path given on the compiler command line as REF_SRC) and only the two host functions
// BMMAcpu (bmm/tensorcore_kernel.cu:38-57) and WMMABOOLCPU
// (bmm/bmma_op_test/main_test.cu:232-254) are re-exported.  Output goes to oracle/_ref/.
#if WHICH == 1
#include REF_SRC
extern "C" void ref_BMMAcpu(const unsigned* A, const unsigned* B, int* C, unsigned m, unsigned n,
                            unsigned k) { BMMAcpu(A, B, C, m, n, k); }

// The reference's own bit-GEMM kernels, launched exactly as bmm/benchmark-bmm.cu:406-453 does
// (same grids and blocks), on DEVICE operands A [m][k/32], B [n][k/32] (the layout its packers
// BMMA_toBit32Row / BMMA_toBit32Col produce), m and n multiples of 32, k a multiple of 128.
// which: 0 = BMMA<4,4>, 1 = BMMApipe<4,4>, 2 = BMMAS<4>.  Returns milliseconds per launch.
extern "C" int ref_gpu_bmm(const unsigned* A, const unsigned* B, int* C, unsigned m, unsigned n,
                           unsigned k, int which, int iters, float* ms_per_launch) {
    if (m % 32 || n % 32 || k % 128 || iters < 1) return 1;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int rep = 0; rep < 2; rep++) {          // first pass warms up
        cudaEventRecord(e0);
        for (int i = 0; i < iters; i++) {
            if (which == 0) BMMA<4, 4><<<dim3(m / 32, n / 32), dim3(32, 4, 4)>>>(A, B, C, m, n, k / 128);
            else if (which == 1) BMMApipe<4, 4><<<dim3(m / 32, n / 32), dim3(32, 4, 4)>>>(A, B, C, m, n, k / 128);
            else BMMAS<4><<<dim3(m / 16, n / 8), dim3(32, 2)>>>(A, B, C, m, n, k);
        }
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess) return 2;
    }
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    *ms_per_launch = ms / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
#else
#define main ref_main_test_main
#include REF_SRC
#undef main
extern "C" void ref_WMMABOOLCPU(const unsigned* A, const unsigned* B, const int* C, int* D,
                                unsigned m, unsigned n, unsigned k) {
    WMMABOOLCPU(A, B, C, D, m, n, k);
}
#endif
