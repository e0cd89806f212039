// Build-time wrapper that exposes the reference's own host popcount loops and GPU kernels through
// a C ABI.  It contains no reference code: the reference source file is #included from where it
// lies (path given on the compiler command line as REF_SRC).  Re-exported: the host functions
// BMMAcpu (bmm/tensorcore_kernel.cu:38-57) and WMMABOOLCPU (bmm/bmma_op_test/main_test.cu:232-254),
// the bit-GEMM kernels of bmm/tensorcore_kernel.cu and the 128-channel bit convolution of
// bconv/bmma_kernel.cu.  Output goes to oracle/_ref/.  Test infrastructure only.
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
#elif WHICH == 3
#include REF_SRC
// The reference's standalone bit convolution, launched as bconv/benchmark-bconv.cu:516-540 does:
// BTC_bin_filter_128 / BTC_bin_input_128 binarise fp32 operands (input NHWC, filter [R*S][C][O]),
// then BTC_Conv2d_balance_128 with one warp per CTA on a grid (OW, OH, N/8 * O/8) writes the int32
// sums [OH][OW][N][O].  C a multiple of 128, N and O multiples of 8.  All pointers are DEVICE
// pointers.  Returns milliseconds per convolution launch (binarisation excluded, as there).
extern "C" int ref_gpu_bconv128(const float* input, const float* filter, int* output, int N, int H, int W,
                                int C, int O, int R, int S, int stride, int pad, int OH, int OW, int iters,
                                float* ms_per_launch) {
    if (C % 128 || N % 8 || O % 8 || iters < 1) return 1;
    unsigned *in_bits = NULL, *f_bits = NULL;
    const size_t in_words = (size_t)H * W * N * (C / 32), f_words = (size_t)R * S * O * (C / 32);
    if (cudaMalloc(&in_bits, in_words * 4) != cudaSuccess || cudaMalloc(&f_bits, f_words * 4) != cudaSuccess) return 4;
    cudaMemset(in_bits, 0, in_words * 4);
    cudaMemset(f_bits, 0, f_words * 4);
    BTC_bin_filter_128<float><<<dim3(R * S, O), 32>>>(filter, f_bits, C, O, S, R);
    BTC_bin_input_128<float><<<dim3(W, H, N), 32>>>(input, in_bits, C, N, W, H);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int rc = 0;
    for (int rep = 0; rep < 2 && rc == 0; rep++) {          // first pass warms up
        cudaEventRecord(e0);
        for (int i = 0; i < iters; i++)
            BTC_Conv2d_balance_128<<<dim3(OW, OH, (N / 8) * (O / 8)), 32>>>(in_bits, f_bits, output, C, O, W, H, S, R, N,
                                                                        stride, stride, OW, OH, pad, pad);
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess) rc = 2;
    }
    float ms = 0;
    if (rc == 0) cudaEventElapsedTime(&ms, e0, e1);
    *ms_per_launch = ms / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(in_bits);
    cudaFree(f_bits);
    if (rc == 0 && cudaGetLastError() != cudaSuccess) rc = 3;
    return rc;
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
