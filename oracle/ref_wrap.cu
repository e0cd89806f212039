// Build-time wrapper that exposes the reference's own host popcount loops through a C ABI.
// It contains no reference code: the reference source file is #included from where it lies
// (path given on the compiler command line as REF_SRC) and only the two host functions
// BMMAcpu (bmm/tensorcore_kernel.cu:38-57) and WMMABOOLCPU
// (bmm/bmma_op_test/main_test.cu:232-254) are re-exported.  Output goes to oracle/_ref/.
#if WHICH == 1
#include REF_SRC
extern "C" void ref_BMMAcpu(const unsigned* A, const unsigned* B, int* C, unsigned m, unsigned n,
                            unsigned k) { BMMAcpu(A, B, C, m, n, k); }
#else
#define main ref_main_test_main
#include REF_SRC
#undef main
extern "C" void ref_WMMABOOLCPU(const unsigned* A, const unsigned* B, const int* C, int* D,
                                unsigned m, unsigned n, unsigned k) {
    WMMABOOLCPU(A, B, C, D, m, n, k);
}
#endif
