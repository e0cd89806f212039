// Forced include (nvcc -include) for building the reference's unchanged network drivers with the
// reference's own headers as a same-box baseline.  Test infrastructure, not part of the library.
//
// The drivers time their one forward launch with CUDA events (START_TIMER / STOP_TIMER,
// utility.h:161-173) but the print of the result is commented out there, and the ImageNet drivers
// select device 1 (imagenet_resnet.cu:205-206).  Without touching the reference's sources, this
// header makes the elapsed time visible on stdout and maps the device index onto the devices that
// exist.  With TCBNN_REF_DUMP=<file> in the environment every device-to-host copy is also written
// to that file (each one replaces the last): the final one is the output layer's download_output()
// (param.h:485-491), i.e. the logits, which the parity test compares.
//
// One CTA per SM.  The reference names a warp by the hardware register %warpid (GET_WARPID,
// utility.h:48) and uses it as the warp's index inside a 1024-thread CTA: In128LayerFMT
// (kernel.cuh:153-172), PackFcWeight128FMT and UnPackFcOutput128FMT (param.h:44-104) compute rows,
// columns and word indices from it.  That holds while one such CTA is resident per SM -- always
// the case on the 1024-threads-per-SM parts the code was written for.  A B200 SM holds 2048
// threads, every launch is sized by the occupancy query (numBlocksPerSm x SMs), and a second
// resident CTA gets %warpid 32..63: the packed FC weights and the unpacked FC activations land in
// the wrong words.  Capping the query's answer at 1 keeps the launches the shape they have on the
// reference's hardware.  (The forward kernel itself already gets 1: 1024 threads x 64 registers.)
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

static inline cudaError_t tcbnn_ref_elapsed(float* ms, cudaEvent_t a, cudaEvent_t b) {
    const cudaError_t e = cudaEventElapsedTime(ms, a, b);
    printf("\nTCBNN_REF_INFERENCE_MS %.4f %s\n", *ms, cudaGetErrorString(cudaGetLastError()));
    return e;
}
static inline int tcbnn_ref_device(int d) {
    int n = 1;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n < 1) n = 1;
    return d % n;
}
static inline cudaError_t tcbnn_ref_set_device(int d) { return cudaSetDevice(tcbnn_ref_device(d)); }
static inline cudaError_t tcbnn_ref_props(cudaDeviceProp* p, int d) {
    return cudaGetDeviceProperties(p, tcbnn_ref_device(d));
}
static inline cudaError_t tcbnn_ref_memcpy(void* dst, const void* src, size_t n, cudaMemcpyKind kind) {
    const cudaError_t e = cudaMemcpy(dst, src, n, kind);
    if (kind == cudaMemcpyDeviceToHost && e == cudaSuccess) {
        const char* path = getenv("TCBNN_REF_DUMP");
        FILE* f = path ? fopen(path, "wb") : NULL;
        if (f) { fwrite(dst, 1, n, f); fclose(f); }
    }
    return e;
}
template <class T>
static inline cudaError_t tcbnn_ref_occupancy(int* blocks, T func, int threads, size_t smem) {
    const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks, func, threads, smem);
    if (*blocks > 1) *blocks = 1;
    return e;
}
#undef cudaGetDeviceProperties
#define cudaEventElapsedTime(ms, a, b) tcbnn_ref_elapsed(ms, a, b)
#define cudaSetDevice(d) tcbnn_ref_set_device(d)
#define cudaGetDeviceProperties(p, d) tcbnn_ref_props(p, d)
#define cudaMemcpy(d, s, n, k) tcbnn_ref_memcpy(d, s, n, k)
#define cudaOccupancyMaxActiveBlocksPerMultiprocessor(n, f, t, s) tcbnn_ref_occupancy(n, f, t, s)
