// Forced include (nvcc -include) for building the reference's unchanged network drivers with the
// reference's own headers as a same-box baseline.  Test infrastructure, not part of the library.
//
// The drivers time their one forward launch with CUDA events (START_TIMER / STOP_TIMER,
// utility.h:161-173) but the print of the result is commented out there, and the ImageNet drivers
// select device 1 (imagenet_resnet.cu:205-206).  Without touching the reference's sources, this
// header makes the elapsed time visible on stdout and maps the device index onto the devices that
// exist.
#pragma once
#include <cstdio>
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
#undef cudaGetDeviceProperties
#define cudaEventElapsedTime(ms, a, b) tcbnn_ref_elapsed(ms, a, b)
#define cudaSetDevice(d) tcbnn_ref_set_device(d)
#define cudaGetDeviceProperties(p, d) tcbnn_ref_props(p, d)
