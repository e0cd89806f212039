// Drop-in replacement for the reference's utility.h (pnnl/TCBNN): same type names, macros and
// helper functions (utility.h:22-246 there), written for the B200 build.  Header-only; each
// driver is a single translation unit, as in the reference.
#ifndef UTILITY_H
#define UTILITY_H

#include <sys/time.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <cuda_runtime.h>

#define NEWFMT   // the "new format" layer functions are the live ones (utility.h:22)

// ---- types (utility.h:25-29) -------------------------------------------------------------
typedef unsigned char uin8;
typedef unsigned short uin16;
typedef unsigned int uin32;
typedef unsigned long long uin64;
typedef uint4 uin128;

// ---- ceil-divide / round-up helpers (utility.h:33-45) -----------------------------------
#define TCBNN_STEP(X, LOG) (((X) + (1 << (LOG)) - 1) >> (LOG))
#define STEP4(X) TCBNN_STEP(X, 2)
#define STEP8(X) TCBNN_STEP(X, 3)
#define STEP16(X) TCBNN_STEP(X, 4)
#define STEP32(X) TCBNN_STEP(X, 5)
#define STEP64(X) TCBNN_STEP(X, 6)
#define STEP128(X) TCBNN_STEP(X, 7)
#define PAD4(X) (STEP4(X) << 2)
#define PAD8(X) (STEP8(X) << 3)
#define PAD16(X) (STEP16(X) << 4)
#define PAD32(X) (STEP32(X) << 5)
#define PAD64(X) (STEP64(X) << 6)
#define PAD128(X) (STEP128(X) << 7)

// lane / warp index of the calling thread (utility.h:47-49); the warp index is the one inside
// the block, which is what the layer loops need
#define GET_LANEID unsigned laneid = threadIdx.x & 31u;
#define GET_WARPID unsigned warpid = threadIdx.x >> 5;
#define FLIPBITS(n, b) ((n) ^ ((1u << (b)) - 1))

// ---- error handling: print and exit, like the reference (utility.h:57-101) -------------------
#define CUDA_SAFE_CALL(err) tcbnn_cuda_safe_call((err), __FILE__, __LINE__)
inline void tcbnn_cuda_safe_call(cudaError_t err, const char* file, int line) {
    if (err != cudaSuccess) {
        fprintf(stderr, "cudaSafeCall() failed at %s:%i : %s\n", file, line, cudaGetErrorString(err));
        exit(-1);
    }
}
#define CUDA_CHECK_KERNEL() tcbnn_cuda_check_kernel(__FILE__, __LINE__)
inline void tcbnn_cuda_check_kernel(const char* file, int line) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        fprintf(stderr, "cudaCheckError() failed at %s:%i : %s\n", file, line, cudaGetErrorString(err));
        exit(-1);
    }
}
#define CHECK_NULL_POINTER(X) tcbnn_check_null((const void*)(X), __FILE__, __LINE__)
inline void tcbnn_check_null(const void* p, const char* file, int line) {
    if (p == NULL) {
        fprintf(stderr, "Error: NULL pointer at %s:%i.\n", file, line);
        exit(-1);
    }
}
#define CHECK_NCCL(cmd)                                                                         \
    do {                                                                                        \
        ncclResult_t r_ = (cmd);                                                                \
        if (r_ != ncclSuccess) {                                                                \
            printf("NCCL error %s: %d '%s'\n", __FILE__, __LINE__, ncclGetErrorString(r_));     \
            exit(EXIT_FAILURE);                                                                 \
        }                                                                                       \
    } while (0)

// ---- allocation (utility.h:107-117) ----------------------------------------------------------
#define SAFE_ALOC_HOST(X, Y) CUDA_SAFE_CALL(cudaMallocHost((void**)&(X), (Y)));
#define SAFE_ALOC_GPU(X, Y) CUDA_SAFE_CALL(cudaMalloc((void**)&(X), (Y)));
#define SAFE_FREE_HOST(X) if ((X) != NULL) { CUDA_SAFE_CALL(cudaFreeHost((X))); (X) = NULL; }
#define SAFE_FREE_GPU(X) if ((X) != NULL) { CUDA_SAFE_CALL(cudaFree((X))); (X) = NULL; }

// ---- timers (utility.h:120-183) ---------------------------------------------------------------
inline double get_cpu_timer() {
    struct timeval tp;
    gettimeofday(&tp, NULL);
    return (double)tp.tv_sec * 1e3 + (double)tp.tv_usec * 1e-3;   // milliseconds
}
typedef struct CPU_Timer {
    CPU_Timer() : start(0.0), stop(0.0) {}
    void start_timer() { start = get_cpu_timer(); }
    void stop_timer() { stop = get_cpu_timer(); }
    double measure() { return stop - start; }
    double start, stop;
} cpu_timer;
typedef struct GPU_Timer {
    GPU_Timer() { CUDA_SAFE_CALL(cudaEventCreate(&start)); CUDA_SAFE_CALL(cudaEventCreate(&stop)); }
    void start_timer() { CUDA_SAFE_CALL(cudaEventRecord(start)); }
    void stop_timer() { CUDA_SAFE_CALL(cudaEventRecord(stop)); }
    double measure() {
        float ms = 0;
        CUDA_SAFE_CALL(cudaEventSynchronize(stop));
        CUDA_SAFE_CALL(cudaEventElapsedTime(&ms, start, stop));
        return (double)ms;
    }
    cudaEvent_t start, stop;
} gpu_timer;
// declare `start`, `stop`, `milliseconds` in the caller's scope, as the drivers expect
#define START_TIMER cudaEvent_t start, stop; cudaEventCreate(&start); cudaEventCreate(&stop); cudaEventRecord(start);
#define STOP_TIMER cudaEventRecord(stop); cudaEventSynchronize(stop); float milliseconds = 0; \
    cudaEventElapsedTime(&milliseconds, start, stop);
#define SET_KERNEL_TIMER uin64 t0 = clock64();
#define TICK_KERNEL_TIMER(X) if (threadIdx.x == 0 && blockIdx.x == 0) \
    printf("Layer-%s takes %lld cycles.\n", (X)->name, clock64() - t0);

// ---- weight file reader and prediction check (utility.h:188-232) ------------------------------
inline void launch_array(FILE* cf, float* array, unsigned array_size) {
    if (cf == NULL) {
        fprintf(stderr, "NULL pointer to the network configuration file.\n");
        exit(1);
    }
    for (unsigned i = 0; i < array_size; i++)
        if (fscanf(cf, "%f", &array[i]) != 1) {
            fprintf(stderr, "network configuration file ended after %u of %u values.\n", i, array_size);
            exit(1);
        }
}
inline void validate_prediction(float* prediction, unsigned* labels, const unsigned categories,
                                const unsigned batch) {
    int top1 = 0, top5 = 0;
    for (unsigned i = 0; i < batch; i++) {
        const float* p = prediction + (size_t)i * categories;
        unsigned better = 0;          // classes scoring above the labelled one
        unsigned arg = 0;
        for (unsigned j = 0; j < categories; j++) {
            if (p[j] > p[labels[i]]) better++;
            if (p[j] > p[arg]) arg = j;
        }
        if (arg == labels[i]) top1++;
        if (better < 5) top5++;
    }
    printf("\n=====Batch Accuracy:%u=======\n", batch);
    printf("Top-1:%f%%\n", float(top1) / batch * 100);
    printf("Top-5:%f%%\n", float(top5) / batch * 100);
}

// ---- vector stores (utility.h:236-246) --------------------------------------------------------
template <typename T>
__device__ __inline__ void store64(const void* addr, T a, T b) {
    *((float2*)addr) = make_float2(*(float*)(&a), *(float*)(&b));
}
template <typename T>
__device__ __inline__ void store128(const void* addr, T a, T b, T c, T d) {
    *((float4*)addr) = make_float4(*(float*)(&a), *(float*)(&b), *(float*)(&c), *(float*)(&d));
}

#endif
