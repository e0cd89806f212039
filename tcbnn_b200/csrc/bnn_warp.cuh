// Warp-level building blocks of the binarised-network layers: the 1-bit tensor-core MMA
// wrapper, fragment conventions and small bit helpers.  Everything here is warp-scoped (no
// block barriers), so the layer loops built on it run unchanged inside any grid: a plain
// launch of the library's own kernels, or a caller's persistent cooperative kernel.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tcbnn {

// mma.sync m16n8k256 on 1-bit operands, AND + popcount, int32 accumulate.
// Fragment ownership (lane = 4*g + t):
//   a0: row g,   k-slice t of the first 128 bits     a1: row g+8, same slice
//   a2: row g,   k-slice t of the second 128 bits    a3: row g+8, same slice
//   b0: col g,   k-slice t of the first 128 bits     b1: col g,   second 128 bits
//   c0: (g, 2t)  c1: (g, 2t+1)  c2: (g+8, 2t)  c3: (g+8, 2t+1)
// A popcount does not care which physical word feeds which slice as long as both operands
// agree, so callers feed a0/a2 (and b0/b1) from one 64-bit load of two adjacent words.
__device__ __forceinline__ void mma_b1_and(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                           uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ldg64(const uint32_t* p) {
    return __ldg(reinterpret_cast<const uint2*>(p));
}

__device__ __forceinline__ int quad_sum(int v) {   // sum over the 4 lanes sharing g
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}
__device__ __forceinline__ uint32_t quad_or(uint32_t v) {
    v |= __shfl_xor_sync(0xffffffffu, v, 1);
    v |= __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// Global warp index / warp count of the running grid (1-D grid, 1-D block).
__device__ __forceinline__ int grid_warp() { return blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); }
__device__ __forceinline__ int grid_warps() { return gridDim.x * (blockDim.x >> 5); }

}  // namespace tcbnn
