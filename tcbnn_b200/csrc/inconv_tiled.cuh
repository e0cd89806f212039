// First layer on fp32 NCHW input (InConv128LayerFMT, kernel.cuh:578-672), block-tiled.
//
// Per in-frame tap the reference adds ((+-f0) + (+-f1)) + (+-f2) to each output channel's
// running fp32 sum, the three signs being that channel's filter bits for the tap
// (kernel.cuh:636-638).  For a given pixel and tap that term takes only 8 different values,
// one per sign pattern.  So a block first tabulates T[pixel][tap][8] in shared memory
// (phase 1, 1/O of the work), then every thread -- one output channel, a few pixels in
// registers -- runs  acc += T[pixel][tap][code(tap, channel)]  (phase 2: one shared load and one
// add per term).  Same operands, same order, same roundings as the reference; out-of-frame
// taps are tabulated as +0.0, which leaves a sum unchanged.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "bnn_layers.cuh"

namespace tcbnn {

constexpr int kInconvThreads = 256;
constexpr int kInconvPixels = 32;      // pre-pool pixels per block iteration

__host__ __device__ inline size_t inconv_tiled_smem(int R, int S, int O) {
    const int opad = ((O + 31) / 32) * 32;
    return (size_t)kInconvPixels * R * S * 8 * 4 + (size_t)R * S * opad + (size_t)opad * 4;
}

template <int PPT>   // pixels per thread = kInconvPixels / (kInconvThreads / opad)
__device__ void inconv_tiled_block(const InConvArgs& c, unsigned char* smem) {
    const int RS = c.R * c.S;
    const int opad = ((c.O + 31) / 32) * 32;
    float* T = reinterpret_cast<float*>(smem);                               // [32][RS][8]
    unsigned char* codes = smem + (size_t)kInconvPixels * RS * 8 * 4;         // [RS][opad]
    float* sthr = reinterpret_cast<float*>(codes + (size_t)RS * opad);       // [opad]
    const int tid = threadIdx.x, lane = tid & 31;
    const int Ow = (c.O + 31) >> 5;
    const int P = c.pool * c.OH, Q = c.pool * c.OW;
    const size_t plane = (size_t)c.H * c.W;

    for (int i = tid; i < RS * opad; i += kInconvThreads) {
        const int tap = i / opad, o = i % opad;
        unsigned code = 0;
        if (o < c.O) {
            const uint32_t* fw = c.fbits + (size_t)tap * 3 * Ow + (o >> 5);
            const int sh = 31 - (o & 31);
            code = (((__ldg(fw) >> sh) & 1u) << 2) | (((__ldg(fw + Ow) >> sh) & 1u) << 1) |
                   ((__ldg(fw + 2 * Ow) >> sh) & 1u);
        }
        codes[i] = (unsigned char)code;
    }
    for (int i = tid; i < opad; i += kInconvThreads) sthr[i] = i < c.O ? __ldg(c.thr + i) : 0.0f;

    const int group = tid / opad;            // which PPT-pixel slice of the block this thread owns
    const int o = tid % opad;
    const long long total = (long long)c.B * P * Q;       // pre-pool pixels
    const long long nblocks = (total + kInconvPixels - 1) / kInconvPixels;

    for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        __syncthreads();                      // previous iteration's readers are done with T
        // ---- phase 1: tabulate the 8 sign patterns per (pixel, tap) ---------------------------
        for (int i = tid; i < kInconvPixels * RS; i += kInconvThreads) {
            const int pb = i / RS, tap = i - pb * RS;
            const long long pix = blk * kInconvPixels + pb;
            float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
            if (pix < total) {
                int n, y, x;
                if (c.pool == 2) {
                    const long long pp = pix >> 2;
                    const int ox = (int)(pp % c.OW); const long long r = pp / c.OW;
                    const int oy = (int)(r % c.OH); n = (int)(r / c.OH);
                    y = 2 * oy + ((int)(pix & 3) >> 1); x = 2 * ox + (int)(pix & 1);
                } else {
                    x = (int)(pix % Q); const long long r = pix / Q;
                    y = (int)(r % P); n = (int)(r / P);
                }
                const int ay = y * c.sh - c.pad_h + tap / c.S, ax = x * c.sw - c.pad_w + tap % c.S;
                if ((unsigned)ay < (unsigned)c.H && (unsigned)ax < (unsigned)c.W) {
                    const float* px = c.x + (size_t)n * 3 * plane + (size_t)ay * c.W + ax;
                    const float f0 = __ldg(px), f1 = __ldg(px + plane), f2 = __ldg(px + 2 * plane);
                    const float pp_ = __fadd_rn(f0, f1), pm = __fadd_rn(f0, -f1);
                    const float mp = __fadd_rn(-f0, f1), mm = __fadd_rn(-f0, -f1);
                    // index = b0<<2 | b1<<1 | b2, bit 1 = '+'
                    lo = make_float4(__fadd_rn(mm, -f2), __fadd_rn(mm, f2), __fadd_rn(mp, -f2),
                                     __fadd_rn(mp, f2));
                    hi = make_float4(__fadd_rn(pm, -f2), __fadd_rn(pm, f2), __fadd_rn(pp_, -f2),
                                     __fadd_rn(pp_, f2));
                }
            }
            float4* dst = reinterpret_cast<float4*>(T + (size_t)i * 8);
            dst[0] = lo;
            dst[1] = hi;
        }
        __syncthreads();
        // ---- phase 2: one output channel per thread, PPT pixels in registers --------------------
        float acc[PPT];
#pragma unroll
        for (int k = 0; k < PPT; k++) acc[k] = 0.0f;
        const float* Tg = T + (size_t)group * PPT * RS * 8;
        for (int tap = 0; tap < RS; tap++) {
            const float* Tt = Tg + tap * 8 + codes[tap * opad + o];
#pragma unroll
            for (int k = 0; k < PPT; k++) acc[k] = __fadd_rn(acc[k], Tt[(size_t)k * RS * 8]);
        }
        // ---- threshold, pool, pack, residual -------------------------------------------------
        const float th = sthr[o];
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < PPT; k++) {
            const long long pix = blk * kInconvPixels + group * PPT + k;
            const bool live = pix < total;
            int n = 0, y = 0, x = 0;
            if (live) {
                if (c.pool == 2) {
                    const long long pp = pix >> 2;
                    const int ox = (int)(pp % c.OW); const long long r = pp / c.OW;
                    const int oy = (int)(r % c.OH); n = (int)(r / c.OH);
                    y = 2 * oy + ((int)(pix & 3) >> 1); x = 2 * ox + (int)(pix & 1);
                } else {
                    x = (int)(pix % Q); const long long r = pix / Q;
                    y = (int)(r % P); n = (int)(r / P);
                }
            }
            const bool bit = live && o < c.O && !(acc[k] < th);           // kernel.cuh:655
            const uint32_t w = __brev(__ballot_sync(0xffffffffu, bit));
            if (live && o < c.O) {
                const size_t opix = ((size_t)n * P + y) * Q + x;
                if (c.res_out) st_res(c.res_out, c.res_out_bytes, opix * c.O + o, (int)acc[k]);  // kernel.cuh:666-668
                if (c.acc_out) c.acc_out[opix * c.O + o] = acc[k];
            }
            if (c.pool == 2) {
                word |= w;
                if ((k & 3) == 3) {
                    if (live && lane == 0)
                        c.out[(size_t)n * c.out_image_stride +
                              ((size_t)(y >> 1) * c.OW + (x >> 1)) * Ow + (o >> 5)] = word;
                    word = 0;
                }
            } else if (live && lane == 0) {
                c.out[(size_t)n * c.out_image_stride + ((size_t)y * c.OW + x) * Ow + (o >> 5)] = w;
            }
        }
    }
}

}  // namespace tcbnn
