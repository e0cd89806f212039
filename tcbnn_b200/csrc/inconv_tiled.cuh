// First layer on fp32 NCHW input (InConv128LayerFMT, kernel.cuh:578-672), block-tiled.
//
// Per in-frame tap the reference adds ((+-f0) + (+-f1)) + (+-f2) to each output channel's
// running fp32 sum, the three signs being that channel's filter bits for the tap
// (kernel.cuh:636-638).  For a given pixel and tap that term takes only 8 different values,
// one per sign pattern.  So a block of 32 pixels first tabulates T[tap][pattern][pixel] in
// shared memory (phase 1: lanes along pixels, warps along taps), then every thread -- one
// output channel, a slab of pixels in registers -- runs  acc[pixel] += T[tap][code][pixel]
// with 128-bit shared loads (phase 2: one load per four adds; rows are padded so that lanes
// with different codes hit different banks).  Same operands, same order, same roundings as
// the reference; out-of-frame taps are tabulated as +0.0, which leaves a sum unchanged.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "bnn_layers.cuh"

namespace tcbnn {

constexpr int kInconvThreads = 256;
constexpr int kInconvPixels = 32;      // pre-pool pixels per block iteration

constexpr int kInconvPitch = kInconvPixels + 4;   // floats per (tap, pattern) row, padded

__host__ __device__ inline size_t inconv_tiled_smem(int R, int S, int O) {
    const int opad = ((O + 31) / 32) * 32;
    return (size_t)R * S * 8 * kInconvPitch * 4 + (size_t)R * S * opad + (size_t)opad * 4 + 3 * 256 * 4;
}

template <int PPT>   // pixels per thread = kInconvPixels / (kInconvThreads / opad)
__device__ void inconv_tiled_block(const InConvArgs& c, unsigned char* smem) {
    const int RS = c.R * c.S;
    const int opad = ((c.O + 31) / 32) * 32;
    float* T = reinterpret_cast<float*>(smem);                                // [RS][8][pitch]
    unsigned char* codes = smem + (size_t)RS * 8 * kInconvPitch * 4;           // [RS][opad]
    float* sthr = reinterpret_cast<float*>(codes + (size_t)RS * opad);        // [opad]
    float* slut = sthr + opad;                                                // [3][256], uint8 input only
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
    if (c.x8)
        for (int i = tid; i < 3 * 256; i += kInconvThreads) slut[i] = __ldg(c.lut + i);

    const int group = tid / opad;            // which PPT-pixel slab of the block this thread owns
    const int o = tid % opad;
    const long long total = (long long)c.B * P * Q;       // pre-pool pixels
    const long long nblocks = (total + kInconvPixels - 1) / kInconvPixels;

    // pre-pool pixel index -> (image, row, column); with 2x2 pooling four consecutive indices
    // are the four positions of one pooling window.  32-bit arithmetic (the host checks that
    // the pixel count fits).
    auto locate = [&](unsigned pix, int& n, int& y, int& x) {
        if (c.pool == 2) {
            const unsigned pp = pix >> 2;
            const unsigned r = pp / (unsigned)c.OW;
            const int ox = (int)(pp - r * c.OW);
            n = (int)(r / (unsigned)c.OH);
            const int oy = (int)(r - (unsigned)n * c.OH);
            y = 2 * oy + ((int)(pix & 3) >> 1); x = 2 * ox + (int)(pix & 1);
        } else {
            const unsigned r = pix / (unsigned)Q;
            x = (int)(pix - r * Q);
            n = (int)(r / (unsigned)P);
            y = (int)(r - (unsigned)n * P);
        }
    };
    // next pixel index in the same order without dividing
    auto advance = [&](int k, int& n, int& y, int& x) {      // k = index being advanced TO
        if (c.pool == 2) {
            if ((k & 3) == 0) {                                // first position of the next window
                x = (x & ~1) + 2; y = y & ~1;
                if (x >= Q) { x = 0; y += 2; if (y >= P) { y = 0; n++; } }
            } else if ((k & 3) == 2) { x -= 1; y += 1; }
            else { x += 1; }
        } else {
            if (++x == Q) { x = 0; if (++y == P) { y = 0; n++; } }
        }
    };

    for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        __syncthreads();                      // previous iteration's readers are done with T
        // ---- phase 1: lane = pixel, warp strides over taps ------------------------------------
        {
            const long long pix = blk * kInconvPixels + lane;
            const bool live = pix < total;
            int n = 0, y = 0, x = 0;
            if (live) locate((unsigned)pix, n, y, x);
            const int y0 = y * c.sh - c.pad_h, x0 = x * c.sw - c.pad_w;
            const float* img = c.x + (size_t)n * 3 * plane;
            const unsigned char* img8 = c.x8 + (size_t)n * 3 * plane;
            for (int tap = warp; tap < RS; tap += kInconvThreads / 32) {
                const int ay = y0 + tap / c.S, ax = x0 + tap % c.S;
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = 0.0f;
                if (live && (unsigned)ay < (unsigned)c.H && (unsigned)ax < (unsigned)c.W) {
                    const size_t po = (size_t)ay * c.W + ax;
                    float f0, f1, f2;
                    if (c.x8) {      // the byte's fp32 value as the caller's reader would have computed it
                        f0 = slut[__ldg(img8 + po)];
                        f1 = slut[256 + __ldg(img8 + po + plane)];
                        f2 = slut[512 + __ldg(img8 + po + 2 * plane)];
                    } else {
                        f0 = __ldg(img + po); f1 = __ldg(img + po + plane); f2 = __ldg(img + po + 2 * plane);
                    }
                    const float pp_ = __fadd_rn(f0, f1), pm = __fadd_rn(f0, -f1);
                    const float mp = __fadd_rn(-f0, f1), mm = __fadd_rn(-f0, -f1);
                    // index = b0<<2 | b1<<1 | b2, bit 1 = '+'
                    v[0] = __fadd_rn(mm, -f2); v[1] = __fadd_rn(mm, f2);
                    v[2] = __fadd_rn(mp, -f2); v[3] = __fadd_rn(mp, f2);
                    v[4] = __fadd_rn(pm, -f2); v[5] = __fadd_rn(pm, f2);
                    v[6] = __fadd_rn(pp_, -f2); v[7] = __fadd_rn(pp_, f2);
                }
                float* dst = T + (size_t)tap * 8 * kInconvPitch + lane;
#pragma unroll
                for (int k = 0; k < 8; k++) dst[k * kInconvPitch] = v[k];
            }
        }
        __syncthreads();
        // ---- phase 2: one output channel per thread, PPT pixels in registers --------------------
        float acc[PPT];
#pragma unroll
        for (int k = 0; k < PPT; k++) acc[k] = 0.0f;
        const float* Tg = T + group * PPT;
        for (int tap = 0; tap < RS; tap++) {
            const float4* row = reinterpret_cast<const float4*>(
                Tg + (size_t)(tap * 8 + codes[tap * opad + o]) * kInconvPitch);
#pragma unroll
            for (int k = 0; k < PPT / 4; k++) {
                const float4 t = row[k];
                acc[4 * k] = __fadd_rn(acc[4 * k], t.x);
                acc[4 * k + 1] = __fadd_rn(acc[4 * k + 1], t.y);
                acc[4 * k + 2] = __fadd_rn(acc[4 * k + 2], t.z);
                acc[4 * k + 3] = __fadd_rn(acc[4 * k + 3], t.w);
            }
        }
        // ---- threshold, pool, pack, residual -------------------------------------------------
        const float th = sthr[o];
        uint32_t word = 0;
        int n = 0, y = 0, x = 0;
        {
            const long long pix0 = blk * kInconvPixels + group * PPT;
            if (pix0 < total) locate((unsigned)pix0, n, y, x);
        }
#pragma unroll
        for (int k = 0; k < PPT; k++) {
            const long long pix = blk * kInconvPixels + group * PPT + k;
            const bool live = pix < total;
            if (k > 0) advance(k, n, y, x);
            const bool bit = live && o < c.O && !(acc[k] < th);           // kernel.cuh:655
            const uint32_t w = __brev(__ballot_sync(0xffffffffu, bit));
            if (live && o < c.O) {
                const size_t opix = ((size_t)n * P + y) * Q + x;
                if (c.res_out) st_res(c.res_out, c.res_out_bytes, opix * c.res_out_ld + o, (int)acc[k]);  // kernel.cuh:666-668
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
