// Layer loops of the binarised-network hot path on the warp-level 1-bit MMA.
//
// Each layer is a __device__ function that strides over warp-sized tasks with the warps of
// whatever grid is running (tasks w, w + grid_warps(), ...).  No block-wide barriers and
// no shared memory are used, so the same code serves the library's own launches and a
// caller's cooperative kernel that runs the layers back to back with grid.sync() between
// them (the way the reference drivers do, imagenet_resnet.cu:56-124).
//
// Arithmetic.  The reference computes popc(a XOR w) on Turing's XOR bit-MMA
// (kernel.cuh:201, 737-749).  On sm_100a the AND form is the faster instruction, so
//   popc(a ^ w) = popc(a) + popc(w) - 2*popc(a & w)
// with popc(a) accumulated from the A fragments on the fly and popc(w) either accumulated
// the same way (GEMM) or read from per-tap tables built when the filter is prepared (conv).
// Out-of-frame conv taps load zeros, so they drop out of all three terms, which is exactly
// the reference's "exclude" rule (kernel.cuh:726, 752-755, 766-768).
#pragma once
#include "bnn_warp.cuh"
#include <climits>

namespace tcbnn {

// Residual tensors are int32 or int16 (element size chosen by the caller, who knows the
// bound of the running shortcut sum); the arithmetic is int32 either way.
__device__ __forceinline__ int ld_res(const void* p, int bytes, size_t i) {
    return bytes == 2 ? (int)__ldg(reinterpret_cast<const short*>(p) + i)
                      : __ldg(reinterpret_cast<const int*>(p) + i);
}
__device__ __forceinline__ void st_res(void* p, int bytes, size_t i, int v) {
    if (bytes == 2) reinterpret_cast<short*>(p)[i] = (short)v;
    else reinterpret_cast<int*>(p)[i] = v;
}

// ----------------------------------------------------------------------------------------
// Bit GEMM family: standalone int32 GEMM (bmm/tensorcore_kernel.cu:138-356), hidden FC
// layer (Fc128LayerFMT, kernel.cuh:174-226) and output layer (Out128LayerFMT, :230-280).
// ----------------------------------------------------------------------------------------
enum GemmMode { GEMM_INT32 = 0, GEMM_FC_BITS = 1, GEMM_OUT_AFFINE = 2, GEMM_PARTIAL = 3 };

struct GemmArgs {
    const uint32_t* A;    // [M][lda] words, bits along K, pad bits 0
    const uint32_t* W;    // [N][ldw] words
    int M, N, K;
    int lda, ldw;         // words, even
    int mode;
    void* out;            // int32 [M][ldo] | bit words [M][ldo] | float [M][ldo]
    int ldo;
    const float* p0;      // thresholds (FC) or scale (OUT)
    const float* p1;      // bias (OUT)
    int splits;           // >1: split K, partial sums go to `partial`
    int32_t* partial;     // [splits][M][N] raw (-2*popc(a) - 2*popc(w) + 4*popc(a&w)) sums
};

// One warp computes a 32 x 32 tile: 2 m-tiles x 4 n-tiles of m16n8k256.
__device__ __forceinline__ void gemm_warp_tile(const GemmArgs& g, int tm, int tn, int split) {
    const int lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
    const int m0 = tm * 32, n0 = tn * 32;
    const int KP = (g.K + 63) >> 6;                     // 64-bit pairs per row
    const int per = ((KP + g.splits - 1) / g.splits + 3) & ~3;
    const int kp0 = split * per;
    const int kp1 = min(KP, kp0 + per);

    int aoff[4], woff[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        aoff[i] = min(m0 + i * 8 + gq, g.M - 1) * g.lda;   // rows past M re-read row M-1
        woff[i] = min(n0 + i * 8 + gq, g.N - 1) * g.ldw;
    }
    int acc[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[a][b][c] = 0;
    int sa[4] = {0, 0, 0, 0}, pw[4] = {0, 0, 0, 0};

    for (int kb = kp0; kb < kp1; kb += 4) {
        const int kp = kb + t;
        const bool ok = kp < kp1;
        uint2 a[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            a[i] = ok ? ldg64(g.A + aoff[i] + 2 * kp) : make_uint2(0u, 0u);
            sa[i] += __popc(a[i].x) + __popc(a[i].y);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint2 b = ok ? ldg64(g.W + woff[j] + 2 * kp) : make_uint2(0u, 0u);
            pw[j] += __popc(b.x) + __popc(b.y);
            mma_b1_and(acc[0][j], a[0].x, a[1].x, a[0].y, a[1].y, b.x, b.y);
            mma_b1_and(acc[1][j], a[2].x, a[3].x, a[2].y, a[3].y, b.x, b.y);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) { sa[i] = quad_sum(sa[i]); pw[i] = quad_sum(pw[i]); }

    // rows held by this thread: i = 2*mt + h -> row m0 + mt*16 + h*8 + gq (= m0 + i*8 + gq)
    // cols held: n0 + j*8 + 2t + e
    uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int pw0 = __shfl_sync(0xffffffffu, pw[j], (2 * t) * 4);
        const int pw1 = __shfl_sync(0xffffffffu, pw[j], (2 * t + 1) * 4);
        const int col = n0 + j * 8 + 2 * t;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int row = m0 + i * 8 + gq;
            const int mt = i >> 1, h = i & 1;
            int v0 = 4 * acc[mt][j][2 * h] - 2 * sa[i] - 2 * pw0;       // = -2*popc(a^w) part
            int v1 = 4 * acc[mt][j][2 * h + 1] - 2 * sa[i] - 2 * pw1;
            if (g.mode == GEMM_PARTIAL) {
                if (row < g.M) {
                    int32_t* p = g.partial + ((size_t)split * g.M + row) * g.N + col;
                    if (col < g.N) p[0] = v0;
                    if (col + 1 < g.N) p[1] = v1;
                }
            } else if (g.mode == GEMM_INT32) {
                if (row < g.M) {
                    int32_t* p = (int32_t*)g.out + (size_t)row * g.ldo + col;
                    if (col < g.N) p[0] = g.K + v0;
                    if (col + 1 < g.N) p[1] = g.K + v1;
                }
            } else if (g.mode == GEMM_FC_BITS) {
                // (float)K - 2*(float)c >= thr[n]  (kernel.cuh:210-213); K + v is that value
                if (col < g.N && (float)(g.K + v0) >= __ldg(g.p0 + col))
                    words[i] |= 0x80000000u >> (j * 8 + 2 * t);
                if (col + 1 < g.N && (float)(g.K + v1) >= __ldg(g.p0 + col + 1))
                    words[i] |= 0x80000000u >> (j * 8 + 2 * t + 1);
            } else {  // GEMM_OUT_AFFINE  (kernel.cuh:270-273), fused multiply-add
                if (row < g.M) {
                    float* p = (float*)g.out + (size_t)row * g.ldo + col;
                    if (col < g.N)
                        p[0] = __fmaf_rn((float)(g.K + v0), __ldg(g.p0 + col), __ldg(g.p1 + col));
                    if (col + 1 < g.N)
                        p[1] = __fmaf_rn((float)(g.K + v1), __ldg(g.p0 + col + 1),
                                         __ldg(g.p1 + col + 1));
                }
            }
        }
    }
    if (g.mode == GEMM_FC_BITS) {
#pragma unroll
        for (int i = 0; i < 4; i++) words[i] = quad_or(words[i]);
        // lane t of each quad stores the word of row i == t
        const uint32_t w = t == 0 ? words[0] : t == 1 ? words[1] : t == 2 ? words[2] : words[3];
        const int row = m0 + t * 8 + gq;
        if (row < g.M) ((uint32_t*)g.out)[(size_t)row * g.ldo + tn] = w;
    }
}

__device__ __forceinline__ void gemm_layer(const GemmArgs& g) {
    const int TM = (g.M + 31) >> 5, TN = (g.N + 31) >> 5;
    const int total = TM * TN * g.splits;
    for (int task = grid_warp(); task < total; task += grid_warps()) {
        const int split = task / (TM * TN);
        const int rem = task - split * (TM * TN);
        gemm_warp_tile(g, rem / TN, rem % TN, split);
    }
}

// Second pass of a split-K GEMM: add the partial slices and apply the epilogue.
// One thread per (row, 32-column word).
__device__ __forceinline__ void gemm_splitk_finish(const GemmArgs& g) {
    const int lane = threadIdx.x & 31;
    const int TN = (g.N + 31) >> 5;
    const int total = g.M * TN;
    for (int task = grid_warp(); task < total; task += grid_warps()) {
        const int row = task / TN, tn = task % TN;
        const int col = tn * 32 + lane;
        int v = 0;
        if (col < g.N)
            for (int s = 0; s < g.splits; s++)
                v += g.partial[((size_t)s * g.M + row) * g.N + col];
        v += g.K;
        if (g.mode == GEMM_INT32) {
            if (col < g.N) ((int32_t*)g.out)[(size_t)row * g.ldo + col] = v;
        } else if (g.mode == GEMM_FC_BITS) {
            const bool bit = col < g.N && (float)v >= __ldg(g.p0 + col);
            const uint32_t w = __brev(__ballot_sync(0xffffffffu, bit));
            if (lane == 0) ((uint32_t*)g.out)[(size_t)row * g.ldo + tn] = w;
        } else {
            if (col < g.N)
                ((float*)g.out)[(size_t)row * g.ldo + col] =
                    __fmaf_rn((float)v, __ldg(g.p0 + col), __ldg(g.p1 + col));
        }
    }
}

// ----------------------------------------------------------------------------------------
// Binary convolution layer (Conv128LayerFMT, kernel.cuh:676-827) as an implicit GEMM:
// rows = output pixels, columns = output channels, K = taps x input channels.
// ----------------------------------------------------------------------------------------
struct ConvArgs {
    const uint32_t* in;      // [B][H][W][Cw] words
    const uint32_t* wq;      // [O][2*KP] words: per tap Cw words (Cw even), zero tail
    const uint32_t* ktab;    // [KP] per 64-bit pair: r<<28 | s<<24 | word offset from window origin
    const int* pwt;          // [R*S][O]  popc of filter o at tap
    const int* pwtot;        // [O]       popc of filter o over all taps
    const float* thr;        // [O]
    int B, H, W, C, Cw, O, R, S, sh, sw, pad_h, pad_w, pool, OH, OW, KP;
    const void* res_in;      // [B][P or 2P][Q or 2Q][res_in_ch] or null
    int res_in_bytes;        // 4 (int32) or 2 (int16)
    int res_in_ch, residual_channels, residual_pool;
    uint32_t* out;           // per image [OH][OW][Ow] words at stride out_image_stride
    long long out_image_stride;
    void* res_out;           // [B][P][Q][res_out_ld] or null
    int res_out_bytes;
    int res_out_ld;          // channel stride of res_out (O, or a padded width)
    int32_t* acc_out;        // [B][P][Q][O] or null (value before residual injection)
};

// One warp: 32 pre-pool pixels x 32 output channels.  With 2x2 pooling the four rows a
// thread owns (i = 0..3 -> rows i*8+g) are the four positions of ONE pooling window, so
// the OR-pool is thread-local and the pooled word is written with a plain store (the
// reference ORs into a zeroed buffer with atomicOr, kernel.cuh:806-815).
__device__ __forceinline__ void conv_warp_tile(const ConvArgs& c, int tp, int tn) {
    const int lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
    const int P = c.pool * c.OH, Q = c.pool * c.OW;
    const int n0 = tn * 32;

    int base[4];            // word offset of the window origin pixel (may be "negative")
    uint32_t pm[4];         // invalid-row mask (bits 0..15) | invalid-col mask (bits 16..31)
    int pb[4], py[4], px[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int b, y, x;
        bool live;
        if (c.pool == 2) {
            long long pp = (long long)tp * 8 + gq;          // pooled pixel
            live = pp < (long long)c.B * c.OH * c.OW;
            int ox = (int)(pp % c.OW); long long r = pp / c.OW;
            int oy = (int)(r % c.OH); b = (int)(r / c.OH);
            y = 2 * oy + (i >> 1); x = 2 * ox + (i & 1);
        } else {
            const long long pix = (long long)tp * 32 + i * 8 + gq;
            live = pix < (long long)c.B * P * Q;
            x = (int)(pix % Q); long long r = pix / Q;
            y = (int)(r % P); b = (int)(r / P);
        }
        const int y0 = y * c.sh - c.pad_h, x0 = x * c.sw - c.pad_w;
        uint32_t m = 0;
        for (int r = 0; r < c.R; r++) if ((unsigned)(y0 + r) >= (unsigned)c.H) m |= 1u << r;
        for (int s = 0; s < c.S; s++) if ((unsigned)(x0 + s) >= (unsigned)c.W) m |= 0x10000u << s;
        m |= 0x8000u;                                     // row 15 marks padding pairs
        if (!live) { m = 0xffffffffu; b = 0; y = 0; x = 0; }
        pm[i] = m; pb[i] = live ? b : -1; py[i] = y; px[i] = x;
        base[i] = live ? ((b * c.H + y0) * c.W + x0) * c.Cw : 0;
    }
    int woff[4];
#pragma unroll
    for (int j = 0; j < 4; j++) woff[j] = min(n0 + j * 8 + gq, c.O - 1) * (2 * c.KP);

    int acc[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int d = 0; d < 4; d++) acc[a][b][d] = 0;
    int sa[4] = {0, 0, 0, 0};

    for (int kb = 0; kb < c.KP; kb += 4) {
        const int kp = kb + t;
        const uint32_t e = __ldg(c.ktab + kp);
        const int r = e >> 28, s = (e >> 24) & 15, off = e & 0xffffff;
        uint2 a[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const bool bad = ((pm[i] >> r) | (pm[i] >> (16 + s))) & 1u;
            a[i] = bad ? make_uint2(0u, 0u) : ldg64(c.in + (base[i] + off));
            sa[i] += __popc(a[i].x) + __popc(a[i].y);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint2 b = ldg64(c.wq + woff[j] + 2 * kp);
            mma_b1_and(acc[0][j], a[0].x, a[1].x, a[0].y, a[1].y, b.x, b.y);
            mma_b1_and(acc[1][j], a[2].x, a[3].x, a[2].y, a[3].y, b.x, b.y);
        }
    }

    uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        sa[i] = quad_sum(sa[i]);
        if (pb[i] < 0) continue;
        const int mt = i >> 1, h = i & 1;
        const uint32_t rinv = pm[i] & ((1u << c.R) - 1u), sinv = (pm[i] >> 16) & ((1u << c.S) - 1u);
        const int kvalid = c.C * (c.R - __popc(rinv)) * (c.S - __popc(sinv));
        const size_t opix = ((size_t)pb[i] * P + py[i]) * Q + px[i];
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int o = n0 + j * 8 + 2 * t + e;
                if (o >= c.O) continue;
                int pwv = __ldg(c.pwtot + o);
                if (rinv | sinv)
                    for (int r = 0; r < c.R; r++)
                        for (int s = 0; s < c.S; s++)
                            if (((rinv >> r) | (sinv >> s)) & 1u)
                                pwv -= __ldg(c.pwt + (r * c.S + s) * c.O + o);
                // C*R*S - exclude*C - 2*popc(a^w) over in-frame taps (kernel.cuh:766-768)
                int res = kvalid - 2 * sa[i] - 2 * pwv + 4 * acc[mt][j][2 * h + e];
                if (c.acc_out) c.acc_out[opix * c.O + o] = res;
                if (c.res_in && o < c.residual_channels) {       // kernel.cuh:770-794
                    int residual = 0;
                    if (o < c.res_in_ch) {
                        if (c.residual_pool) {
                            residual = INT_MIN;
                            for (int u = 0; u < 2; u++)
                                for (int v = 0; v < 2; v++)
                                    residual = max(residual, ld_res(c.res_in, c.res_in_bytes,
                                        (((size_t)pb[i] * 2 * P + (2 * py[i] + u)) * 2 * Q +
                                         (2 * px[i] + v)) * c.res_in_ch + o));
                        } else {
                            residual = ld_res(c.res_in, c.res_in_bytes, opix * c.res_in_ch + o);
                        }
                    }
                    res += residual;
                }
                if (!((float)res < __ldg(c.thr + o)))            // kernel.cuh:795-796
                    words[c.pool == 2 ? 0 : i] |= 0x80000000u >> (j * 8 + 2 * t + e);
                if (c.res_out) st_res(c.res_out, c.res_out_bytes, opix * c.res_out_ld + o, res);  // kernel.cuh:818-824
            }
        }
    }
    const int Ow = (c.O + 31) >> 5;
    if (c.pool == 2) {
        const uint32_t w = quad_or(words[0]);
        if (t == 0 && pb[0] >= 0)
            c.out[(size_t)pb[0] * c.out_image_stride +
                  ((size_t)(py[0] >> 1) * c.OW + (px[0] >> 1)) * Ow + tn] = w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) words[i] = quad_or(words[i]);
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (t == i && pb[i] >= 0)
                c.out[(size_t)pb[i] * c.out_image_stride +
                      ((size_t)py[i] * c.OW + px[i]) * Ow + tn] = words[i];
    }
}

__device__ __forceinline__ void conv_layer(const ConvArgs& c) {
    const long long rows = c.pool == 2 ? (long long)c.B * c.OH * c.OW * 4
                                       : (long long)c.B * c.OH * c.OW;
    const int TP = (int)((rows + 31) / 32);
    const int TN = (c.O + 31) >> 5;
    const long long total = (long long)TP * TN;
    for (long long task = grid_warp(); task < total; task += grid_warps())
        conv_warp_tile(c, (int)(task / TN), (int)(task % TN));
}

// ----------------------------------------------------------------------------------------
// First layer on fp32 NCHW input (InConv128LayerFMT, kernel.cuh:578-672).
// One warp per (pooled) output pixel, lane = output channel within a group of 32.
// ----------------------------------------------------------------------------------------
struct InConvArgs {
    const float* x;          // [B][3][H][W]
    const unsigned char* x8; // alternative input: uint8 [B][3][H][W] (x is null) ...
    const float* lut;        // ... with the fp32 value of every byte per channel, [3][256]
    const uint32_t* fbits;   // [R*S][3][Ow] words, out-channel o at bit 31-o%32 (param.h:613-632)
    const float* thr;        // [O]
    int B, H, W, O, R, S, sh, sw, pad_h, pad_w, pool, OH, OW;
    uint32_t* out;
    long long out_image_stride;
    void* res_out;           // [B][P][Q][res_out_ld], (int)acc truncation (kernel.cuh:666-668)
    int res_out_bytes;       // 4 or 2
    int res_out_ld;          // channel stride of res_out (O, or a padded width)
    float* acc_out;          // optional fp32 accumulators
};

template <int OG>   // OG = ceil(O/32) groups held in registers
__device__ __forceinline__ void inconv_warp_pixel(const InConvArgs& c, long long task) {
    const int lane = threadIdx.x & 31;
    const int P = c.pool * c.OH, Q = c.pool * c.OW;
    const int ox = (int)(task % c.OW); long long r0 = task / c.OW;
    const int oy = (int)(r0 % c.OH); const int b = (int)(r0 / c.OH);
    const size_t plane = (size_t)c.H * c.W;
    const float* xb = c.x + (size_t)b * 3 * plane;
    uint32_t words[OG];
#pragma unroll
    for (int k = 0; k < OG; k++) words[k] = 0u;
    for (int wy = 0; wy < c.pool; wy++)
        for (int wx = 0; wx < c.pool; wx++) {
            const int y = oy * c.pool + wy, x = ox * c.pool + wx;
            const int y0 = y * c.sh - c.pad_h, x0 = x * c.sw - c.pad_w;
            float acc[OG];
#pragma unroll
            for (int k = 0; k < OG; k++) acc[k] = 0.0f;
            for (int r = 0; r < c.R; r++) {
                const int ay = y0 + r;
                if ((unsigned)ay >= (unsigned)c.H) continue;
                for (int s = 0; s < c.S; s++) {
                    const int ax = x0 + s;
                    if ((unsigned)ax >= (unsigned)c.W) continue;
                    const float f0 = __ldg(xb + (size_t)ay * c.W + ax);
                    const float f1 = __ldg(xb + plane + (size_t)ay * c.W + ax);
                    const float f2 = __ldg(xb + 2 * plane + (size_t)ay * c.W + ax);
                    const uint32_t* fw = c.fbits + (size_t)(r * c.S + s) * 3 * OG;
#pragma unroll
                    for (int k = 0; k < OG; k++) {
                        const uint32_t l0 = __ldg(fw + k), l1 = __ldg(fw + OG + k),
                                       l2 = __ldg(fw + 2 * OG + k);
                        // ((+-f0) + (+-f1)) + (+-f2), then added to the running sum
                        // (kernel.cuh:636-638); plain adds, nothing to contract.
                        const float t0 = ((l0 >> (31 - lane)) & 1u) ? f0 : -f0;
                        const float t1 = ((l1 >> (31 - lane)) & 1u) ? f1 : -f1;
                        const float t2 = ((l2 >> (31 - lane)) & 1u) ? f2 : -f2;
                        acc[k] = __fadd_rn(acc[k], __fadd_rn(__fadd_rn(t0, t1), t2));
                    }
                }
            }
            const size_t opix = ((size_t)b * P + y) * Q + x;
#pragma unroll
            for (int k = 0; k < OG; k++) {
                const int o = k * 32 + lane;
                const bool bit = o < c.O && !(acc[k] < __ldg(c.thr + min(o, c.O - 1)));
                words[k] |= __brev(__ballot_sync(0xffffffffu, bit));
                if (o < c.O) {
                    if (c.res_out) st_res(c.res_out, c.res_out_bytes, opix * c.res_out_ld + o, (int)acc[k]);
                    if (c.acc_out) c.acc_out[opix * c.O + o] = acc[k];
                }
            }
        }
    if (lane == 0) {
        uint32_t* o = c.out + (size_t)b * c.out_image_stride + ((size_t)oy * c.OW + ox) * OG;
#pragma unroll
        for (int k = 0; k < OG; k++) o[k] = words[k];
    }
}

__device__ __forceinline__ void inconv_layer(const InConvArgs& c) {
    const long long total = (long long)c.B * c.OH * c.OW;
    const int og = (c.O + 31) >> 5;
    for (long long task = grid_warp(); task < total; task += grid_warps()) {
        switch (og) {
            case 1: inconv_warp_pixel<1>(c, task); break;
            case 2: inconv_warp_pixel<2>(c, task); break;
            case 3: inconv_warp_pixel<3>(c, task); break;
            case 4: inconv_warp_pixel<4>(c, task); break;
            default: break;   // rejected on the host
        }
    }
}

// ----------------------------------------------------------------------------------------
// Packers.
// ----------------------------------------------------------------------------------------
// fp32 rows -> bit rows, bit = (x >= 0)  (In128LayerFMT, kernel.cuh:153-172).
// One warp per (row, 128-column block): four coalesced 128-byte reads, four ballots, one
// 16-byte store.
__device__ __forceinline__ void pack_rows(const float* x, int rows, int cols, int ld_words,
                                          uint32_t* out) {
    const int lane = threadIdx.x & 31;
    const int blocks = ld_words >> 2;                       // ld_words is a multiple of 4
    const long long total = (long long)rows * blocks;
    for (long long task = grid_warp(); task < total; task += grid_warps()) {
        const int row = (int)(task / blocks), blk = (int)(task % blocks);
        const float* xr = x + (size_t)row * cols;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int col = blk * 128 + i * 32 + lane;
            const float f = col < cols ? __ldg(xr + col) : -1.0f;
            w[i] = __brev(__ballot_sync(0xffffffffu, f >= 0));
        }
        if (lane == 0)
            *reinterpret_cast<uint4*>(out + (size_t)row * ld_words + blk * 4) =
                make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// bit i of the low byte of b -> bit 4 * i
__device__ __forceinline__ uint32_t spread4(uint32_t b) {
    uint32_t x = b & 0xFFu;
    x = (x | (x << 12)) & 0x000F000Fu;
    x = (x | (x << 6)) & 0x03030303u;
    x = (x | (x << 3)) & 0x11111111u;
    return x;
}

// The same packing for rows whose length is a multiple of 4 floats on a 16-byte aligned base: a
// lane reads 16 bytes (four consecutive columns), a warp one 128-column block per load, and a
// task is eight consecutive blocks of one row, all eight loads (4 KB) issued before the first is
// used -- with 64 warps per SM that keeps up to 256 KB in flight.  Four ballots give one bit per
// (lane, component); lane L interleaves eight lanes' four bits into word L & 3 of block L >> 2.
// rows * ceil(blocks / 8) must fit in 31 bits (the caller checks).
__device__ __forceinline__ void pack_rows_vec(const float* x, int rows, int cols, int ld_words,
                                              uint32_t* out) {
    constexpr int U = 8;
    const int lane = threadIdx.x & 31;
    const unsigned blocks = (unsigned)ld_words >> 2, chunks = (blocks + U - 1) / U;
    const unsigned total = (unsigned)rows * chunks, step = (unsigned)grid_warps();
    for (unsigned task = (unsigned)grid_warp(); task < total; task += step) {
        const unsigned row = task / chunks, blk0 = (task - row * chunks) * U;
        const float* xr = x + (size_t)row * cols;
        float4 f[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int col = (int)(blk0 + u) * 128 + 4 * lane;
            f[u] = col < cols ? __ldg(reinterpret_cast<const float4*>(xr + col)) : make_float4(-1.0f, -1.0f, -1.0f, -1.0f);
        }
        // lane L produces word L & 3 of block L >> 2: it keeps that block's four ballots
        uint32_t m0 = 0, m1 = 0, m2 = 0, m3 = 0;
        const int myu = lane >> 2;
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t b0 = __ballot_sync(0xffffffffu, f[u].x >= 0), b1 = __ballot_sync(0xffffffffu, f[u].y >= 0);
            const uint32_t b2 = __ballot_sync(0xffffffffu, f[u].z >= 0), b3 = __ballot_sync(0xffffffffu, f[u].w >= 0);
            if (myu == u) { m0 = b0; m1 = b1; m2 = b2; m3 = b3; }
        }
        const int sh = 8 * (lane & 3);
        const uint32_t v = spread4(m0 >> sh) | (spread4(m1 >> sh) << 1) | (spread4(m2 >> sh) << 2) |
                           (spread4(m3 >> sh) << 3);           // column k of the word at bit k
        if (blk0 + myu < blocks) out[(size_t)row * ld_words + blk0 * 4 + lane] = __brev(v);   // 128 contiguous bytes
    }
}

// bit rows -> +-1 floats (UnPackFcOutput128FMT, param.h:87-104).
__device__ __forceinline__ void unpack_rows(const uint32_t* in, int rows, int cols, int ld_words,
                                            float* out) {
    const long long total = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / cols), col = (int)(i % cols);
        const uint32_t w = __ldg(in + (size_t)r * ld_words + (col >> 5));
        out[i] = 2 * (float)((w >> (31 - (col & 31))) & 1u) - 1;
    }
}

// fp32 src[inner][outer-major..] -> bit rows: generic "transpose and binarise".
// dst[o][wd] bit (31-i) = src[(base(wd) + i) * stride + o] >= 0, i < count(wd).
// Used for FC weights W[K][N] -> [N][ld] (PackFcWeight128FMT, param.h:44-63) and conv
// filters F[R*S][C][O] -> [O][R*S][Cw] (PackFiltersByInChannels128FMT, param.h:560-581).
// Threads run along o, so the fp32 reads are coalesced.
__device__ __forceinline__ void pack_fc_weight(const float* W, int K, int N, int ld_words,
                                               uint32_t* out) {
    const long long total = (long long)N * ld_words;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i % N), wd = (int)(i / N);
        uint32_t w = 0;
        for (int b = 0; b < 32; b++) {
            const int k = wd * 32 + b;
            if (k < K && __ldg(W + (size_t)k * N + n) >= 0) w |= 0x80000000u >> b;
        }
        out[(size_t)n * ld_words + wd] = w;
    }
}

__device__ __forceinline__ void pack_conv_filter(const float* F, int RS, int C, int O,
                                                 uint32_t* out) {
    const int Cw = (C + 31) >> 5;
    const long long total = (long long)O * RS * Cw;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int o = (int)(i % O);
        const int wd = (int)(i / O);           // tap*Cw + cw
        const int tap = wd / Cw, cw = wd % Cw;
        uint32_t w = 0;
        for (int b = 0; b < 32; b++) {
            const int ch = cw * 32 + b;
            if (ch < C && __ldg(F + ((size_t)tap * C + ch) * O + o) >= 0) w |= 0x80000000u >> b;
        }
        out[(size_t)o * RS * Cw + wd] = w;
    }
}

// First-layer filter: fp32 F[R*S][3][O] -> [R*S][3][Ow] words over output channels
// (PackFiltersByOutChannels32, param.h:613-632).
__device__ __forceinline__ void pack_inconv_filter(const float* F, int RS, int O, uint32_t* out) {
    const int Ow = (O + 31) >> 5;
    const int total = RS * 3 * Ow;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % Ow, tc = i / Ow;
        uint32_t w = 0;
        for (int b = 0; b < 32; b++) {
            const int o = k * 32 + b;
            if (o < O && __ldg(F + (size_t)tc * O + o) >= 0) w |= 0x80000000u >> b;
        }
        out[i] = w;
    }
}

// Conv filter preparation: pads [O][R*S][Cw] to [O][2*KP], builds the per-tap popcount
// tables and the pair table the implicit-GEMM loop walks.
__device__ __forceinline__ void conv_prepare(const uint32_t* fbits, int O, int R, int S, int Cw,
                                             int W_in, int KP, uint32_t* wq, uint32_t* ktab,
                                             int* pwt, int* pwtot) {
    const int RS = R * S;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
    for (long long i = tid; i < (long long)O * 2 * KP; i += nth) {
        const int o = (int)(i / (2 * KP)), wd = (int)(i % (2 * KP));
        wq[i] = wd < RS * Cw ? fbits[(size_t)o * RS * Cw + wd] : 0u;
    }
    for (int kp = tid; kp < KP; kp += nth) {
        const int wd = 2 * kp;
        uint32_t e;
        if (wd < RS * Cw) {
            const int tap = wd / Cw, cw = wd % Cw, r = tap / S, s = tap % S;
            e = ((uint32_t)r << 28) | ((uint32_t)s << 24) | (uint32_t)((r * W_in + s) * Cw + cw);
        } else {
            e = 15u << 28;                       // padding pair: row 15 is always "invalid"
        }
        ktab[kp] = e;
    }
    for (int i = tid; i < O; i += nth) {
        int tot = 0;
        for (int tap = 0; tap < RS; tap++) {
            int p = 0;
            for (int cw = 0; cw < Cw; cw++) p += __popc(fbits[((size_t)i * RS + tap) * Cw + cw]);
            pwt[tap * O + i] = p;
            tot += p;
        }
        pwtot[i] = tot;
    }
}

}  // namespace tcbnn
