// tcgen05 binary convolution for wide layers (C >= 256): activation-stationary schedule.
//
// bconv_umma_ws.cuh keeps a CTA's filter block resident and streams positions past it; with
// C = 256 / 512 only 64 / 32 output channels of filter fit, the MMA's N is that small, and the
// tensor pipe runs at 67 % / 36 % of its rate while every position is expanded once per n-tile.
// Here the roles are swapped.  A CTA owns 256 consecutive raster positions (two 128-row
// sub-tiles): their +-1 bytes for ALL input channels are expanded once and stay in shared
// memory.  The filter streams past them in 8 KB units (128 output channels x 64 input channels
// x one tap) through a ring filled by bulk asynchronous copies (cp.async.bulk + mbarrier
// complete_tx), each unit feeding four N=128 MMAs (two sub-tiles x two k-steps) -- the shape
// at which the tensor pipe reaches its peak.  Accumulators: 2 sub-tiles x 128 columns, double
// buffered across n-tiles (all 512 TMEM columns).
//
//   warps 0-7   epilogue    (warps 0-3 sub-tile 0, warps 4-7 sub-tile 1; thread = raster position)
//   warps 8-13  expanders   (once per task: all 64-channel blocks of the 256+halo positions)
//   warp  14    filter loader (one lane issues the bulk copies)
//   warp  15    MMA issuer  (one lane)
//
// Same arithmetic, raster, descriptors and bounded waits as bconv_umma_ws.cuh.  Stride 1 only.
#pragma once
#include "bconv_umma_ws.cuh"

namespace tcbnn {
namespace umma {

constexpr int kAsNT = 128;                 // output channels per filter unit / accumulator
constexpr int kAsMaxSlots = 18;            // filter ring: 6, 9 or 18 units (whole rows of a 3x3 filter)
constexpr int kAsUnitBytes = kAsNT * 64;   // 128 out x 64 in x 1 tap, int8
constexpr int kAsEpiThreads = 256;
constexpr int kAsExpThreads = 192;
constexpr int kAsThreads = kAsEpiThreads + kAsExpThreads + 64;
constexpr int kAsMaxPos = 2;               // raster positions per expander thread (NPOS <= 384)

__host__ __device__ inline size_t as_smem_bytes(int npos, int C, int O, int RS, int slots) {
    return (size_t)(C / 16) * npos * 16 + (size_t)slots * kAsUnitBytes + (size_t)O * 4 + RS * 8 +
           64 * 8 + 64;
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// global -> shared bulk copy; completion is counted in bytes on the mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int DUMMY>
__device__ void conv_umma_as_cta(const ConvWsArgs& a, unsigned char* smem) {
    constexpr int NT = kAsNT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RS = a.R * a.S, NCB = a.C >> 6, NNT = a.O / NT;
    const uint32_t cb_bytes = 4u * a.NPOS * 16u;              // one 64-channel block of the patch

    unsigned char* sA = smem;
    unsigned char* sB = smem + (size_t)NCB * cb_bytes;
    const int NS = a.as_slots;
    const int GT = RS == 9 ? 3 : 1;                           // taps per filter group (a row of a 3x3 filter)
    const int NG = NS / GT;                                   // groups in the ring
    const uint32_t group_bytes = (uint32_t)GT * kAsUnitBytes;
    int* sThr = reinterpret_cast<int*>(sB + (size_t)NS * kAsUnitBytes);
    uint32_t* sTapK = reinterpret_cast<uint32_t*>(sThr + a.O);
    uint64_t* sBar = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(sTapK + 2 * RS) + 7) & ~(uintptr_t)7);
    // barriers: a_full[8] | a_empty | c_full[2] | c_empty[2] | b_full[18] | b_empty[18]
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 49);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sTmem + 1);
    const uint32_t bar0 = smem_u32(sBar);
    auto BAR_AFULL = [&](int cb) { return bar0 + 8u * cb; };
    const uint32_t BAR_AEMPTY = bar0 + 8u * 8;
    auto BAR_CFULL = [&](int b) { return bar0 + 8u * (9 + b); };
    auto BAR_CEMPTY = [&](int b) { return bar0 + 8u * (11 + b); };
    auto BAR_BFULL = [&](int s) { return bar0 + 8u * (13 + s); };
    auto BAR_BEMPTY = [&](int s) { return bar0 + 8u * (13 + kAsMaxSlots + s); };

    const int NV = (int)a.NV;
    const int ntasks = (NV + 255) / 256;

    if (tid == 0) {
        for (int i = 0; i < 8; i++) mbar_init(BAR_AFULL(i), kAsExpThreads / 32);
        for (int i = 0; i < kAsMaxSlots; i++) { mbar_init(BAR_BFULL(i), 1); mbar_init(BAR_BEMPTY(i), 1); }
        mbar_init(BAR_AEMPTY, 1);
        for (int b = 0; b < 2; b++) { mbar_init(BAR_CFULL(b), 1); mbar_init(BAR_CEMPTY(b), 8); }
        *sAbort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 15) tmem_alloc(smem_u32(sTmem), 512);
    for (int i = tid; i < a.O; i += kAsThreads) {
        // integer form of  !((float)v < thr)  (kernel.cuh:795-796): v >= ceil(thr)
        const float t = __ldg(a.thr + i);
        int it = INT_MIN;
        if (t == t) it = t >= 2147483520.0f ? INT_MAX : t <= -2147483648.0f ? INT_MIN : (int)ceilf(t);
        sThr[i] = it;
    }
    for (int t = tid; t < RS; t += kAsThreads) {
        const uint32_t byte_off = (uint32_t)((t / a.S) * a.PW + (t % a.S)) * 16u;
        sTapK[2 * t] = byte_off >> 4;
        sTapK[2 * t + 1] = (byte_off + 2u * (uint32_t)a.NPOS * 16u) >> 4;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *sTmem;
    const WsWait wait{sAbort, a.err_flag};
    // work items: (task of 256 positions, part of the n-tiles); items of a CTA: blockIdx.x, +gridDim.x ..
    const int split = a.as_split, nts_per = NNT / split;
    const int nitems = ntasks * split;

    if (tid >= kAsEpiThreads && tid < kAsEpiThreads + kAsExpThreads) {
        // =============================== expanders ==========================================
        const int et = tid - kAsEpiThreads;
        const int Cw = a.C >> 5;
        uint32_t ic = 0;
        long long tr_wait = 0;
        const long long tr_t0 = clock64();
        for (int item = blockIdx.x; item < nitems; item += gridDim.x, ic++) {
            const int task = item / split;
            const int base = task * 256 - (a.back_y * a.PW + a.back_x);
            int ptr[kAsMaxPos];
            bool val[kAsMaxPos];
#pragma unroll
            for (int j = 0; j < kAsMaxPos; j++) {
                const int q = et + j * kAsExpThreads, gq = base + q;
                ptr[j] = 0; val[j] = false;
                if (q < a.NPOS && gq >= 0 && gq < NV) {
                    const int vy = fastdiv(gq, a.pw_mul, a.pw_sh), vx = gq - vy * a.PW;
                    const int n = fastdiv(vy, a.vh_mul, a.vh_sh), vr = vy - n * a.VH;
                    if (vr < a.OHg && vx < a.OWg && vr < a.H && vx < a.W) {
                        ptr[j] = ((n * a.H + vr) * a.W + vx) * Cw;
                        val[j] = true;
                    }
                }
            }
            // all channels of this thread's positions; the loads fly while the MMAs of the
            // previous item still read the patch
            uint2 bits[kAsMaxPos][8];
#pragma unroll
            for (int j = 0; j < kAsMaxPos; j++)
#pragma unroll
                for (int cb = 0; cb < 8; cb++)
                    bits[j][cb] = (val[j] && cb < NCB) ? ldg64(a.in + ptr[j] + cb * 2) : make_uint2(0u, 0u);
            if (!wait.timed(BAR_AEMPTY, (ic & 1) ^ 1, tr_wait)) break;
#pragma unroll
            for (int cb = 0; cb < 8; cb++) {
                if (cb >= NCB) continue;
                uint4* blk = reinterpret_cast<uint4*>(sA + (size_t)cb * cb_bytes);
#pragma unroll
                for (int j = 0; j < kAsMaxPos; j++) {
                    const int q = et + j * kAsExpThreads;
                    if (q >= a.NPOS) continue;
                    uint4* dst = blk + q;
                    if (val[j]) {
                        dst[0] = expand16(bits[j][cb].x >> 16);
                        dst[(size_t)a.NPOS] = expand16(bits[j][cb].x & 0xFFFFu);
                        dst[(size_t)2 * a.NPOS] = expand16(bits[j][cb].y >> 16);
                        dst[(size_t)3 * a.NPOS] = expand16(bits[j][cb].y & 0xFFFFu);
                    } else {
                        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                        dst[0] = z; dst[(size_t)a.NPOS] = z;
                        dst[(size_t)2 * a.NPOS] = z; dst[(size_t)3 * a.NPOS] = z;
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR_AFULL(cb));
            }
        }
        if (a.trace && blockIdx.x == 0 && et == 0) { a.trace[0] = clock64() - tr_t0; a.trace[1] = tr_wait; a.trace[2] = ic; }
    } else if (warp == 14) {
        // =============================== filter loader ======================================
        // The filter moves in groups of GT taps (a filter row of a 3x3 filter: 24 KB, one copy,
        // one barrier), so that the MMA warp waits and commits once per 12 MMAs.
        if (lane == 0) {
            int slot = 0;
            uint32_t ph = 0, issued = 0;                 // ph: parity of the current pass over the ring
            bool ok = true;
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x) {
                const int part = item % split;
                for (int nt = part * nts_per; nt < (part + 1) * nts_per && ok; nt++) {
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(a.wi8) +
                                               (size_t)nt * NCB * RS * kAsUnitBytes;
                    for (int k = 0; k < NCB * RS; k += GT) {
                        ok = wait(BAR_BEMPTY(slot), ph ^ 1);
                        if (!ok) break;
                        mbar_expect_tx(BAR_BFULL(slot), group_bytes);
                        bulk_g2s(smem_u32(sB + (size_t)slot * group_bytes), src + (size_t)k * kAsUnitBytes,
                                 group_bytes, BAR_BFULL(slot));
                        issued++;
                        if (++slot == NG) { slot = 0; ph ^= 1; }
                    }
                }
            }
            if (!ok) {
                // giving up: wait (bounded) for the copies still in flight before the CTA exits;
                // slots below `slot` were last filled in this pass, the others in the one before
                for (int s2 = 0; s2 < NG; s2++) {
                    const bool this_pass = s2 < slot;
                    if (!this_pass && issued < (uint32_t)NG) continue;       // never filled
                    const uint32_t par = this_pass ? ph : ph ^ 1;
                    for (int i = 0; i < (1 << 20); i++)
                        if (mbar_try_wait(BAR_BFULL(s2), par)) break;
                }
            }
        }
        __syncwarp();
    } else if (warp == 15) {
        // =============================== MMA issuer =========================================
        // A 128x128x32 MMA occupies the tensor pipe for 64 clocks and the pipe does not run ahead
        // of the issuing thread by much: whatever that thread executes between two MMAs is time
        // the pipe idles.  So the whole warp runs the control flow converged (waits by all lanes
        // with the non-blocking barrier test), one elected lane issues, and a wait / commit pair
        // covers a group of taps (12 MMAs for a 3x3 filter).
        {
            const bool leader = elect_one();
            const uint32_t lboA = (uint32_t)a.NPOS * 16u, lboB = NT * 16u;
            const uint64_t descA0 = smem_desc(smem_u32(sA), lboA, 128u);
            const uint64_t descB0 = smem_desc(smem_u32(sB), lboB, 128u);
            const uint32_t aHi = (uint32_t)(descA0 >> 32), bHi = (uint32_t)(descB0 >> 32);
            const uint32_t aLo0 = (uint32_t)descA0, bLo0 = (uint32_t)descB0;
            constexpr uint32_t stepKB = (2u * NT * 16u) >> 4;   // second k-step of a tap
            constexpr uint32_t stepTap = kAsUnitBytes >> 4;
            constexpr uint32_t stepSub = (128u * 16u) >> 4;     // second 128-row sub-tile
            const uint32_t stepCb = cb_bytes >> 4, stepGroup = group_bytes >> 4;
            constexpr uint32_t IDESC = idesc_i8(NT);
            const bool rs9 = RS == 9;
            uint32_t ak[18];
#pragma unroll
            for (int i = 0; i < 18; i++) ak[i] = rs9 ? sTapK[i] : 0u;
            uint32_t cc = 0, ic = 0, units = 0;
            int slot = 0;
            uint32_t bph = 0;
            bool ok = true;
            long long tr_wc = 0, tr_wa = 0;
            const long long tr_t0 = clock64();
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ic++) {
                for (int nti = 0; nti < nts_per && ok; nti++, cc++) {
                    const int buf = cc & 1;
                    ok = wait.timed(BAR_CEMPTY(buf), ((cc >> 1) & 1) ^ 1, tr_wc);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d0 = tmem + buf * 256, d1 = d0 + 128;
                    for (int cb = 0; cb < NCB && ok; cb++) {
                        if (nti == 0) {
                            ok = wait.timed(BAR_AFULL(cb), ic & 1, tr_wa);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        const uint32_t aCb = aLo0 + cb * stepCb;
                        if (rs9) {
#pragma unroll
                            for (int g = 0; g < 3; g++) {
                                ok = ok && wait.spin(BAR_BFULL(slot), bph);
                                if (!ok) break;
                                tc_fence_after();
                                if (leader) {
                                    const uint32_t bG = bLo0 + slot * stepGroup;
#pragma unroll
                                    for (int j = 0; j < 3; j++) {
                                        const int t = 3 * g + j;
                                        const uint32_t acc = (t == 0 && cb == 0) ? 0u : 1u;
                                        const uint32_t bLo = bG + j * stepTap;
                                        mma_i8_split(d0, aCb + ak[2 * t], aHi, bLo, bHi, IDESC, acc);
                                        mma_i8_split(d1, aCb + ak[2 * t] + stepSub, aHi, bLo, bHi, IDESC, acc);
                                        mma_i8_split(d0, aCb + ak[2 * t + 1], aHi, bLo + stepKB, bHi, IDESC, 1u);
                                        mma_i8_split(d1, aCb + ak[2 * t + 1] + stepSub, aHi, bLo + stepKB, bHi, IDESC, 1u);
                                    }
                                    mma_commit(BAR_BEMPTY(slot));   // group free once these MMAs have read it
                                }
                                units++;
                                if (++slot == NG) { slot = 0; bph ^= 1; }
                            }
                        } else {
                            for (int t = 0; t < RS; t++) {          // GT == 1: one tap per group
                                ok = wait.spin(BAR_BFULL(slot), bph);
                                if (!ok) break;
                                tc_fence_after();
                                if (leader) {
                                    const uint2 ao = *reinterpret_cast<const uint2*>(sTapK + 2 * t);
                                    const uint32_t bLo = bLo0 + slot * stepGroup;
                                    const uint32_t acc = (cb | t) ? 1u : 0u;
                                    mma_i8_split(d0, aCb + ao.x, aHi, bLo, bHi, IDESC, acc);
                                    mma_i8_split(d1, aCb + ao.x + stepSub, aHi, bLo, bHi, IDESC, acc);
                                    mma_i8_split(d0, aCb + ao.y, aHi, bLo + stepKB, bHi, IDESC, 1u);
                                    mma_i8_split(d1, aCb + ao.y + stepSub, aHi, bLo + stepKB, bHi, IDESC, 1u);
                                    mma_commit(BAR_BEMPTY(slot));
                                }
                                units++;
                                if (++slot == NG) { slot = 0; bph ^= 1; }
                            }
                        }
                    }
                    if (ok && leader) mma_commit(BAR_CFULL(buf));   // both sub-tile accumulators complete
                }
                if (ok && leader) mma_commit(BAR_AEMPTY);           // the patch may be overwritten
            }
            if (a.trace && blockIdx.x == 0 && leader) { a.trace[3] = clock64() - tr_t0; a.trace[4] = tr_wc; a.trace[5] = tr_wa; a.trace[10] = units; }
        }
        __syncwarp();
    } else if (tid < kAsEpiThreads) {
        // =============================== epilogue ===========================================
        const int row = tid & 127, sub = tid >> 7, quad = warp & 3;
        const int Ow = a.O >> 5;
        const int lim = a.res_in ? min(a.residual_channels, a.res_in_ch) : 0;
        uint32_t cc = 0;
        bool ok = true, overflow = false;
        long long tr_w = 0;
        const long long tr_t0 = clock64();
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x) {
            const int task = item / split, part = item - task * split;
            const int p = task * 256 + sub * 128 + row;
            bool live = false;
            int n = 0, y = 0, x = 0;
            if (p < NV) {
                const int vy = fastdiv(p, a.pw_mul, a.pw_sh);
                x = p - vy * a.PW;
                n = fastdiv(vy, a.vh_mul, a.vh_sh);
                y = vy - n * a.VH;
                live = x < a.OWg && y < a.OHg;
            }
            const size_t opix = ((size_t)n * a.OHg + y) * a.OWg + x;
            // 2x2 window of a pooled residual (kernel.cuh:773-783)
            const size_t rp00 = (((size_t)n * 2 * a.OHg + 2 * y) * 2 * a.OWg + 2 * x) * a.res_in_ch;
            const size_t rprow = (size_t)2 * a.OWg * a.res_in_ch;
            // int16 residuals: the 32 channels [o0, o0+32) of this thread's pixel as packed
            // pairs, all loads of a group issued together (zeros where nothing is injected)
            const bool res16 = a.res_in && a.res_in_bytes == 2 && (a.res_in_ch & 7) == 0 && (lim & 7) == 0;
            auto fetch16 = [&](uint4 (&r)[4], int o0) {
                const short* base = reinterpret_cast<const short*>(a.res_in);
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                if (a.residual_pool) {
                    uint4 w[4][4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const bool on = live && o0 + 8 * j < lim;
                        const short* q = base + rp00 + o0 + 8 * j;
                        w[0][j] = on ? __ldg(reinterpret_cast<const uint4*>(q)) : z;
                        w[1][j] = on ? __ldg(reinterpret_cast<const uint4*>(q + a.res_in_ch)) : z;
                        w[2][j] = on ? __ldg(reinterpret_cast<const uint4*>(q + rprow)) : z;
                        w[3][j] = on ? __ldg(reinterpret_cast<const uint4*>(q + rprow + a.res_in_ch)) : z;
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        r[j].x = __vmaxs2(__vmaxs2(w[0][j].x, w[1][j].x), __vmaxs2(w[2][j].x, w[3][j].x));
                        r[j].y = __vmaxs2(__vmaxs2(w[0][j].y, w[1][j].y), __vmaxs2(w[2][j].y, w[3][j].y));
                        r[j].z = __vmaxs2(__vmaxs2(w[0][j].z, w[1][j].z), __vmaxs2(w[2][j].z, w[3][j].z));
                        r[j].w = __vmaxs2(__vmaxs2(w[0][j].w, w[1][j].w), __vmaxs2(w[2][j].w, w[3][j].w));
                    }
                } else {
                    const short* q = base + opix * a.res_in_ch + o0;
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        r[j] = (live && o0 + 8 * j < lim) ? __ldg(reinterpret_cast<const uint4*>(q + 8 * j)) : z;
                }
            };
            for (int nti = 0; nti < nts_per && ok; nti++, cc++) {
                const int nt = part * nts_per + nti, buf = cc & 1;
                uint4 rnext[4];
                const bool res16_nt = res16 && nt * NT < lim;          // uniform over the CTA
                if (res16_nt) fetch16(rnext, nt * NT);                 // flies during the wait
                ok = wait.timed(BAR_CFULL(buf), (cc >> 1) & 1, tr_w);
                if (!ok) break;
                tc_fence_after();
                uint32_t words[4];
#pragma unroll
                for (int nb = 0; nb < 4; nb++) {
                    const int o0 = nt * NT + nb * 32;
                    uint4 rcur[4];
                    if (res16_nt) {
                        // plain residuals are prefetched one group ahead; pooled ones (four loads
                        // per value) are fetched and reduced here, before the accumulator is
                        // read, so that they do not sit in registers next to it
                        if (a.residual_pool && nb > 0) fetch16(rnext, o0);
#pragma unroll
                        for (int j = 0; j < 4; j++) rcur[j] = rnext[j];
                        if (!a.residual_pool && nb < 3) fetch16(rnext, o0 + 32);
                    }
                    int v[32];
                    tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + buf * 256 + sub * 128 + nb * 32, v);
                    tmem_ld_wait();
                    if (nb == 3) {                            // this warp is done with the accumulator
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(BAR_CEMPTY(buf));
                    }
                    if (live && a.acc_out) {
                        int4* dst = reinterpret_cast<int4*>(a.acc_out + opix * a.O + o0);
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            dst[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                    if (res16_nt) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            v[8 * j] += (int)(short)(rcur[j].x & 0xFFFFu);
                            v[8 * j + 1] += (int)(short)(rcur[j].x >> 16);
                            v[8 * j + 2] += (int)(short)(rcur[j].y & 0xFFFFu);
                            v[8 * j + 3] += (int)(short)(rcur[j].y >> 16);
                            v[8 * j + 4] += (int)(short)(rcur[j].z & 0xFFFFu);
                            v[8 * j + 5] += (int)(short)(rcur[j].z >> 16);
                            v[8 * j + 6] += (int)(short)(rcur[j].w & 0xFFFFu);
                            v[8 * j + 7] += (int)(short)(rcur[j].w >> 16);
                        }
                    } else if (a.res_in && live && o0 < lim) {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int o = o0 + 4 * j;
                            if (o >= lim) continue;
                            int4 r;
                            if (a.residual_pool) {
                                r = max4(max4(ld_res4(a.res_in, a.res_in_bytes, rp00 + o),
                                              ld_res4(a.res_in, a.res_in_bytes, rp00 + a.res_in_ch + o)),
                                         max4(ld_res4(a.res_in, a.res_in_bytes, rp00 + rprow + o),
                                              ld_res4(a.res_in, a.res_in_bytes, rp00 + rprow + a.res_in_ch + o)));
                            } else {
                                r = ld_res4(a.res_in, a.res_in_bytes, opix * a.res_in_ch + o);
                            }
                            v[4 * j] += r.x; v[4 * j + 1] += r.y; v[4 * j + 2] += r.z; v[4 * j + 3] += r.w;
                        }
                    }
                    uint32_t word = 0;
                    const int4* th4 = reinterpret_cast<const int4*>(sThr + o0);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int4 th = th4[j];
                        if (v[4 * j] >= th.x) word |= 0x80000000u >> (4 * j);
                        if (v[4 * j + 1] >= th.y) word |= 0x80000000u >> (4 * j + 1);
                        if (v[4 * j + 2] >= th.z) word |= 0x80000000u >> (4 * j + 2);
                        if (v[4 * j + 3] >= th.w) word |= 0x80000000u >> (4 * j + 3);
                    }
                    words[nb] = word;
                    if (a.res_out && live) {
                        const size_t idx = opix * a.O + o0;
                        if (a.res_out_bytes == 2) {
                            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<short*>(a.res_out) + idx);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint32_t w[4];
#pragma unroll
                                for (int kk = 0; kk < 4; kk++) {
                                    const int lo = v[8 * j + 2 * kk], hi = v[8 * j + 2 * kk + 1];
                                    overflow |= max(abs(lo), abs(hi)) > 32767;
                                    w[kk] = ((uint32_t)lo & 0xFFFFu) | ((uint32_t)hi << 16);
                                }
                                dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
                            int4* dst = reinterpret_cast<int4*>(reinterpret_cast<int*>(a.res_out) + idx);
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                dst[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                    }
                }
                if (live) {
                    uint32_t* dst = a.out + (size_t)n * a.out_image_stride +
                                    ((size_t)y * a.OWg + x) * Ow + nt * (NT >> 5);
                    if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
                    } else {
                        dst[0] = words[0]; dst[1] = words[1]; dst[2] = words[2]; dst[3] = words[3];
                    }
                }
            }
        }
        if (overflow) atomicExch(a.err_flag, 2);
        if (a.trace && blockIdx.x == 0 && tid == 0) { a.trace[6] = clock64() - tr_t0; a.trace[7] = tr_w; a.trace[8] = cc; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 15) tmem_dealloc(tmem, 512);
}

}  // namespace umma
}  // namespace tcbnn
