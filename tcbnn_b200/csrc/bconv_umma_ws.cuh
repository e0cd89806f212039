// Warp-specialised, persistent tcgen05 binary convolution (stride 1 and stride 2).
//
// Arithmetic and raster trick: see bconv_umma.cuh (read that header first).  Packed bits become
// +-1 bytes in the no-swizzle K-major core-matrix layout, taps are start-address offsets,
// int8 x int8 -> int32 accumulates in tensor memory.  One CTA per SM runs
//
//   warps 0-7   epilogue   : prefetch the residual rows, wait for an accumulator, tcgen05.ld,
//                            add / threshold / pack, store bits and the new residual
//                            (warp w reads TMEM lanes 32*(w%4).., column groups of parity w/4)
//   warps 8-14  expanders  : packed input bits (prefetched three stages ahead in registers) ->
//                            +-1 bytes of one 64-channel block of the patch, ring of stages
//   warp  15    MMA issuer : one lane issues 9 taps x 2 k-steps per stage, commits the stage
//                            back to the expanders and the finished tile to the epilogue
//
// with mbarriers between them, two accumulators in tensor memory (epilogue of tile i overlaps
// the MMAs of tile i+1) and the filter block of the CTA's n-tile resident in shared memory.
//
// Stride 2: the input is de-interleaved into its four (row parity, column parity) planes, each a
// raster with the OUTPUT pitch; tap (r, s) then reads plane ((r-pad)&1, (s-pad)&1) at a fixed
// raster offset, so it is again just a descriptor start address.
//
// Every wait is bounded: a wait that gives up raises the CTA's abort flag and the layer's
// status word, all roles drain, tensor memory is released, the kernel returns.
#pragma once
#include "bconv_umma.cuh"

namespace tcbnn {
namespace umma {

struct ConvWsArgs {
    const uint32_t* in;       // [B][H][W][C/32]
    const uint4* wi8;         // [n-tile][64-ch block][tap][4 chunks][NT][16 B]
    const uint4* wf4;         // 4-bit form for bconv_umma_pre.cuh: [n-tile][64-ch block][tap][2 chunks][NT][16 B]
    const float* thr;         // [O]
    int B, H, W, C, O, R, S, pad_h, pad_w, stride;
    int OHg, OWg;             // outputs per image (pre-pool == post-pool here)
    int PW, VH;               // raster pitch and rows per image (output grid + zero band)
    uint32_t pw_mul, pw_sh, vh_mul, vh_sh;   // x / PW and x / VH by multiply-shift (x < 2^31)
    int NPOS;                 // raster positions per plane patch (multiple of 8)
    int back_y, back_x;       // patch origin = tile start - (back_y*PW + back_x)
    long long NV;             // raster positions over the batch
    int ntiles_n;
    // loader-fed kernel: the first nt_heavy n-tiles (those an injected, pooled residual falls into)
    // get per_heavy CTAs each, the others per_light; 0 = every n-tile the same share of the grid
    int nt_heavy, per_heavy, per_light;
    int as_split;             // activation-stationary kernel: parts the n-tiles of a task are split into
    int as_slots;             // ... and units in its filter ring (9 or 18)
    const uint4* pre;         // pre-expanded input planes (bconv_umma_pre.cuh), else null
    long long pre_positions, pre_front;
    int pre_stages;           // patch ring depth of that kernel
    int pre_cbs;              // 64-channel blocks per stage of that ring (1, 2 or 4)
    // optional: also write the output as +-1 nibbles into the next layer's input planes
    // (bconv_umma_pre.cuh layout over THAT layer's raster; dead slots stay as the caller zeroed them)
    uint4* nxt; long long nxt_positions, nxt_front; int nxt_PW, nxt_VH;
    int nxt_nplane;           // 1, or 4 when that layer has stride 2 (one plane per row / column parity)
    const void* res_in; int res_in_bytes, res_in_ch, residual_channels, residual_pool;
    // int16 residual tensors may be laid out by 8-channel chunk, [ch/8][pixels][8], instead of NHWC
    // (bconv_umma_pre.cuh, direct epilogue only): npix = pixels of the whole tensor
    int res_in_chunked, res_out_chunked; long long res_in_npix, res_out_npix;
    uint32_t* out; long long out_image_stride;
    void* res_out; int res_out_bytes; int32_t* acc_out;
    int res_out_proven;       // the caller vouches that every saved int16 value fits: no range check
    int* err_flag;
    long long* trace;         // optional: block 0 writes per-role cycle counters (see tcbnn_conv_set_trace)
};

constexpr int kWsEpiThreads = 256;
constexpr int kWsExpThreads = 224;       // 7 warps; with the issuer warp the CTA is 16 warps
constexpr int kWsThreads = kWsEpiThreads + kWsExpThreads + 32;
constexpr int kWsMaxEnt = 4;          // (positions per expander thread) x planes

__host__ __device__ inline int ws_stages(int stride) { return stride == 2 ? 2 : 3; }
__host__ __device__ inline size_t ws_stage_bytes(int stride, int npos) {
    return (size_t)(stride == 2 ? 4 : 1) * 4 * npos * 16;
}
__host__ __device__ inline size_t ws_smem_bytes(int stride, int npos, int C, int RS, int nt) {
    return ws_stages(stride) * ws_stage_bytes(stride, npos) + (size_t)RS * C * nt + nt * 4 +
           RS * 12 + 16 * 8 + 64;
}

// filter bits [O][R*S][Cw] -> int8 blocks in the order the kernel keeps them in shared memory
__device__ __forceinline__ void prepare_filter_ws(const uint32_t* fbits, int O, int RS, int C,
                                                  int nt, uint4* out) {
    const int Cw = C >> 5, ncb = C >> 6;
    const long long total = (long long)O * RS * (C >> 4);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i % nt);
        long long r = i / nt;
        const int c4 = (int)(r & 3); r >>= 2;
        const int tap = (int)(r % RS); r /= RS;
        const int cb = (int)(r % ncb);
        const int tile = (int)(r / ncb);
        const int o = tile * nt + n;
        const uint32_t w = fbits[((size_t)o * RS + tap) * Cw + cb * 2 + (c4 >> 1)];
        out[i] = expand16((c4 & 1) ? (w & 0xFFFFu) : (w >> 16));
    }
}

// floor(x / d) for 0 <= x < 2^31 with mul = ceil(2^sh / d), sh = 31 + ceil(log2 d)
__device__ __forceinline__ int fastdiv(int x, uint32_t mul, uint32_t sh) {
    return (int)(((unsigned long long)(uint32_t)x * mul) >> sh);
}
__host__ inline void fastdiv_setup(int d, uint32_t* mul, uint32_t* sh) {
    uint32_t s = 0;
    while ((1u << s) < (uint32_t)d) s++;
    *sh = 31 + s;
    *mul = (uint32_t)((((unsigned long long)1 << (31 + s)) + d - 1) / d);
}

// filter bits [O][R*S][Cw] -> e2m1 nibble blocks in the order bconv_umma_pre.cuh keeps them in
// shared memory: [n-tile][64-ch block][tap][32-ch chunk][n][16 B]
__device__ __forceinline__ void prepare_filter_f4(const uint32_t* fbits, int O, int RS, int C,
                                                  int nt, uint4* out) {
    const int Cw = C >> 5, ncb = C >> 6;
    const long long total = (long long)O * RS * Cw;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i % nt);
        long long r = i / nt;
        const int c2 = (int)(r & 1); r >>= 1;
        const int tap = (int)(r % RS); r /= RS;
        const int cb = (int)(r % ncb);
        const int tile = (int)(r / ncb);
        const int o = tile * nt + n;
        out[i] = expand32_f4(fbits[((size_t)o * RS + tap) * Cw + cb * 2 + c2]);
    }
}

// Writes the +-1 nibbles of `nbits` output channels (8, 16 or 32; first channel o0, a multiple of
// nbits; channel c at bit nbits-1-c of `word`) of output pixel (n, y, x) into the next layer's
// planes: one 16-byte slot per raster position and 32-channel chunk (expand32_f4 order).
__device__ __forceinline__ void store_next_planes(const ConvWsArgs& a, int n, int y, int x, int o0,
                                                  uint32_t word, int nbits) {
    int pl = 0;
    if (a.nxt_nplane == 4) {                    // stride-2 consumer: pixel (y, x) lives in plane (y&1, x&1) at (y/2, x/2)
        pl = (y & 1) * 2 + (x & 1);
        y >>= 1; x >>= 1;
    }
    uint4* base = a.nxt + ((size_t)(o0 >> 5) * a.nxt_nplane + pl) * a.nxt_positions + a.nxt_front +
                  ((long long)n * a.nxt_VH + y) * a.nxt_PW + x;
    if (nbits == 32) {
        base[0] = expand32_f4(word);
    } else if (nbits == 16) {                   // half a chunk: channels 0-15 are its first 8 bytes
        reinterpret_cast<uint2*>(base)[(o0 >> 4) & 1] = make_uint2(expand8_f4(word >> 8), expand8_f4(word));
    } else {                                    // 8 channels: one 32-bit word of the slot
        reinterpret_cast<uint32_t*>(base)[(o0 >> 3) & 3] = expand8_f4(word);
    }
}

struct WsWait {
    volatile int* abort;
    int* err;
    __device__ __forceinline__ bool operator()(uint32_t bar, uint32_t parity) const {
        for (int i = 0; i < (1 << 24); i++) {
            if (mbar_try_wait(bar, parity)) return true;
            if ((i & 1023) == 1023 && *abort) return false;
        }
        *abort = 1;
        atomicExch(err, 1);
        return false;
    }
    // for the MMA warp, whose every instruction delays the next MMA: one non-blocking test first
    // (measured cheaper than try_wait when the phase is already complete, the case that matters),
    // then the suspending wait, which leaves the issue slots to the other warps
    __device__ __forceinline__ bool spin(uint32_t bar, uint32_t parity) const {
        if (mbar_test_wait(bar, parity)) return true;
        return (*this)(bar, parity);
    }
    // the same for roles that can afford to look less often: sleeps between polls, so that many
    // waiting warps do not keep the shared-memory pipe busy with barrier reads
    __device__ __forceinline__ bool relaxed(uint32_t bar, uint32_t parity) const {
        for (int i = 0; i < (1 << 22); i++) {
            if (mbar_try_wait(bar, parity)) return true;
            __nanosleep(64);
            if ((i & 255) == 255 && *abort) return false;
        }
        *abort = 1;
        atomicExch(err, 1);
        return false;
    }
    // same, adding the cycles spent waiting to `acc` (tracing)
    __device__ __forceinline__ bool timed(uint32_t bar, uint32_t parity, long long& acc) const {
        const long long t0 = clock64();
        const bool ok = (*this)(bar, parity);
        acc += clock64() - t0;
        return ok;
    }
};

template <int NT, int STRIDE>
__device__ void conv_umma_ws_cta(const ConvWsArgs& a, unsigned char* smem) {
    constexpr int NSTAGE = STRIDE == 2 ? 2 : 3;
    constexpr int NPLANE = STRIDE == 2 ? 4 : 1;
    constexpr uint32_t TM_COLS = 2 * NT < 32 ? 32 : 2 * NT;
    constexpr int NB = NT / 32;                       // 32-column groups per accumulator
    constexpr int EPI_GROUPS = NB >= 2 ? 2 : 1;       // epilogue warp groups with work
    constexpr int NB_PER = NB / EPI_GROUPS;
    constexpr int MMA_WARP = (kWsEpiThreads + kWsExpThreads) / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RS = a.R * a.S, NCB = a.C >> 6;
    const uint32_t plane_bytes = 4u * a.NPOS * 16u, stage_bytes = NPLANE * plane_bytes;

    unsigned char* sAraw = smem;
    uint4* sB = reinterpret_cast<uint4*>(smem + (size_t)NSTAGE * stage_bytes);
    int* sThr = reinterpret_cast<int*>(sB + (size_t)RS * (a.C >> 4) * NT);
    int* sTap = sThr + NT;
    uint32_t* sTapK = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sTap + RS) + 7) & ~(uintptr_t)7);
    uint64_t* sBar = reinterpret_cast<uint64_t*>(sTapK + 2 * RS);
    // barriers: a_full[NSTAGE], a_empty[NSTAGE], acc_full[2], acc_empty[2]
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 2 * NSTAGE + 4);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sTmem + 1);
    const uint32_t bar0 = smem_u32(sBar);
    auto BAR_AFULL = [&](int s) { return bar0 + 8u * s; };
    auto BAR_AEMPTY = [&](int s) { return bar0 + 8u * (NSTAGE + s); };
    auto BAR_CFULL = [&](int b) { return bar0 + 8u * (2 * NSTAGE + b); };
    auto BAR_CEMPTY = [&](int b) { return bar0 + 8u * (2 * NSTAGE + 2 + b); };

    // this CTA's n-tile and m-tile sequence (all raster arithmetic fits 32 bits: host checks)
    const int nt = blockIdx.x % a.ntiles_n;
    const int mfirst = blockIdx.x / a.ntiles_n, mstep = gridDim.x / a.ntiles_n;
    const int NV = (int)a.NV;
    const int mtiles = (NV + 127) / 128;
    const int obase = nt * NT;

    // ---- one-time setup -------------------------------------------------------------------
    if (tid == 0) {
        for (int s = 0; s < NSTAGE; s++) { mbar_init(BAR_AFULL(s), kWsExpThreads / 32); mbar_init(BAR_AEMPTY(s), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(BAR_CFULL(b), 1); mbar_init(BAR_CEMPTY(b), 4 * EPI_GROUPS); }
        *sAbort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(smem_u32(sTmem), TM_COLS);
    {
        const uint4* src = a.wi8 + (size_t)nt * RS * (a.C >> 4) * NT;
        const int nB = RS * (a.C >> 4) * NT;
        for (int i = tid; i < nB; i += kWsThreads) sB[i] = __ldg(src + i);
        for (int i = tid; i < NT; i += kWsThreads) {
            // integer form of  !((float)v < thr)  (kernel.cuh:795-796): v >= ceil(thr);
            // NaN never compares less, so the bit is always set
            int it = INT_MIN;
            if (obase + i < a.O) {
                const float t = __ldg(a.thr + obase + i);
                if (t == t) it = t >= 2147483520.0f ? INT_MAX : t <= -2147483648.0f ? INT_MIN : (int)ceilf(t);
            }
            sThr[i] = it;
        }
        for (int t = tid; t < RS; t += kWsThreads) {
            const int r = t / a.S, s = t % a.S;
            int plane = 0, off;
            if (STRIDE == 2) {
                const int ty = r - a.pad_h, tx = s - a.pad_w;
                const int py = ty & 1, px = tx & 1;
                const int dy = (ty - py) / 2, dx = (tx - px) / 2;
                plane = py * 2 + px;
                off = (dy + a.back_y) * a.PW + (dx + a.back_x);
            } else {
                off = r * a.PW + s;
            }
            sTap[t] = (plane << 24) | off;
            // A-descriptor address increments (bytes >> 4) of this tap's two k-steps
            const uint32_t byte_off = (uint32_t)plane * plane_bytes + (uint32_t)off * 16u;
            sTapK[2 * t] = byte_off >> 4;
            sTapK[2 * t + 1] = (byte_off + 2u * (uint32_t)a.NPOS * 16u) >> 4;
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *sTmem;
    const WsWait wait{sAbort, a.err_flag};

    if (tid >= kWsEpiThreads && tid < kWsEpiThreads + kWsExpThreads) {
        // =============================== expanders ==========================================
        const int et = tid - kWsEpiThreads;
        const int Cw = a.C >> 5;
        const int nq = (a.NPOS + kWsExpThreads - 1) / kWsExpThreads;      // positions per thread
        const int nent = nq * NPLANE;
        // The loader runs three stages ahead of the expander.  A stage's bits wait in one of four
        // register buffers (with a per-entry "pixel exists" mask); the stage loop is unrolled
        // by four so that buffers are addressed statically and no buffer is ever copied -- a
        // copy would make the thread wait for the load it has just issued.
        int ptr[kWsMaxEnt];                                 // loader: word offset of the pixel
        uint32_t pmask = 0;
        uint2 qa[kWsMaxEnt], qb[kWsMaxEnt], qc[kWsMaxEnt], qd[kWsMaxEnt];
        uint32_t ma = 0, mb = 0, mc = 0, md = 0;
        auto map_tile = [&](int m) {
            const int base = m * 128 - (a.back_y * a.PW + a.back_x);
            pmask = 0;
#pragma unroll
            for (int j = 0; j < kWsMaxEnt; j++) {
                ptr[j] = 0;
                if (j >= nent) continue;
                const int qi = j / NPLANE, pl = j % NPLANE;
                const int q = et + qi * kWsExpThreads;
                const int gq = base + q;
                if (q < a.NPOS && gq >= 0 && gq < NV) {
                    const int vy = fastdiv(gq, a.pw_mul, a.pw_sh), vx = gq - vy * a.PW;
                    const int n = fastdiv(vy, a.vh_mul, a.vh_sh), vr = vy - n * a.VH;
                    const int iy = STRIDE == 2 ? 2 * vr + (pl >> 1) : vr;
                    const int ix = STRIDE == 2 ? 2 * vx + (pl & 1) : vx;
                    if (vr < a.OHg && vx < a.OWg && iy < a.H && ix < a.W) {
                        ptr[j] = ((n * a.H + iy) * a.W + ix) * Cw;
                        pmask |= 1u << j;
                    }
                }
            }
        };
        // loader position (lm, lcb); load_next fetches that stage's bits and advances
        int lm = mfirst, lcb = 0;
        bool lvalid = lm < mtiles;
        if (lvalid) map_tile(lm);
        auto load_next = [&](uint2 (&dst)[kWsMaxEnt], uint32_t& dm) {
            dm = 0;
            if (!lvalid) return;
            dm = pmask;
#pragma unroll
            for (int j = 0; j < kWsMaxEnt; j++)
                dst[j] = ((pmask >> j) & 1u) ? ldg64(a.in + ptr[j] + lcb * 2) : make_uint2(0u, 0u);
            if (++lcb == NCB) {
                lcb = 0;
                lm += mstep;
                lvalid = lm < mtiles;
                if (lvalid) map_tile(lm);
            }
        };
        const int my_tiles = mfirst < mtiles ? (mtiles - mfirst + mstep - 1) / mstep : 0;
        const uint32_t nstages = (uint32_t)my_tiles * NCB;
        uint32_t it = 0;
        long long tr_wait = 0, tr_load = 0, tr_exp = 0, tr_fence = 0;
        // one stage: refill `fill` (three stages ahead), expand `use` into ring slot it % NSTAGE
        auto step = [&](uint2 (&use)[kWsMaxEnt], uint32_t um, uint2 (&fill)[kWsMaxEnt], uint32_t& fm) -> bool {
            const long long c0 = clock64();
            load_next(fill, fm);
            const long long c1 = clock64();
            tr_load += c1 - c0;
            const int s = it % NSTAGE;
            if (!wait.timed(BAR_AEMPTY(s), ((it / NSTAGE) & 1) ^ 1, tr_wait)) return false;
            const long long c2 = clock64();
            uint4* stage = reinterpret_cast<uint4*>(sAraw + (size_t)s * stage_bytes);
#pragma unroll
            for (int j = 0; j < kWsMaxEnt; j++) {
                if (j >= nent) continue;
                const int qi = j / NPLANE, pl = j % NPLANE;
                const int q = et + qi * kWsExpThreads;
                if (q >= a.NPOS) continue;
                uint4* dst = stage + (size_t)pl * 4 * a.NPOS + q;
                if ((um >> j) & 1u) {
                    dst[0] = expand16(use[j].x >> 16);
                    dst[(size_t)a.NPOS] = expand16(use[j].x & 0xFFFFu);
                    dst[(size_t)2 * a.NPOS] = expand16(use[j].y >> 16);
                    dst[(size_t)3 * a.NPOS] = expand16(use[j].y & 0xFFFFu);
                } else {
                    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                    dst[0] = z; dst[(size_t)a.NPOS] = z;
                    dst[(size_t)2 * a.NPOS] = z; dst[(size_t)3 * a.NPOS] = z;
                }
            }
            const long long c3 = clock64();
            tr_exp += c3 - c2;
            fence_proxy_async();                        // each writer publishes its own stores,
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_AFULL(s));   // then one arrival per warp
            tr_fence += clock64() - c3;
            it++;
            return true;
        };
        const long long tr_t0 = clock64();
        load_next(qa, ma);
        load_next(qb, mb);
        load_next(qc, mc);
        while (it < nstages) {
            if (!step(qa, ma, qd, md)) break;
            if (it >= nstages) break;
            if (!step(qb, mb, qa, ma)) break;
            if (it >= nstages) break;
            if (!step(qc, mc, qb, mb)) break;
            if (it >= nstages) break;
            if (!step(qd, md, qc, mc)) break;
        }
        if (a.trace && blockIdx.x == 0 && et == 0) { a.trace[0] = clock64() - tr_t0; a.trace[1] = tr_wait; a.trace[2] = nstages; a.trace[9] = tr_load; a.trace[10] = tr_exp; a.trace[11] = tr_fence; }
    } else if (warp == MMA_WARP) {
        // =============================== MMA issuer =========================================
        // Where the MMAs are the critical path (n-tile of 128 or more, or several channel blocks per
        // tile) the whole warp runs the control flow converged and polls the barriers, and one
        // elected lane issues: what the issuing thread executes between two MMAs is time the
        // tensor pipe idles, and a lone lane in a diverged warp pays far more per branch and per
        // wait.  Narrow layers wait for their epilogue instead and measured faster with a single
        // lane in the loop (the other 31 parked at the __syncwarp below).
        const bool converged = NT >= 128 || NCB >= 2;
        const bool elected = elect_one();
        if (converged || lane == 0) {
            const bool leader = converged ? elected : true;
            // Descriptors differ only in their 14-bit address field (low word), so the issue
            // loop adds precomputed (byte offset >> 4) values to two base descriptors: the A
            // offset of (tap, k-step) comes from a table (held in registers for 3x3 filters),
            // the B descriptor advances by one k-step (two 16-channel chunks) per MMA.
            const uint32_t lboA = (uint32_t)a.NPOS * 16u, lboB = NT * 16u;
            const uint64_t descA0 = smem_desc(smem_u32(sAraw), lboA, 128u);
            const uint64_t descB0 = smem_desc(smem_u32(sB), lboB, 128u);
            const uint32_t aHi = (uint32_t)(descA0 >> 32), bHi = (uint32_t)(descB0 >> 32);
            const uint32_t aLo0 = (uint32_t)descA0, bLo0 = (uint32_t)descB0;
            const uint32_t stepB = (2u * lboB) >> 4, stepStage = stage_bytes >> 4;
            constexpr uint32_t IDESC = idesc_i8(NT);
            const bool rs9 = RS == 9;
            uint32_t tapk[18];
#pragma unroll
            for (int i = 0; i < 18; i++) tapk[i] = rs9 ? sTapK[i] : 0u;
            uint32_t it = 0, tc = 0;
            bool ok = true;
            long long tr_wc = 0, tr_wa = 0;
            const long long tr_t0 = clock64();
            for (int m = mfirst; m < mtiles && ok; m += mstep, tc++) {
                const int b = tc & 1;
                ok = a.trace ? wait.timed(BAR_CEMPTY(b), ((tc >> 1) & 1) ^ 1, tr_wc) : wait.spin(BAR_CEMPTY(b), ((tc >> 1) & 1) ^ 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + b * NT;
                uint32_t acc = 0;
                uint32_t bLo = bLo0;
                for (int cb = 0; cb < NCB && ok; cb++, it++) {
                    const int s = it % NSTAGE;
                    ok = a.trace ? wait.timed(BAR_AFULL(s), (it / NSTAGE) & 1, tr_wa) : wait.spin(BAR_AFULL(s), (it / NSTAGE) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t aLo = aLo0 + s * stepStage;
                    if (leader) {
                    if (rs9) {
#pragma unroll
                        for (int i = 0; i < 18; i++)
                            mma_i8_split(d, aLo + tapk[i], aHi, bLo + i * stepB, bHi, IDESC, i == 0 ? acc : 1u);
                        bLo += 18 * stepB;
                    } else {
                        for (int t = 0; t < RS; t++) {
                            const uint2 ao = *reinterpret_cast<const uint2*>(sTapK + 2 * t);
                            mma_i8_split(d, aLo + ao.x, aHi, bLo, bHi, IDESC, acc);
                            mma_i8_split(d, aLo + ao.y, aHi, bLo + stepB, bHi, IDESC, 1u);
                            acc = 1;
                            bLo += 2 * stepB;
                        }
                    }
                    acc = 1;
                    mma_commit(BAR_AEMPTY(s));          // stage free once these MMAs have read it
                    }
                }
                if (ok && leader) mma_commit(BAR_CFULL(b));       // accumulator complete
            }
            if (a.trace && blockIdx.x == 0 && leader) { a.trace[3] = clock64() - tr_t0; a.trace[4] = tr_wc; a.trace[5] = tr_wa; }
        }
        __syncwarp();
    } else if (tid < 128 * EPI_GROUPS) {
        // =============================== epilogue ===========================================
        const int row = tid & 127, grp = tid >> 7, quad = warp & 3;
        const int Ow = (a.O + 31) >> 5;
        const int lim = a.res_in ? min(a.residual_channels, a.res_in_ch) : 0;
        uint32_t tc = 0;
        bool ok = true;
        bool overflow = false;
        long long tr_w = 0, tr_tld = 0, tr_body = 0;
        const long long tr_t0 = clock64();
        // 32 int16 residual channels [o0, o0+32) of one output pixel as 8 packed pairs-of-pairs
        // (zeros where nothing is injected); 2x2 max for pooled residuals (kernel.cuh:773-783)
        auto fetch_res16 = [&](uint2 (&r)[8], int n_, int y_, int x_, size_t opix_, bool live_, int o0) {
            const short* base = reinterpret_cast<const short*>(a.res_in);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                uint2 v = make_uint2(0u, 0u);
                const int o = o0 + 4 * j;
                if (live_ && o < lim) {
                    if (a.residual_pool) {
                        const size_t b00 = (((size_t)n_ * 2 * a.OHg + 2 * y_) * 2 * a.OWg + 2 * x_) *
                                           a.res_in_ch + o;
                        const size_t rowp = (size_t)2 * a.OWg * a.res_in_ch;
                        const uint2 p0 = __ldg(reinterpret_cast<const uint2*>(base + b00));
                        const uint2 p1 = __ldg(reinterpret_cast<const uint2*>(base + b00 + a.res_in_ch));
                        const uint2 p2 = __ldg(reinterpret_cast<const uint2*>(base + b00 + rowp));
                        const uint2 p3 = __ldg(reinterpret_cast<const uint2*>(base + b00 + rowp + a.res_in_ch));
                        v.x = __vmaxs2(__vmaxs2(p0.x, p1.x), __vmaxs2(p2.x, p3.x));
                        v.y = __vmaxs2(__vmaxs2(p0.y, p1.y), __vmaxs2(p2.y, p3.y));
                    } else {
                        v = __ldg(reinterpret_cast<const uint2*>(base + opix_ * a.res_in_ch + o));
                    }
                }
                r[j] = v;
            }
        };
        // general path: add the residual of channels [o0, o0+32) straight from memory
        auto add_res_inplace = [&](int (&v)[32], int n_, int y_, int x_, size_t opix_, bool live_, int o0) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                int4 r = make_int4(0, 0, 0, 0);
                const int o = o0 + 4 * j;
                if (live_ && o < lim) {
                    if (a.residual_pool) {
                        const size_t b00 = (((size_t)n_ * 2 * a.OHg + 2 * y_) * 2 * a.OWg + 2 * x_) *
                                           a.res_in_ch + o;
                        const size_t rowp = (size_t)2 * a.OWg * a.res_in_ch;
                        r = max4(max4(ld_res4(a.res_in, a.res_in_bytes, b00),
                                      ld_res4(a.res_in, a.res_in_bytes, b00 + a.res_in_ch)),
                                 max4(ld_res4(a.res_in, a.res_in_bytes, b00 + rowp),
                                      ld_res4(a.res_in, a.res_in_bytes, b00 + rowp + a.res_in_ch)));
                    } else {
                        r = ld_res4(a.res_in, a.res_in_bytes, opix_ * a.res_in_ch + o);
                    }
                }
                v[4 * j] += r.x; v[4 * j + 1] += r.y; v[4 * j + 2] += r.z; v[4 * j + 3] += r.w;
            }
        };
        uint2 rnext[8];
#pragma unroll
        for (int j = 0; j < 8; j++) rnext[j] = make_uint2(0u, 0u);
        for (int m = mfirst; m < mtiles && ok; m += mstep, tc++) {
            const int b = tc & 1;
            const int p = m * 128 + row;
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
            // ---- residual prefetch --------------------------------------------------------
            // The residual of this thread's row is fetched one tile ahead (packed int16 pairs
            // stay packed in registers until they are added), so its memory latency overlaps
            // the previous tile's epilogue instead of stalling this one.  int32 residuals and
            // the rare case of several column groups per thread are loaded in place.
            if (a.res_in && m == mfirst && NB_PER == 1 && a.res_in_bytes == 2)
                fetch_res16(rnext, n, y, x, opix, live, obase + grp * 32);
            uint2 rcur16[8];
            if (a.res_in && NB_PER == 1 && a.res_in_bytes == 2) {
#pragma unroll
                for (int j = 0; j < 8; j++) rcur16[j] = rnext[j];
                const int mn = m + mstep;
                if (mn < mtiles) {                         // next tile's row, same column group
                    const int pn = mn * 128 + row;
                    bool ln = false;
                    int nn = 0, yn = 0, xn = 0;
                    if (pn < NV) {
                        const int vy = fastdiv(pn, a.pw_mul, a.pw_sh);
                        xn = pn - vy * a.PW;
                        nn = fastdiv(vy, a.vh_mul, a.vh_sh);
                        yn = vy - nn * a.VH;
                        ln = xn < a.OWg && yn < a.OHg;
                    }
                    fetch_res16(rnext, nn, yn, xn, ((size_t)nn * a.OHg + yn) * a.OWg + xn, ln, obase + grp * 32);
                }
            }
            ok = wait.timed(BAR_CFULL(b), (tc >> 1) & 1, tr_w);
            if (!ok) break;
            tc_fence_after();
            const long long e0 = clock64();
            uint32_t words[NB_PER];
#pragma unroll
            for (int k = 0; k < NB_PER; k++) {
                const int nb = grp + k * EPI_GROUPS;
                int v[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + b * NT + nb * 32, v);
                tmem_ld_wait();
                if (k == 0) tr_tld += clock64() - e0;
                if (k == NB_PER - 1) {                    // this warp is done with the accumulator
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR_CEMPTY(b));
                }
                const int o0 = obase + nb * 32;
                if (live && a.acc_out) {
                    int4* dst = reinterpret_cast<int4*>(a.acc_out + opix * a.O + o0);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        dst[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
                if (a.res_in) {
                    if (NB_PER == 1 && a.res_in_bytes == 2) {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            v[4 * j] += (int)(short)(rcur16[j].x & 0xFFFFu);
                            v[4 * j + 1] += (int)(short)(rcur16[j].x >> 16);
                            v[4 * j + 2] += (int)(short)(rcur16[j].y & 0xFFFFu);
                            v[4 * j + 3] += (int)(short)(rcur16[j].y >> 16);
                        }
                    } else {
                        add_res_inplace(v, n, y, x, opix, live, o0);
                    }
                }
                uint32_t word = 0;
                const int4* th4 = reinterpret_cast<const int4*>(sThr + nb * 32);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int4 th = th4[j];                  // one broadcast load per 4 channels
                    if (v[4 * j] >= th.x) word |= 0x80000000u >> (4 * j);
                    if (v[4 * j + 1] >= th.y) word |= 0x80000000u >> (4 * j + 1);
                    if (v[4 * j + 2] >= th.z) word |= 0x80000000u >> (4 * j + 2);
                    if (v[4 * j + 3] >= th.w) word |= 0x80000000u >> (4 * j + 3);
                }
                words[k] = word;
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
                                ((size_t)y * a.OWg + x) * Ow + (obase >> 5);
#pragma unroll
                for (int k = 0; k < NB_PER; k++) dst[grp + k * EPI_GROUPS] = words[k];
                if (a.nxt) {
#pragma unroll
                    for (int k = 0; k < NB_PER; k++)
                        store_next_planes(a, n, y, x, obase + (grp + k * EPI_GROUPS) * 32, words[k], 32);
                }
            }
            tr_body += clock64() - e0;
        }
        if (overflow) atomicExch(a.err_flag, 2);
        if (a.trace && blockIdx.x == 0 && tid == 0) { a.trace[6] = clock64() - tr_t0; a.trace[7] = tr_w; a.trace[8] = tc; a.trace[12] = tr_tld; a.trace[13] = tr_body; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace umma
}  // namespace tcbnn
