// tcgen05 binary convolution fed from a pre-expanded input (stride 1, C <= 512), 4-bit operands:
// tcgen05.mma kind::mxf4 on +-1.0 as e2m1 with unit block scales (bconv_umma.cuh), 128 x NT x 64
// per instruction -- one MMA per filter tap and 64-channel block.
//
// In bconv_umma_ws.cuh seven warps of every CTA turn packed bits into +-1 bytes, stage by
// stage, next to the epilogue warps; with 16 warps per SM that chain of dependent scalar
// instructions is what the layers wait for.  Here the expansion is done by whoever produces the
// input -- the previous layer's epilogue, or a separate streaming pass (expand_raster below: full
// occupancy, HBM-bound, 8 bytes in and 32 out per pixel and 64-channel block) -- which writes it
// as +-1 nibbles straight in the layout the MMA wants: for every 32-channel chunk a plane
// [raster position][16 bytes] over the zero-padded virtual raster of bconv_umma.cuh, zeros on the
// dead bands.  A tile's patch is then two contiguous runs per 64-channel block, which one thread
// fetches with bulk asynchronous copies (cp.async.bulk + mbarrier complete_tx).  With half a byte
// per channel the filter block of 128 output channels stays resident up to 256 input channels
// (64 output channels at 512), so the wide layers run filter-stationary too.  The CTA becomes
//
//   warps 0-15  epilogue   : warp w reads TMEM lanes 32*(w%4).., columns (w/4) * NT/4 ..
//   warp  16    loader     : one lane, bulk copies of the patch planes into the stage ring
//   warp  17    MMA issuer : one lane, as in bconv_umma_ws.cuh
//
// i.e. twice the epilogue threads on every accumulator, each holding a quarter of its columns.
// The scratch planes come from the caller (tcbnn_conv_workspace_bytes).
#pragma once
#include "bconv_umma_as.cuh"

namespace tcbnn {
namespace umma {

constexpr int kPreEpiThreads = 512;         // epilogue threads of the one-CTA-per-SM form (16 warps)
// One MMA-issuing warp.  (Two issuers on alternate tiles were tried and are wrong as well as no
// faster: an mbarrier wait names its phase by parity only, so a waiter must see every phase of a
// barrier; with two consumers alternating on the same ring slot the one that runs ahead finds the
// parity of the phase before last already complete and reads a slot that has not been refilled.)
constexpr int kPreMmaWarps = 1;
constexpr int kPreThreads = kPreEpiThreads + 32 + 32 * kPreMmaWarps;
// EPIW, the kernel's third template argument, is the number of epilogue warps: 16 (one CTA per SM,
// all of tensor memory) or 8 (n-tile 64 only: each thread then takes 32 columns instead of 16, the
// CTA allocates half of tensor memory and two CTAs share an SM -- twice the independent
// loader / issuer / epilogue pipelines, so that one CTA's barrier round trips and epilogue
// latency are covered by the other's work, and half the per-thread bookkeeping per output).
__host__ __device__ constexpr int pre_threads(int epiw) { return epiw * 32 + 32 + 32 * kPreMmaWarps; }
constexpr int kPreMaxStages = 8;           // patch ring depth is chosen by the host from the shared memory left

// positions of zero padding in front of the planes (a tile's patch starts up to back_y*PW+back_x
// positions before its first output position) and the rounded-up plane length
__host__ __device__ inline long long pre_front(int back_y, int back_x, int PW) {
    return ((long long)back_y * PW + back_x + 7) & ~7LL;
}
__host__ __device__ inline long long pre_plane_positions(long long NV, int npos, long long front) {
    return ((front + ((NV + 127) / 128) * 128 + npos + 7) & ~7LL);
}
// nplane: 1 for stride 1, 4 for stride 2 (the input's four row / column parity planes)
__host__ __device__ inline size_t pre_smem_bytes(int npos, int C, int RS, int nt, int stages, int nplane) {
    return (size_t)stages * nplane * 2 * npos * 16 + (size_t)RS * C * nt / 2 + nt * 8 + RS * 8 + 40 * 8 + 64;
}
// two buffers of a tile's int16 residual rows (128 rows x nt channels), staged in shared memory
__host__ __device__ inline size_t pre_res_stage_bytes(int nt) { return (size_t)2 * 128 * nt * 2 + 128; }

// packed bits [B][H][W][C/32] -> planes [C/32][nplane][plane_positions][16 B] of +-1 nibbles, zero
// where the raster position is padding or outside the batch.  Stride 1: one plane, the raster of
// the input.  Stride 2: four planes, plane (py, px) holds input pixel (2*vr + py, 2*vx + px) at
// raster position (vr, vx) of the OUTPUT grid, so that a filter tap is again a fixed offset.
__device__ __forceinline__ void expand_raster(const ConvWsArgs& a, uint4* planes, long long plane_positions,
                                              long long front) {
    const int NCB = a.C >> 6, Cw = a.C >> 5;
    const int nplane = a.stride == 2 ? 4 : 1;
    const long long total = plane_positions * NCB * nplane;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int cp = (int)(i / plane_positions);             // (channel block, plane)
        const int cb = cp / nplane, pl = cp - cb * nplane;
        const long long slot = i - (long long)cp * plane_positions;
        const long long gq = slot - front;
        uint4 e0 = make_uint4(0u, 0u, 0u, 0u), e1 = e0;
        if (gq >= 0 && gq < a.NV) {
            const int vy = fastdiv((int)gq, a.pw_mul, a.pw_sh), vx = (int)gq - vy * a.PW;
            const int n = fastdiv(vy, a.vh_mul, a.vh_sh), vr = vy - n * a.VH;
            const int iy = nplane == 4 ? 2 * vr + (pl >> 1) : vr, ix = nplane == 4 ? 2 * vx + (pl & 1) : vx;
            if (vr < a.OHg && vx < a.OWg && iy < a.H && ix < a.W) {
                const uint2 b = ldg64(a.in + ((size_t)(n * a.H + iy) * a.W + ix) * Cw + cb * 2);
                e0 = expand32_f4(b.x); e1 = expand32_f4(b.y);
            }
        }
        uint4* dst = planes + ((size_t)(cb * 2) * nplane + pl) * plane_positions + slot;
        dst[0] = e0;
        dst[(size_t)nplane * plane_positions] = e1;
    }
}

// Staged epilogue: int16 residual rows travel through shared memory.  The four epilogue warps that
// share 32 rows of a tile (same TMEM lane quadrant, different column groups) form a group: the live
// pixels among its rows are consecutive rows of the residual tensors, so the group's 128 threads
// move them as whole 128-byte lines (cp.async in, 16-byte stores out: 4 lines per instruction) into
// a buffer of its own whose 16-byte chunks are XOR-swizzled by row, and every thread then reads /
// overwrites its own pixel's chunks there without bank conflicts.  The incoming rows of the next
// tile fly while this tile is computed; the outgoing rows leave one tile late; the four groups
// meet only among themselves (one mbarrier each), never CTA-wide.  (Without it each lane moves 16-byte pieces of its own row: 32
// lines per instruction, which made L1TEX the busiest unit of these layers.)
//
// EPI selects the epilogue the kernel is compiled with, so that each carries only its own
// registers (18 warps leave 96 per thread): 0 = plain (no residual in or out, no integer output:
// the fp32 accumulator is compared with the fp32 threshold as it is), 1 = residual rows moved
// directly between registers and global memory (any element size, pooled residuals, partial
// channel ranges), 2 = staged int16 residual rows as described above.
//
// Tile-per-group epilogues (3 = no residual, 4 = chunk-major int16 residuals in and / or out): the
// forms above put all 16 epilogue warps on every tile, so that a thread holds 16 or 32 of its
// pixel's columns and pays the per-tile bookkeeping (raster position -> pixel, addresses, barrier
// waits: some 200 instructions) for that few outputs -- most of what these warps issue.  Here a
// group of 4 warps (8 at an n-tile of 128) owns a whole tile and the groups take tiles in turn: a
// thread walks 64 columns of its pixel in passes of 32, the bookkeeping is paid once per 64
// outputs, and the groups work on different accumulators at the same time (NT = 64: 4 groups on
// 7 accumulators; NT = 128: 2 groups on 3).  With one thread per pixel every tensor is touched in
// whole lines: chunk-major residuals, 16-byte plane slots, 8 bytes of packed bits -- so nothing is
// staged, and a pooled residual is read in place (four lines per chunk) instead of by a pass of
// its own.
constexpr int kEpiPlain = 0, kEpiDirect = 1, kEpiStaged = 2, kEpiTile = 3, kEpiTileRes = 4;
template <int NT, int EPI, int EPIW>
__device__ void conv_umma_pre_cta(const ConvWsArgs& a, unsigned char* smem) {
    constexpr bool RSTAGE = EPI == kEpiStaged;
    constexpr int kEpiThreads = EPIW * 32, kThreadsCta = pre_threads(EPIW);
    static_assert(EPIW == 16 || (EPIW == 8 && NT == 64 && EPI != kEpiStaged), "8 epilogue warps: n-tile 64, no staging");
    constexpr bool TILE = EPI == kEpiTile || EPI == kEpiTileRes;
    constexpr int CPT = NT < 64 ? NT : 64;            // tile-per-group: columns of a tile per thread
    constexpr int WPG = 4 * (NT / CPT);               // ... warps of a group (all rows x all columns of a tile)
    constexpr int NG = EPIW / WPG;                    // ... groups, each on a tile of its own
    // Tensor memory: accumulators (7 at NT = 64) below column 480, the unit block scales of the
    // 4-bit MMA above it; the patch ring is as deep as shared memory allows, so that no role waits
    // on another's latency.
    constexpr uint32_t TM_COLS = EPIW == 16 ? 512 : 256, SF_COL = TM_COLS - 32;
    constexpr int NACC = NT >= 128 ? (TILE ? 3 : 2)   // measured: deeper does not pay at NT = 128 when all warps share a tile
                                   : ((SF_COL / NT) > 8 ? 8 : (SF_COL / NT));
    const int NSTAGE = a.pre_stages;
    constexpr int COLS = NT / (EPIW / 4);             // accumulator columns per epilogue thread
    static_assert(COLS == 8 || COLS == 16 || COLS == 32, "n-tile of 32, 64 or 128");
    constexpr int LOAD_WARP = EPIW, MMA_WARP = LOAD_WARP + 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RS = a.R * a.S, NCB = a.C >> 6;
    const int NPLANE = a.stride == 2 ? 4 : 1;
    const uint32_t plane_bytes = 2u * a.NPOS * 16u;           // two 32-channel chunk planes
    const uint32_t block_bytes = NPLANE * plane_bytes;        // one 64-channel block of a tile's patch
    // A stage holds one, two or four blocks: the issuing thread's wait / commit round per stage is
    // time the tensor pipe idles, so layers with several blocks pay it once per 2 or 4 x RS MMAs.
    const int CBS = a.pre_cbs;
    const uint32_t stage_bytes = (uint32_t)CBS * block_bytes;

    unsigned char* sAraw = smem;
    uint4* sB = reinterpret_cast<uint4*>(smem + (size_t)NSTAGE * stage_bytes);
    int* sThr = reinterpret_cast<int*>(sB + (size_t)RS * (a.C >> 5) * NT);
    float* sThrF = reinterpret_cast<float*>(sThr + NT);       // the thresholds as given (fp32)
    uint32_t* sTapK = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sThrF + NT) + 7) & ~(uintptr_t)7);
    uint64_t* sBar = reinterpret_cast<uint64_t*>(sTapK + 2 * RS);
    // barriers: a_full[8], a_empty[8], acc_full[8], acc_empty[8], epilogue groups [4], drain
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 40);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sTmem + 1);
    unsigned char* sRes = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sTmem + 2) + 127) & ~(uintptr_t)127);
    const uint32_t bar0 = smem_u32(sBar);
    auto BAR_EPI = [&](int g) { return bar0 + 8u * (32 + g); };    // rendezvous of an epilogue group (staged epilogue)
    const uint32_t BAR_DRAIN = bar0 + 8u * 36;         // MMAs still in flight when the issuer gives up
    auto BAR_AFULL = [&](int s) { return bar0 + 8u * s; };
    auto BAR_AEMPTY = [&](int s) { return bar0 + 8u * (8 + s); };
    auto BAR_CFULL = [&](int b) { return bar0 + 8u * (16 + b); };
    auto BAR_CEMPTY = [&](int b) { return bar0 + 8u * (24 + b); };

    // CTA -> (n-tile, first m-tile, stride over m-tiles).  Normally every n-tile gets the same
    // share of the grid; where only the first n-tiles carry the epilogue's expensive part (a pooled
    // residual injected into the first channels) the host gives those more CTAs each.
    int nt, mfirst, mstep;
    if (a.nt_heavy > 0) {
        const int nh = a.nt_heavy * a.per_heavy;
        if ((int)blockIdx.x < nh) {
            nt = blockIdx.x % a.nt_heavy; mfirst = blockIdx.x / a.nt_heavy; mstep = a.per_heavy;
        } else {
            const int r = blockIdx.x - nh, nl = a.ntiles_n - a.nt_heavy;
            nt = a.nt_heavy + r % nl; mfirst = r / nl; mstep = a.per_light;
        }
    } else {
        nt = blockIdx.x % a.ntiles_n; mfirst = blockIdx.x / a.ntiles_n; mstep = gridDim.x / a.ntiles_n;
    }
    const int NV = (int)a.NV;
    const int mtiles = (NV + 127) / 128;
    const int obase = nt * NT;

    if (tid == 0) {
        for (int s = 0; s < 8; s++) { mbar_init(BAR_AFULL(s), 1); mbar_init(BAR_AEMPTY(s), 1); }
        for (int b = 0; b < 8; b++) { mbar_init(BAR_CFULL(b), 1); mbar_init(BAR_CEMPTY(b), TILE ? WPG : EPIW); }
        for (int g = 0; g < 4; g++) mbar_init(BAR_EPI(g), EPIW / 4);
        mbar_init(BAR_DRAIN, 1);
        *sAbort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(smem_u32(sTmem), TM_COLS);
    {
        const uint4* src = a.wf4 + (size_t)nt * RS * (a.C >> 5) * NT;
        const int nB = RS * (a.C >> 5) * NT;
        for (int i = tid; i < nB; i += kThreadsCta) sB[i] = __ldg(src + i);
        for (int i = tid; i < NT; i += kThreadsCta) {
            // integer form of  !((float)v < thr)  (kernel.cuh:795-796): v >= ceil(thr)
            int it = INT_MIN;
            float tf = __int_as_float(0x7FC00000);       // NaN: never "less", the bit is always set
            if (obase + i < a.O) {
                const float t = __ldg(a.thr + obase + i);
                tf = t;
                if (t == t) it = t >= 2147483520.0f ? INT_MAX : t <= -2147483648.0f ? INT_MIN : (int)ceilf(t);
            }
            sThr[i] = it;
            sThrF[i] = tf;
        }
        for (int t = tid; t < RS; t += kThreadsCta) {
            // offset of the tap's operand inside a stage, in 16-byte units
            const int r = t / a.S, sx = t % a.S;
            if (NPLANE == 4) {
                const int ty = r - a.pad_h, tx = sx - a.pad_w;
                const int py = ty & 1, px = tx & 1;
                const int dy = (ty - py) / 2, dx = (tx - px) / 2;
                sTapK[t] = (uint32_t)(py * 2 + px) * (plane_bytes >> 4) + (uint32_t)((dy + a.back_y) * a.PW + (dx + a.back_x));
            } else {
                sTapK[t] = (uint32_t)(r * a.PW + sx);
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *sTmem;
    if (warp < 4) tmem_fill_unit_scales(tmem, SF_COL);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const WsWait wait{sAbort, a.err_flag};

    if (warp == LOAD_WARP) {
        // =============================== patch loader =======================================
        // Lane 0 waits for a free stage and announces the bytes; up to eight lanes then issue the
        // stage's bulk copies between them.  A thread is busy 100-200 clocks per copy whatever its
        // size, and a stage of a stride-2 layer is 8 to 32 copies (four parity planes x two chunks
        // per 64-channel block): one lane issuing them all took longer than the stage's MMAs.
        {
            constexpr int kIssueLanes = 8;
            const long long back = (long long)a.back_y * a.PW + a.back_x;
            const int ncopy = CBS * NPLANE * 2;
            uint32_t it = 0, sph = 0;
            int s = 0;
            bool ok = true;
            for (int m = mfirst; m < mtiles && ok; m += mstep) {
                const long long slot0 = (long long)m * 128 - back + a.pre_front;
                for (int cb = 0; cb < NCB; cb += CBS, it++) {
                    // the ring is several tiles deep: lane 0 mostly waits for a slot, and sleeps
                    // between polls so that it does not take issue slots from the epilogue warps
                    if (lane == 0) ok = wait.relaxed(BAR_AEMPTY(s), sph ^ 1);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    if (lane == 0) mbar_expect_tx(BAR_AFULL(s), stage_bytes);
                    __syncwarp();
                    const uint32_t dst = smem_u32(sAraw + (size_t)s * stage_bytes);
                    if (lane < kIssueLanes) {
                        for (int i = lane; i < ncopy; i += kIssueLanes) {
                            const int c = i & 1, pl = (i >> 1) % NPLANE, sub = (i >> 1) / NPLANE;
                            bulk_g2s(dst + (uint32_t)sub * block_bytes + (uint32_t)(pl * 2 + c) * (uint32_t)a.NPOS * 16u,
                                     a.pre + ((size_t)((cb + sub) * 2 + c) * NPLANE + pl) * a.pre_positions + slot0,
                                     (uint32_t)a.NPOS * 16u, BAR_AFULL(s));
                        }
                    }
                    if (++s == NSTAGE) { s = 0; sph ^= 1; }
                }
            }
            if (!ok && lane == 0) {
                // giving up: wait (bounded) for the copies still in flight before the CTA exits;
                // stages below `s` were last filled in this pass over the ring, the others in the one before
                for (int s2 = 0; s2 < NSTAGE; s2++) {
                    const bool this_pass = s2 < s;
                    if (!this_pass && it < (uint32_t)NSTAGE) continue;
                    for (int i = 0; i < (1 << 20); i++)
                        if (mbar_try_wait(BAR_AFULL(s2), this_pass ? sph : sph ^ 1)) break;
                }
            }
        }
        __syncwarp();
    } else if (warp >= MMA_WARP && warp < MMA_WARP + kPreMmaWarps) {
        // =============================== MMA issuer =========================================
        // The whole warp runs the control flow converged and polls the barriers, and one elected
        // lane issues: what the issuing thread executes between two MMAs is time the tensor pipe
        // idles, and a lone lane in a diverged warp pays far more per branch and per wait.
        constexpr bool converged = true;
        const bool elected = elect_one();
        if (converged || lane == 0) {
            const bool leader = converged ? elected : true;
            const uint32_t lboA = (uint32_t)a.NPOS * 16u, lboB = NT * 16u;
            const uint64_t descA0 = smem_desc(smem_u32(sAraw), lboA, 128u);
            const uint64_t descB0 = smem_desc(smem_u32(sB), lboB, 128u);
            const uint32_t aHi = (uint32_t)(descA0 >> 32), bHi = (uint32_t)(descB0 >> 32);
            const uint32_t aLo0 = (uint32_t)descA0, bLo0 = (uint32_t)descB0;
            const uint32_t stepB = (2u * lboB) >> 4, stepStage = stage_bytes >> 4;   // one tap = two chunks of B
            const uint32_t stepBlock = block_bytes >> 4;
            constexpr uint32_t IDESC = idesc_f4(NT);
            const uint32_t sfa = tmem + SF_COL, sfb = tmem + SF_COL + 16;
            const bool rs9 = RS == 9;
            uint32_t tapk[9];                              // 3x3 filters: the tap offsets in registers
#pragma unroll
            for (int t = 0; t < 9; t++) tapk[t] = rs9 ? sTapK[t] : 0u;
            const uint32_t w2 = (uint32_t)(warp - MMA_WARP);
            uint32_t it = 0;
            bool ok = true;
            long long tr_wc = 0, tr_wa = 0;
            const long long tr_t0 = clock64();
            // ring slot, accumulator and their phases as running counters: a division by the
            // ring depth per stage would sit between two groups of MMAs
            static_assert(kPreMmaWarps == 1, "the counters below assume one issuing warp");
            int s = 0, b = 0;
            uint32_t sph = 0, bph = 0;
            for (uint32_t tc = w2; (long long)mfirst + (long long)tc * mstep < mtiles && ok; tc += kPreMmaWarps) {
                ok = a.trace ? wait.timed(BAR_CEMPTY(b), bph ^ 1, tr_wc) : wait.spin(BAR_CEMPTY(b), bph ^ 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + b * NT;
                uint32_t acc = 0;
                uint32_t bLo = bLo0;
                for (int cb = 0; cb < NCB && ok; cb += CBS, it++) {
                    ok = a.trace ? wait.timed(BAR_AFULL(s), sph, tr_wa) : wait.spin(BAR_AFULL(s), sph);
                    if (!ok) break;
                    tc_fence_after();
                    if (leader) {
                    for (int sub = 0; sub < CBS; sub++) {
                        const uint32_t aLo = aLo0 + s * stepStage + sub * stepBlock;
                        if (rs9) {
#pragma unroll
                            for (int t = 0; t < 9; t++)
                                mma_f4_split(d, aLo + tapk[t], aHi, bLo + t * stepB, bHi, IDESC, t == 0 ? acc : 1u, sfa, sfb);
                            bLo += 9 * stepB;
                        } else {
                            for (int t = 0; t < RS; t++) {
                                mma_f4_split(d, aLo + sTapK[t], aHi, bLo, bHi, IDESC, acc, sfa, sfb);
                                acc = 1;
                                bLo += stepB;
                            }
                        }
                        acc = 1;
                    }
                    mma_commit(BAR_AEMPTY(s));          // stage free once these MMAs have read it
                    }
                    if (++s == NSTAGE) { s = 0; sph ^= 1u; }
                }
                if (ok && leader) mma_commit(BAR_CFULL(b));       // accumulator complete
                if (++b == NACC) { b = 0; bph ^= 1u; }
            }
            if (!ok && leader) {
                // giving up: the MMAs already issued must have finished before tensor memory is freed
                mma_commit(BAR_DRAIN);
                for (int i = 0; i < (1 << 20); i++)
                    if (mbar_try_wait(BAR_DRAIN, 0)) break;
            }
            if (a.trace && blockIdx.x == 0 && leader && w2 == 0) { a.trace[3] = clock64() - tr_t0; a.trace[4] = tr_wc; a.trace[5] = tr_wa; a.trace[2] = it; }
        }
        __syncwarp();
    } else if (TILE && tid < kEpiThreads) {
        // =============================== epilogue, a tile per group ==========================
        constexpr bool RES = EPI == kEpiTileRes;
        constexpr int PASSES = CPT / 32;
        const int grp = warp / WPG, quad = warp & 3, half = (warp % WPG) >> 2;
        const int row = quad * 32 + lane;
        const int Ow = (a.O + 31) >> 5;
        // Pass k of a thread covers the tile's 32-column block k (groups of 4 warps) or 2k + half
        // (groups of 8: the two halves interleave, so that a residual injected into the first
        // channels only -- the first block of a stage -- is shared between them).
        constexpr int HSTEP = WPG / 4;                     // 32-column blocks between a thread's passes
        const int o0 = obase + half * 32;                  // this thread's first output channel
        const int lim = (RES && a.res_in) ? min(a.residual_channels, a.res_in_ch) : 0;
        const bool has_in = RES && a.res_in && o0 < lim;
        const uint4* rin = reinterpret_cast<const uint4*>(a.res_in) + (size_t)(o0 >> 3) * a.res_in_npix;
        uint4* rout = reinterpret_cast<uint4*>(a.res_out) + (size_t)(o0 >> 3) * a.res_out_npix;
        bool ok = true, overflow = false;
        uint32_t done = 0;
        long long tr_w = 0;
        const long long tr_t0 = clock64();
        for (uint32_t tc = grp; (long long)mfirst + (long long)tc * mstep < mtiles && ok; tc += NG, done++) {
            const int m = mfirst + (int)tc * mstep;
            const int b = (int)(tc % NACC);
            const uint32_t bph = (tc / NACC) & 1u;
            // raster position -> output pixel
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
            // injected residual of pass k (channels o0 + 32k ..): zeros where nothing is injected;
            // 2x2 max for pooled residuals (kernel.cuh:773-783)
            uint4 r[4];
            auto fetch = [&](int k) {
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                if (a.residual_pool) {
                    const size_t i00 = ((size_t)n * 2 * a.OHg + 2 * y) * 2 * a.OWg + 2 * x, rw = (size_t)2 * a.OWg;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        r[j] = z;
                        if (live && o0 + 32 * HSTEP * k + 8 * j < lim) {
                            const uint4* q = rin + (size_t)(4 * HSTEP * k + j) * a.res_in_npix + i00;
                            const uint4 w0 = __ldg(q), w1 = __ldg(q + 1), w2 = __ldg(q + rw), w3 = __ldg(q + rw + 1);
                            r[j].x = __vmaxs2(__vmaxs2(w0.x, w1.x), __vmaxs2(w2.x, w3.x));
                            r[j].y = __vmaxs2(__vmaxs2(w0.y, w1.y), __vmaxs2(w2.y, w3.y));
                            r[j].z = __vmaxs2(__vmaxs2(w0.z, w1.z), __vmaxs2(w2.z, w3.z));
                            r[j].w = __vmaxs2(__vmaxs2(w0.w, w1.w), __vmaxs2(w2.w, w3.w));
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        r[j] = (live && o0 + 32 * HSTEP * k + 8 * j < lim)
                                   ? __ldg(rin + (size_t)(4 * HSTEP * k + j) * a.res_in_npix + opix) : z;
                }
            };
            if (RES && has_in) fetch(0);                   // flies while the accumulator is awaited
            ok = (a.trace && blockIdx.x == 0) ? wait.timed(BAR_CFULL(b), bph, tr_w) : wait.relaxed(BAR_CFULL(b), bph);
            if (!ok) break;
            tc_fence_after();
            uint32_t words[PASSES];
#pragma unroll
            for (int k = 0; k < PASSES; k++) {
                int v[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + b * NT + (HSTEP * k + half) * 32, v);
                tmem_ld_wait();
                if (k == PASSES - 1) {
                    tc_fence_before();                     // this warp is done with the accumulator
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR_CEMPTY(b));
                }
                uint32_t word = 0;                         // channel c of the pass at bit 31 - c
                if (!RES) {
                    // the reference's comparison as it stands, !((float)value < threshold)
                    // (kernel.cuh:795-796), on the fp32 accumulator
                    const float4* tf4 = reinterpret_cast<const float4*>(sThrF + (HSTEP * k + half) * 32);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float4 th = tf4[j];
                        if (!(__int_as_float(v[4 * j]) < th.x)) word |= 0x80000000u >> (4 * j);
                        if (!(__int_as_float(v[4 * j + 1]) < th.y)) word |= 0x80000000u >> (4 * j + 1);
                        if (!(__int_as_float(v[4 * j + 2]) < th.z)) word |= 0x80000000u >> (4 * j + 2);
                        if (!(__int_as_float(v[4 * j + 3]) < th.w)) word |= 0x80000000u >> (4 * j + 3);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = f4_acc_to_int(v[j]);   // fp32 accumulators, exact integers
                    if (has_in) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            v[8 * j] += (int)(short)(r[j].x & 0xFFFFu);
                            v[8 * j + 1] += (int)(short)(r[j].x >> 16);
                            v[8 * j + 2] += (int)(short)(r[j].y & 0xFFFFu);
                            v[8 * j + 3] += (int)(short)(r[j].y >> 16);
                            v[8 * j + 4] += (int)(short)(r[j].z & 0xFFFFu);
                            v[8 * j + 5] += (int)(short)(r[j].z >> 16);
                            v[8 * j + 6] += (int)(short)(r[j].w & 0xFFFFu);
                            v[8 * j + 7] += (int)(short)(r[j].w >> 16);
                        }
                        if (k + 1 < PASSES) fetch(k + 1);  // the next pass's residual flies during this one's arithmetic
                    }
                    const int4* th4 = reinterpret_cast<const int4*>(sThr + (HSTEP * k + half) * 32);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int4 th = th4[j];
                        if (v[4 * j] >= th.x) word |= 0x80000000u >> (4 * j);
                        if (v[4 * j + 1] >= th.y) word |= 0x80000000u >> (4 * j + 1);
                        if (v[4 * j + 2] >= th.z) word |= 0x80000000u >> (4 * j + 2);
                        if (v[4 * j + 3] >= th.w) word |= 0x80000000u >> (4 * j + 3);
                    }
                    if (a.res_out && live) {
                        if (!a.res_out_proven) {           // a real branch: two instructions per value
                            uint32_t ovf = 0;              // |v| of every value ORed together
#pragma unroll
                            for (int j = 0; j < 32; j++) ovf |= (uint32_t)(v[j] ^ (v[j] >> 31));
                            overflow |= ovf > 32767u;      // some value outside [-32768, 32767]
                        }
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint32_t w[4];
#pragma unroll
                            for (int kk = 0; kk < 4; kk++)
                                w[kk] = ((uint32_t)v[8 * j + 2 * kk] & 0xFFFFu) | ((uint32_t)v[8 * j + 2 * kk + 1] << 16);
                            rout[(size_t)(4 * HSTEP * k + j) * a.res_out_npix + opix] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
                words[k] = word;
                if (a.nxt && live) store_next_planes(a, n, y, x, o0 + 32 * HSTEP * k, word, 32);
            }
            if (live) {
                // bits of channel o live at bit 31 - o%32 of word o/32
                uint32_t* wp = a.out + (size_t)n * a.out_image_stride + ((size_t)y * a.OWg + x) * Ow + (o0 >> 5);
                if (PASSES == 2 && HSTEP == 1 && (reinterpret_cast<uintptr_t>(wp) & 7) == 0) {
                    *reinterpret_cast<uint2*>(wp) = make_uint2(words[0], words[PASSES - 1]);
                } else {
#pragma unroll
                    for (int k = 0; k < PASSES; k++) wp[HSTEP * k] = words[k];
                }
            }
        }
        if (overflow) atomicExch(a.err_flag, 2);
        if (a.trace && blockIdx.x == 0 && tid == 0) { a.trace[6] = clock64() - tr_t0; a.trace[7] = tr_w; a.trace[8] = done; }
    } else if (!TILE && tid < kEpiThreads) {
        // =============================== epilogue ===========================================
        constexpr int NQ = COLS / 8;                       // 8-channel groups (one uint4 of int16) per thread
        const int row = tid & 127, quad = warp & 3, cg = warp >> 2;
        const int Ow = (a.O + 31) >> 5;
        const int lim = a.res_in ? min(a.residual_channels, a.res_in_ch) : 0;
        const int o0 = obase + cg * COLS;                  // this thread's first output channel
        const bool res16 = EPI == kEpiDirect && a.res_in && a.res_in_bytes == 2 && (a.res_in_ch & 7) == 0 && (lim & 7) == 0;
        uint32_t tc = 0;
        bool ok = true, overflow = false;
        long long tr_w = 0;
        const long long tr_t0 = clock64();
        struct Pix { bool live; int n, y, x; size_t opix; };
        auto locate = [&](int m) {
            Pix q{false, 0, 0, 0, 0};
            const int p = m * 128 + row;
            if (p < NV) {
                const int vy = fastdiv(p, a.pw_mul, a.pw_sh);
                q.x = p - vy * a.PW;
                q.n = fastdiv(vy, a.vh_mul, a.vh_sh);
                q.y = vy - q.n * a.VH;
                q.live = q.x < a.OWg && q.y < a.OHg;
            }
            q.opix = ((size_t)q.n * a.OHg + q.y) * a.OWg + q.x;
            return q;
        };
        // ---- staged residual rows (RSTAGE; the host enables it only for int16 tensors, an n-tile
        //      that lies entirely inside or outside the injected channels, NT of 64 or 128) --------
        constexpr uint32_t ROWB = NT * 2;                  // bytes of one pixel's residual segment
        constexpr int NCOPY = (32 * ROWB) / (128 * 16);    // 16-byte pieces per thread and tile (group: 32 rows, 128 threads)
        const int gtid = cg * 32 + lane;                   // this thread's index in its group
        const int grow0 = quad * 32;                       // the group's first row of a tile
        const bool st_in = RSTAGE && a.res_in && obase < lim;
        const bool st_out = RSTAGE && a.res_out;
        // output pixels in front of raster position p (live pixels are consecutive tensor rows)
        auto live_before = [&](int p) -> long long {
            if (p >= NV) return (long long)a.B * a.OHg * a.OWg;
            const int vy = fastdiv(p, a.pw_mul, a.pw_sh), x = p - vy * a.PW;
            const int n = fastdiv(vy, a.vh_mul, a.vh_sh), y = vy - n * a.VH;
            return ((long long)n * a.OHg + min(y, a.OHg)) * a.OWg + (y < a.OHg ? min(x, a.OWg) : 0);
        };
        // shared-memory address of 16-byte chunk `c` of staged row `r`: chunks XOR-swizzled by row
        auto st_addr = [&](int buf, int r, int c) -> uint32_t {
            return smem_u32(sRes) + (uint32_t)(quad * 2 + buf) * (32u * ROWB) + (uint32_t)r * ROWB +
                   (uint32_t)(((c & ~7) | ((c ^ r) & 7)) << 4);
        };
        // bytes of a pixel's incoming segment: the whole n-tile, or the part of it that receives a
        // residual (a producer with fewer channels, e.g. 64 of this layer's 128); a multiple of 16
        const uint32_t rowb_in = st_in ? (uint32_t)min(NT, lim - obase) * 2u : ROWB;
        auto issue_in = [&](long long p0, int nl, int buf) {   // cp.async of a tile's incoming rows
            if (!st_in) return;
            const char* g = reinterpret_cast<const char*>(a.res_in) + ((size_t)p0 * a.res_in_ch + obase) * 2;
#pragma unroll
            for (int k = 0; k < NCOPY; k++) {
                // the same thread -> (row, chunk) map as store_out: a thread refills exactly the
                // bytes it has just drained, whatever the width of the incoming rows
                const uint32_t off = (uint32_t)(gtid + k * 128) * 16u;
                const int r = off / ROWB, c = (off % ROWB) >> 4;
                if (r < nl && (uint32_t)(c << 4) < rowb_in)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(st_addr(buf, r, c)),
                                 "l"(g + (size_t)r * a.res_in_ch * 2 + (c << 4)) : "memory");
            }
        };
        auto store_out = [&](long long p0, int nl, int buf) {  // a tile's outgoing rows, whole lines
            if (!st_out) return;
            char* g = reinterpret_cast<char*>(a.res_out) + ((size_t)p0 * a.O + obase) * 2;
#pragma unroll
            for (int k = 0; k < NCOPY; k++) {
                const uint32_t off = (uint32_t)(gtid + k * 128) * 16u;
                const int r = off / ROWB, c = (off % ROWB) >> 4;
                if (r < nl) {
                    uint4 v4;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v4.x), "=r"(v4.y), "=r"(v4.z), "=r"(v4.w)
                                 : "r"(st_addr(buf, r, c)) : "memory");
                    *reinterpret_cast<uint4*>(g + (size_t)r * a.O * 2 + (c << 4)) = v4;
                }
            }
        };
        uint32_t eph = 0;                                  // phase of the epilogue rendezvous
        auto rendezvous = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_EPI(quad));
            const bool r = wait(BAR_EPI(quad), eph);
            eph ^= 1;
            return r;
        };
        // int16 residual of channels [o0, o0+COLS) of one pixel, packed (zeros where nothing is
        // injected); 2x2 max for pooled residuals (kernel.cuh:773-783)
        auto fetch16 = [&](uint4 (&r)[NQ], const Pix& q) {
            const short* base = reinterpret_cast<const short*>(a.res_in);
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            if (a.res_in_chunked) {
                // [channel chunk][pixel][8 channels]: consecutive lanes (pixels) read consecutive
                // 16 bytes, so a warp's load touches four whole lines instead of 32 pieces of lines
                const uint4* cb = reinterpret_cast<const uint4*>(a.res_in) + (size_t)(o0 >> 3) * a.res_in_npix;
                if (a.residual_pool) {
                    const size_t i00 = ((size_t)q.n * 2 * a.OHg + 2 * q.y) * 2 * a.OWg + 2 * q.x, rw = (size_t)2 * a.OWg;
#pragma unroll
                    for (int j = 0; j < NQ; j++) {
                        r[j] = z;
                        if (q.live && o0 + 8 * j < lim) {
                            const uint4* p = cb + (size_t)j * a.res_in_npix + i00;
                            const uint4 w0 = __ldg(p), w1 = __ldg(p + 1), w2 = __ldg(p + rw), w3 = __ldg(p + rw + 1);
                            r[j].x = __vmaxs2(__vmaxs2(w0.x, w1.x), __vmaxs2(w2.x, w3.x));
                            r[j].y = __vmaxs2(__vmaxs2(w0.y, w1.y), __vmaxs2(w2.y, w3.y));
                            r[j].z = __vmaxs2(__vmaxs2(w0.z, w1.z), __vmaxs2(w2.z, w3.z));
                            r[j].w = __vmaxs2(__vmaxs2(w0.w, w1.w), __vmaxs2(w2.w, w3.w));
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NQ; j++)
                        r[j] = (q.live && o0 + 8 * j < lim) ? __ldg(cb + (size_t)j * a.res_in_npix + q.opix) : z;
                }
            } else if (a.residual_pool) {
                const size_t b00 = (((size_t)q.n * 2 * a.OHg + 2 * q.y) * 2 * a.OWg + 2 * q.x) * a.res_in_ch + o0;
                const size_t rowp = (size_t)2 * a.OWg * a.res_in_ch;
#pragma unroll
                for (int h = 0; h < NQ; h += 2) {              // 8 loads in flight at a time
                    uint4 w[4][2];
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        const bool on = h + j < NQ && q.live && o0 + 8 * (h + j) < lim;
                        const short* s = base + b00 + 8 * (h + j);
                        w[0][j] = on ? __ldg(reinterpret_cast<const uint4*>(s)) : z;
                        w[1][j] = on ? __ldg(reinterpret_cast<const uint4*>(s + a.res_in_ch)) : z;
                        w[2][j] = on ? __ldg(reinterpret_cast<const uint4*>(s + rowp)) : z;
                        w[3][j] = on ? __ldg(reinterpret_cast<const uint4*>(s + rowp + a.res_in_ch)) : z;
                    }
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        if (h + j >= NQ) continue;
                        r[h + j].x = __vmaxs2(__vmaxs2(w[0][j].x, w[1][j].x), __vmaxs2(w[2][j].x, w[3][j].x));
                        r[h + j].y = __vmaxs2(__vmaxs2(w[0][j].y, w[1][j].y), __vmaxs2(w[2][j].y, w[3][j].y));
                        r[h + j].z = __vmaxs2(__vmaxs2(w[0][j].z, w[1][j].z), __vmaxs2(w[2][j].z, w[3][j].z));
                        r[h + j].w = __vmaxs2(__vmaxs2(w[0][j].w, w[1][j].w), __vmaxs2(w[2][j].w, w[3][j].w));
                    }
                }
            } else {
                const short* s = base + q.opix * a.res_in_ch + o0;
#pragma unroll
                for (int j = 0; j < NQ; j++)
                    r[j] = (q.live && o0 + 8 * j < lim) ? __ldg(reinterpret_cast<const uint4*>(s + 8 * j)) : z;
            }
        };
        auto add16 = [&](int (&v)[COLS], const uint4 (&r)[NQ]) {
#pragma unroll
            for (int j = 0; j < NQ; j++) {
                v[8 * j] += (int)(short)(r[j].x & 0xFFFFu);
                v[8 * j + 1] += (int)(short)(r[j].x >> 16);
                v[8 * j + 2] += (int)(short)(r[j].y & 0xFFFFu);
                v[8 * j + 3] += (int)(short)(r[j].y >> 16);
                v[8 * j + 4] += (int)(short)(r[j].z & 0xFFFFu);
                v[8 * j + 5] += (int)(short)(r[j].z >> 16);
                v[8 * j + 6] += (int)(short)(r[j].w & 0xFFFFu);
                v[8 * j + 7] += (int)(short)(r[j].w >> 16);
            }
        };
        // packed output bits (and the next layer's planes) of this thread's channels of one pixel
        auto store_bits = [&](const Pix& q, uint32_t word) {
            // bits of channel o live at bit 31 - o%32 of word o/32 (little-endian bytes)
            unsigned char* wp = reinterpret_cast<unsigned char*>(
                a.out + (size_t)q.n * a.out_image_stride + ((size_t)q.y * a.OWg + q.x) * Ow + (o0 >> 5));
            if (COLS == 32) *reinterpret_cast<uint32_t*>(wp) = word;
            else if (COLS == 16) *reinterpret_cast<unsigned short*>(wp + ((o0 & 16) ? 0 : 2)) = (unsigned short)word;
            else wp[3 - ((o0 & 31) >> 3)] = (unsigned char)word;
            if (a.nxt) store_next_planes(a, q.n, q.y, q.x, o0, word, COLS);
        };
        constexpr bool plain = EPI == kEpiPlain;
        uint4 rnext[NQ];
#pragma unroll
        for (int j = 0; j < NQ; j++) rnext[j] = make_uint4(0u, 0u, 0u, 0u);
        Pix cur = locate(mfirst);
        if (res16 && mfirst < mtiles) fetch16(rnext, cur);
        // first pixel and number of live pixels of the group's rows of the current, previous and next tile
        long long p0_cur = 0, p0_prev = 0, p0_next = 0;
        int nl_cur = 0, nl_prev = -1, nl_next = 0;
        if (RSTAGE && mfirst < mtiles) {
            p0_cur = live_before(mfirst * 128 + grow0);
            nl_cur = (int)(live_before(mfirst * 128 + grow0 + 32) - p0_cur);
            issue_in(p0_cur, nl_cur, 0);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        int b = 0, mprev = -1;
        uint32_t bph = 0;
        for (int m = mfirst; m < mtiles && ok; m += mstep, tc++) {
            const Pix q = cur;
            uint4 rcur[NQ];
#pragma unroll
            for (int j = 0; j < NQ; j++) rcur[j] = rnext[j];
            if (m + mstep < mtiles) {                      // next tile's row: its residual flies during this tile
                cur = locate(m + mstep);
                if (res16) fetch16(rnext, cur);
            }
            ok = wait.timed(BAR_CFULL(b), bph, tr_w);
            if (!ok) break;
            tc_fence_after();
            int v[COLS];
            tmem_ld_cols<COLS>(tmem + ((uint32_t)(quad * 32) << 16) + b * NT + cg * COLS, v);
            tmem_ld_wait();
            tc_fence_before();                             // this warp is done with the accumulator
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_CEMPTY(b));
            if (++b == NACC) { b = 0; bph ^= 1; }
            if (plain) {
                // no residual and no integer output: the reference's comparison as it stands,
                // !((float)value < threshold) (kernel.cuh:795-796), on the fp32 accumulator
                uint32_t word = 0;
                const float4* tf4 = reinterpret_cast<const float4*>(sThrF + cg * COLS);
#pragma unroll
                for (int j = 0; j < COLS / 4; j++) {
                    const float4 th = tf4[j];
                    if (!(__int_as_float(v[4 * j]) < th.x)) word |= (1u << (COLS - 1)) >> (4 * j);
                    if (!(__int_as_float(v[4 * j + 1]) < th.y)) word |= (1u << (COLS - 1)) >> (4 * j + 1);
                    if (!(__int_as_float(v[4 * j + 2]) < th.z)) word |= (1u << (COLS - 1)) >> (4 * j + 2);
                    if (!(__int_as_float(v[4 * j + 3]) < th.w)) word |= (1u << (COLS - 1)) >> (4 * j + 3);
                }
                if (q.live) store_bits(q, word);
                mprev = m;
                continue;
            }
#pragma unroll
            for (int j = 0; j < COLS; j++) v[j] = f4_acc_to_int(v[j]);     // fp32 accumulators, exact integers
            if (q.live && a.acc_out) {
                int4* dst = reinterpret_cast<int4*>(a.acc_out + q.opix * a.O + o0);
#pragma unroll
                for (int j = 0; j < COLS / 4; j++)
                    dst[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
            const int sbuf = (int)(tc & 1);
            int lrow = 0;
            if (RSTAGE) {
                // this tile's incoming rows have landed (mine: wait_group; everyone's: rendezvous),
                // and every thread has written its part of the previous tile's outgoing rows
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                ok = rendezvous();
                if (!ok) break;
                if (nl_prev >= 0) store_out(p0_prev, nl_prev, sbuf ^ 1);
                if (m + mstep < mtiles) {
                    p0_next = live_before((m + mstep) * 128 + grow0);
                    nl_next = (int)(live_before((m + mstep) * 128 + grow0 + 32) - p0_next);
                    issue_in(p0_next, nl_next, sbuf ^ 1);  // the buffer this thread has just drained
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                lrow = (int)((long long)q.opix - p0_cur);
                if (st_in && q.live && o0 < lim) {
                    uint4 r[NQ];
#pragma unroll
                    for (int j = 0; j < NQ; j++) {
                        r[j] = make_uint4(0u, 0u, 0u, 0u);
                        if (o0 + 8 * j < lim)
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[j].x), "=r"(r[j].y), "=r"(r[j].z), "=r"(r[j].w)
                                         : "r"(st_addr(sbuf, lrow, cg * NQ + j)) : "memory");
                    }
                    add16(v, r);
                }
            } else if (res16) {
                add16(v, rcur);
            } else if (a.res_in && q.live && o0 < lim) {
#pragma unroll
                for (int j = 0; j < COLS / 4; j++) {
                    const int o = o0 + 4 * j;
                    if (o >= lim) continue;
                    int4 r;
                    if (a.residual_pool) {
                        const size_t b00 = (((size_t)q.n * 2 * a.OHg + 2 * q.y) * 2 * a.OWg + 2 * q.x) * a.res_in_ch + o;
                        const size_t rowp = (size_t)2 * a.OWg * a.res_in_ch;
                        r = max4(max4(ld_res4(a.res_in, a.res_in_bytes, b00),
                                      ld_res4(a.res_in, a.res_in_bytes, b00 + a.res_in_ch)),
                                 max4(ld_res4(a.res_in, a.res_in_bytes, b00 + rowp),
                                      ld_res4(a.res_in, a.res_in_bytes, b00 + rowp + a.res_in_ch)));
                    } else {
                        r = ld_res4(a.res_in, a.res_in_bytes, q.opix * a.res_in_ch + o);
                    }
                    v[4 * j] += r.x; v[4 * j + 1] += r.y; v[4 * j + 2] += r.z; v[4 * j + 3] += r.w;
                }
            }
            uint32_t word = 0;                             // channel c of this thread at bit COLS-1-c
            const int4* th4 = reinterpret_cast<const int4*>(sThr + cg * COLS);
#pragma unroll
            for (int j = 0; j < COLS / 4; j++) {
                const int4 th = th4[j];
                if (v[4 * j] >= th.x) word |= (1u << (COLS - 1)) >> (4 * j);
                if (v[4 * j + 1] >= th.y) word |= (1u << (COLS - 1)) >> (4 * j + 1);
                if (v[4 * j + 2] >= th.z) word |= (1u << (COLS - 1)) >> (4 * j + 2);
                if (v[4 * j + 3] >= th.w) word |= (1u << (COLS - 1)) >> (4 * j + 3);
            }
            if (a.res_out && q.live) {
                const size_t idx = q.opix * a.O + o0;
                if (a.res_out_bytes == 2) {
                    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<short*>(a.res_out) + idx);
                    if (!a.res_out_proven) {               // a real branch: two instructions per value
                        uint32_t ovf = 0;                  // |v| of every value ORed together
#pragma unroll
                        for (int j = 0; j < COLS; j++) ovf |= (uint32_t)(v[j] ^ (v[j] >> 31));
                        overflow |= ovf > 32767u;          // some value outside [-32768, 32767]
                    }
#pragma unroll
                    for (int j = 0; j < NQ; j++) {
                        uint32_t w[4];
#pragma unroll
                        for (int kk = 0; kk < 4; kk++) {
                            const int lo = v[8 * j + 2 * kk], hi = v[8 * j + 2 * kk + 1];
                            w[kk] = ((uint32_t)lo & 0xFFFFu) | ((uint32_t)hi << 16);
                        }
                        if (RSTAGE)                        // into the staged row, in place of what was read
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(st_addr(sbuf, lrow, cg * NQ + j)),
                                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        else if (a.res_out_chunked)
                            reinterpret_cast<uint4*>(a.res_out)[(size_t)((o0 >> 3) + j) * a.res_out_npix + q.opix] =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        else
                            dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
                    int4* dst = reinterpret_cast<int4*>(reinterpret_cast<int*>(a.res_out) + idx);
#pragma unroll
                    for (int j = 0; j < COLS / 4; j++)
                        dst[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            if (q.live) store_bits(q, word);
            mprev = m;
            p0_prev = p0_cur; nl_prev = nl_cur;
            p0_cur = p0_next; nl_cur = nl_next;
        }
        if (RSTAGE) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");      // nothing of this thread's in flight at exit
            if (ok && mprev >= 0 && rendezvous()) store_out(p0_prev, nl_prev, (int)((tc - 1) & 1));
        }
        if (overflow) atomicExch(a.err_flag, 2);
        if (a.trace && blockIdx.x == 0 && tid == 0) { a.trace[6] = clock64() - tr_t0; a.trace[7] = tr_w; a.trace[8] = tc; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace umma
}  // namespace tcbnn
