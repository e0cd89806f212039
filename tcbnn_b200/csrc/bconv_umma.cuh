// Binary convolution on the 5th-generation tensor cores: tcgen05.mma kind::i8 with the
// accumulators in tensor memory.
//
// The layer is the same Conv128LayerFMT arithmetic (kernel.cuh:676-827) as the warp-MMA
// path in bnn_layers.cuh.  Here the packed input bits are expanded to +-1 bytes in shared
// memory and the contraction is an exact int8 x int8 -> int32 implicit GEMM, so the
// accumulator IS the reference's `C*R*S - exclude*C - 2*popc(a^w)`: out-of-frame taps are
// zero bytes and contribute nothing, no popcount identities or correction tables needed.
//
// Implicit GEMM without im2col.  Pixels of the whole batch are laid out in one "virtual"
// zero-padded raster of pitch PW = W + pad columns and VH = H + pad rows per image (one shared
// band of zeros between neighbouring rows / images).  A tile is 128 consecutive raster
// positions; the +-1 bytes of the positions it touches (tile + halo) sit in shared memory as
//     A[channel chunk of 16][raster position][16 bytes]
// which is the no-swizzle K-major core-matrix layout of the UMMA shared-memory descriptor
// (8 rows x 16 bytes contiguous, next 8 rows +128 B, next 16 channels +LBO).  In that layout
// filter tap (r, s) is nothing but a start-address offset of ((r*PW + s) * 16) bytes, so the
// nine taps reuse one expanded patch.  Positions that fall on the zero bands produce junk
// rows that are simply not stored.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <climits>

namespace tcbnn {
namespace umma {

// ---- small PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking form: a plain read of the barrier's phase, cheaper for a thread that expects the
// phase to be complete already.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// One lane of a converged warp (the whole warp must execute this).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
// Bounded wait: gives up after `limit` polls and reports failure instead of hanging.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err_flag) {
    for (int i = 0; i < (1 << 22); i++)
        if (mbar_try_wait(bar, parity)) return true;
    if (err_flag) atomicExch(err_flag, 1);
    return false;
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], int8 operands, int32 accumulate; one thread issues.
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Same instruction with the two descriptors handed over as (low, high) register pairs, so the
// issue loop only does 32-bit adds on the address field; no memory clobber (ordering against
// the data comes from the mbarrier waits and fences around the loop).
__device__ __forceinline__ void mma_i8_split(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                             uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
// Same for 16 and 8 columns, and a width-generic front.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr) : "memory");
}
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, int (&r)[N]);
template <> __device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, int (&r)[32]) { tmem_ld32(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, int (&r)[16]) { tmem_ld16(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_cols<8>(uint32_t taddr, int (&r)[8]) { tmem_ld8(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: rows 16 B apart inside a core matrix,
// `sbo` bytes between 8-row groups, `lbo` bytes between 16-byte K chunks.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// Instruction descriptor: int8 x int8 -> int32, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_i8(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

// 16 packed bits -> 16 bytes of +1 / -1.  Which bit lands in which byte is a fixed
// permutation; activations and filters both go through this function, so it cancels.
__device__ __forceinline__ uint4 expand16(uint32_t h) {
    uint32_t v[4];
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const uint32_t nb = (h >> (4 * g)) & 0xFu;
        const uint32_t y = (nb * 0x00204081u) & 0x01010101u;      // one bit per byte
        v[g] = ~(y * 0xFEu);                                      // 1 -> 0x01, 0 -> 0xFF
    }
    return make_uint4(v[0], v[1], v[2], v[3]);
}

// Four consecutive residual channels (element index i, a multiple of 4) widened to int32.
__device__ __forceinline__ int4 ld_res4(const void* p, int bytes, size_t i) {
    if (bytes == 2) {
        const uint2 q = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const short*>(p) + i));
        return make_int4((int)(short)(q.x & 0xFFFFu), (int)(short)(q.x >> 16),
                         (int)(short)(q.y & 0xFFFFu), (int)(short)(q.y >> 16));
    }
    return __ldg(reinterpret_cast<const int4*>(reinterpret_cast<const int*>(p) + i));
}
__device__ __forceinline__ int4 max4(int4 a, int4 b) {
    return make_int4(max(a.x, b.x), max(a.y, b.y), max(a.z, b.z), max(a.w, b.w));
}

// ---- filter preparation -------------------------------------------------------------------
// bits [O][R*S][Cw] -> int8 blocks [n-tile][tap][chunk][n in tile][16 bytes], the order the
// kernel keeps them in shared memory.
__device__ __forceinline__ void prepare_filter_i8(const uint32_t* fbits, int O, int RS, int C,
                                                  int n_tile, uint4* out) {
    const int Cw = (C + 31) >> 5, chunks = C >> 4;
    const long long total = (long long)O * RS * chunks;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i % n_tile);
        long long r = i / n_tile;
        const int chunk = (int)(r % chunks); r /= chunks;
        const int tap = (int)(r % RS);
        const int nt = (int)(r / RS);
        const int o = nt * n_tile + n;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (o < O) {
            const uint32_t w = fbits[((size_t)o * RS + tap) * Cw + (chunk >> 1)];
            v = expand16((chunk & 1) ? (w & 0xFFFFu) : (w >> 16));
        }
        out[i] = v;
    }
}

struct ConvUmmaArgs {
    const uint32_t* in;      // [B][H][W][Cw]
    const uint4* wi8;        // prepared int8 filter blocks
    const float* thr;        // [O]
    int B, H, W, C, O, R, S, pad_h, pad_w;
    int PW, VH;              // raster pitch / rows per image
    int NPOS;                // patch positions held in shared memory (multiple of 8)
    long long NV;            // raster positions over the batch
    const void* res_in; int res_in_bytes, res_in_ch, residual_channels, residual_pool;
    uint32_t* out; long long out_image_stride;
    void* res_out; int res_out_bytes; int32_t* acc_out;
    int* err_flag;           // 1: a bounded wait gave up, 2: a residual did not fit int16
};

// One CTA of 128 threads; stride-1 conv, no pooling.  Phases per tile: expand the patch,
// issue the MMAs (one thread), read the accumulators back and run the epilogue.  Overlap
// between phases comes from co-resident CTAs.
template <int C, int NT>
__device__ void conv_umma_cta(const ConvUmmaArgs& a, unsigned char* smem) {
    constexpr int CH = C / 16;                 // 16-channel chunks
    constexpr int KS = C / 32;                 // MMA k-steps per tap
    constexpr uint32_t TM_COLS = NT < 32 ? 32 : NT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RS = a.R * a.S;
    const int ntiles_n = (a.O + NT - 1) / NT;

    // shared memory carve-up: [A patch | residual staging tile][B filter][thresholds]
    // [row -> output pixel][barrier][tmem ptr].  The staging tile (int32 [128][NT+4]) reuses
    // the patch, which is dead once the tile's MMAs have completed.
    constexpr int PITCH = NT + 4;
    const size_t a_bytes = (size_t)CH * a.NPOS * 16, r_bytes = (size_t)128 * PITCH * 4;
    uint4* sA = reinterpret_cast<uint4*>(smem);
    int* sR = reinterpret_cast<int*>(smem);
    uint4* sB = reinterpret_cast<uint4*>(smem + (a_bytes > r_bytes ? a_bytes : r_bytes));
    float* sThr = reinterpret_cast<float*>(sB + (size_t)RS * CH * NT);
    int* sRow = reinterpret_cast<int*>(sThr + NT);
    uint64_t* sBar = reinterpret_cast<uint64_t*>(sRow + 128);
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 1);

    if (warp == 0) tmem_alloc(smem_u32(sTmem), TM_COLS);
    if (tid == 0) mbar_init(smem_u32(sBar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *sTmem;
    uint32_t phase = 0;
    bool ok = true;

    const long long mtiles = (a.NV + 127) / 128;
    const long long total = mtiles * ntiles_n;
    int cur_nt = -1;
    for (long long task = blockIdx.x; task < total && ok; task += gridDim.x) {
        // n-tile major order so a CTA keeps its filter block as long as possible
        const int nt = (int)(task / mtiles);
        const long long mt = task - (long long)nt * mtiles;
        if (nt != cur_nt) {
            const uint4* src = a.wi8 + (size_t)nt * RS * CH * NT;
            for (int i = tid; i < RS * CH * NT; i += 128) sB[i] = __ldg(src + i);
            for (int i = tid; i < NT; i += 128) {
                const int o = nt * NT + i;
                sThr[i] = o < a.O ? __ldg(a.thr + o) : 0.0f;
            }
            cur_nt = nt;
        }
        // ---- expand the patch -----------------------------------------------------------
        const long long p0 = mt * 128;
        const long long q0 = p0 - (long long)a.pad_h * a.PW - a.pad_w;
        for (int q = tid; q < a.NPOS; q += 128) {
            const long long gq = q0 + q;
            const uint32_t* px = nullptr;
            if (gq >= 0 && gq < a.NV) {
                const long long vy = gq / a.PW;
                const int vx = (int)(gq - vy * a.PW);
                const int n = (int)(vy / a.VH);
                const int y = (int)(vy - (long long)n * a.VH);
                if (vx < a.W && y < a.H)
                    px = a.in + (((size_t)n * a.H + y) * a.W + vx) * (C / 32);
            }
#pragma unroll
            for (int w = 0; w < C / 32; w++) {
                if (px) {
                    const uint32_t bits = __ldg(px + w);
                    sA[(size_t)(2 * w) * a.NPOS + q] = expand16(bits >> 16);
                    sA[(size_t)(2 * w + 1) * a.NPOS + q] = expand16(bits & 0xFFFFu);
                } else {
                    sA[(size_t)(2 * w) * a.NPOS + q] = make_uint4(0u, 0u, 0u, 0u);
                    sA[(size_t)(2 * w + 1) * a.NPOS + q] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- MMAs: one thread ----------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
            const uint32_t aBase = smem_u32(sA), bBase = smem_u32(sB);
            const uint32_t lboA = (uint32_t)a.NPOS * 16u, lboB = NT * 16u;
            uint32_t acc = 0;
            for (int r = 0; r < a.R; r++)
                for (int s = 0; s < a.S; s++) {
                    const uint32_t tapA = aBase + (uint32_t)(r * a.PW + s) * 16u;
                    const uint32_t tapB = bBase + (uint32_t)((r * a.S + s) * CH) * NT * 16u;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        mma_i8(tmem, smem_desc(tapA + 2 * ks * lboA, lboA, 128u),
                               smem_desc(tapB + 2 * ks * lboB, lboB, 128u), idesc_i8(NT), acc);
                        acc = 1;
                    }
                }
            mma_commit(smem_u32(sBar));
        }
        ok = mbar_wait(smem_u32(sBar), phase, a.err_flag);
        ok = __syncthreads_and(ok ? 1 : 0) != 0;      // all threads agree before going on
        phase ^= 1;
        tc_fence_after();
        // ---- epilogue: thread <-> raster position p0 + tid ---------------------------------------
        const long long p = p0 + tid;
        bool live = false;
        int n = 0, y = 0, x = 0;
        if (p < a.NV) {
            const long long vy = p / a.PW;
            x = (int)(p - vy * a.PW);
            n = (int)(vy / a.VH);
            y = (int)(vy - (long long)n * a.VH);
            live = x < a.W && y < a.H;
        }
        const size_t opix = ((size_t)n * a.H + y) * a.W + x;
        const int Ow = (a.O + 31) >> 5;
        const int obase = nt * NT;
        sRow[tid] = live ? (int)opix : -1;
        __syncthreads();                       // patch is dead (MMAs done), row table visible
        constexpr int UPR = NT / 4;            // 4-channel units per staged row
        constexpr int UNROLL = 8;
        if (ok && a.res_in) {
            // residual tile -> shared memory: consecutive threads take consecutive 4-channel
            // units (whole rows are contiguous in memory), UNROLL independent loads in flight
            const int lim = min(a.residual_channels, a.res_in_ch);
            for (int u0 = tid; u0 < 128 * UPR; u0 += 128 * UNROLL) {
                int4 val[UNROLL];
#pragma unroll
                for (int k = 0; k < UNROLL; k++) {
                    const int u = u0 + k * 128;
                    val[k] = make_int4(0, 0, 0, 0);
                    if (u < 128 * UPR) {
                        const int r = u / UPR, o = obase + (u % UPR) * 4;
                        const int op = sRow[r];
                        if (op >= 0 && o < lim) {
                            if (a.residual_pool) {      // max over the 2x2 window (kernel.cuh:773-783)
                                const int px = op % a.W, t2 = op / a.W, py = t2 % a.H, pn = t2 / a.H;
                                const size_t b00 = (((size_t)pn * 2 * a.H + 2 * py) * 2 * a.W + 2 * px) *
                                                   a.res_in_ch + o;
                                const size_t rowp = (size_t)2 * a.W * a.res_in_ch;
                                val[k] = max4(max4(ld_res4(a.res_in, a.res_in_bytes, b00),
                                                   ld_res4(a.res_in, a.res_in_bytes, b00 + a.res_in_ch)),
                                              max4(ld_res4(a.res_in, a.res_in_bytes, b00 + rowp),
                                                   ld_res4(a.res_in, a.res_in_bytes, b00 + rowp + a.res_in_ch)));
                            } else {
                                val[k] = ld_res4(a.res_in, a.res_in_bytes, (size_t)op * a.res_in_ch + o);
                            }
                        }
                    }
                }
#pragma unroll
                for (int k = 0; k < UNROLL; k++) {
                    const int u = u0 + k * 128;
                    if (u < 128 * UPR)
                        *reinterpret_cast<int4*>(sR + (u / UPR) * PITCH + (u % UPR) * 4) = val[k];
                }
            }
            __syncthreads();
        }
        if (ok) {
            uint32_t words[NT / 32];
#pragma unroll
            for (int nb = 0; nb < NT / 32; nb++) {
                int v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + nb * 32, v);
                tmem_ld_wait();
                const int o0 = obase + nb * 32;
                int4* srow = reinterpret_cast<int4*>(sR + tid * PITCH + nb * 32);
                if (live && a.acc_out) {
                    int4* dst = reinterpret_cast<int4*>(a.acc_out + opix * a.O + o0);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        dst[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
                if (a.res_in) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int4 rr = srow[j];
                        v[4 * j] += rr.x; v[4 * j + 1] += rr.y; v[4 * j + 2] += rr.z; v[4 * j + 3] += rr.w;
                    }
                }
                uint32_t word = 0;
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (!((float)v[j] < sThr[nb * 32 + j])) word |= 0x80000000u >> j;
                words[nb] = word;
                if (a.res_out) {
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        srow[j] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            if (live) {
                uint32_t* dst = a.out + (size_t)n * a.out_image_stride +
                                ((size_t)y * a.W + x) * Ow + (obase >> 5);
#pragma unroll
                for (int nb = 0; nb < NT / 32; nb++) dst[nb] = words[nb];
            }
            if (a.res_out) {
                __syncthreads();
                bool overflow = false;
                for (int u = tid; u < 128 * UPR; u += 128) {
                    const int r = u / UPR, c4 = (u % UPR) * 4;
                    const int op = sRow[r];
                    if (op < 0) continue;
                    const int4 v4 = *reinterpret_cast<const int4*>(sR + r * PITCH + c4);
                    const size_t idx = (size_t)op * a.O + obase + c4;
                    if (a.res_out_bytes == 2) {
                        overflow |= max(max(abs(v4.x), abs(v4.y)), max(abs(v4.z), abs(v4.w))) > 32767;
                        *reinterpret_cast<uint2*>(reinterpret_cast<short*>(a.res_out) + idx) =
                            make_uint2(((uint32_t)v4.x & 0xFFFFu) | ((uint32_t)v4.y << 16),
                                       ((uint32_t)v4.z & 0xFFFFu) | ((uint32_t)v4.w << 16));
                    } else {
                        *reinterpret_cast<int4*>(reinterpret_cast<int*>(a.res_out) + idx) = v4;
                    }
                }
                if (overflow) atomicExch(a.err_flag, 2);
            }
        }
        tc_fence_before();
        __syncthreads();       // accumulators and patch are free again
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace umma
}  // namespace tcbnn
