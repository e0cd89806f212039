// Bit GEMM on tcgen05: C[m][n] = sum_k a[m][k] * w[n][k] over +-1 values, i.e. the reference's
// K - 2*popc(a ^ w) (bmm/tensorcore_kernel.cu:138-356; Fc128LayerFMT / Out128LayerFMT,
// kernel.cuh:174-280 on top of it), as an exact int8 x int8 -> int32 MMA.
//
// Two streaming passes first write both operands as +-1 bytes (0 for padding: rows past the end,
// bits past K) in 8 KB units [128-row tile][64-bit k-block][16-bit chunk][row][16 B], the
// no-swizzle K-major operand layout, so that a unit is one bulk copy and one MMA operand.
// The GEMM CTA owns a 256 x 128 tile (two 128-row sub-tiles of A against one tile of W) over a
// range of k-blocks (split K):
//
//   warps 0-7  epilogue : after the last k-block, tcgen05.ld and store the int32 partial sums
//   warp  8    loader   : one lane, three bulk copies per k-block into a ring of 24 KB stages
//   warp  9    MMA      : converged warp, elected lane: 4 N=128 MMAs per stage
//
// The split-K partial sums go through gemm_splitk_finish (bnn_layers.cuh), which applies the
// output mode (int32 / threshold bits / scale + bias).
#pragma once
#include "bconv_umma_pre.cuh"

namespace tcbnn {
namespace umma {

constexpr int kGemmThreads = 320;
constexpr int kGemmStages = 6;
constexpr int kGemmUnit = 8192;                        // 128 rows x 64 k, int8
constexpr size_t kGemmSmem = (size_t)kGemmStages * 3 * kGemmUnit + 32 * 8 + 64;

struct GemmUmmaArgs {
    const unsigned char* ea;   // expanded A: [MT][KB] units
    const unsigned char* ew;   // expanded W: [NT][KB] units
    int M, N, KB, MT, NT, splits, per;   // per: k-blocks per split
    int32_t* partial;          // [splits][M][N]
    int* status;               // set to 1 when a bounded wait gives up
};

// packed bits [rows][ld words] (bit k of a row at bit 31 - k%32 of word k/32) -> units
__device__ __forceinline__ void expand_rows(const uint32_t* bits, int rows, int ld, int K, int RT, int KB,
                                            uint4* out) {
    const long long total = (long long)RT * KB * 4 * 128;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i & 127);
        const int chunk = (int)((i >> 7) & 3);
        const long long u = i >> 9;
        const int kb = (int)(u % KB), rt = (int)(u / KB);
        const int r = rt * 128 + row, k0 = kb * 64 + chunk * 16;
        uint4 e = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows && k0 < K) {
            const uint32_t w = __ldg(bits + (size_t)r * ld + (k0 >> 5));
            e = expand16((k0 & 16) ? (w & 0xFFFFu) : (w >> 16));
            const int valid = K - k0;                   // element c of the chunk sits in byte 15 - c
            if (valid < 16) {
                uint32_t v[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
                for (int b = 0; b < 16; b++)
                    if (b < 16 - valid) v[b >> 2] &= ~(0xFFu << (8 * (b & 3)));
                e = make_uint4(v[0], v[1], v[2], v[3]);
            }
        }
        out[i] = e;
    }
}

__device__ __forceinline__ void gemm_umma_cta(const GemmUmmaArgs& g, unsigned char* smem) {
    constexpr int NST = kGemmStages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint64_t* sBar = reinterpret_cast<uint64_t*>(smem + (size_t)NST * 3 * kGemmUnit);
    // barriers: full[NST] | empty[NST] | acc_full
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 2 * NST + 1);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sTmem + 1);
    const uint32_t bar0 = smem_u32(sBar);
    auto BAR_FULL = [&](int s) { return bar0 + 8u * s; };
    auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (NST + s); };
    const uint32_t BAR_ACC = bar0 + 8u * (2 * NST);

    // tile of this CTA: blockIdx.x = (split * tiles_m2 + tm2) * NT + tn
    const int tiles_m2 = (g.MT + 1) >> 1;
    const int tn = blockIdx.x % g.NT;
    const int tm2 = (blockIdx.x / g.NT) % tiles_m2;
    const int split = blockIdx.x / (g.NT * tiles_m2);
    const int kb0 = split * g.per, kb1 = min(g.KB, kb0 + g.per);
    const bool two = tm2 * 2 + 1 < g.MT;               // second 128-row sub-tile exists

    if (tid == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(BAR_FULL(s), 1); mbar_init(BAR_EMPTY(s), 1); }
        mbar_init(BAR_ACC, 1);
        *sAbort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) tmem_alloc(smem_u32(sTmem), 256);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *sTmem;
    const WsWait wait{sAbort, g.status};

    if (warp == 8) {
        // =============================== loader =============================================
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0, issued = 0;
            bool ok = true;
            const uint32_t bytes = (two ? 3u : 2u) * kGemmUnit;
            for (int kb = kb0; kb < kb1; kb++) {
                ok = wait(BAR_EMPTY(s), ph ^ 1);
                if (!ok) break;
                mbar_expect_tx(BAR_FULL(s), bytes);
                const uint32_t dst = smem_u32(smem + (size_t)s * 3 * kGemmUnit);
                bulk_g2s(dst, g.ea + ((size_t)(tm2 * 2) * g.KB + kb) * kGemmUnit, kGemmUnit, BAR_FULL(s));
                if (two)
                    bulk_g2s(dst + kGemmUnit, g.ea + ((size_t)(tm2 * 2 + 1) * g.KB + kb) * kGemmUnit, kGemmUnit, BAR_FULL(s));
                bulk_g2s(dst + 2 * kGemmUnit, g.ew + ((size_t)tn * g.KB + kb) * kGemmUnit, kGemmUnit, BAR_FULL(s));
                issued++;
                if (++s == NST) { s = 0; ph ^= 1; }
            }
            if (!ok) {
                // giving up: wait (bounded) for the copies still in flight before the CTA exits
                for (int s2 = 0; s2 < NST; s2++) {
                    const bool this_pass = s2 < s;
                    if (!this_pass && issued < (uint32_t)NST) continue;
                    for (int i = 0; i < (1 << 20); i++)
                        if (mbar_try_wait(BAR_FULL(s2), this_pass ? ph : ph ^ 1)) break;
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // =============================== MMA issuer =========================================
        const bool leader = elect_one();
        constexpr uint32_t IDESC = idesc_i8(128);
        const uint64_t desc0 = smem_desc(smem_u32(smem), 128 * 16, 128u);
        const uint32_t hi = (uint32_t)(desc0 >> 32), lo0 = (uint32_t)desc0;
        constexpr uint32_t stepStage = (3 * kGemmUnit) >> 4, stepUnit = kGemmUnit >> 4, stepK = (2 * 128 * 16) >> 4;
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int kb = kb0; kb < kb1 && ok; kb++) {
            ok = wait.spin(BAR_FULL(s), ph);
            if (!ok) break;
            tc_fence_after();
            if (leader) {
                const uint32_t a = lo0 + s * stepStage, b = a + 2 * stepUnit;
                const uint32_t acc = kb > kb0 ? 1u : 0u;
                mma_i8_split(tmem, a, hi, b, hi, IDESC, acc);
                mma_i8_split(tmem, a + stepK, hi, b + stepK, hi, IDESC, 1u);
                if (two) {
                    mma_i8_split(tmem + 128, a + stepUnit, hi, b, hi, IDESC, acc);
                    mma_i8_split(tmem + 128, a + stepUnit + stepK, hi, b + stepK, hi, IDESC, 1u);
                }
                mma_commit(BAR_EMPTY(s));
            }
            if (++s == NST) { s = 0; ph ^= 1; }
        }
        if (ok && leader) mma_commit(BAR_ACC);
        __syncwarp();
    } else {
        // =============================== epilogue ===========================================
        const int sub = warp >> 2, quad = warp & 3;
        const int m = (tm2 * 2 + sub) * 128 + quad * 32 + lane;
        const bool have = sub == 0 || two;
        if (wait.relaxed(BAR_ACC, 0) && have) {
            tc_fence_after();
            int32_t* dst = g.partial + ((size_t)split * g.M + m) * g.N + tn * 128;
            const bool vec = (g.N & 3) == 0;
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
                int v[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + sub * 128 + nb * 32, v);
                tmem_ld_wait();
                if (m < g.M) {
                    const int n0 = tn * 128 + nb * 32;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        if (vec && n0 + 4 * j + 3 < g.N) {
                            *reinterpret_cast<int4*>(dst + nb * 32 + 4 * j) = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                if (n0 + 4 * j + k < g.N) dst[nb * 32 + 4 * j + k] = v[4 * j + k];
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, 256);
}

}  // namespace umma
}  // namespace tcbnn
