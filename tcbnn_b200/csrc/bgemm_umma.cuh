// Bit GEMM on tcgen05: C[m][n] = sum_k a[m][k] * w[n][k] over +-1 values, i.e. the reference's
// K - 2*popc(a ^ w) (bmm/tensorcore_kernel.cu:138-356; Fc128LayerFMT / Out128LayerFMT,
// kernel.cuh:174-280 on top of it), as an exact 4-bit MMA: tcgen05.mma kind::mxf4 on +-1.0 as e2m1
// nibbles with unit block scales (bconv_umma.cuh), fp32 accumulators holding exact integers.
//
// One streaming pass first writes both operands as +-1 nibbles (0 for padding: rows past the end,
// bits past K) in 4 KB units [128-row tile][64-bit k-block][32-bit chunk][row][16 B], the
// no-swizzle K-major operand layout, so that a unit is one bulk copy and one MMA operand.
// The GEMM CTA owns a 128 x 128 or a 256 x 128 tile (one or two 128-row sub-tiles of A against one
// tile of W) over a range of k-blocks:
//
//   warps 0-7  epilogue : after the last k-block, tcgen05.ld and either finish the layer (one
//                         split: int32 / threshold bits / scale + bias straight from the
//                         accumulator) or store int32 partial sums for gemm_splitk_finish
//   warp  8    loader A : one lane, one bulk copy per sub-tile and stage (a stage holds up to
//                         kGemmKU consecutive k-blocks, contiguous in the expanded operand)
//   warp  9    MMA      : converged warp, elected lane: one N=128 MMA per sub-tile and k-block
//   warp  10   loader W : one lane, one bulk copy per stage
//
// A thread that issues a bulk copy is busy for 100-200 clocks per copy whatever its size, and
// copies issued by different warps overlap (tcbnn_bulk_copy_rate measures both): hence few, large
// copies and one issuing warp per operand.
#pragma once
#include "bconv_umma_pre.cuh"

namespace tcbnn {
namespace umma {

constexpr int kGemmThreads = 352;
constexpr int kGemmUnit = 4096;                        // 128 rows x 64 k, 4 bits each
constexpr int kGemmKU = 4;                             // k-blocks per stage
// Per tile shape (PAIR: 256 x 128, else 128 x 128): ring depth, bytes of a stage, tensor-memory
// columns (accumulators, then 32 columns of unit scales at the top).  The ring sizes also fix how
// many CTAs share an SM: one 256 x 128 CTA (all 512 columns), two 128 x 128 CTAs (256 each), so
// that no CTA ever waits for tensor memory held by a neighbour.
// stages: 4 for a 256 x 128 CTA; 128 x 128 CTAs take 3 when two of them share an SM, 6 alone
__host__ __device__ constexpr int gemm_stage_bytes(bool pair) { return (pair ? 3 : 2) * kGemmKU * kGemmUnit; }
__host__ __device__ constexpr uint32_t gemm_tmem_cols(bool pair) { return pair ? 512u : 256u; }
__host__ __device__ constexpr size_t gemm_smem(bool pair, int stages) {
    return (size_t)stages * gemm_stage_bytes(pair) + 32 * 8 + 64;
}

struct GemmUmmaArgs {
    const unsigned char* ea;   // expanded A: [MT][KB] units
    const unsigned char* ew;   // expanded W: [NT][KB] units
    int M, N, KB, MT, NT, splits, per;   // per: k-blocks per split
    int32_t* partial;          // [splits][M][N], used when splits > 1
    // splits == 1: the layer is finished in the epilogue (GemmMode of bnn_layers.cuh)
    int mode; void* out; int ldo; const float* p0; const float* p1;
    int nst;                   // stages in the ring (the launch's dynamic shared memory holds them)
    int* status;               // set to 1 when a bounded wait gives up
    long long* trace;          // null, or 16 counters: CTA 0 writes [9..15] (clocks; see the C header)
};

// bit i of b set -> nibble i of the result = 0xF (the nibble order of expand8_f4)
__device__ __forceinline__ uint32_t nibble_mask8(uint32_t b) {
    uint32_t x = b & 0xFFu;
    x = (x | (x << 12)) & 0x000F000Fu;
    x = (x | (x << 6)) & 0x03030303u;
    x = (x | (x << 3)) & 0x11111111u;
    return x * 0xFu;
}

// packed bits [rows][ld words] (bit k of a row at bit 31 - k%32 of word k/32) -> units; one launch
// expands both operands.  A task is (128-row tile, group of four k-blocks): 256 threads, two per
// row, each reading the 16 bytes (four 32-bit chunks) of its row that fall into its half of the
// group -- a whole 32-byte sector per row -- and writing four 16-byte slots; for a given chunk the
// threads of a warp write two runs of 256 contiguous bytes.  Tasks [0, RT_a * KG) belong to A, the
// rest to W (KG = groups per row tile).  lda / ldw are even, so the 8-byte loads are aligned.
__device__ __forceinline__ void expand_rows_pair(const uint32_t* a_bits, int a_rows, int a_ld, int RT_a,
                                                 const uint32_t* w_bits, int w_rows, int w_ld, int RT_w,
                                                 int K, int KB, uint4* out_a, uint4* out_w) {
    // the GEMM that consumes these units may be set up meanwhile (it waits before its first copy)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int KG = (KB + 3) >> 2;
    const int tasks = (RT_a + RT_w) * KG;
    const int t = threadIdx.x, row = t >> 1, half = t & 1;
    for (int task = blockIdx.x; task < tasks; task += gridDim.x) {
        const bool isw = task >= RT_a * KG;
        const int tk = isw ? task - RT_a * KG : task;
        const int rt = tk / KG, kg = tk - rt * KG;
        const uint32_t* bits = isw ? w_bits : a_bits;
        const int rows = isw ? w_rows : a_rows, ld = isw ? w_ld : a_ld;
        uint4* out = (isw ? out_w : out_a) + (size_t)rt * KB * 256;      // 256 slots of 16 bytes per unit
        const int r = rt * 128 + row;
        const int w0 = kg * 8 + half * 4;                                // first 32-bit chunk of this thread
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (r < rows) {
            const uint32_t* src = bits + (size_t)r * ld + w0;
            if (w0 + 1 < ld) { const uint2 q = __ldg(reinterpret_cast<const uint2*>(src)); w[0] = q.x; w[1] = q.y; }
            else if (w0 < ld) w[0] = __ldg(src);
            if (w0 + 3 < ld) { const uint2 q = __ldg(reinterpret_cast<const uint2*>(src + 2)); w[2] = q.x; w[3] = q.y; }
            else if (w0 + 2 < ld) w[2] = __ldg(src + 2);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = w0 + j, kb = c >> 1;                           // chunk -> k-block
            if (kb >= KB) break;
            const int k0 = c * 32;
            uint4 e = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows && k0 < K) {
                e = expand32_f4(w[j]);
                const int valid = K - k0;                                // elements of this chunk that exist
                if (valid < 32) {                                        // the rest is padding: 0, not -1
                    const uint32_t m = 0xFFFFFFFFu << (32 - valid);
                    e.x &= nibble_mask8(m >> 24); e.y &= nibble_mask8(m >> 16);
                    e.z &= nibble_mask8(m >> 8);  e.w &= nibble_mask8(m);
                }
            }
            out[(size_t)kb * 256 + (c & 1) * 128 + row] = e;
        }
    }
}

template <bool PAIR>
__device__ __forceinline__ void gemm_umma_cta(const GemmUmmaArgs& g, unsigned char* smem) {
    constexpr int STAGE = gemm_stage_bytes(PAIR);
    const int NST = g.nst;                              // at most 8
    constexpr uint32_t TM_COLS = gemm_tmem_cols(PAIR), SF_COL = TM_COLS - 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long tr_cta0 = clock64();
    uint64_t* sBar = reinterpret_cast<uint64_t*>(smem + (size_t)NST * STAGE);
    // barriers: full[NST] | empty[NST] | acc_full | drain
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 2 * NST + 2);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sTmem + 1);
    const uint32_t bar0 = smem_u32(sBar);
    auto BAR_FULL = [&](int s) { return bar0 + 8u * s; };
    auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (NST + s); };
    const uint32_t BAR_ACC = bar0 + 8u * (2 * NST), BAR_DRAIN = bar0 + 8u * (2 * NST + 1);

    // tile of this CTA: blockIdx.x = (split * tiles_m + tm) * NT + tn; tm counts pairs of sub-tiles when PAIR
    const int tiles_m = PAIR ? (g.MT + 1) >> 1 : g.MT;
    const int tn = blockIdx.x % g.NT;
    const int tm = (blockIdx.x / g.NT) % tiles_m;
    const int split = blockIdx.x / (g.NT * tiles_m);
    const int kb0 = split * g.per, kb1 = min(g.KB, kb0 + g.per);
    const int rt0 = PAIR ? tm * 2 : tm;                 // first 128-row tile of A
    const bool two = PAIR && rt0 + 1 < g.MT;            // second 128-row sub-tile exists

    if (tid == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(BAR_FULL(s), 2); mbar_init(BAR_EMPTY(s), 1); }
        mbar_init(BAR_ACC, 1);
        mbar_init(BAR_DRAIN, 1);
        *sAbort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) tmem_alloc(smem_u32(sTmem), TM_COLS);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *sTmem;
    if (warp < 4) tmem_fill_unit_scales(tmem, SF_COL);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const WsWait wait{sAbort, g.status};
    // Launched as a programmatic dependent of the expansion pass, the CTA has come this far while
    // that pass was still running; its units are complete (and visible) once this returns.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr uint32_t OFF_W = (PAIR ? 2u : 1u) * kGemmKU * kGemmUnit;     // W's place inside a stage
    const bool tr = g.trace != nullptr && blockIdx.x == 0;

    if (warp == 8 || warp == 10) {
        // =============================== loaders ============================================
        if (lane == 0) {
            const bool isw = warp == 10;
            int s = 0;
            uint32_t ph = 0, issued = 0;
            bool ok = true;
            long long tr_w = 0;
            for (int kb = kb0; kb < kb1; kb += kGemmKU) {
                const uint32_t nkb = (uint32_t)min(kGemmKU, kb1 - kb);
                ok = tr ? wait.timed(BAR_EMPTY(s), ph ^ 1, tr_w) : wait(BAR_EMPTY(s), ph ^ 1);
                if (!ok) break;
                const uint32_t dst = smem_u32(smem + (size_t)s * STAGE);
                if (isw) {
                    mbar_expect_tx(BAR_FULL(s), nkb * kGemmUnit);
                    bulk_g2s(dst + OFF_W, g.ew + ((size_t)tn * g.KB + kb) * kGemmUnit, nkb * kGemmUnit, BAR_FULL(s));
                } else {
                    mbar_expect_tx(BAR_FULL(s), (two ? 2u : 1u) * nkb * kGemmUnit);
                    bulk_g2s(dst, g.ea + ((size_t)rt0 * g.KB + kb) * kGemmUnit, nkb * kGemmUnit, BAR_FULL(s));
                    if (two)
                        bulk_g2s(dst + kGemmKU * kGemmUnit, g.ea + ((size_t)(rt0 + 1) * g.KB + kb) * kGemmUnit,
                                 nkb * kGemmUnit, BAR_FULL(s));
                }
                issued++;
                if (++s == NST) { s = 0; ph ^= 1; }
            }
            if (tr && !isw) g.trace[10] = tr_w;
            if (!ok) {
                // giving up: wait (bounded) for the copies still in flight before the CTA exits.  A
                // stage's barrier completes once both loaders' copies have landed; if the other
                // loader never got that far the polls run out, which takes longer than any copy.
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
        constexpr uint32_t IDESC = idesc_f4(128);
        const uint64_t desc0 = smem_desc(smem_u32(smem), 128 * 16, 128u);
        const uint32_t hi = (uint32_t)(desc0 >> 32), lo0 = (uint32_t)desc0;
        constexpr uint32_t stepStage = STAGE >> 4, stepUnit = kGemmUnit >> 4, offW = OFF_W >> 4,
                           offA2 = (kGemmKU * kGemmUnit) >> 4;
        const uint32_t sfa = tmem + SF_COL, sfb = tmem + SF_COL + 16;
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        long long tr_w = 0;
        const long long tr_t0 = clock64();
        for (int kb = kb0; kb < kb1 && ok; kb += kGemmKU) {
            const int nkb = min(kGemmKU, kb1 - kb);
            ok = tr ? wait.timed(BAR_FULL(s), ph, tr_w) : wait.spin(BAR_FULL(s), ph);
            if (!ok) break;
            tc_fence_after();
            if (leader) {
                const uint32_t a = lo0 + s * stepStage, b = a + offW;
#pragma unroll
                for (int j = 0; j < kGemmKU; j++) {
                    if (j < nkb) {
                        const uint32_t acc = (kb > kb0 || j > 0) ? 1u : 0u;
                        mma_f4_split(tmem, a + j * stepUnit, hi, b + j * stepUnit, hi, IDESC, acc, sfa, sfb);
                        if (two)
                            mma_f4_split(tmem + 128, a + offA2 + j * stepUnit, hi, b + j * stepUnit, hi, IDESC, acc, sfa, sfb);
                    }
                }
                mma_commit(BAR_EMPTY(s));
            }
            if (++s == NST) { s = 0; ph ^= 1; }
        }
        if (ok && leader) mma_commit(BAR_ACC);
        if (tr && leader) { g.trace[11] = clock64() - tr_t0; g.trace[12] = tr_w; g.trace[14] = kb1 - kb0; }
        if (!ok && leader) {
            // giving up: the MMAs already issued must have finished before tensor memory is freed
            mma_commit(BAR_DRAIN);
            for (int i = 0; i < (1 << 20); i++)
                if (mbar_try_wait(BAR_DRAIN, 0)) break;
        }
        __syncwarp();
    } else if (warp < 8) {
        // =============================== epilogue ===========================================
        const int sub = warp >> 2, quad = warp & 3;
        const int m = (rt0 + sub) * 128 + quad * 32 + lane;
        const bool have = sub == 0 || two;
        const long long tr_t0 = clock64();
        const bool acc_ok = wait.relaxed(BAR_ACC, 0);
        if (g.trace != nullptr && blockIdx.x == 0 && tid == 0) g.trace[13] = clock64() - tr_t0;
        const long long tr_t1 = clock64();
        if (acc_ok && have) {
            tc_fence_after();
            const bool vec = (g.N & 3) == 0;
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
                int v[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + sub * 128 + nb * 32, v);
                tmem_ld_wait();
                const int n0 = tn * 128 + nb * 32;
                if (m >= g.M || n0 >= g.N) continue;
                if (g.splits > 1 || g.mode == GEMM_INT32) {
                    // int32 sums: the split-K partials, or C itself
                    int32_t* dst = g.splits > 1 ? g.partial + ((size_t)split * g.M + m) * g.N + n0
                                                : reinterpret_cast<int32_t*>(g.out) + (size_t)m * g.ldo + n0;
                    const bool v4 = g.splits > 1 ? vec : ((g.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int c0 = f4_acc_to_int(v[4 * j]), c1 = f4_acc_to_int(v[4 * j + 1]);
                        const int c2 = f4_acc_to_int(v[4 * j + 2]), c3 = f4_acc_to_int(v[4 * j + 3]);
                        if (v4 && n0 + 4 * j + 3 < g.N) {
                            *reinterpret_cast<int4*>(dst + 4 * j) = make_int4(c0, c1, c2, c3);
                        } else {
                            const int cc[4] = {c0, c1, c2, c3};
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                if (n0 + 4 * j + k < g.N) dst[4 * j + k] = cc[k];
                        }
                    }
                } else if (g.mode == GEMM_FC_BITS) {
                    // (float)K - 2*(float)c >= thr[n] (kernel.cuh:210-213): the accumulator is that value
                    uint32_t word = 0;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (n0 + j < g.N && __int_as_float(v[j]) >= __ldg(g.p0 + n0 + j)) word |= 0x80000000u >> j;
                    reinterpret_cast<uint32_t*>(g.out)[(size_t)m * g.ldo + (n0 >> 5)] = word;
                } else {
                    // scale and bias (kernel.cuh:270-273), fused multiply-add
                    float* dst = reinterpret_cast<float*>(g.out) + (size_t)m * g.ldo + n0;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (n0 + j < g.N) dst[j] = fmaf(__int_as_float(v[j]), __ldg(g.p0 + n0 + j), __ldg(g.p1 + n0 + j));
                }
            }
        }
        if (g.trace != nullptr && blockIdx.x == 0 && tid == 0) g.trace[15] = clock64() - tr_t1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, TM_COLS);
    if (g.trace != nullptr && blockIdx.x == 0 && tid == 0) g.trace[9] = clock64() - tr_cta0;
}

}  // namespace umma
}  // namespace tcbnn
