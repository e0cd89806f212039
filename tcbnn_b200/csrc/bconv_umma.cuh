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
//
// This header holds the PTX wrappers, descriptors and bit -> byte expansion shared by the kernels:
// bconv_umma_ws.cuh (filter-stationary), bconv_umma_as.cuh (activation-stationary),
// bconv_umma_pre.cuh (fed from a pre-expanded input), bgemm_umma.cuh (bit GEMM).
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

// ---- 4-bit operands: tcgen05.mma kind::mxf4 ------------------------------------------------
// +1 / -1 are exact in e2m1 (0x2 / 0xA), zero is 0x0, and with unit ue8m0 block scales (byte 0x7F)
// the fp32 accumulator of a +-1 contraction is the exact integer sum (every partial sum is an
// integer far below 2^24).  An MMA is 128 x N x 64: twice the MAC rate of kind::i8 at half the
// operand bytes (measured by tcbnn_mma_peak kind 7).  Layout as for int8, K-major without
// swizzle, except that a 16-byte core-matrix row now holds 32 channels and one MMA spans two of
// them (`lbo` apart).
// 8 packed bits -> 8 nibbles (bit i -> nibble i; 1 -> +1.0, 0 -> -1.0)
__host__ __device__ __forceinline__ uint32_t expand8_f4(uint32_t b) {
    uint32_t x = b & 0xFFu;
    x = (x | (x << 12)) & 0x000F000Fu;
    x = (x | (x << 6)) & 0x03030303u;
    x = (x | (x << 3)) & 0x11111111u;
    return 0xAAAAAAAAu ^ (x << 3);
}
// 32 packed bits -> 16 bytes; bits 31..24 (the chunk's channels 0-7) land in .x, 7..0 in .w.
// Activations and filters both go through this function, so the order inside a word cancels.
__host__ __device__ __forceinline__ uint4 expand32_f4(uint32_t w) {
    return make_uint4(expand8_f4(w >> 24), expand8_f4(w >> 16), expand8_f4(w >> 8), expand8_f4(w));
}
// Instruction descriptor of the block-scaled kinds: e2m1 x e2m1, ue8m0 scales, K-major, M = 128,
// K = 64, scale-factor ids 0.
__host__ __device__ constexpr uint32_t idesc_f4(int n) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
}
// D[tmem] (+)= A * B with the scale factors read from tensor memory at sfa / sfb; descriptors as
// (low, high) register pairs like mma_i8_split.
__device__ __forceinline__ void mma_f4_split(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                             uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], da, db, %5, [%7], [%8], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(sfa), "r"(sfb));
}
// Columns [col, col + 32) of the calling warp's 32 lanes of tensor memory := unit scales (every
// byte 0x7F), so a scale reads as 1.0 wherever in the region the hardware looks it up.  Whole
// warp; warps 0-3 of a warpgroup cover the 128 lanes between them (warp w -> lanes 32*(w%4)..).
__device__ __forceinline__ void tmem_fill_unit_scales(uint32_t tmem, uint32_t col) {
    const uint32_t base = tmem + ((uint32_t)(((threadIdx.x >> 5) & 3) * 32) << 16) + col;
#pragma unroll
    for (int c = 0; c < 32; c += 8)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};"
                     ::"r"(base + c), "r"(0x7F7F7F7Fu) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// fp32 accumulator holding an integer of magnitude below 2^22 -> that integer, exactly
__device__ __forceinline__ int f4_acc_to_int(int raw) {
    return __float_as_int(__int_as_float(raw) + 12582912.0f) - 0x4B400000;
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

}  // namespace umma
}  // namespace tcbnn
