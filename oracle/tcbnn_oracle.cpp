// CPU oracle for the binarised-network hot path: a plain C++ restatement of the
// reference's layer arithmetic (pnnl/TCBNN kernel.cuh / param.h / bmm/tensorcore_kernel.cu).
//
// THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the CUDA path is compared
// against and the timed CPU baseline; nothing in the shipped library calls it.
//
// Parity status: the popcount GEMM core is pinned against the reference's own host
// functions (BMMAcpu, bmm/tensorcore_kernel.cu:38-57 and WMMABOOLCPU,
// bmm/bmma_op_test/main_test.cu:232-254) compiled from their sources, and against the
// reference's one seeded known-answer recipe (srand(4)+rand(), main_test.cu:293-298).
// The layer epilogues (threshold, pooling, residual, first-layer fp32 path) have no golden
// vectors anywhere in the reference: for those this oracle is "parity unpinned" and
// follows the cited reference lines statement by statement.
//
// Data formats (shared with the CUDA library so words can be compared directly):
//   * bit rows: element e of a row lives in 32-bit word e/32 at bit (31 - e%32), i.e. the
//     order produced by __brev(__ballot_sync(..)) in the reference packers (param.h:60).
//     bit 1 <-> +1, bit 0 <-> -1; pad bits are 0 in every operand.
//   * FC activations / weights: [rows][ld] words, ld >= ceil(K/32).
//   * conv activations: NHWC, [B][H][W][Cw] words with Cw = ceil(C/32).
//   * conv filters: [O][R*S][Cw] words (tap-major, then input channel).
//   * residuals and accumulators: NHWC int32 [B][P][Q][O] (no channel padding).
// The reference keeps the same bits in its HWNC / 8x128-tile "FMT" orders
// (kernel.cuh:650-660, 798-816); the values are layout independent.
#include <cstdint>
#include <cstring>
#include <cmath>
#include <climits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks for all cores
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline int popc32(uint32_t x) { return __builtin_popcount(x); }

// ---------------------------------------------------------------------------------------
// Packing.  bit = (x >= 0) as in In128LayerFMT (kernel.cuh:165-168: out-of-range -> -1.0f
// -> bit 0) and PackFcWeight128FMT (param.h:58-60).
// ---------------------------------------------------------------------------------------
void orc_pack_rows(const float* x, int rows, int cols, int ld_words, uint32_t* out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        uint32_t* o = out + (size_t)r * ld_words;
        for (int w = 0; w < ld_words; w++) o[w] = 0;
        for (int c = 0; c < cols; c++)
            if (x[(size_t)r * cols + c] >= 0) o[c >> 5] |= 1u << (31 - (c & 31));
    }
}

// FC weight: fp32 W[K][N] (row-major, as read by launch_array, param.h:272-274) ->
// bit rows [N][ld] over K (param.h:44-63).
void orc_pack_fc_weight(const float* W, int K, int N, int ld_words, uint32_t* out) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        uint32_t* o = out + (size_t)n * ld_words;
        for (int w = 0; w < ld_words; w++) o[w] = 0;
        for (int k = 0; k < K; k++)
            if (W[(size_t)k * N + n] >= 0) o[k >> 5] |= 1u << (31 - (k & 31));
    }
}

// Conv filter: fp32 F[R*S][C][O] (param.h:573-575) -> bits [O][R*S][Cw].
void orc_pack_conv_filter(const float* F, int RS, int C, int O, uint32_t* out) {
    const int Cw = (C + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        uint32_t* dst = out + (size_t)o * RS * Cw;
        for (int i = 0; i < RS * Cw; i++) dst[i] = 0;
        for (int t = 0; t < RS; t++)
            for (int c = 0; c < C; c++)
                if (F[((size_t)t * C + c) * O + o] >= 0)
                    dst[t * Cw + (c >> 5)] |= 1u << (31 - (c & 31));
    }
}

// bits -> +-1 floats (UnPackFcOutput128FMT, param.h:102; UnpackConvOutput32FMT, param.h:685).
void orc_unpack_rows(const uint32_t* in, int rows, int cols, int ld_words, float* out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) {
            uint32_t w = in[(size_t)r * ld_words + (c >> 5)];
            out[(size_t)r * cols + c] = 2 * (float)((w >> (31 - (c & 31))) & 1u) - 1;
        }
}

// ---------------------------------------------------------------------------------------
// Bit GEMM.  acc[m][n] = sum_k popc(A[m][k] ^ B[n][k]) (tensorcore_kernel.cu:38-57),
// C = K - 2*acc (tensorcore_kernel.cu:331).
// ---------------------------------------------------------------------------------------
static inline int xor_popc_row(const uint32_t* a, const uint32_t* b, int words) {
    int s = 0;
    int w = 0;
    for (; w + 1 < words; w += 2) {
        uint64_t x, y;
        memcpy(&x, a + w, 8);
        memcpy(&y, b + w, 8);
        s += __builtin_popcountll(x ^ y);
    }
    for (; w < words; w++) s += popc32(a[w] ^ b[w]);
    return s;
}

void orc_bgemm_popc(const uint32_t* A, const uint32_t* B, int M, int N, int K, int lda, int ldb,
                    int32_t* acc) {
    const int words = (K + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++)
            acc[(size_t)m * N + n] = xor_popc_row(A + (size_t)m * lda, B + (size_t)n * ldb, words);
}

void orc_bgemm(const uint32_t* A, const uint32_t* B, int M, int N, int K, int lda, int ldb,
               int32_t* C) {
    const int words = (K + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++)
            C[(size_t)m * N + n] =
                K - 2 * xor_popc_row(A + (size_t)m * lda, B + (size_t)n * ldb, words);
}

// Hidden FC layer (Fc128LayerFMT, kernel.cuh:197-224):
//   bit[m][n] = ((float)K - 2*(float)acc >= thr[n]); pad columns stay 0.
void orc_fc_layer(const uint32_t* A, const uint32_t* W, const float* thr, int M, int K, int N,
                  int lda, int ldw, int ldo, uint32_t* out) {
    const int words = (K + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        uint32_t* o = out + (size_t)m * ldo;
        for (int w = 0; w < ldo; w++) o[w] = 0;
        for (int n = 0; n < N; n++) {
            int c = xor_popc_row(A + (size_t)m * lda, W + (size_t)n * ldw, words);
            bool v = (((float)K) - 2 * (float)c) >= thr[n];
            if (v) o[n >> 5] |= 1u << (31 - (n & 31));
        }
    }
}

// Output layer (Out128LayerFMT, kernel.cuh:270-273):
//   out[m][n] = ((float)K - (float)acc*2.0f) * scale[n] + bias[n].
// The multiply-add is evaluated fused (the reference is built with nvcc's default
// -fmad=true, which contracts it); K - 2*acc is exact in fp32 either way.
void orc_out_layer(const uint32_t* A, const uint32_t* W, const float* scale, const float* bias,
                   int M, int K, int N, int lda, int ldw, float* out) {
    const int words = (K + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            int c = xor_popc_row(A + (size_t)m * lda, W + (size_t)n * ldw, words);
            float t = (float)K - (float)c * 2.0f;
            out[(size_t)m * N + n] = fmaf(t, scale[n], bias[n]);
        }
}

// ---------------------------------------------------------------------------------------
// Conv shape arithmetic (param.h:719-728 and 897-906).
// ---------------------------------------------------------------------------------------
void orc_conv_shape(int H, int W, int R, int S, int sh, int sw, int padding, int ph, int pw,
                    int* pad_h, int* pad_w, int* P, int* Q, int* OH, int* OW) {
    *pad_h = padding ? ((((H + sh - (H % sh)) / sh - 1) * sh + R - H) / 2) : 0;
    *pad_w = padding ? ((((W + sw - (W % sw)) / sw - 1) * sw + S - W) / 2) : 0;
    int bh = padding ? (H + sh - 1) / sh : ((H - R) / sh + 1);
    int bw = padding ? (W + sw - 1) / sw : ((W - S) / sw + 1);
    *OH = (bh + ph - 1) / ph;
    *OW = (bw + pw - 1) / pw;
    // the layer kernels iterate over pool*output pre-pool pixels (kernel.cuh:685-686)
    *P = ph * (*OH);
    *Q = pw * (*OW);
}

// ---------------------------------------------------------------------------------------
// Binary conv layer (Conv128LayerFMT, kernel.cuh:676-827).
//   acc   = sum over in-frame taps of popc(a ^ w)                       (:720-757)
//   res   = C*R*S - exclude*C - 2*acc                                   (:766-768)
//   res  += residual (plain, or max over the 2x2 window when residual_pool) for
//           o < residual_channels                                       (:770-794)
//   bit   = !((float)res < thr[o]) OR-ed into the pooled pixel          (:795-816)
//   res_out = res (after injection) when save_residual                  (:818-824)
// in  : [B][H][W][Cw], filt: [O][R*S][Cw], out: [B] images of out_image_stride words each
//       holding [OH][OW][Ow] (Ow = ceil(O/32)); res_in: [B][P or 2P][Q or 2Q][res_in_ch].
// acc_out (optional): res before residual injection, [B][P][Q][O].
// Residual channels the producer never wrote read as 0 (the reference memsets the
// PAD128-wide buffer, param.h:979-980).
// ---------------------------------------------------------------------------------------
void orc_conv_layer(const uint32_t* in, const uint32_t* filt, const float* thr,
                    int B, int H, int W, int C, int O, int R, int S, int sh, int sw,
                    int pad_h, int pad_w, int ph, int pw, int OH, int OW,
                    const int32_t* res_in, int res_in_ch, int residual_channels,
                    int residual_pool,
                    uint32_t* out, long out_image_stride, int32_t* res_out, int32_t* acc_out) {
    const int Cw = (C + 31) / 32, Ow = (O + 31) / 32;
    const int P = ph * OH, Q = pw * OW;
    for (int b = 0; b < B; b++) memset(out + (size_t)b * out_image_stride, 0,
                                       sizeof(uint32_t) * (size_t)OH * OW * Ow);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int y = 0; y < P; y++) {
            std::vector<const uint32_t*> win(R * S);
            for (int x = 0; x < Q; x++) {
                int exclude = 0;
                for (int r = 0; r < R; r++)
                    for (int s = 0; s < S; s++) {
                        int ay = y * sh - pad_h + r, ax = x * sw - pad_w + s;
                        if (ay >= 0 && ay < H && ax >= 0 && ax < W)
                            win[r * S + s] = in + (((size_t)b * H + ay) * W + ax) * Cw;
                        else { win[r * S + s] = nullptr; exclude++; }
                    }
                uint32_t* opix = out + (size_t)b * out_image_stride +
                                 ((size_t)(y / ph) * OW + (x / pw)) * Ow;
                for (int o = 0; o < O; o++) {
                    const uint32_t* wf = filt + (size_t)o * R * S * Cw;
                    int acc = 0;
                    for (int t = 0; t < R * S; t++)
                        if (win[t]) acc += xor_popc_row(win[t], wf + (size_t)t * Cw, Cw);
                    int res = C * R * S - exclude * C - 2 * acc;
                    size_t oidx = (((size_t)b * P + y) * Q + x) * O + o;
                    if (acc_out) acc_out[oidx] = res;
                    if (res_in && o < residual_channels) {
                        int residual = 0;
                        if (residual_pool) {
                            residual = INT_MIN;
                            for (int i = 0; i < 2; i++)
                                for (int j = 0; j < 2; j++) {
                                    int v = (o < res_in_ch)
                                        ? res_in[(((size_t)b * 2 * P + (2 * y + i)) * 2 * Q +
                                                  (2 * x + j)) * res_in_ch + o]
                                        : 0;
                                    residual = v > residual ? v : residual;
                                }
                        } else {
                            residual = (o < res_in_ch)
                                ? res_in[(((size_t)b * P + y) * Q + x) * res_in_ch + o] : 0;
                        }
                        res += residual;
                    }
                    bool bit = !((float)res < thr[o]);
                    if (bit) {
#pragma omp atomic
                        opix[o >> 5] |= 1u << (31 - (o & 31));
                    }
                    if (res_out) res_out[oidx] = res;
                }
            }
        }
}

// ---------------------------------------------------------------------------------------
// First (fp32-input) conv layer (InConv128LayerFMT, kernel.cuh:578-672).
//   x: NCHW fp32 [B][3][H][W] (:620-625); filter signs from fp32 F[R*S][3][O], bit=(f>=0)
//   (param.h:626-628).  Per in-frame tap, in r-then-s order (:609-643):
//       acc[o] += ((w0? f0:-f0) + (w1? f1:-f1)) + (w2? f2:-f2)
//   bit = !(acc < thr[o]) OR-ed into the pooled pixel (:655-660);
//   residual = (int)acc, truncation toward zero (:666-668).
// ---------------------------------------------------------------------------------------
void orc_inconv_layer(const float* x, const float* F, const float* thr,
                      int B, int H, int W, int O, int R, int S, int sh, int sw,
                      int pad_h, int pad_w, int ph, int pw, int OH, int OW,
                      uint32_t* out, long out_image_stride, int32_t* res_out, float* acc_out) {
    const int Ow = (O + 31) / 32;
    const int P = ph * OH, Q = pw * OW;
    for (int b = 0; b < B; b++) memset(out + (size_t)b * out_image_stride, 0,
                                       sizeof(uint32_t) * (size_t)OH * OW * Ow);
    // sign tables: sg[t][c][o] = +1 / -1
    std::vector<float> sg((size_t)R * S * 3 * O);
    for (size_t i = 0; i < sg.size(); i++) sg[i] = F[i] >= 0 ? 1.0f : -1.0f;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int y = 0; y < P; y++) {
            std::vector<float> acc(O);
            for (int xq = 0; xq < Q; xq++) {
                for (int o = 0; o < O; o++) acc[o] = 0.0f;
                for (int r = 0; r < R; r++) {
                    int ay = y * sh - pad_h + r;
                    if (ay < 0 || ay >= H) continue;
                    for (int s = 0; s < S; s++) {
                        int ax = xq * sw - pad_w + s;
                        if (ax < 0 || ax >= W) continue;
                        float f0 = x[(((size_t)b * 3 + 0) * H + ay) * W + ax];
                        float f1 = x[(((size_t)b * 3 + 1) * H + ay) * W + ax];
                        float f2 = x[(((size_t)b * 3 + 2) * H + ay) * W + ax];
                        const float* w = &sg[(size_t)(r * S + s) * 3 * O];
                        for (int o = 0; o < O; o++) {
                            float t01 = (w[o] > 0 ? f0 : -f0) + (w[O + o] > 0 ? f1 : -f1);
                            float t = t01 + (w[2 * O + o] > 0 ? f2 : -f2);
                            acc[o] = acc[o] + t;
                        }
                    }
                }
                uint32_t* opix = out + (size_t)b * out_image_stride +
                                 ((size_t)(y / ph) * OW + (xq / pw)) * Ow;
                for (int o = 0; o < O; o++) {
                    size_t oidx = (((size_t)b * P + y) * Q + xq) * O + o;
                    bool bit = !(acc[o] < thr[o]);
                    if (bit) {
#pragma omp atomic
                        opix[o >> 5] |= 1u << (31 - (o & 31));
                    }
                    if (res_out) res_out[oidx] = (int32_t)acc[o];
                    if (acc_out) acc_out[oidx] = acc[o];
                }
            }
        }
}

// 64-bit mixing counter generator used by tests and benches to make identical inputs on the
// CPU and GPU sides without files (splitmix64 finaliser of seed and index).
static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
void orc_fill_words(uint32_t* dst, size_t n, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = (uint32_t)(mix64(seed * 0x100000001B3ull + i) >> 32);
}

}  // extern "C"
