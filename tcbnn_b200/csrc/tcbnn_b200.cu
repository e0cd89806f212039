// libtcbnn_b200.so: kernels and C ABI of the binarised-network hot path (see
// include/tcbnn_b200.h for the contract of each entry point).
#include "../../include/tcbnn_b200.h"
#include "bnn_layers.cuh"
#include "bconv_umma.cuh"
#include "bconv_umma_ws.cuh"
#include "bconv_umma_as.cuh"
#include "bconv_umma_pre.cuh"
#include "bgemm_umma.cuh"
#include "inconv_spec.cuh"
#include "inconv_tiled.cuh"
#include <cstdio>
#include <cstdarg>
#include <cstring>
#include <atomic>
#include <mutex>
#include <vector>

using namespace tcbnn;

namespace {

thread_local char g_err[512] = "";

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return 1;
}

#define CUDA_TRY(expr)                                                              \
    do {                                                                            \
        cudaError_t e_ = (expr);                                                    \
        if (e_ != cudaSuccess)                                                      \
            return fail("%s failed: %s", #expr, cudaGetErrorString(e_));            \
    } while (0)

int sm_count(int* sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail("no CUDA device: %s", cudaGetErrorString(e));
    // per-device caches are shared by every host thread that drives a GPU of its own
    static std::atomic<int> cache[64];
    if (dev >= 0 && dev < 64) {
        const int c = cache[dev].load(std::memory_order_relaxed);
        if (c) { *sms = c; return 0; }
    }
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || n <= 0) return fail("cannot query SM count: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) cache[dev].store(n, std::memory_order_relaxed);
    *sms = n;
    return 0;
}

// First-use configuration of a kernel on the current device (opt-in shared memory size): done once
// per device, under a lock, because callers may drive several GPUs from threads of one process.
std::mutex g_configure_mutex;
template <class F>
int configure_once(bool (&done)[64], F&& configure) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_configure_mutex);
    if (dev >= 0 && dev < 64 && done[dev]) return 0;
    const cudaError_t e = configure();
    if (e != cudaSuccess) return fail("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return 0;
}

constexpr int kThreads = 256;          // 8 warps per CTA
constexpr int kCtasPerSm = 2;          // 16 resident warps per SM, up to 128 registers each

// grid for `tasks` warp-sized tasks on a persistent warp-strided loop
int warp_grid(long long tasks, int sms) {
    long long ctas = (tasks + (kThreads / 32) - 1) / (kThreads / 32);
    long long cap = (long long)kCtasPerSm * sms;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return (int)ctas;
}

__global__ void __launch_bounds__(kThreads, kCtasPerSm) k_gemm(GemmArgs g) { gemm_layer(g); }
__global__ void __launch_bounds__(kThreads, kCtasPerSm) k_gemm_finish(GemmArgs g) { gemm_splitk_finish(g); }
__global__ void __launch_bounds__(kThreads, kCtasPerSm) k_conv(ConvArgs c) { conv_layer(c); }
__global__ void __launch_bounds__(kThreads, kCtasPerSm) k_inconv(InConvArgs c) { inconv_layer(c); }
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
k_pack_rows(const float* x, int rows, int cols, int ld, uint32_t* out) {
    pack_rows(x, rows, cols, ld, out);
}
__global__ void __launch_bounds__(kThreads, 8)
k_pack_rows_vec(const float* x, int rows, int cols, int ld, uint32_t* out) {
    pack_rows_vec(x, rows, cols, ld, out);
}
__global__ void k_unpack_rows(const uint32_t* in, int rows, int cols, int ld, float* out) {
    unpack_rows(in, rows, cols, ld, out);
}
__global__ void k_pack_fc_weight(const float* W, int K, int N, int ld, uint32_t* out) {
    pack_fc_weight(W, K, N, ld, out);
}
__global__ void k_pack_conv_filter(const float* F, int RS, int C, int O, uint32_t* out) {
    pack_conv_filter(F, RS, C, O, out);
}
__global__ void k_pack_inconv_filter(const float* F, int RS, int O, uint32_t* out) {
    pack_inconv_filter(F, RS, O, out);
}
__global__ void k_conv_prepare(const uint32_t* fbits, int O, int R, int S, int Cw, int W_in, int KP,
                               uint32_t* wq, uint32_t* ktab, int* pwt, int* pwtot) {
    conv_prepare(fbits, O, R, S, Cw, W_in, KP, wq, ktab, pwt, pwtot);
}

int launch_check(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

int elementwise_grid(long long n, int sms) {
    long long b = (n + 255) / 256;
    long long cap = 8LL * sms;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

// ---- split-K policy ---------------------------------------------------------------------
int gemm_splits(int M, int N, int K, int sms) {
    const long long tiles = (long long)((M + 31) / 32) * ((N + 31) / 32);
    const long long slots = (long long)sms * kCtasPerSm * (kThreads / 32);
    const int KP = (K + 63) / 64;
    if (tiles * 2 > slots || KP < 32) return 1;
    long long s = (slots + tiles - 1) / tiles;
    if (s > KP / 8) s = KP / 8;
    if (s > 32) s = 32;
    return s < 1 ? 1 : (int)s;
}

// ---- tcgen05 bit GEMM (bgemm_umma.cuh) -----------------------------------------------------
long long* g_conv_trace = nullptr;   // device buffer for per-role cycle counters, or null
int g_gemm_force_pair = -1, g_gemm_force_splits = -1;   // tcbnn_set_gemm_plan: -1 = from the model
__device__ int g_gemm_status;        // 1 after a bounded wait inside k_gemm_umma gave up

__global__ void __launch_bounds__(256) k_expand_rows(const uint32_t* a_bits, int a_rows, int a_ld, int RT_a,
                                                     const uint32_t* w_bits, int w_rows, int w_ld, int RT_w,
                                                     int K, int KB, uint4* out_a, uint4* out_w) {
    umma::expand_rows_pair(a_bits, a_rows, a_ld, RT_a, w_bits, w_rows, w_ld, RT_w, K, KB, out_a, out_w);
}
template <bool PAIR>
__global__ void __launch_bounds__(umma::kGemmThreads, 1) k_gemm_umma(umma::GemmUmmaArgs g) {
    extern __shared__ __align__(128) unsigned char dyn_smem_gemm[];
    umma::gemm_umma_cta<PAIR>(g, dyn_smem_gemm);
}

struct GemmUmmaPlan {
    bool use;
    bool pair;            // 256 x 128 tiles (two sub-tiles of A per CTA) instead of 128 x 128
    int stages;           // ring depth; fixes the dynamic shared memory and with it the CTAs per SM
    int MT, NT, KB, splits, per;
    size_t off_ea, off_ew, off_partial, bytes;
};

// Tile shape and split count of the tcgen05 path from a clock model of its launches, calibrated
// on the kernel's own cycle counters (tcbnn_conv_set_trace): a k-block costs a lone 128 x 128 CTA
// about 150 clocks, each of two such CTAs sharing an SM 250, a 256 x 128 CTA 180 (the loads, not
// the MMAs, set the pace); set-up and epilogue cost a CTA 6500, 8000 and 11000 clocks; more than
// one split adds the finishing launch and the partial sums' round trip.
GemmUmmaPlan gemm_umma_plan(int M, int N, int K, int sms) {
    GemmUmmaPlan p = {};
    // below 2^30 multiply-adds the single launch of the warp-level kernel wins (measured; a plan
    // forced through tcbnn_set_gemm_plan waives that); the fp32 accumulators hold K exactly up to 2^22
    const bool forced = g_gemm_force_pair >= 0 || g_gemm_force_splits > 0;
    p.use = M >= 128 && N >= 64 && K >= 512 && K < (1 << 22) && ((long long)M * N * K >= (1LL << 30) || forced);
    if (!p.use) return p;
    p.MT = (M + 127) / 128; p.NT = (N + 127) / 128; p.KB = (K + 63) / 64;
    double best = 1e30;
    for (int pair = 0; pair < 2; pair++) {
        if (g_gemm_force_pair >= 0 && pair != g_gemm_force_pair) continue;
        if (pair && p.MT < 2 && g_gemm_force_pair < 0) continue;
        const long long tiles = (long long)(pair ? (p.MT + 1) / 2 : p.MT) * p.NT;
        for (int want = 1; want <= 32 && (want <= (p.KB + 3) / 4 || g_gemm_force_splits > 0); want++) {
            const int per = (p.KB + want - 1) / want;
            const int splits = (p.KB + per - 1) / per;                    // no empty split
            if (splits != want && want > 1) continue;
            if (g_gemm_force_splits > 0 && want != (g_gemm_force_splits < p.KB ? g_gemm_force_splits : p.KB)) continue;
            const long long ctas = tiles * splits;
            const bool shared_sm = !pair && ctas > sms;                   // two 128 x 128 CTAs per SM
            const long long resident = (long long)sms * (shared_sm ? 2 : 1);
            const long long waves = (ctas + resident - 1) / resident;
            const double kblock = pair ? 180.0 : (shared_sm ? 250.0 : 150.0);
            const double fixed = pair ? 11000.0 : (shared_sm ? 8000.0 : 6500.0);
            double clk = (double)waves * (per * kblock + fixed);
            if (splits > 1) clk += 12000.0 + 6.0 * splits * (double)M * N * 4.0 / 3000.0;
            if (clk < best) { best = clk; p.pair = pair != 0; p.splits = splits; p.per = per; }
        }
    }
    if (p.splits < 1) { p.use = false; return p; }      // a forced plan no slicing of K gives
    {
        const long long ctas = (long long)(p.pair ? (p.MT + 1) / 2 : p.MT) * p.NT * p.splits;
        p.stages = p.pair ? 4 : (ctas > sms ? 3 : 6);
    }
    size_t o = 0;
    p.off_ea = o;      o += (size_t)p.MT * p.KB * umma::kGemmUnit;  o = (o + 255) & ~(size_t)255;
    p.off_ew = o;      o += (size_t)p.NT * p.KB * umma::kGemmUnit;  o = (o + 255) & ~(size_t)255;
    p.off_partial = o; o += p.splits > 1 ? (size_t)p.splits * M * N * sizeof(int32_t) : 0;
    p.bytes = o;
    return p;
}

int run_gemm_umma(const GemmArgs& g, const GemmUmmaPlan& p, void* workspace, int sms, cudaStream_t st) {
    static bool configured[64] = {false};
    if (configure_once(configured, [] {
            cudaError_t e = cudaFuncSetAttribute(k_gemm_umma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)umma::gemm_smem(true, 4));
            if (e != cudaSuccess) return e;
            return cudaFuncSetAttribute(k_gemm_umma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)umma::gemm_smem(false, 6));
        }))
        return 1;
    char* w = (char*)workspace;
    {
        const long long tasks = (long long)(p.MT + p.NT) * ((p.KB + 3) / 4);   // one CTA per task, up to 8 per SM
        const int grid = (int)(tasks < (long long)sms * 8 ? tasks : (long long)sms * 8);
        k_expand_rows<<<grid, 256, 0, st>>>(g.A, g.M, g.lda, p.MT, g.W, g.N, g.ldw, p.NT, g.K, p.KB,
                                            (uint4*)(w + p.off_ea), (uint4*)(w + p.off_ew));
    }
    if (launch_check("gemm (operand expansion)")) return 1;
    umma::GemmUmmaArgs a;
    a.ea = (const unsigned char*)(w + p.off_ea); a.ew = (const unsigned char*)(w + p.off_ew);
    a.M = g.M; a.N = g.N; a.KB = p.KB; a.MT = p.MT; a.NT = p.NT; a.splits = p.splits; a.per = p.per;
    a.partial = p.splits > 1 ? (int32_t*)(w + p.off_partial) : nullptr;
    a.mode = g.mode; a.out = g.out; a.ldo = g.ldo; a.p0 = g.p0; a.p1 = g.p1;
    a.trace = g_conv_trace;
    a.nst = p.stages;
    {
        static int* status_addr[64] = {nullptr};
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(g_configure_mutex);
        if (dev < 0 || dev >= 64 || !status_addr[dev]) {
            int* q = nullptr;
            CUDA_TRY(cudaGetSymbolAddress((void**)&q, g_gemm_status));
            if (dev >= 0 && dev < 64) status_addr[dev] = q;
            a.status = q;
        } else {
            a.status = status_addr[dev];
        }
    }
    {
        // a programmatic dependent of the expansion launch: set-up (barriers, tensor memory, unit
        // scales) overlaps the expansion pass, the kernel waits for it before its first copy
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((p.pair ? (p.MT + 1) / 2 : p.MT) * p.NT * p.splits));
        cfg.blockDim = dim3(umma::kGemmThreads);
        cfg.dynamicSmemBytes = umma::gemm_smem(p.pair, p.stages);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = p.pair ? cudaLaunchKernelEx(&cfg, k_gemm_umma<true>, a)
                                     : cudaLaunchKernelEx(&cfg, k_gemm_umma<false>, a);
        if (e != cudaSuccess) return fail("gemm (tcgen05): %s", cudaGetErrorString(e));
    }
    if (launch_check("gemm (tcgen05)")) return 1;
    if (p.splits == 1) return 0;                         // the GEMM's epilogue finished the layer
    GemmArgs f = g;
    f.K = 0;                                             // the partial sums are already K - 2*popc
    f.splits = p.splits;
    f.partial = a.partial;
    k_gemm_finish<<<warp_grid((long long)g.M * ((g.N + 31) / 32), sms), kThreads, 0, st>>>(f);
    return launch_check("gemm (tcgen05) finish");
}

int g_gemm_path = 0;     // 0 automatic, 1 warp-level b1 MMA only

int run_gemm(GemmArgs g, void* workspace, size_t workspace_bytes, cudaStream_t st) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return fail("gemm: M, N, K must be positive");
    if ((g.lda & 1) || (g.ldw & 1)) return fail("gemm: lda and ldw must be even (64-bit loads)");
    if (g.lda * 32 < g.K || g.ldw * 32 < g.K) return fail("gemm: leading dimension shorter than K");
    if ((long long)g.M * g.lda >= (1LL << 31) || (long long)g.N * g.ldw >= (1LL << 31))
        return fail("gemm: operand larger than 2^31 words");
    if (((uintptr_t)g.A & 7) || ((uintptr_t)g.W & 7)) return fail("gemm: operands must be 8-byte aligned");
    int sms;
    if (sm_count(&sms)) return 1;
    const GemmUmmaPlan plan = gemm_umma_plan(g.M, g.N, g.K, sms);
    if (plan.use && g_gemm_path != 1 && workspace && workspace_bytes >= plan.bytes && ((uintptr_t)workspace & 255) == 0)
        return run_gemm_umma(g, plan, workspace, sms, st);
    int splits = gemm_splits(g.M, g.N, g.K, sms);
    const size_t need = (size_t)splits * g.M * g.N * sizeof(int32_t);
    if (splits > 1 && (workspace == nullptr || workspace_bytes < need)) splits = 1;
    const long long tiles = (long long)((g.M + 31) / 32) * ((g.N + 31) / 32);
    if (splits == 1) {
        g.splits = 1;
        g.partial = nullptr;
        k_gemm<<<warp_grid(tiles, sms), kThreads, 0, st>>>(g);
        return launch_check("gemm");
    }
    GemmArgs p = g;
    p.mode = GEMM_PARTIAL;
    p.splits = splits;
    p.partial = (int32_t*)workspace;
    k_gemm<<<warp_grid(tiles * splits, sms), kThreads, 0, st>>>(p);
    if (launch_check("gemm split-K")) return 1;
    g.splits = splits;
    g.partial = (int32_t*)workspace;
    k_gemm_finish<<<warp_grid((long long)g.M * ((g.N + 31) / 32), sms), kThreads, 0, st>>>(g);
    return launch_check("gemm split-K finish");
}

// ---- prepared conv filter blob ------------------------------------------------------------
struct PreparedLayout {
    int KP;               // 64-bit pairs per filter row, multiple of 4
    size_t off_wq, off_ktab, off_pwt, off_pwtot, off_err, off_wi8, bytes;
    int umma_nt;          // n-tile of the tcgen05 path, 0 when the layer is not eligible
    bool ws_ok;           // the filter-stationary kernel with in-CTA expansion can take the layer
    int umma_npos;        // raster positions of the shared-memory patch (per plane)
    size_t umma_smem;     // dynamic shared memory of the tcgen05 kernel
    int umma_pw, umma_vh, umma_back_y, umma_back_x;   // raster geometry
    // activation-stationary tcgen05 kernel (wide stride-1 layers): its own filter copy in
    // 128-channel n-tiles (shared with the other kernel's when that one also uses 128)
    // kernel fed from a pre-expanded input (narrow stride-1 layers): needs a caller workspace
    size_t pre_bytes;     // workspace size, 0 when the layer is not eligible
    size_t pre_smem;
    int pre_stages;
    int pre_nt;           // its n-tile (output channels of the resident filter block)
    size_t off_wf4;       // its filter copy: e2m1 nibbles
    long long pre_positions, pre_front;
    int as_npos;          // 0 when the layer is not eligible
    size_t pool_bytes;    // scratch the activation-stationary kernel can use to pre-pool a residual
    size_t prepool_bytes; // pooled layers: their pre-pool output bits (the OR-pooling pass reads them)
    int as_slots;         // units in its filter ring
    size_t as_smem, off_wi8_as;
};

int conv_check(const tcbnn_conv_desc* d, bool binary) {
    if (!d) return fail("conv: null descriptor");
    if (d->B <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->O <= 0 || d->R <= 0 || d->S <= 0)
        return fail("conv: sizes must be positive");
    if (d->R > 15 || d->S > 15) return fail("conv: filter larger than 15x15 is not supported");
    if (d->stride_h <= 0 || d->stride_w <= 0) return fail("conv: stride must be positive");
    if (d->pool != 1 && d->pool != 2) return fail("conv: pool must be 1 or 2");
    if (binary && (((d->C + 31) / 32) & 1))
        return fail("conv: input channels must fill an even number of 32-bit words (C=%d)", d->C);
    if (!binary && d->C != 3) return fail("inconv: input channels must be 3");
    if (!binary && d->O > 128) return fail("inconv: more than 128 output channels not supported");
    if (d->OH <= 0 || d->OW <= 0) return fail("conv: call tcbnn_conv_shape first");
    const long long in_words = (long long)d->B * d->H * d->W * ((d->C + 31) / 32);
    if (binary && in_words >= (1LL << 31)) return fail("conv: input larger than 2^31 words");
    if ((long long)d->B * d->OH * d->OW * d->pool * d->pool >= (1LL << 31))
        return fail("conv: more than 2^31 output pixels");
    return 0;
}

PreparedLayout prepared_layout(const tcbnn_conv_desc* d) {
    PreparedLayout L;
    const int Cw = (d->C + 31) / 32;
    const int words = d->R * d->S * Cw;
    L.KP = ((words + 7) / 8) * 4;
    size_t o = 0;
    L.off_wq = o;    o += (size_t)d->O * 2 * L.KP * 4;  o = (o + 255) & ~(size_t)255;
    L.off_ktab = o;  o += (size_t)L.KP * 4;             o = (o + 255) & ~(size_t)255;
    L.off_pwt = o;   o += (size_t)d->R * d->S * d->O * 4; o = (o + 255) & ~(size_t)255;
    L.off_pwtot = o; o += (size_t)d->O * 4;             o = (o + 255) & ~(size_t)255;
    L.off_err = o;   o += 256;
    // tcgen05 path: stride 1 or 2, "same" padding, no pooling, channels in blocks of 64,
    // filter block of one n-tile resident in shared memory
    L.umma_nt = 0; L.umma_npos = 0; L.umma_smem = 0; L.off_wi8 = o; L.ws_ok = false;
    L.umma_pw = L.umma_vh = L.umma_back_y = L.umma_back_x = 0;
    L.as_npos = 0; L.as_smem = 0; L.as_slots = 0; L.off_wi8_as = o;
    L.pre_bytes = 0; L.pre_smem = 0; L.pre_stages = 0; L.pool_bytes = 0; L.pre_positions = 0; L.pre_front = 0;
    L.pre_nt = 0; L.off_wf4 = o;
    // (a pooled layer runs the tcgen05 kernels on its pre-pool grid, followed by an OR-pooling pass)
    const int OHu = d->OH * d->pool, OWu = d->OW * d->pool;
    if (d->stride_h == d->stride_w && (d->stride_h == 1 || d->stride_h == 2) &&
        d->padding && d->C % 64 == 0 && d->O % 32 == 0) {
        const int st = d->stride_h;
        // tap (r,s) reads raster offset (dy,dx) of a plane; extremes over the taps
        const int back_y = st == 2 ? (d->pad_h + 1) / 2 : d->pad_h;
        const int back_x = st == 2 ? (d->pad_w + 1) / 2 : d->pad_w;
        const int fwd_y = st == 2 ? (d->R - 1 - d->pad_h >= 0 ? (d->R - 1 - d->pad_h) / 2 : 0)
                                  : d->R - 1 - d->pad_h;
        const int fwd_x = st == 2 ? (d->S - 1 - d->pad_w >= 0 ? (d->S - 1 - d->pad_w) / 2 : 0)
                                  : d->S - 1 - d->pad_w;
        const int PW = OWu + (back_x > fwd_x ? back_x : fwd_x);
        const int VH = OHu + (back_y > fwd_y ? back_y : fwd_y);
        const int npos = (128 + (back_y + fwd_y) * PW + back_x + fwd_x + 7) & ~7;
        const int max_npos = st == 2 ? umma::kWsExpThreads : 2 * umma::kWsExpThreads;
        const long long nv = (long long)d->B * VH * PW;
        const long long in_words = (long long)d->B * d->H * d->W * (d->C / 32);
        if (fwd_y >= 0 && fwd_x >= 0 && nv + 1024 < (1LL << 31) && in_words < (1LL << 31)) {
            for (int nt = 256; nt >= 32 && npos <= max_npos; nt >>= 1) {
                if (d->O % nt) continue;
                const size_t smem = umma::ws_smem_bytes(st, npos, d->C, d->R * d->S, nt);
                if (smem > 227 * 1024) continue;
                L.umma_nt = nt; L.umma_npos = npos; L.umma_smem = smem;
                L.umma_pw = PW; L.umma_vh = VH; L.umma_back_y = back_y; L.umma_back_x = back_x;
                o += (size_t)d->R * d->S * d->C * d->O;      o = (o + 255) & ~(size_t)255;
                break;
            }
            L.ws_ok = L.umma_nt != 0;
            const int nplane = st == 2 ? 4 : 1;
            if (d->C <= 512 && (nplane * 2 * npos * 16) < (1 << 18)) {
                // loader-fed 4-bit kernel: the largest n-tile whose filter block leaves room for a
                // patch ring of at least three stages
                for (int nt = 128; nt >= 32 && !L.pre_nt; nt >>= 1) {
                    if (d->O % nt) continue;
                    int stages = nt >= 128 ? 4 : umma::kPreMaxStages;
                    while (stages > 3 && umma::pre_smem_bytes(npos, d->C, d->R * d->S, nt, stages, nplane) > 227 * 1024) stages--;
                    const size_t smem_pre = umma::pre_smem_bytes(npos, d->C, d->R * d->S, nt, stages, nplane);
                    if (smem_pre > 227 * 1024) continue;
                    L.pre_nt = nt; L.pre_stages = stages; L.pre_smem = smem_pre;
                    L.umma_npos = npos;
                    L.umma_pw = PW; L.umma_vh = VH; L.umma_back_y = back_y; L.umma_back_x = back_x;
                    L.pre_front = umma::pre_front(back_y, back_x, PW);
                    L.pre_positions = umma::pre_plane_positions(nv, npos, L.pre_front);
                    L.pre_bytes = (size_t)(d->C / 32) * nplane * (size_t)L.pre_positions * 16;    // C/32 x nplane planes of 16-byte slots
                    L.off_wf4 = o;
                    o += (size_t)d->R * d->S * d->C * d->O / 2;  o = (o + 255) & ~(size_t)255;
                }
            }
            // wide layers: keep 256 positions x all channels resident, stream the filter
            const int npos_as = (256 + (back_y + fwd_y) * PW + back_x + fwd_x + 7) & ~7;
            int slots_as = umma::kAsMaxSlots;
            if (umma::as_smem_bytes(npos_as, d->C, d->O, d->R * d->S, slots_as) > 227 * 1024) slots_as = 9;
            if (umma::as_smem_bytes(npos_as, d->C, d->O, d->R * d->S, slots_as) > 227 * 1024) slots_as = 6;
            const size_t smem_as = umma::as_smem_bytes(npos_as, d->C, d->O, d->R * d->S, slots_as);
            // (at 128 channels the filter-stationary kernel is as fast: measured)
            if (st == 1 && d->C >= 256 && d->C <= 512 && d->O % umma::kAsNT == 0 &&
                npos_as <= umma::kAsMaxPos * umma::kAsExpThreads && smem_as <= 227 * 1024) {
                L.as_npos = npos_as; L.as_smem = smem_as; L.as_slots = slots_as;
                L.pool_bytes = d->pool == 1 ? (size_t)d->B * d->OH * d->OW * d->O * 4 : 0;
                L.umma_pw = PW; L.umma_vh = VH; L.umma_back_y = back_y; L.umma_back_x = back_x;
                if (L.umma_nt == umma::kAsNT) {
                    L.off_wi8_as = L.off_wi8;
                } else {
                    L.off_wi8_as = o;
                    o += (size_t)d->R * d->S * d->C * d->O;  o = (o + 255) & ~(size_t)255;
                }
            }
        }
    }
    // the loader-fed kernel pre-pools an injected residual too (scratch behind its planes)
    if (L.pre_nt && d->pool == 1) L.pool_bytes = (size_t)d->B * d->OH * d->OW * d->O * 2;
    L.prepool_bytes = 0;
    if (d->pool != 1 && (L.umma_nt || L.as_npos || L.pre_nt))
        L.prepool_bytes = ((size_t)d->B * OHu * OWu * ((d->O + 31) / 32) * 4 + 255) & ~(size_t)255;
    L.bytes = o;
    return L;
}

// Scratch in front of a pooled layer's pre-pool bits: the input planes of the loader-fed kernel
// followed by its pooled-residual scratch, or the activation-stationary kernel's pooled residual.
size_t planes_padded(const PreparedLayout& L) { return (L.pre_bytes + 255) & ~(size_t)255; }
size_t main_ws_bytes(const PreparedLayout& L) {
    if (L.pre_bytes) return planes_padded(L) + ((L.pool_bytes + 255) & ~(size_t)255);
    return (L.pool_bytes + 255) & ~(size_t)255;
}

template <int PPT>
__global__ void __launch_bounds__(kInconvThreads) k_inconv_tiled(InConvArgs c) {
    extern __shared__ __align__(16) unsigned char dyn_smem_inconv[];
    inconv_tiled_block<PPT>(c, dyn_smem_inconv);
}

template <int PPT>
int launch_inconv_tiled(const InConvArgs& c, size_t smem, int sms, cudaStream_t st) {
    static bool configured[64] = {false};
    if (configure_once(configured, [] {
            return cudaFuncSetAttribute(k_inconv_tiled<PPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        }))
        return 1;
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    const long long total = (long long)c.B * c.OH * c.OW * c.pool * c.pool;
    long long grid = (total + kInconvPixels - 1) / kInconvPixels;
    if (grid > (long long)sms * per_sm) grid = (long long)sms * per_sm;
    k_inconv_tiled<PPT><<<(int)grid, kInconvThreads, smem, st>>>(c);
    return launch_check("inconv_layer (tiled)");
}

int g_conv_two_ctas = 1;  // loader-fed kernel, n-tile 64: two CTAs of eight epilogue warps per SM when they fit
int g_conv_res_stage = 1; // loader-fed kernel: stage int16 residual rows in shared memory when possible
int g_conv_tile = 1;      // loader-fed kernel: the tile-per-group epilogues where the tensors allow them
int g_conv_cbs = 1;       // loader-fed kernel: four or two 64-channel blocks per stage where they fit
int g_conv_uneven = 1;    // loader-fed kernel: more CTAs for the n-tiles that carry a pooled residual

// The tile-per-group epilogues of the loader-fed kernel take residuals only in the chunk-major
// int16 layout and write no int32 accumulators.
bool pre_tile_ok(const void* res_in, int res_in_bytes, int res_in_chunked, const void* res_out, int res_out_bytes,
                 int res_out_chunked, const void* acc_out) {
    return g_conv_tile && !acc_out && (!res_in || (res_in_chunked && res_in_bytes == 2)) &&
           (!res_out || (res_out_chunked && res_out_bytes == 2));
}
int g_conv_path = 0;     // 0 auto, 1 warp-level b1 MMA, 2 tcgen05 (error if not eligible), 3 = 2 without the activation-stationary kernel

template <int NT, int STRIDE>
__global__ void __launch_bounds__(umma::kWsThreads, 1) k_conv_umma_ws(umma::ConvWsArgs a) {
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    umma::conv_umma_ws_cta<NT, STRIDE>(a, dyn_smem);
}
__global__ void k_prepare_filter_ws(const uint32_t* fbits, int O, int RS, int C, int nt, uint4* out) {
    umma::prepare_filter_ws(fbits, O, RS, C, nt, out);
}
__global__ void k_prepare_filter_f4(const uint32_t* fbits, int O, int RS, int C, int nt, uint4* out) {
    umma::prepare_filter_f4(fbits, O, RS, C, nt, out);
}

template <int NT, int STRIDE>
int launch_conv_umma_ws(umma::ConvWsArgs& a, size_t smem, int sms, cudaStream_t st) {
    static bool configured[64] = {false};
    if (configure_once(configured, [] {
            return cudaFuncSetAttribute(k_conv_umma_ws<NT, STRIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        }))
        return 1;
    a.ntiles_n = a.O / NT;
    if (a.ntiles_n > sms) return fail("conv_layer: more n-tiles than SMs");
    const long long mtiles = (a.NV + 127) / 128;
    long long per = sms / a.ntiles_n;                 // CTAs per n-tile
    if (per > mtiles) per = mtiles;
    k_conv_umma_ws<NT, STRIDE><<<(int)(per * a.ntiles_n), umma::kWsThreads, smem, st>>>(a);
    return launch_check("conv_layer (tcgen05)");
}

template <int NT, int EPI, int EPIW>
__global__ void __launch_bounds__(umma::pre_threads(EPIW), EPIW == 8 ? 2 : 1) k_conv_umma_pre(umma::ConvWsArgs a) {
    extern __shared__ __align__(128) unsigned char dyn_smem_pre[];
    umma::conv_umma_pre_cta<NT, EPI, EPIW>(a, dyn_smem_pre);
}
__global__ void __launch_bounds__(256) k_expand_raster(umma::ConvWsArgs a, uint4* planes, long long positions,
                                                       long long front) {
    umma::expand_raster(a, planes, positions, front);
}

template <int NT, int EPI, int EPIW>
int launch_conv_umma_pre_k(umma::ConvWsArgs& a, size_t smem, int sms, cudaStream_t st) {
    static bool configured[64] = {false};
    if (configure_once(configured, [] {
            return cudaFuncSetAttribute(k_conv_umma_pre<NT, EPI, EPIW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        EPIW == 8 ? 113 * 1024 : 227 * 1024);
        }))
        return 1;
    a.ntiles_n = a.O / NT;
    if (a.ntiles_n > sms) return fail("conv_layer: more n-tiles than SMs");
    const long long mtiles = (a.NV + 127) / 128;
    const long long budget = (long long)(EPIW == 8 ? 2 : 1) * sms;        // one or two CTAs per SM
    long long per = budget / a.ntiles_n;                                  // CTAs per n-tile
    if (per > mtiles) per = mtiles;
    long long grid = per * a.ntiles_n;
    a.nt_heavy = 0; a.per_heavy = a.per_light = (int)per;
    if (EPI == umma::kEpiTileRes && g_conv_uneven && a.res_in && a.residual_pool) {
        // A pooled residual injected into the first channels only (the first block of a stage):
        // the n-tiles it falls into take about 1.75 times as long per tile as the others when the
        // tile's own MMAs are few (measured at 14 x 14 x 256: 0.141 ms against 0.081 for the same
        // layer without pooling), so they get that many more CTAs each.
        const int lim = a.residual_channels < a.res_in_ch ? a.residual_channels : a.res_in_ch;
        const int heavy = (lim + NT - 1) / NT, light = a.ntiles_n - heavy;
        if (heavy > 0 && light > 0 && (a.C >> 6) * a.R * a.S <= 36) {
            long long pl = (long long)((double)budget / (1.75 * heavy + light));
            if (pl < 1) pl = 1;
            long long ph = (budget - light * pl) / heavy;
            if (ph > mtiles) ph = mtiles;
            if (pl > mtiles) pl = mtiles;
            if (ph >= 1) {
                a.nt_heavy = heavy; a.per_heavy = (int)ph; a.per_light = (int)pl;
                grid = heavy * ph + light * pl;
            }
        }
    }
    k_conv_umma_pre<NT, EPI, EPIW><<<(int)grid, umma::pre_threads(EPIW), smem, st>>>(a);
    return launch_check("conv_layer (tcgen05, pre-expanded input)");
}

// n-tile 64: two CTAs of eight epilogue warps per SM when the filter block and a patch ring of at
// least three stages fit half of the shared memory.  Measured at batch 1024, 56 x 56 x 64 -> 64
// (two CTAs / one): all-warps-per-tile epilogues 0.119 / 0.154 ms plain and 0.40 / 0.33 with
// residual rows moved directly (32 columns of residual per thread spill), so those stay on one
// CTA; tile-per-group epilogues 0.105 / 0.143 plain and 0.223 / 0.255 with chunk-major residuals.
template <int EPI>
int launch_conv_umma_pre_64(umma::ConvWsArgs& a, size_t smem, int sms, cudaStream_t st) {
    if (g_conv_two_ctas && (EPI == umma::kEpiPlain || EPI == umma::kEpiTile || EPI == umma::kEpiTileRes || g_conv_two_ctas == 2)) {
        int stages = a.pre_stages;
        const int nplane = (a.stride == 2 ? 4 : 1) * a.pre_cbs;
        while (stages > 3 && umma::pre_smem_bytes(a.NPOS, a.C, a.R * a.S, 64, stages, nplane) > 113 * 1024) stages--;
        const size_t need = umma::pre_smem_bytes(a.NPOS, a.C, a.R * a.S, 64, stages, nplane);
        if (need <= 113 * 1024) {
            a.pre_stages = stages;
            return launch_conv_umma_pre_k<64, EPI, 8>(a, need, sms, st);
        }
    }
    return launch_conv_umma_pre_k<64, EPI, 16>(a, smem, sms, st);
}

// npos, C, RS of the layer are needed to size the patch ring again when the residual rows are staged
template <int NT>
int launch_conv_umma_pre(umma::ConvWsArgs& a, size_t smem, int sms, cudaStream_t st, bool expand) {
    if (expand) {
        const long long units = a.pre_positions * (a.C >> 6) * (a.stride == 2 ? 4 : 1);
        k_expand_raster<<<elementwise_grid(units, sms), 256, 0, st>>>(a, const_cast<uint4*>(a.pre), a.pre_positions,
                                                                   a.pre_front);
        if (launch_check("conv_layer (input expansion)")) return 1;
    }
    if (pre_tile_ok(a.res_in, a.res_in_bytes, a.res_in_chunked, a.res_out, a.res_out_bytes, a.res_out_chunked, a.acc_out)) {
        const bool plain = !a.res_in && !a.res_out;
        if constexpr (NT == 64) {
            return plain ? launch_conv_umma_pre_64<umma::kEpiTile>(a, smem, sms, st)
                         : launch_conv_umma_pre_64<umma::kEpiTileRes>(a, smem, sms, st);
        } else {
            return plain ? launch_conv_umma_pre_k<NT, umma::kEpiTile, 16>(a, smem, sms, st)
                         : launch_conv_umma_pre_k<NT, umma::kEpiTileRes, 16>(a, smem, sms, st);
        }
    }
    if constexpr (NT >= 64) {
        // int16 residual rows through shared memory (see conv_umma_pre_cta) when the tensors allow
        // it and the two row buffers fit beside a patch ring of at least two stages.  Measured at
        // batch 1024 (staged / direct): 28 x 28 x 128 0.186 / 0.215 ms, 14 x 14 x 256 0.112 /
        // 0.138, 7 x 7 x 512 0.127 / 0.120, 56 x 56 x 64 (n-tile 64) 0.425 / 0.327 -- the once-per-tile
        // rendezvous of the 16 epilogue warps costs more than the narrow rows save there.
        const int lim = a.res_in ? (a.residual_channels < a.res_in_ch ? a.residual_channels : a.res_in_ch) : 0;
        const bool in_ok = !a.res_in || (a.res_in_bytes == 2 && !a.res_in_chunked && !a.residual_pool && a.res_in_ch % 8 == 0 &&
                                         ((uintptr_t)a.res_in & 15) == 0 && lim % 8 == 0);
        const bool out_ok = !a.res_out || (a.res_out_bytes == 2 && !a.res_out_chunked && ((uintptr_t)a.res_out & 15) == 0);
        if ((a.res_in || a.res_out) && in_ok && out_ok && g_conv_res_stage && (NT >= 128 || g_conv_res_stage == 2)) {
            int stages = a.pre_stages;
            const int RS = a.R * a.S;
            const int nplane = (a.stride == 2 ? 4 : 1) * a.pre_cbs;
            while (stages > 2 && umma::pre_smem_bytes(a.NPOS, a.C, RS, NT, stages, nplane) + umma::pre_res_stage_bytes(NT) > 227 * 1024)
                stages--;
            const size_t need = umma::pre_smem_bytes(a.NPOS, a.C, RS, NT, stages, nplane) + umma::pre_res_stage_bytes(NT);
            if (need <= 227 * 1024) {
                a.pre_stages = stages;
                return launch_conv_umma_pre_k<NT, umma::kEpiStaged, 16>(a, need, sms, st);
            }
        }
    }
    const bool plain = !a.res_in && !a.res_out && !a.acc_out;
    if constexpr (NT == 64) {
        return plain ? launch_conv_umma_pre_64<umma::kEpiPlain>(a, smem, sms, st)
                     : launch_conv_umma_pre_64<umma::kEpiDirect>(a, smem, sms, st);
    } else {
        return plain ? launch_conv_umma_pre_k<NT, umma::kEpiPlain, 16>(a, smem, sms, st)
                     : launch_conv_umma_pre_k<NT, umma::kEpiDirect, 16>(a, smem, sms, st);
    }
}

// The *_bytes arguments of the conv entry points name the residual's element format: 4 = int32
// NHWC, 2 = int16 NHWC, TCBNN_RES_INT16_CHUNKED = int16 laid out by 8-channel chunk.
// TCBNN_RES_PROVEN on an int16 format: the caller vouches for the range, no check per value.
bool residual_format(int code, int* bytes, int* chunked, int* proven = nullptr) {
    const int fmt = code & ~TCBNN_RES_PROVEN;
    if (proven) *proven = (code & TCBNN_RES_PROVEN) != 0 && fmt != 4;
    *chunked = fmt == TCBNN_RES_INT16_CHUNKED;
    *bytes = *chunked ? 2 : fmt;
    return fmt == 2 || fmt == 4 || fmt == TCBNN_RES_INT16_CHUNKED;
}

// 2x2 max of a chunked int16 residual [ch/8][B*2P*2Q][8] -> NHWC [B][P][Q][ch].  A block takes 32
// consecutive output pixels x all chunks: it reads chunk by chunk (consecutive lanes = consecutive
// pixels: whole lines), turns the tile through shared memory (16-byte slots XOR-swizzled by pixel),
// and writes pixel by pixel (consecutive lanes = consecutive chunks of a row: whole lines again).
constexpr int kPoolChunkedMaxCh8 = 32;
__global__ void __launch_bounds__(256) k_pool_residual16_chunked(const uint4* in, uint4* out, int B, int P, int Q, int ch8) {
    __shared__ uint4 tile[32 * kPoolChunkedMaxCh8];
    const long long npix = (long long)B * P * Q, npix_in = npix * 4;
    const long long ntiles = (npix + 31) / 32;
    const int units = 32 * ch8;
    const int swz = (ch8 & (ch8 - 1)) == 0 ? (ch8 < 8 ? ch8 - 1 : 7) : 0;    // power-of-two chunk counts only
    for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const long long pix0 = t * 32;
        for (int u = threadIdx.x; u < units; u += 256) {
            const int c = u >> 5, pl = u & 31;
            const long long pix = pix0 + pl;
            uint4 m = make_uint4(0u, 0u, 0u, 0u);
            if (pix < npix) {
                long long r = pix;
                const int x = (int)(r % Q); r /= Q;
                const int y = (int)(r % P);
                const long long n = r / P;
                const uint4* s0 = in + (long long)c * npix_in + (n * 2 * P + 2 * y) * 2 * Q + 2 * x;
                const uint4* s1 = s0 + 2 * Q;
                const uint4 a = __ldg(s0), b = __ldg(s0 + 1), e = __ldg(s1), f = __ldg(s1 + 1);
                m.x = __vmaxs2(__vmaxs2(a.x, b.x), __vmaxs2(e.x, f.x));
                m.y = __vmaxs2(__vmaxs2(a.y, b.y), __vmaxs2(e.y, f.y));
                m.z = __vmaxs2(__vmaxs2(a.z, b.z), __vmaxs2(e.z, f.z));
                m.w = __vmaxs2(__vmaxs2(a.w, b.w), __vmaxs2(e.w, f.w));
            }
            tile[pl * ch8 + (c ^ (pl & swz))] = m;
        }
        __syncthreads();
        for (int u = threadIdx.x; u < units; u += 256) {
            const int pl = u / ch8, c = u - pl * ch8;
            if (pix0 + pl < npix) out[(pix0 + pl) * ch8 + c] = tile[pl * ch8 + (c ^ (pl & swz))];
        }
        __syncthreads();
    }
}

// 2x2 max of an int16 residual [B][2P][2Q][ch] -> [B][P][Q][ch] (kernel.cuh:773-783), 8 channels
// per thread: the activation-stationary kernel then reads one row per pixel instead of four.
__global__ void __launch_bounds__(256) k_pool_residual16(const uint4* in, uint4* out, int B, int P, int Q, int ch8) {
    const long long total = (long long)B * P * Q * ch8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % ch8);
        long long r = i / ch8;
        const int x = (int)(r % Q); r /= Q;
        const int y = (int)(r % P);
        const long long n = r / P;
        const uint4* s0 = in + ((n * 2 * P + 2 * y) * 2 * Q + 2 * x) * ch8 + c;
        const uint4* s1 = s0 + (long long)2 * Q * ch8;
        const uint4 a = __ldg(s0), b = __ldg(s0 + ch8), e = __ldg(s1), f = __ldg(s1 + ch8);
        uint4 m;
        m.x = __vmaxs2(__vmaxs2(a.x, b.x), __vmaxs2(e.x, f.x));
        m.y = __vmaxs2(__vmaxs2(a.y, b.y), __vmaxs2(e.y, f.y));
        m.z = __vmaxs2(__vmaxs2(a.z, b.z), __vmaxs2(e.z, f.z));
        m.w = __vmaxs2(__vmaxs2(a.w, b.w), __vmaxs2(e.w, f.w));
        out[i] = m;
    }
}

// OR over 2x2 windows of packed output bits [B][2P][2Q][Ow] -> [B][P][Q][Ow] (kernel.cuh:756-770
// pools by OR-ing the window's bits): the tcgen05 kernels compute a pooled layer on its pre-pool
// grid, this pass reduces it.
__global__ void __launch_bounds__(256) k_pool_bits(const uint32_t* in, uint32_t* out, int B, int P, int Q, int Ow,
                                                  long long out_image_stride) {
    const long long total = (long long)B * P * Q * Ow;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int w = (int)(i % Ow);
        long long r = i / Ow;
        const int x = (int)(r % Q); r /= Q;
        const int y = (int)(r % P);
        const long long n = r / P;
        const uint32_t* s0 = in + ((n * 2 * P + 2 * y) * 2 * Q + 2 * x) * Ow + w;
        const uint32_t* s1 = s0 + (long long)2 * Q * Ow;
        out[n * out_image_stride + ((long long)y * Q + x) * Ow + w] = __ldg(s0) | __ldg(s0 + Ow) | __ldg(s1) | __ldg(s1 + Ow);
    }
}

__global__ void __launch_bounds__(umma::kAsThreads, 1) k_conv_umma_as(umma::ConvWsArgs a) {
    extern __shared__ __align__(128) unsigned char dyn_smem_as[];
    umma::conv_umma_as_cta<0>(a, dyn_smem_as);
}

int launch_conv_umma_as(umma::ConvWsArgs& a, size_t smem, int sms, cudaStream_t st) {
    static bool configured[64] = {false};
    if (configure_once(configured, [] {
            return cudaFuncSetAttribute(k_conv_umma_as, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        }))
        return 1;
    // Split the n-tiles of a task over several work items when that fills the last wave of
    // CTAs better (the patch is then expanded once per part, which is cheap).
    const long long ntasks = (a.NV + 255) / 256;
    const int nnt = a.O / umma::kAsNT;
    int best = 1;
    double best_cost = 1e300;
    for (int sp = 1; sp <= nnt; sp++) {
        if (nnt % sp) continue;
        const long long items = ntasks * sp;
        const long long waves = (items + sms - 1) / sms;
        const double cost = (double)waves * ((double)nnt / sp + 0.15);   // 0.15: expansion + fill
        if (cost < best_cost - 1e-9) { best_cost = cost; best = sp; }
    }
    a.as_split = best;
    const long long items = ntasks * best;
    const int grid = (int)(items < sms ? items : sms);
    k_conv_umma_as<<<grid, umma::kAsThreads, smem, st>>>(a);
    return launch_check("conv_layer (tcgen05, activation-stationary)");
}

// ---- MMA issue-rate probe ----------------------------------------------------------------
template <int KIND>
__global__ void k_mma_peak(int iters, unsigned seed, int* sink) {
    unsigned a[4], b[2];
    int c[8][4];
    for (int i = 0; i < 4; i++) a[i] = seed * (threadIdx.x + i + 1);
    for (int i = 0; i < 2; i++) b[i] = seed * (threadIdx.x * 7 + i + 3);
    for (int j = 0; j < 8; j++)
        for (int i = 0; i < 4; i++) c[j][i] = 0;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (KIND == 0) mma_b1_and(c[j], a[0], a[1], a[2], a[3], b[0], b[1]);
            if (KIND == 1)
                asm volatile(
                    "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.xor.popc "
                    "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                    : "+r"(c[j][0]), "+r"(c[j][1]), "+r"(c[j][2]), "+r"(c[j][3])
                    : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
            if (KIND == 2)
                asm volatile(
                    "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
                    "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                    : "+r"(c[j][0]), "+r"(c[j][1]), "+r"(c[j][2]), "+r"(c[j][3])
                    : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
        }
    }
    int s = 0;
    for (int j = 0; j < 8; j++)
        for (int i = 0; i < 4; i++) s += c[j][i];
    if (s == 0x7fffffff) sink[0] = s;
}


// tcgen05.mma kind::i8 M=128 N=256 K=32 issued back to back by one thread per SM on resident
// shared-memory operands: the int8 tensor-core ceiling the conv kernel is measured against.
__global__ void __launch_bounds__(128) k_umma_peak(int iters, long long* cycles, int* err) {
    extern __shared__ __align__(1024) unsigned char peak_smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tm;
    if (threadIdx.x < 32) umma::tmem_alloc(umma::smem_u32(&tm), 256);
    if (threadIdx.x == 0) umma::mbar_init(umma::smem_u32(&bar), 1);
    for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) ((uint32_t*)peak_smem)[i] = 0x01FF01FFu;
    umma::fence_proxy_async();
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    if (threadIdx.x == 0) {
        const uint64_t da = umma::smem_desc(umma::smem_u32(peak_smem), 128 * 16, 128);
        const uint64_t db = umma::smem_desc(umma::smem_u32(peak_smem + 16384), 256 * 16, 128);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++)
            umma::mma_i8(tm, da + 2 * (i & 3), db + 2 * (i & 3), umma::idesc_i8(256), 1u);
        umma::mma_commit(umma::smem_u32(&bar));
        if (!umma::mbar_wait(umma::smem_u32(&bar), 0, err)) { /* status already recorded */ }
        if (blockIdx.x == 0) cycles[0] = clock64() - t0;
    }
    umma::tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) umma::tmem_dealloc(tm, 256);
}

// tcgen05.mma kind::mxf4 (e2m1 operands, ue8m0 block scales, fp32 accumulate) M=128 N=256 K=64,
// back to back like k_umma_peak.  +-1.0 is exact in e2m1 (0x2 / 0xA) and a unit scale is the
// ue8m0 byte 0x7F; the scale region of tensor memory is filled with that byte throughout, so every
// scale reads as 1.0 wherever the hardware looks.  A is all +1, B all -1: every accumulator must
// end at -64 * iters, which the kernel checks on one row per warp (sample[]).
__global__ void __launch_bounds__(128) k_umma_peak_mxf4(int iters, long long* cycles, int* err, float* sample) {
    extern __shared__ __align__(1024) unsigned char peak_smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tm;
    if (threadIdx.x < 32) umma::tmem_alloc(umma::smem_u32(&tm), 512);
    if (threadIdx.x == 0) umma::mbar_init(umma::smem_u32(&bar), 1);
    for (int i = threadIdx.x; i < 16384 / 4; i += blockDim.x) ((uint32_t*)peak_smem)[i] = 0x22222222u;            // A: +1
    for (int i = threadIdx.x; i < 32768 / 4; i += blockDim.x) ((uint32_t*)(peak_smem + 16384))[i] = 0xAAAAAAAAu;  // B: -1
    umma::fence_proxy_async();
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem = tm;
    {   // unit scales: columns 256..511 of this warp's 32 lanes
        const uint32_t lane_base = (uint32_t)((threadIdx.x >> 5) * 32) << 16;
        for (int c = 256; c < 512; c += 8)
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};"
                         ::"r"(tmem + lane_base + c), "r"(0x7F7F7F7Fu) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    if (threadIdx.x == 0) {
        // K-major, no swizzle: a 16-byte row of a core matrix holds 32 elements; K = 64 is two core
        // matrices `lbo` apart
        const uint64_t da = umma::smem_desc(umma::smem_u32(peak_smem), 128 * 16, 128);
        const uint64_t db = umma::smem_desc(umma::smem_u32(peak_smem + 16384), 256 * 16, 128);
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
            const uint32_t acc = i ? 1u : 0u;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "setp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(tmem + 256u), "r"(tmem + 384u) : "memory");
        }
        umma::mma_commit(umma::smem_u32(&bar));
        if (!umma::mbar_wait(umma::smem_u32(&bar), 0, err)) { /* status already recorded */ }
        if (blockIdx.x == 0) cycles[0] = clock64() - t0;
    }
    __syncthreads();
    umma::tc_fence_after();
    {
        int r[8];
        umma::tmem_ld8(tmem + ((uint32_t)((threadIdx.x >> 5) * 32) << 16) + 248u, r);
        umma::tmem_ld_wait();
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 5) sample[threadIdx.x >> 5] = __int_as_float(r[7]);
    }
    umma::tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) umma::tmem_dealloc(tmem, 512);
}

// What the position of the A operand costs: 128 x n x 64 MMAs (kind::mxf4, K-major without swizzle)
// back to back, A's descriptor starting `a_off16` 16-byte rows into its buffer -- the conv kernels
// address a filter tap by such an offset, so most of their operands start in the middle of an
// 8-row core matrix.  CTA 0 reports its clocks.
__global__ void __launch_bounds__(128) k_umma_operand_probe(int n, int a_off16, int iters, long long* cycles, int* err) {
    extern __shared__ __align__(1024) unsigned char peak_smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tm;
    if (threadIdx.x < 32) umma::tmem_alloc(umma::smem_u32(&tm), 512);
    if (threadIdx.x == 0) umma::mbar_init(umma::smem_u32(&bar), 1);
    for (int i = threadIdx.x; i < 49152 / 4; i += blockDim.x) ((uint32_t*)peak_smem)[i] = 0x22222222u;
    umma::fence_proxy_async();
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem = tm;
    umma::tmem_fill_unit_scales(tmem, 480);
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    if (threadIdx.x == 0) {
        // A: two chunk planes of 320 rows (room for the offset), B behind them: two planes of n rows
        const uint64_t da = umma::smem_desc(umma::smem_u32(peak_smem) + 16u * (uint32_t)a_off16, 320 * 16, 128);
        const uint64_t db = umma::smem_desc(umma::smem_u32(peak_smem + 16384), (uint32_t)n * 16, 128);
        const uint32_t idesc = umma::idesc_f4(n);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i += 8) {
#pragma unroll
            for (int u = 0; u < 8; u++)
                umma::mma_f4_split(tmem, (uint32_t)da, (uint32_t)(da >> 32), (uint32_t)db, (uint32_t)(db >> 32), idesc,
                                   (i | u) ? 1u : 0u, tmem + 480u, tmem + 496u);
        }
        umma::mma_commit(umma::smem_u32(&bar));
        if (!umma::mbar_wait(umma::smem_u32(&bar), 0, err)) { /* status already recorded */ }
        if (blockIdx.x == 0) cycles[0] = clock64() - t0;
    }
    umma::tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) umma::tmem_dealloc(tmem, 512);
}

// What the issuing thread's bookkeeping costs: 128x128x32 MMAs in groups of `group`, with per
// group nothing (MODE 0), a try_wait on a completed barrier plus a commit by a lone lane inside
// `if (threadIdx.x == 0)` (MODE 1), or a test_wait by the converged warp plus a commit by the lane
// elect.sync picks (MODE 2) -- the three ways an MMA warp can be written.
template <int MODE>
__global__ void __launch_bounds__(128) k_umma_issue(int iters, int group, long long* cycles, int* err) {
    extern __shared__ __align__(1024) unsigned char peak_smem[];
    __shared__ uint64_t bar_done, bar_ready, bar_commit;
    __shared__ uint32_t tm;
    if (threadIdx.x < 32) umma::tmem_alloc(umma::smem_u32(&tm), 256);
    if (threadIdx.x == 0) {
        umma::mbar_init(umma::smem_u32(&bar_done), 1);
        umma::mbar_init(umma::smem_u32(&bar_ready), 1);      // never arrived on: parity 1 reads as complete
        umma::mbar_init(umma::smem_u32(&bar_commit), 1);
    }
    for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) ((uint32_t*)peak_smem)[i] = 0x01FF01FFu;
    umma::fence_proxy_async();
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    if (threadIdx.x < 32) {
        const uint64_t da = umma::smem_desc(umma::smem_u32(peak_smem), 128 * 16, 128);
        const uint64_t db = umma::smem_desc(umma::smem_u32(peak_smem + 16384), 128 * 16, 128);
        const bool elected = umma::elect_one();
        const bool in_loop = MODE == 2 ? true : threadIdx.x == 0;
        const bool leader = MODE == 2 ? elected : threadIdx.x == 0;
        if (in_loop) {
            const long long t0 = clock64();
            for (int i = 0; i < iters; i += group) {
                if (MODE == 1) { for (int w = 0; w < 1000; w++) if (umma::mbar_try_wait(umma::smem_u32(&bar_ready), 1)) break; }
                if (MODE == 2) { for (int w = 0; w < 1000; w++) if (umma::mbar_test_wait(umma::smem_u32(&bar_ready), 1)) break; }
                if (leader) {
                    for (int k = 0; k < group; k++)
                        umma::mma_i8(tm + ((k & 1) ? 128 : 0), da + 2 * (k & 3), db + 2 * (k & 3), umma::idesc_i8(128), 1u);
                    if (MODE != 0) umma::mma_commit(umma::smem_u32(&bar_commit));
                }
            }
            if (leader) {
                umma::mma_commit(umma::smem_u32(&bar_done));
                if (!umma::mbar_wait(umma::smem_u32(&bar_done), 0, err)) { /* status already recorded */ }
                if (blockIdx.x == 0) cycles[0] = clock64() - t0;
            }
        }
        __syncwarp();
    }
    umma::tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) umma::tmem_dealloc(tm, 256);
}

// ---- what a wait that gives up looks like ----------------------------------------------------
// One CTA allocates tensor memory like the conv kernels, initialises an mbarrier that expects one
// arrival, and polls it `polls` times with the kernels' own poll instruction.  Nobody arrives: the wait runs out, the thread records status 1, the CTA frees its
// tensor memory and returns -- the path every bounded wait of the tcgen05 kernels takes when its
// partner never shows up.  Nothing faults and nothing hangs; the context stays usable.
__global__ void __launch_bounds__(128) k_wait_probe(int polls, int* status, int* polled) {
    __shared__ uint64_t bar;
    __shared__ uint32_t tm;
    if (threadIdx.x < 32) umma::tmem_alloc(umma::smem_u32(&tm), 32);
    if (threadIdx.x == 0) {
        umma::mbar_init(umma::smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    if (threadIdx.x == 0) {
        int i = 0;
        bool done = false;
        for (; i < polls && !done; i++) done = umma::mbar_try_wait(umma::smem_u32(&bar), 0);
        *polled = i;
        if (!done) atomicExch(status, 1);
    }
    umma::tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) umma::tmem_dealloc(tm, 32);
}

// ---- how fast one SM pulls bulk copies out of L2 ---------------------------------------------
// Each CTA runs `iters` rounds over its own part of an L2-resident buffer: lane 0 of each of its
// `warps` warps issues `depth` bulk copies of `bytes` back to back into that warp's ring in shared
// memory, then waits for all of them.  Reports per CTA the clocks warp 0 spent issuing and its
// clocks in total.  Every wait is bounded.
__global__ void __launch_bounds__(128) k_bulk_probe(const unsigned char* src, int bytes, int depth, int warps,
                                                    int iters, long long* clocks, int* status) {
    extern __shared__ __align__(128) unsigned char probe_smem[];
    __shared__ uint64_t bars[4][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int w = 0; w < 4; w++)
            for (int s = 0; s < 16; s++) umma::mbar_init(umma::smem_u32(&bars[w][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    umma::fence_proxy_async();
    __syncthreads();
    if (warp < warps && lane == 0) {
        const size_t span = (size_t)bytes * depth * 8;                 // this warp's window of the buffer
        const unsigned char* mine = src + ((size_t)blockIdx.x * warps + warp) * span;
        unsigned char* ring = probe_smem + (size_t)warp * depth * bytes;
        bool ok = true;
        long long issue = 0, total = 0;
        for (int i = 0; i < iters && ok; i++) {
            const long long t0 = clock64();
            for (int s = 0; s < depth; s++) {
                umma::mbar_expect_tx(umma::smem_u32(&bars[warp][s]), (uint32_t)bytes);
                umma::bulk_g2s(umma::smem_u32(ring + (size_t)s * bytes), mine + (size_t)((i & 7) * depth + s) * bytes,
                               (uint32_t)bytes, umma::smem_u32(&bars[warp][s]));
            }
            const long long t1 = clock64();
            for (int s = 0; s < depth && ok; s++) ok = umma::mbar_wait(umma::smem_u32(&bars[warp][s]), i & 1, status);
            issue += t1 - t0;
            total += clock64() - t0;
        }
        if (warp == 0) { clocks[2 * blockIdx.x] = issue; clocks[2 * blockIdx.x + 1] = total; }
    }
}

// ---- fixed scratch for callers that cannot allocate ---------------------------------------
// Split-K partial sums for tcbnn_fc_layer_noalloc live in this array instead of a caller
// workspace.  It is part of the loaded module: every GPU that loads the library keeps these
// bytes resident until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, never a device address,
// so the address each device uses is looked up once (with that device current) and cached.
std::mutex g_scratch_mutex;
void* g_scratch_ptr[64] = {nullptr};

int static_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail("no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail("fc_layer_noalloc: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail("cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" {

int tcbnn_version(void) { return 100; }
const char* tcbnn_last_error(void) { return g_err; }

int tcbnn_pack_rows(const float* x, int rows, int cols, int ld_words, uint32_t* out, void* stream) {
    if (rows <= 0 || cols <= 0) return fail("pack_rows: empty input");
    if ((ld_words & 3) || ld_words * 32 < cols) return fail("pack_rows: ld_words must be a multiple of 4 and cover cols");
    if ((uintptr_t)out & 15) return fail("pack_rows: output must be 16-byte aligned");
    int sms;
    if (sm_count(&sms)) return 1;
    const long long tasks = (long long)rows * (ld_words / 4);
    const long long vtasks = (long long)rows * ((ld_words / 4 + 7) / 8);
    if ((cols & 3) == 0 && ((uintptr_t)x & 15) == 0 && vtasks < (1LL << 31)) {   // 16-byte loads, eight blocks per task
        // memory-bound and light on registers: all 64 warps an SM holds (8 CTAs)
        long long ctas = (vtasks + kThreads / 32 - 1) / (kThreads / 32);
        if (ctas > 8LL * sms) ctas = 8LL * sms;
        k_pack_rows_vec<<<(int)ctas, kThreads, 0, (cudaStream_t)stream>>>(x, rows, cols, ld_words, out);
    } else
        k_pack_rows<<<warp_grid(tasks, sms), kThreads, 0, (cudaStream_t)stream>>>(x, rows, cols, ld_words, out);
    return launch_check("pack_rows");
}

int tcbnn_unpack_rows(const uint32_t* in, int rows, int cols, int ld_words, float* out, void* stream) {
    if (rows <= 0 || cols <= 0) return fail("unpack_rows: empty input");
    int sms;
    if (sm_count(&sms)) return 1;
    k_unpack_rows<<<elementwise_grid((long long)rows * cols, sms), 256, 0, (cudaStream_t)stream>>>(
        in, rows, cols, ld_words, out);
    return launch_check("unpack_rows");
}

int tcbnn_pack_fc_weight(const float* W, int K, int N, int ld_words, uint32_t* out, void* stream) {
    if (K <= 0 || N <= 0 || ld_words * 32 < K) return fail("pack_fc_weight: bad sizes");
    int sms;
    if (sm_count(&sms)) return 1;
    k_pack_fc_weight<<<elementwise_grid((long long)N * ld_words, sms), 256, 0, (cudaStream_t)stream>>>(
        W, K, N, ld_words, out);
    return launch_check("pack_fc_weight");
}

int tcbnn_pack_conv_filter(const float* F, int RS, int C, int O, uint32_t* out, void* stream) {
    if (RS <= 0 || C <= 0 || O <= 0) return fail("pack_conv_filter: bad sizes");
    int sms;
    if (sm_count(&sms)) return 1;
    k_pack_conv_filter<<<elementwise_grid((long long)O * RS * ((C + 31) / 32), sms), 256, 0,
                         (cudaStream_t)stream>>>(F, RS, C, O, out);
    return launch_check("pack_conv_filter");
}

int tcbnn_pack_inconv_filter(const float* F, int RS, int O, uint32_t* out, void* stream) {
    if (RS <= 0 || O <= 0) return fail("pack_inconv_filter: bad sizes");
    int sms;
    if (sm_count(&sms)) return 1;
    k_pack_inconv_filter<<<elementwise_grid((long long)RS * 3 * ((O + 31) / 32), sms), 256, 0,
                           (cudaStream_t)stream>>>(F, RS, O, out);
    return launch_check("pack_inconv_filter");
}

size_t tcbnn_gemm_workspace_bytes(int M, int N, int K) {
    int sms;
    if (M <= 0 || N <= 0 || K <= 0 || sm_count(&sms)) return 0;
    const int s = gemm_splits(M, N, K, sms);
    const size_t split_k = s > 1 ? (size_t)s * M * N * sizeof(int32_t) : 0;
    const GemmUmmaPlan plan = gemm_umma_plan(M, N, K, sms);
    return plan.use && plan.bytes > split_k ? plan.bytes : split_k;
}

int tcbnn_gemm_launches(int M, int N, int K, size_t workspace_bytes) {
    int sms;
    if (M <= 0 || N <= 0 || K <= 0 || sm_count(&sms)) return 0;
    const GemmUmmaPlan plan = gemm_umma_plan(M, N, K, sms);
    if (plan.use && g_gemm_path != 1 && workspace_bytes >= plan.bytes) return plan.splits > 1 ? 3 : 2;   // expansion, GEMM, finish
    const int s = gemm_splits(M, N, K, sms);
    return (s > 1 && workspace_bytes >= (size_t)s * M * N * sizeof(int32_t)) ? 2 : 1;
}

int tcbnn_set_gemm_path(int path) {
    if (path < 0 || path > 1) return fail("set_gemm_path: 0 = automatic, 1 = warp-level b1 MMA only");
    g_gemm_path = path;
    return 0;
}

int tcbnn_set_gemm_plan(int pair, int splits) {
    if (pair < -1 || pair > 1 || splits < -1 || splits == 0 || splits > 32)
        return fail("set_gemm_plan: pair is -1, 0 or 1; splits is -1 or 1..32");
    g_gemm_force_pair = pair;
    g_gemm_force_splits = splits;
    return 0;
}

int tcbnn_gemm_status(int* status) {
    if (!status) return fail("gemm_status: null pointer");
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemcpyFromSymbol(status, g_gemm_status, sizeof(int)));
    if (*status) {                                       // reading a failure clears it
        const int zero = 0;
        CUDA_TRY(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
    }
    return 0;
}

int tcbnn_bgemm(const uint32_t* A, const uint32_t* B, int M, int N, int K, int lda, int ldb,
                int32_t* C, int ldc, void* workspace, size_t workspace_bytes, void* stream) {
    if (ldc < N) return fail("bgemm: ldc < N");
    GemmArgs g{A, B, M, N, K, lda, ldb, GEMM_INT32, C, ldc, nullptr, nullptr, 1, nullptr};
    return run_gemm(g, workspace, workspace_bytes, (cudaStream_t)stream);
}

int tcbnn_fc_layer(const uint32_t* A, const uint32_t* W, const float* thr, int M, int K, int N,
                   int lda, int ldw, uint32_t* out, int ldo, void* workspace,
                   size_t workspace_bytes, void* stream) {
    if (ldo * 32 < N) return fail("fc_layer: ldo too small");
    GemmArgs g{A, W, M, N, K, lda, ldw, GEMM_FC_BITS, out, ldo, thr, nullptr, 1, nullptr};
    return run_gemm(g, workspace, workspace_bytes, (cudaStream_t)stream);
}

int tcbnn_out_layer(const uint32_t* A, const uint32_t* W, const float* scale, const float* bias,
                    int M, int K, int N, int lda, int ldw, float* out, int ldo, void* workspace,
                    size_t workspace_bytes, void* stream) {
    if (ldo < N) return fail("out_layer: ldo < N");
    GemmArgs g{A, W, M, N, K, lda, ldw, GEMM_OUT_AFFINE, out, ldo, scale, bias, 1, nullptr};
    return run_gemm(g, workspace, workspace_bytes, (cudaStream_t)stream);
}

int tcbnn_conv_shape(tcbnn_conv_desc* d) {
    if (!d) return fail("conv_shape: null descriptor");
    if (d->H <= 0 || d->W <= 0 || d->R <= 0 || d->S <= 0 || d->stride_h <= 0 || d->stride_w <= 0 ||
        d->pool <= 0)
        return fail("conv_shape: sizes must be positive");
    const int H = d->H, W = d->W, sh = d->stride_h, sw = d->stride_w;
    d->pad_h = d->padding ? ((((H + sh - (H % sh)) / sh - 1) * sh + d->R - H) / 2) : 0;
    d->pad_w = d->padding ? ((((W + sw - (W % sw)) / sw - 1) * sw + d->S - W) / 2) : 0;
    const int bh = d->padding ? (H + sh - 1) / sh : ((H - d->R) / sh + 1);
    const int bw = d->padding ? (W + sw - 1) / sw : ((W - d->S) / sw + 1);
    d->OH = (bh + d->pool - 1) / d->pool;
    d->OW = (bw + d->pool - 1) / d->pool;
    return 0;
}

size_t tcbnn_conv_prepared_bytes(const tcbnn_conv_desc* d) {
    if (conv_check(d, true)) return 0;
    return prepared_layout(d).bytes;
}

int tcbnn_conv_prepare(const tcbnn_conv_desc* d, const uint32_t* filter_bits, void* prepared,
                       void* stream) {
    if (conv_check(d, true)) return 1;
    if ((uintptr_t)prepared & 255) return fail("conv_prepare: blob must be 256-byte aligned");
    const PreparedLayout L = prepared_layout(d);
    char* p = (char*)prepared;
    int sms;
    if (sm_count(&sms)) return 1;
    k_conv_prepare<<<elementwise_grid((long long)d->O * 2 * L.KP, sms), 256, 0, (cudaStream_t)stream>>>(
        filter_bits, d->O, d->R, d->S, (d->C + 31) / 32, d->W, L.KP, (uint32_t*)(p + L.off_wq),
        (uint32_t*)(p + L.off_ktab), (int*)(p + L.off_pwt), (int*)(p + L.off_pwtot));
    if (launch_check("conv_prepare")) return 1;
    CUDA_TRY(cudaMemsetAsync(p + L.off_err, 0, 256, (cudaStream_t)stream));
    if (L.umma_nt) {
        const long long units = (long long)d->O * d->R * d->S * (d->C / 16);
        k_prepare_filter_ws<<<elementwise_grid(units, sms), 256, 0, (cudaStream_t)stream>>>(
            filter_bits, d->O, d->R * d->S, d->C, L.umma_nt, (uint4*)(p + L.off_wi8));
        if (launch_check("conv_prepare (int8 filter)")) return 1;
    }
    if (L.pre_nt) {
        const long long units = (long long)d->O * d->R * d->S * (d->C / 32);
        k_prepare_filter_f4<<<elementwise_grid(units, sms), 256, 0, (cudaStream_t)stream>>>(
            filter_bits, d->O, d->R * d->S, d->C, L.pre_nt, (uint4*)(p + L.off_wf4));
        if (launch_check("conv_prepare (4-bit filter)")) return 1;
    }
    if (L.as_npos && (!L.umma_nt || L.off_wi8_as != L.off_wi8)) {
        const long long units = (long long)d->O * d->R * d->S * (d->C / 16);
        k_prepare_filter_ws<<<elementwise_grid(units, sms), 256, 0, (cudaStream_t)stream>>>(
            filter_bits, d->O, d->R * d->S, d->C, umma::kAsNT, (uint4*)(p + L.off_wi8_as));
        if (launch_check("conv_prepare (int8 filter, 128-channel tiles)")) return 1;
    }
    return 0;
}

size_t tcbnn_conv_workspace_bytes(const tcbnn_conv_desc* d) {
    if (conv_check(d, true)) return 0;
    const PreparedLayout L = prepared_layout(d);
    return main_ws_bytes(L) + L.prepool_bytes;
}

size_t tcbnn_conv_planes_bytes(const tcbnn_conv_desc* d) {
    if (conv_check(d, true)) return 0;
    return prepared_layout(d).pre_bytes;
}

int tcbnn_conv_layer(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                     const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                     int residual_channels, int residual_pool, uint32_t* out,
                     long long out_image_stride, void* res_out, int res_out_bytes,
                     int32_t* acc_out, void* stream) {
    return tcbnn_conv_layer_w(d, in, prepared, thr, res_in, res_in_bytes, res_in_ch, residual_channels,
                              residual_pool, out, out_image_stride, res_out, res_out_bytes, acc_out,
                              nullptr, 0, stream);
}

int tcbnn_conv_layer_w(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                       const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                       int residual_channels, int residual_pool, uint32_t* out,
                       long long out_image_stride, void* res_out, int res_out_bytes,
                       int32_t* acc_out, void* workspace, size_t workspace_bytes, void* stream) {
    return tcbnn_conv_layer_x(d, in, prepared, thr, res_in, res_in_bytes, res_in_ch, residual_channels,
                              residual_pool, out, out_image_stride, res_out, res_out_bytes, acc_out,
                              workspace, workspace_bytes, 0, nullptr, nullptr, 0, stream);
}

// the next layer's input planes, as its descriptor lays them out
struct NextPlanes { uint4* planes; long long positions, front; int PW, VH, nplane; };

// Checks that `next` can take `d`'s output as pre-expanded input and describes its planes.
static int next_planes_of(const tcbnn_conv_desc* d, int out_h, int out_w, const tcbnn_conv_desc* next,
                          void* planes, size_t planes_bytes, NextPlanes* nx) {
    if (conv_check(next, true)) return 1;
    const PreparedLayout N = prepared_layout(next);
    if (!N.pre_bytes) return fail("next layer takes no pre-expanded input (tcbnn_conv_planes_bytes is 0)");
    if (next->B != d->B || next->H != out_h || next->W != out_w || next->C != d->O)
        return fail("next layer's input %dx%dx%dx%d is not this layer's output %dx%dx%dx%d", next->B, next->H,
                    next->W, next->C, d->B, out_h, out_w, d->O);
    if (!planes || planes_bytes < N.pre_bytes) return fail("next layer's planes: %zu bytes given, %zu needed", planes_bytes, N.pre_bytes);
    if ((uintptr_t)planes & 255) return fail("next layer's planes must be 256-byte aligned");
    nx->planes = (uint4*)planes; nx->positions = N.pre_positions; nx->front = N.pre_front;
    nx->PW = N.umma_pw; nx->VH = N.umma_vh; nx->nplane = next->stride_h == 2 ? 4 : 1;
    return 0;
}

// Expansion pass of `next` run on bits that are already in memory (the producing kernel could not
// write the planes itself).
static int expand_for_next(const tcbnn_conv_desc* next, const uint32_t* bits, const NextPlanes& nx, cudaStream_t st) {
    umma::ConvWsArgs a = {};
    a.in = bits; a.B = next->B; a.H = next->H; a.W = next->W; a.C = next->C;
    a.stride = next->stride_h; a.OHg = next->OH * next->pool; a.OWg = next->OW * next->pool;
    a.PW = nx.PW; a.VH = nx.VH; a.NV = (long long)next->B * nx.VH * nx.PW;
    umma::fastdiv_setup(a.PW, &a.pw_mul, &a.pw_sh);
    umma::fastdiv_setup(a.VH, &a.vh_mul, &a.vh_sh);
    int sms;
    if (sm_count(&sms)) return 1;
    k_expand_raster<<<elementwise_grid(nx.positions * (next->C >> 6) * nx.nplane, sms), 256, 0, st>>>(a, nx.planes, nx.positions, nx.front);
    return launch_check("expansion for the next layer");
}

static int conv_layer_impl(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                           const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                           int residual_channels, int residual_pool, uint32_t* out,
                           long long out_image_stride, void* res_out, int res_out_bytes,
                           int32_t* acc_out, void* workspace, size_t workspace_bytes, int workspace_ready,
                           const NextPlanes* nx, bool* fed, void* stream) {
    *fed = false;
    if (conv_check(d, true)) return 1;
    const int Ow = (d->O + 31) / 32;
    if (out_image_stride < (long long)d->OH * d->OW * Ow) return fail("conv_layer: out_image_stride too small");
    if ((res_out || res_in) && d->pool != 1) return fail("conv_layer: residuals need pool == 1");
    if (res_in && (res_in_ch <= 0 || residual_channels <= 0)) return fail("conv_layer: residual channel counts must be positive");
    int res_in_chunked = 0, res_out_chunked = 0, res_out_proven = 0;
    if (res_in && !residual_format(res_in_bytes, &res_in_bytes, &res_in_chunked))
        return fail("conv_layer: res_in_bytes must be 2, 4 or TCBNN_RES_INT16_CHUNKED");
    if (res_out && !residual_format(res_out_bytes, &res_out_bytes, &res_out_chunked, &res_out_proven))
        return fail("conv_layer: res_out_bytes must be 2, 4 or TCBNN_RES_INT16_CHUNKED");
    if (!res_in) res_in_chunked = 0;
    if (!res_out) res_out_chunked = 0;
    if ((uintptr_t)in & 7) return fail("conv_layer: input must be 8-byte aligned");
    const PreparedLayout L = prepared_layout(d);
    const char* p = (const char*)prepared;
    const bool use_pre = L.pre_bytes && workspace && g_conv_path != 3;
    if (res_in_chunked || res_out_chunked) {
        // only the loader-fed kernel reads and writes that layout
        if (!use_pre || g_conv_path == 1 || d->pool != 1)
            return fail("conv_layer: chunked residuals need the loader-fed tcgen05 kernel (a layer with tcbnn_conv_planes_bytes != 0, "
                        "called with its workspace, no pooling)");
        const int lim_in = residual_channels < res_in_ch ? residual_channels : res_in_ch;
        if (res_in_chunked && (res_in_ch % 8 || lim_in % 8 || ((uintptr_t)res_in & 15)))
            return fail("conv_layer: a chunked residual needs channel counts in multiples of 8 and a 16-byte aligned tensor");
        if (res_out_chunked && (d->O % 8 || ((uintptr_t)res_out & 15)))
            return fail("conv_layer: a chunked residual needs channel counts in multiples of 8 and a 16-byte aligned tensor");
    }
    const bool use_as = L.as_npos && g_conv_path != 3 && !use_pre;
    const bool have_tc = use_as || use_pre || L.ws_ok;
    if (g_conv_path >= 2 && !have_tc) return fail("conv_layer: layer is not eligible for the tcgen05 path (or needs its workspace)");
    // the tcgen05 epilogue moves residuals in 4-channel vectors
    const bool res_vec_ok = !res_in || (res_in_ch % 4 == 0 && residual_channels % 4 == 0 &&
                                        ((uintptr_t)res_in & 15) == 0);
    if (g_conv_path >= 2 && !res_vec_ok) return fail("conv_layer: residual layout not eligible for the tcgen05 path");
    // a pooled layer needs room behind the kernel's own scratch for its pre-pool bits
    const size_t main_ws = main_ws_bytes(L);
    const bool pooled = d->pool != 1;
    const bool pooled_ok = !pooled || (workspace && workspace_bytes >= main_ws + L.prepool_bytes &&
                                       ((uintptr_t)workspace & 255) == 0);
    if (g_conv_path >= 2 && !pooled_ok) return fail("conv_layer: a pooled layer needs its workspace for the tcgen05 path");
    if (have_tc && g_conv_path != 1 && res_vec_ok && pooled_ok &&
        (!res_out || ((uintptr_t)res_out & 15) == 0)) {
      const int P = d->OH * d->pool, Q = d->OW * d->pool;
      uint32_t* prepool = pooled ? (uint32_t*)((char*)workspace + main_ws) : nullptr;
      int sms;
      if (sm_count(&sms)) return 1;
      cudaStream_t st = (cudaStream_t)stream;
      auto launch_tc = [&]() -> int {
        umma::ConvWsArgs a;
        a.in = in; a.wi8 = (const uint4*)(p + L.off_wi8); a.wf4 = (const uint4*)(p + L.off_wf4); a.thr = thr;
        a.B = d->B; a.H = d->H; a.W = d->W; a.C = d->C; a.O = d->O; a.R = d->R; a.S = d->S;
        a.pad_h = d->pad_h; a.pad_w = d->pad_w; a.stride = d->stride_h;
        a.OHg = P; a.OWg = Q;
        a.PW = L.umma_pw; a.VH = L.umma_vh; a.NPOS = L.umma_npos;
        a.back_y = L.umma_back_y; a.back_x = L.umma_back_x;
        a.NV = (long long)d->B * a.VH * a.PW;
        umma::fastdiv_setup(a.PW, &a.pw_mul, &a.pw_sh);
        umma::fastdiv_setup(a.VH, &a.vh_mul, &a.vh_sh);
        a.res_in = res_in; a.res_in_bytes = res_in_bytes; a.res_in_ch = res_in_ch;
        a.res_in_chunked = res_in_chunked; a.res_out_chunked = res_out_chunked;
        a.res_out_proven = res_out ? res_out_proven : 0;
        a.res_in_npix = (long long)d->B * d->OH * d->OW * (residual_pool ? 4 : 1);
        a.res_out_npix = (long long)d->B * d->OH * d->OW;
        a.residual_channels = residual_channels; a.residual_pool = residual_pool;
        a.out = pooled ? prepool : out;
        a.out_image_stride = pooled ? (long long)P * Q * Ow : out_image_stride;
        a.res_out = res_out;
        a.res_out_bytes = res_out_bytes; a.acc_out = acc_out;
        a.err_flag = (int*)(p + L.off_err);
        a.trace = g_conv_trace;
        a.pre = nullptr; a.pre_positions = 0; a.pre_front = 0;
        a.pre_stages = 0; a.pre_cbs = 1;
        a.nxt = nullptr; a.nxt_positions = 0; a.nxt_front = 0; a.nxt_PW = 0; a.nxt_VH = 0; a.nxt_nplane = 1;
        if (nx && !use_as && !pooled) {     // (a pooled layer's kernel sees the pre-pool grid)
            a.nxt = nx->planes; a.nxt_positions = nx->positions; a.nxt_front = nx->front;
            a.nxt_PW = nx->PW; a.nxt_VH = nx->VH; a.nxt_nplane = nx->nplane;
            *fed = true;
        }
        if (use_as) {
            a.NPOS = L.as_npos; a.as_slots = L.as_slots;
            a.wi8 = (const uint4*)(p + L.off_wi8_as);
            // a pooled int16 residual is reduced by a streaming pass first when there is scratch
            // for it: four scattered 16-byte loads per value inside the epilogue cost more
            const size_t pooled_res_bytes = (size_t)d->B * d->OH * d->OW * (size_t)res_in_ch * 2;
            if (res_in && residual_pool && res_in_bytes == 2 && res_in_ch % 8 == 0 && workspace &&
                workspace_bytes >= pooled_res_bytes && ((uintptr_t)workspace & 15) == 0) {
                const long long units = (long long)d->B * d->OH * d->OW * (res_in_ch / 8);
                k_pool_residual16<<<elementwise_grid(units, sms), 256, 0, st>>>((const uint4*)res_in, (uint4*)workspace,
                                                                             d->B, d->OH, d->OW, res_in_ch / 8);
                if (launch_check("conv_layer (residual pooling)")) return 1;
                a.res_in = workspace; a.residual_pool = 0;
            }
            return launch_conv_umma_as(a, L.as_smem, sms, st);
        }
        if (use_pre) {
            if (workspace_bytes < L.pre_bytes)
                return fail("conv_layer: workspace of %zu bytes, the layer needs %zu", workspace_bytes, L.pre_bytes);
            if ((uintptr_t)workspace & 255) return fail("conv_layer: workspace must be 256-byte aligned");
            a.pre = (const uint4*)workspace; a.pre_positions = L.pre_positions; a.pre_front = L.pre_front;
            a.pre_stages = L.pre_stages;
            a.pre_cbs = 1;
            size_t pre_smem = L.pre_smem;
            if (g_conv_cbs) {
                // four or two 64-channel blocks per stage where at least three such stages fit
                const int RS = d->R * d->S;
                for (int cbs = 4; cbs >= 2 && a.pre_cbs == 1; cbs >>= 1) {
                    if ((d->C / 64) % cbs) continue;
                    const int np = (d->stride_h == 2 ? 4 : 1) * cbs;
                    int stages = 6;
                    while (stages > 3 && umma::pre_smem_bytes(L.umma_npos, d->C, RS, L.pre_nt, stages, np) > 227 * 1024) stages--;
                    const size_t need = umma::pre_smem_bytes(L.umma_npos, d->C, RS, L.pre_nt, stages, np);
                    if (need <= 227 * 1024) { a.pre_cbs = cbs; a.pre_stages = stages; pre_smem = need; }
                }
                // (a stride-2 layer next to a 147 KB filter block: two stages of two blocks still
                // halve the issuing thread's wait / commit rounds)
                if (a.pre_cbs == 1 && (d->C / 64) % 2 == 0) {
                    const size_t need = umma::pre_smem_bytes(L.umma_npos, d->C, RS, L.pre_nt, 2, (d->stride_h == 2 ? 4 : 1) * 2);
                    if (need <= 227 * 1024) { a.pre_cbs = 2; a.pre_stages = 2; pre_smem = need; }
                }
            }
            // a pooled int16 residual is reduced by a streaming pass first when the workspace has
            // the room behind the planes: four scattered loads per value in the epilogue cost more
            const size_t pooled_res_bytes = (size_t)d->B * d->OH * d->OW * (size_t)res_in_ch * 2;
            // (the tile-per-group epilogues read a pooled chunk-major residual in place: whole lines)
            if (res_in && residual_pool && res_in_bytes == 2 && res_in_ch % 8 == 0 && !pooled &&
                !pre_tile_ok(res_in, res_in_bytes, res_in_chunked, res_out, res_out_bytes, res_out_chunked, acc_out) &&
                (!res_in_chunked || res_in_ch / 8 <= kPoolChunkedMaxCh8) &&
                pooled_res_bytes <= L.pool_bytes && workspace_bytes >= planes_padded(L) + pooled_res_bytes) {
                char* pooled_res = (char*)workspace + planes_padded(L);
                const long long units = (long long)d->B * d->OH * d->OW * (res_in_ch / 8);
                if (res_in_chunked)
                    k_pool_residual16_chunked<<<elementwise_grid(units, sms), 256, 0, st>>>(
                        (const uint4*)res_in, (uint4*)pooled_res, d->B, d->OH, d->OW, res_in_ch / 8);   // (res_in_ch / 8 <= 32: checked above)
                else
                    k_pool_residual16<<<elementwise_grid(units, sms), 256, 0, st>>>((const uint4*)res_in, (uint4*)pooled_res,
                                                                                 d->B, d->OH, d->OW, res_in_ch / 8);
                if (launch_check("conv_layer (residual pooling)")) return 1;
                a.res_in = pooled_res; a.residual_pool = 0;
                a.res_in_chunked = 0; a.res_in_npix = (long long)d->B * d->OH * d->OW;     // the pooled copy is NHWC
            }
            if (L.pre_nt == 32) return launch_conv_umma_pre<32>(a, pre_smem, sms, st, !workspace_ready);
            if (L.pre_nt == 64) return launch_conv_umma_pre<64>(a, pre_smem, sms, st, !workspace_ready);
            if (L.pre_nt == 128) return launch_conv_umma_pre<128>(a, pre_smem, sms, st, !workspace_ready);
        }
#define TCBNN_WS_CASE(NN, SS) \
        if (L.umma_nt == NN && d->stride_h == SS) return launch_conv_umma_ws<NN, SS>(a, L.umma_smem, sms, st);
        TCBNN_WS_CASE(32, 1) TCBNN_WS_CASE(64, 1) TCBNN_WS_CASE(128, 1) TCBNN_WS_CASE(256, 1)
        TCBNN_WS_CASE(32, 2) TCBNN_WS_CASE(64, 2) TCBNN_WS_CASE(128, 2) TCBNN_WS_CASE(256, 2)
#undef TCBNN_WS_CASE
        return fail("conv_layer: no tcgen05 instance for n-tile=%d stride=%d", L.umma_nt, d->stride_h);
      };
      if (launch_tc()) return 1;
      if (pooled) {
          k_pool_bits<<<elementwise_grid((long long)d->B * d->OH * d->OW * Ow, sms), 256, 0, st>>>(
              prepool, out, d->B, d->OH, d->OW, Ow, out_image_stride);
          return launch_check("conv_layer (OR pooling)");
      }
      return 0;
    }
    if (res_in_chunked || res_out_chunked)
        return fail("conv_layer: this call cannot take the tcgen05 path it needs for chunked residuals (alignment, residual layout)");
    ConvArgs c;
    c.in = in;
    c.wq = (const uint32_t*)(p + L.off_wq);
    c.ktab = (const uint32_t*)(p + L.off_ktab);
    c.pwt = (const int*)(p + L.off_pwt);
    c.pwtot = (const int*)(p + L.off_pwtot);
    c.thr = thr;
    c.B = d->B; c.H = d->H; c.W = d->W; c.C = d->C; c.Cw = (d->C + 31) / 32; c.O = d->O;
    c.R = d->R; c.S = d->S; c.sh = d->stride_h; c.sw = d->stride_w;
    c.pad_h = d->pad_h; c.pad_w = d->pad_w; c.pool = d->pool; c.OH = d->OH; c.OW = d->OW;
    c.KP = L.KP;
    c.res_in = res_in; c.res_in_bytes = res_in_bytes; c.res_in_ch = res_in_ch;
    c.residual_channels = residual_channels; c.residual_pool = residual_pool;
    c.out = out; c.out_image_stride = out_image_stride; c.res_out = res_out;
    c.res_out_bytes = res_out_bytes; c.res_out_ld = d->O; c.acc_out = acc_out;
    int sms;
    if (sm_count(&sms)) return 1;
    const long long rows = (long long)d->B * d->OH * d->OW * d->pool * d->pool;
    const long long tasks = ((rows + 31) / 32) * Ow;
    k_conv<<<warp_grid(tasks, sms), kThreads, 0, (cudaStream_t)stream>>>(c);
    return launch_check("conv_layer");
}

int tcbnn_conv_layer_x(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                       const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                       int residual_channels, int residual_pool, uint32_t* out,
                       long long out_image_stride, void* res_out, int res_out_bytes,
                       int32_t* acc_out, void* workspace, size_t workspace_bytes, int workspace_ready,
                       const tcbnn_conv_desc* next, void* next_planes, size_t next_planes_bytes,
                       void* stream) {
    NextPlanes nx;
    if (next) {
        if (conv_check(d, true)) return 1;
        if (next_planes_of(d, d->OH, d->OW, next, next_planes, next_planes_bytes, &nx)) return 1;
        if (out_image_stride != (long long)d->OH * d->OW * ((d->O + 31) / 32))
            return fail("conv_layer: feeding the next layer needs a dense output (out_image_stride == OH*OW*ceil(O/32))");
    }
    if (workspace_ready && !workspace) return fail("conv_layer: workspace_ready without a workspace");
    bool fed = false;
    if (conv_layer_impl(d, in, prepared, thr, res_in, res_in_bytes, res_in_ch, residual_channels, residual_pool,
                        out, out_image_stride, res_out, res_out_bytes, acc_out, workspace, workspace_bytes,
                        workspace_ready, next ? &nx : nullptr, &fed, stream))
        return 1;
    if (next && !fed) return expand_for_next(next, out, nx, (cudaStream_t)stream);
    return 0;
}

int tcbnn_conv_prefers_chunked_residual(const tcbnn_conv_desc* d) {
    if (conv_check(d, true)) return 0;
    const PreparedLayout L = prepared_layout(d);
    // the loader-fed kernel's tile-per-group epilogue: one thread per pixel, whole lines per warp
    return L.pre_nt != 0 && d->pool == 1 && d->O % 8 == 0 ? 1 : 0;
}

int tcbnn_set_conv_path(int path) {
    if (path < 0 || path > 10)
        return fail("set_conv_path: 0 = automatic, 1 = warp-level b1 MMA, 2 = tcgen05, 3 = tcgen05 filter-stationary kernel only, "
                    "4 / 5 = automatic with residual staging never / wherever possible, 6 = automatic, one CTA per SM only, "
                    "7 = automatic without the tile-per-group epilogues, 8 = automatic, two CTAs per SM wherever they fit, "
                    "9 = automatic, one 64-channel block per stage, 10 = automatic, every n-tile the same number of CTAs");
    g_conv_path = path >= 4 ? 0 : path;
    g_conv_res_stage = path == 4 ? 0 : path == 5 ? 2 : 1;
    g_conv_two_ctas = path == 6 ? 0 : path == 8 ? 2 : 1;
    g_conv_tile = path == 7 ? 0 : 1;
    g_conv_cbs = path == 9 ? 0 : 1;
    g_conv_uneven = path == 10 ? 0 : 1;
    return 0;
}

int tcbnn_conv_set_trace(void* device_buffer) {
    g_conv_trace = (long long*)device_buffer;
    return 0;
}

int tcbnn_conv_status(const tcbnn_conv_desc* d, const void* prepared, int* status) {
    if (conv_check(d, true)) return 1;
    if (!status) return fail("conv_status: null status");
    const PreparedLayout L = prepared_layout(d);
    CUDA_TRY(cudaMemcpy(status, (const char*)prepared + L.off_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status)                                         // reading a failure clears it
        CUDA_TRY(cudaMemset((char*)const_cast<void*>(prepared) + L.off_err, 0, sizeof(int)));
    return 0;
}

static int run_inconv(const tcbnn_conv_desc* d, const float* x, const unsigned char* x8, const float* lut,
                      const uint32_t* filter_bits, const float* thr, uint32_t* out,
                      long long out_image_stride, void* res_out, int res_out_bytes, float* acc_out,
                      void* stream) {
    if (conv_check(d, false)) return 1;
    if (res_out && res_out_bytes != 2 && res_out_bytes != 4) return fail("inconv_layer: res_out_bytes must be 2 or 4");
    const int Ow = (d->O + 31) / 32;
    if (out_image_stride < (long long)d->OH * d->OW * Ow) return fail("inconv_layer: out_image_stride too small");
    InConvArgs c;
    c.x = x; c.x8 = x8; c.lut = lut; c.fbits = filter_bits; c.thr = thr;
    c.B = d->B; c.H = d->H; c.W = d->W; c.O = d->O; c.R = d->R; c.S = d->S;
    c.sh = d->stride_h; c.sw = d->stride_w; c.pad_h = d->pad_h; c.pad_w = d->pad_w;
    c.pool = d->pool; c.OH = d->OH; c.OW = d->OW;
    c.out = out; c.out_image_stride = out_image_stride; c.res_out = res_out;
    c.res_out_bytes = res_out_bytes; c.res_out_ld = d->O; c.acc_out = acc_out;
    int sms;
    if (sm_count(&sms)) return 1;
    const int opad = ((d->O + 31) / 32) * 32;
    const size_t smem = inconv_tiled_smem(d->R, d->S, d->O);
    if ((g_conv_path != 1 || x8) && smem <= 200 * 1024 && kInconvThreads % opad == 0) {
        const int ppt = kInconvPixels / (kInconvThreads / opad);
        if (ppt == 4) return launch_inconv_tiled<4>(c, smem, sms, (cudaStream_t)stream);
        if (ppt == 8) return launch_inconv_tiled<8>(c, smem, sms, (cudaStream_t)stream);
        if (ppt == 16) return launch_inconv_tiled<16>(c, smem, sms, (cudaStream_t)stream);
    }
    if (x8) return fail("inconv_layer_u8: this shape has no uint8-input kernel (filter too large or %d output channels)", d->O);
    k_inconv<<<warp_grid((long long)d->B * d->OH * d->OW, sms), kThreads, 0, (cudaStream_t)stream>>>(c);
    return launch_check("inconv_layer");
}

int tcbnn_inconv_layer(const tcbnn_conv_desc* d, const float* x, const uint32_t* filter_bits,
                       const float* thr, uint32_t* out, long long out_image_stride,
                       void* res_out, int res_out_bytes, float* acc_out, void* stream) {
    return run_inconv(d, x, nullptr, nullptr, filter_bits, thr, out, out_image_stride, res_out,
                      res_out_bytes, acc_out, stream);
}

int tcbnn_inconv_layer_u8(const tcbnn_conv_desc* d, const uint8_t* x, const float* lut,
                          const uint32_t* filter_bits, const float* thr, uint32_t* out,
                          long long out_image_stride, void* res_out, int res_out_bytes,
                          float* acc_out, void* stream) {
    if (!x || !lut) return fail("inconv_layer_u8: null input or table");
    return run_inconv(d, nullptr, x, lut, filter_bits, thr, out, out_image_stride, res_out,
                      res_out_bytes, acc_out, stream);
}

// ---- first layer specialised to one filter (run-time compiled) -----------------------------
// Compiles (and loads, unless only_compile) one variant of the handle's kernel; variant = u8 * 2 + vec.
static int spec_build(spec::SpecHandle* h, int variant, bool only_compile) {
    std::lock_guard<std::mutex> lock(h->mu);
    if (h->kernel[variant]) return 0;
    const std::string src = spec::generate_source(*h, h->codes, h->thr_bits, variant);
    std::vector<char> cubin;
    std::string err;
    if (!spec::compile_cubin(src, cubin, err)) return fail("inconv_specialize: %s", err.c_str());
    if (only_compile) return 0;
    CUDA_TRY(cudaLibraryLoadData(&h->lib[variant], cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    CUDA_TRY(cudaLibraryGetKernel(&h->kernel[variant], h->lib[variant], "tcbnn_spec"));
    return 0;
}

static int spec_check(const tcbnn_conv_desc* d) {
    if (conv_check(d, false)) return 1;
    if (d->O > spec::kSpecMaxO)
        return fail("inconv_specialize: at most %d output channels", spec::kSpecMaxO);
    return 0;
}

int tcbnn_inconv_specialize(const tcbnn_conv_desc* d, const uint32_t* filter_bits, const float* thr,
                            void* stream, void** handle) {
    if (!handle) return fail("inconv_specialize: null handle pointer");
    *handle = nullptr;
    if (spec_check(d)) return 1;
    const int RS = d->R * d->S, Ow = (d->O + 31) / 32;
    std::vector<uint32_t> fb((size_t)RS * 3 * Ow), thr_bits(d->O);
    CUDA_TRY(cudaMemcpyAsync(fb.data(), filter_bits, fb.size() * 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    CUDA_TRY(cudaMemcpyAsync(thr_bits.data(), thr, (size_t)d->O * 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    if (!spec::nvrtc().ok) return fail("inconv_specialize: libnvrtc could not be opened (set TCBNN_NVRTC to its path)");
    spec::SpecHandle* h = new spec::SpecHandle();
    h->O = d->O; h->R = d->R; h->S = d->S; h->sh = d->stride_h; h->sw = d->stride_w;
    h->pad_h = d->pad_h; h->pad_w = d->pad_w; h->pool = d->pool;
    h->thr_bits = thr_bits;
    h->codes.resize((size_t)RS * d->O);
    for (int t = 0; t < RS; t++)
        for (int o = 0; o < d->O; o++) {
            const uint32_t* fw = fb.data() + (size_t)t * 3 * Ow + (o >> 5);      // param.h:613-632
            const int sh = 31 - (o & 31);
            h->codes[(size_t)t * d->O + o] = (unsigned char)((((fw[0] >> sh) & 1u) << 2) | (((fw[Ow] >> sh) & 1u) << 1) |
                                                             ((fw[2 * Ow] >> sh) & 1u));
        }
    *handle = h;
    return 0;
}

int tcbnn_inconv_specialized_layer(void* handle, const tcbnn_conv_desc* d, const float* x,
                                   const uint8_t* x8, const float* lut, uint32_t* out,
                                   long long out_image_stride, void* res_out, int res_out_bytes,
                                   float* acc_out, void* stream) {
    return tcbnn_inconv_specialized_layer_x(handle, d, x, x8, lut, out, out_image_stride, res_out, res_out_bytes,
                                            acc_out, nullptr, nullptr, 0, stream);
}

int tcbnn_inconv_specialized_layer_x(void* handle, const tcbnn_conv_desc* d, const float* x,
                                     const uint8_t* x8, const float* lut, uint32_t* out,
                                     long long out_image_stride, void* res_out, int res_out_bytes,
                                     float* acc_out, const tcbnn_conv_desc* next, void* next_planes,
                                     size_t next_planes_bytes, void* stream) {
    if (!handle) return fail("inconv_specialized_layer: null handle");
    if (conv_check(d, false)) return 1;
    spec::SpecHandle* h = (spec::SpecHandle*)handle;
    if (d->O != h->O || d->R != h->R || d->S != h->S || d->stride_h != h->sh || d->stride_w != h->sw ||
        d->pad_h != h->pad_h || d->pad_w != h->pad_w || d->pool != h->pool)
        return fail("inconv_specialized_layer: descriptor does not match the one the kernel was built for");
    if ((x != nullptr) == (x8 != nullptr)) return fail("inconv_specialized_layer: give fp32 images or uint8 images");
    if (x8 && !lut) return fail("inconv_specialized_layer: uint8 images need the value table");
    int res_out_chunked = 0;
    if (res_out && !residual_format(res_out_bytes, &res_out_bytes, &res_out_chunked))
        return fail("inconv_specialized_layer: res_out_bytes must be 2, 4 or TCBNN_RES_INT16_CHUNKED");
    if (res_out && res_out_chunked && (d->O % 8 || d->pool != 1 || ((uintptr_t)res_out & 15)))
        return fail("inconv_specialized_layer: a chunked residual needs a multiple of 8 channels, no pooling and a 16-byte aligned tensor");
    const int Ow = (d->O + 31) / 32;
    if (out_image_stride < (long long)d->OH * d->OW * Ow) return fail("inconv_specialized_layer: out_image_stride too small");
    spec::SpecArgs c;
    c.x = x; c.x8 = x8; c.lut = lut; c.B = d->B; c.H = d->H; c.W = d->W; c.OH = d->OH; c.OW = d->OW;
    c.out = out; c.out_image_stride = out_image_stride; c.res_out = res_out;
    c.res_out_bytes = res_out_bytes; c.res_out_ld = d->O; c.acc_out = acc_out;
    c.res_out_chunked = res_out ? res_out_chunked : 0;
    c.total = (unsigned)((long long)d->B * d->OH * d->OW * d->pool * d->pool);
    c.nxt = nullptr; c.nxt_positions = 0; c.nxt_front = 0; c.nxt_PW = 0; c.nxt_VH = 0;
    NextPlanes nx;
    bool expand_after = false;
    if (next) {
        if (next_planes_of(d, d->OH, d->OW, next, next_planes, next_planes_bytes, &nx)) return 1;
        if (nx.nplane == 1) {
            c.nxt = nx.planes; c.nxt_positions = nx.positions; c.nxt_front = nx.front; c.nxt_PW = nx.PW; c.nxt_VH = nx.VH;
        } else {
            expand_after = true;                  // the generated kernel writes stride-1 planes only
        }
    }
    void* params[] = {&c};
    const unsigned grid = (c.total + spec::kSpecThreads - 1) / spec::kSpecThreads;
    // aligned row loads when the geometry allows (stride 4, rows a multiple of 4 pixels, aligned base)
    const bool vec = h->sw == 4 && d->W % 4 == 0 && (x ? ((uintptr_t)x & 15) == 0 : ((uintptr_t)x8 & 3) == 0);
    const int variant = (x ? 0 : 2) + (vec ? 1 : 0);
    if (spec_build(h, variant, false)) return 1;       // first use compiles it (checked under the handle's lock)
    CUDA_TRY(cudaLaunchKernel((const void*)h->kernel[variant], dim3(grid, (h->O + 63) / 64), dim3(spec::kSpecThreads),
                              params, 0, (cudaStream_t)stream));
    if (launch_check("inconv_specialized_layer")) return 1;
    if (expand_after) return expand_for_next(next, out, nx, (cudaStream_t)stream);
    return 0;
}

int tcbnn_inconv_release(void* handle) {
    if (!handle) return 0;
    spec::SpecHandle* h = (spec::SpecHandle*)handle;
    for (int v = 0; v < 4; v++)
        if (h->lib[v]) cudaLibraryUnload(h->lib[v]);
    delete h;
    return 0;
}

int tcbnn_inconv_specialize_selftest(const tcbnn_conv_desc* d, unsigned seed, long long* source_bytes) {
    if (spec_check(d)) return 1;
    const int RS = d->R * d->S;
    spec::SpecHandle h;
    h.O = d->O; h.R = d->R; h.S = d->S; h.sh = d->stride_h; h.sw = d->stride_w;
    h.pad_h = d->pad_h; h.pad_w = d->pad_w; h.pool = d->pool;
    h.codes.resize((size_t)RS * d->O);
    h.thr_bits.resize(d->O);
    unsigned s = seed * 2654435761u + 12345u;
    for (auto& c : h.codes) { s = s * 1664525u + 1013904223u; c = (unsigned char)((s >> 24) & 7u); }
    for (auto& t : h.thr_bits) { s = s * 1664525u + 1013904223u; t = 0x40000000u ^ (s & 0x807FFFFFu); }
    // the uint8 variant with row loads where the stride allows them, the plain fp32 one otherwise
    const int variant = d->stride_w == 4 ? 3 : 0;
    if (source_bytes) *source_bytes = (long long)spec::generate_source(h, h.codes, h.thr_bits, variant).size();
    return spec_build(&h, variant, true);
}

int tcbnn_mma_peak(int kind, int warps_per_sm, int iters, double* tops) {
    if (!tops || iters <= 0 || warps_per_sm <= 0 || kind < 0 || kind > 7) return fail("mma_peak: bad arguments");
    int sms;
    if (sm_count(&sms)) return 1;
    cudaEvent_t e0, e1;
    CUDA_TRY(cudaEventCreate(&e0));
    CUDA_TRY(cudaEventCreate(&e1));
    float best = 1e30f;
    if (kind >= 3) {
        long long* buf = nullptr;
        CUDA_TRY(cudaMalloc(&buf, 32));
        CUDA_TRY(cudaMemset(buf, 0, 32));
        if (kind == 7 && iters > (1 << 18)) return fail("mma_peak: at most 2^18 iterations for kind 7 (exact fp32 sums)");
        CUDA_TRY(cudaFuncSetAttribute(k_umma_peak_mxf4, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024));
        CUDA_TRY(cudaFuncSetAttribute(k_umma_peak, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024));
        CUDA_TRY(cudaFuncSetAttribute(k_umma_issue<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024));
        CUDA_TRY(cudaFuncSetAttribute(k_umma_issue<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024));
        CUDA_TRY(cudaFuncSetAttribute(k_umma_issue<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024));
        const int group = warps_per_sm;            // kinds 4-6: MMAs per wait/commit group
        if (kind > 3 && kind < 7) iters = (iters / group) * group;
        if (iters <= 0) return fail("mma_peak: fewer iterations than MMAs per group");
        for (int rep = 0; rep < 4; rep++) {
            cudaEventRecord(e0);
            if (kind == 3) k_umma_peak<<<sms, 128, 48 * 1024>>>(iters, buf, (int*)(buf + 1));
            if (kind == 4) k_umma_issue<0><<<sms, 128, 48 * 1024>>>(iters, group, buf, (int*)(buf + 1));
            if (kind == 5) k_umma_issue<1><<<sms, 128, 48 * 1024>>>(iters, group, buf, (int*)(buf + 1));
            if (kind == 6) k_umma_issue<2><<<sms, 128, 48 * 1024>>>(iters, group, buf, (int*)(buf + 1));
            if (kind == 7) k_umma_peak_mxf4<<<sms, 128, 48 * 1024>>>(iters, buf, (int*)(buf + 1), (float*)(buf + 2));
            cudaEventRecord(e1);
            CUDA_TRY(cudaEventSynchronize(e1));
            float ms = 0;
            cudaEventElapsedTime(&ms, e0, e1);
            if (rep > 0 && ms < best) best = ms;
        }
        int status = 0;
        CUDA_TRY(cudaMemcpy(&status, buf + 1, sizeof(int), cudaMemcpyDeviceToHost));
        float sample[4] = {0, 0, 0, 0};
        CUDA_TRY(cudaMemcpy(sample, buf + 2, sizeof(sample), cudaMemcpyDeviceToHost));
        cudaFree(buf);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        if (status) return fail("mma_peak: a bounded wait in the tcgen05 probe gave up");
        if (kind == 7) {
            for (int w = 0; w < 4; w++)
                if (sample[w] != -64.0f * iters)
                    return fail("mma_peak: kind::mxf4 accumulator is %g, expected %g (+-1 operands, unit scales)",
                                (double)sample[w], -64.0 * iters);
            *tops = (double)sms * iters * 2.0 * 128 * 256 * 64 / (best * 1e-3) / 1e12;
            return 0;
        }
        *tops = (double)sms * iters * 2.0 * 128 * (kind == 3 ? 256 : 128) * 32 / (best * 1e-3) / 1e12;
        return 0;
    }
    int* sink = nullptr;
    CUDA_TRY(cudaMalloc(&sink, 4));
    const int threads = 256, ctas = sms * warps_per_sm * 32 / threads;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(e0);
        if (kind == 0) k_mma_peak<0><<<ctas, threads>>>(iters, 1u, sink);
        if (kind == 1) k_mma_peak<1><<<ctas, threads>>>(iters, 1u, sink);
        if (kind == 2) k_mma_peak<2><<<ctas, threads>>>(iters, 1u, sink);
        cudaEventRecord(e1);
        CUDA_TRY(cudaEventSynchronize(e1));
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    const double ops = (kind == 2 ? 2.0 * 16 * 8 * 32 : 2.0 * 16 * 8 * 256);
    *tops = (double)ctas * (threads / 32) * iters * 8 * ops / (best * 1e-3) / 1e12;
    return 0;
}

int tcbnn_bulk_copy_rate(int bytes, int depth, int warps, int ctas, int iters, double* issue_clocks_per_copy,
                         double* bytes_per_clock) {
    if (!bytes_per_clock || !issue_clocks_per_copy || bytes < 16 || bytes % 16 != 0 || depth < 1 || depth > 16 ||
        warps < 1 || warps > 4 || ctas < 1 || iters < 1 || iters > (1 << 20) ||
        (size_t)bytes * depth * warps > 200 * 1024)
        return fail("bulk_copy_rate: bytes a multiple of 16, depth 1..16, warps 1..4, bytes*depth*warps <= 200 KB, "
                    "iters <= 2^20");
    const size_t span = (size_t)bytes * depth * 8, total = span * (size_t)ctas * warps;
    if (total > ((size_t)1 << 30)) return fail("bulk_copy_rate: buffer would exceed 1 GB");
    unsigned char* src = nullptr;
    long long* clocks = nullptr;
    const size_t nclk = sizeof(long long) * (2 * (size_t)ctas + 1);
    CUDA_TRY(cudaMalloc(&src, total));
    if (cudaMalloc(&clocks, nclk) != cudaSuccess) { cudaFree(src); return fail("bulk_copy_rate: out of memory"); }
    cudaMemset(src, 1, total);
    cudaMemset(clocks, 0, nclk);
    int* status = (int*)(clocks + 2 * ctas);
    cudaError_t e = cudaFuncSetAttribute(k_bulk_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    for (int rep = 0; rep < 2 && e == cudaSuccess; rep++) {   // the first pass warms L2
        k_bulk_probe<<<ctas, 128, (size_t)bytes * depth * warps>>>(src, bytes, depth, warps, iters, clocks, status);
        e = cudaDeviceSynchronize();
    }
    std::vector<long long> h(2 * (size_t)ctas + 1);
    if (e == cudaSuccess) e = cudaMemcpy(h.data(), clocks, nclk, cudaMemcpyDeviceToHost);
    cudaFree(src);
    cudaFree(clocks);
    if (e != cudaSuccess) return fail("bulk_copy_rate: %s", cudaGetErrorString(e));
    if (*(int*)&h[2 * (size_t)ctas]) return fail("bulk_copy_rate: a bounded wait gave up");
    long long worst = 1, issue = 0;
    for (int i = 0; i < ctas; i++) {
        if (h[2 * i + 1] > worst) { worst = h[2 * i + 1]; issue = h[2 * i]; }
    }
    *bytes_per_clock = (double)bytes * depth * warps * iters / (double)worst;
    *issue_clocks_per_copy = (double)issue / ((double)depth * iters);
    return 0;
}

int tcbnn_mma_operand_probe(int n, int a_off16, int iters, double* clocks_per_mma) {
    if (!clocks_per_mma || n < 16 || n > 256 || n % 16 || a_off16 < 0 || a_off16 > 128 || iters < 8 || iters > (1 << 18))
        return fail("mma_operand_probe: n a multiple of 16 up to 256, offset 0..128 rows, 8..2^18 iterations");
    int sms;
    if (sm_count(&sms)) return 1;
    long long* buf = nullptr;
    CUDA_TRY(cudaMalloc(&buf, 16));
    CUDA_TRY(cudaMemset(buf, 0, 16));
    cudaError_t e = cudaFuncSetAttribute(k_umma_operand_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024);
    iters &= ~7;
    for (int rep = 0; rep < 2 && e == cudaSuccess; rep++) {
        k_umma_operand_probe<<<sms, 128, 48 * 1024>>>(n, a_off16, iters, buf, (int*)(buf + 1));
        e = cudaDeviceSynchronize();
    }
    long long host[2] = {0, 0};
    if (e == cudaSuccess) e = cudaMemcpy(host, buf, sizeof host, cudaMemcpyDeviceToHost);
    cudaFree(buf);
    if (e != cudaSuccess) return fail("mma_operand_probe: %s", cudaGetErrorString(e));
    if ((int)host[1]) return fail("mma_operand_probe: a bounded wait gave up");
    *clocks_per_mma = (double)host[0] / iters;
    return 0;
}

int tcbnn_wait_probe(int polls, int* status) {
    if (!status || polls <= 0 || polls > (1 << 24)) return fail("wait_probe: polls must be in 1..2^24");
    int* buf = nullptr;
    CUDA_TRY(cudaMalloc(&buf, 8));
    CUDA_TRY(cudaMemset(buf, 0, 8));
    k_wait_probe<<<1, 128>>>(polls, buf, buf + 1);
    if (launch_check("wait_probe")) { cudaFree(buf); return 1; }
    int host[2] = {0, 0};
    const cudaError_t e = cudaMemcpy(host, buf, sizeof host, cudaMemcpyDeviceToHost);   // synchronises
    cudaFree(buf);
    if (e != cudaSuccess) return fail("wait_probe: %s", cudaGetErrorString(e));
    if (host[0] == 1 && host[1] != polls) return fail("wait_probe: gave up after %d of %d polls", host[1], polls);
    *status = host[0];
    return 0;
}

size_t tcbnn_noalloc_scratch_bytes(void) { return kStaticScratchBytes; }

int tcbnn_fc_layer_noalloc(const uint32_t* A, const uint32_t* W, const float* thr, int M, int K,
                           int N, int lda, int ldw, uint32_t* out, int ldo, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return fail("fc_layer_noalloc: M, N, K must be positive");
    if (ldo * 32 < N) return fail("fc_layer_noalloc: ldo too small");
    int sms;
    if (sm_count(&sms)) return 1;
    const int splits = gemm_splits(M, N, K, sms);
    const size_t need = splits > 1 ? (size_t)splits * M * N * sizeof(int32_t) : 0;
    if (need > kStaticScratchBytes)
        return fail("fc_layer_noalloc: this shape needs %zu bytes of split-K scratch, the built-in "
                    "scratch holds %zu; use tcbnn_fc_layer with a caller workspace",
                    need, (size_t)kStaticScratchBytes);
    void* scratch = nullptr;
    if (static_scratch(&scratch)) return 1;
    GemmArgs g{A, W, M, N, K, lda, ldw, GEMM_FC_BITS, out, ldo, thr, nullptr, 1, nullptr};
    return run_gemm(g, scratch, kStaticScratchBytes, (cudaStream_t)stream);
}

}  // extern "C"
