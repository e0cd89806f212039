// First layer specialised to one filter: run-time compiled kernel (host side).
//
// InConv128LayerFMT (kernel.cuh:578-672) adds, per in-frame tap and output channel, the term
// ((+-f0) + (+-f1)) + (+-f2) to a running fp32 sum; the three signs are that channel's filter
// bits.  With the filter read at run time the term has to be fetched by a data-dependent index
// (inconv_tiled.cuh keeps an 8-entry table per tap in shared memory and is bound by the 128
// bytes per clock an SM can move from shared memory to registers: one 4-byte operand per add).
// A first-layer filter is fixed for the life of a model, so here the filter is compiled into
// the instruction stream: one thread owns one pixel, computes the four distinct magnitudes of
// the term in registers ((f0+f1)+-f2, (f0-f1)+-f2; the other four are their negations, which
// an add takes for free) and runs one register-to-register add per (tap, channel) whose
// operand is chosen by the generator.  No table, no shared-memory traffic: the bound becomes
// the fp32 add rate.  Operands, order of the adds and roundings are those of the reference.
//
// The source is generated below, compiled with NVRTC for sm_100a (libnvrtc is opened with
// dlopen, so the library itself does not depend on it) and loaded with cudaLibraryLoadData.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>
#include <dlfcn.h>
#include <cuda_runtime.h>

namespace tcbnn {
namespace spec {

constexpr int kSpecThreads = 256;
constexpr int kSpecMaxO = 128;

// Kernel arguments; the same struct is declared in the generated source.
struct SpecArgs {
    const float* x;            // [B][3][H][W] fp32, or null
    const unsigned char* x8;   // [B][3][H][W] uint8 with lut, when x is null
    const float* lut;          // [3][256]
    int B, H, W, OH, OW;       // OH, OW: outputs after pooling
    uint32_t* out;
    long long out_image_stride;
    void* res_out;
    int res_out_bytes, res_out_ld;
    float* acc_out;
    unsigned total;            // pre-pool pixels
    // optional: the output also as +-1 nibbles in the next layer's input planes (bconv_umma_pre.cuh)
    uint4* nxt; long long nxt_positions, nxt_front; int nxt_PW, nxt_VH;
    int res_out_chunked;      // int16 residual laid out [channel chunk of 8][pixel][8] instead of NHWC
};

// One kernel per (input type, load style), compiled when first used: a 7x7x64 kernel takes
// 1.5 - 4 s to compile and most callers only ever use one of the four.
struct SpecHandle {
    int O, R, S, sh, sw, pad_h, pad_w, pool;
    std::vector<unsigned char> codes;
    std::vector<uint32_t> thr_bits;
    std::mutex mu;
    cudaLibrary_t lib[4] = {nullptr, nullptr, nullptr, nullptr};       // index = u8 * 2 + vec
    cudaKernel_t kernel[4] = {nullptr, nullptr, nullptr, nullptr};
};

inline void emit(std::string& s, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    s += buf;
}

// codes[tap][o] = b0<<2 | b1<<1 | b2 (bit 1 = '+'), thr_bits[o] = the threshold's bit pattern
// variant = u8 * 2 + vec: which of the four kernels the source defines (entry point tcbnn_spec)
inline std::string generate_source(const SpecHandle& h, const std::vector<unsigned char>& codes,
                                   const std::vector<uint32_t>& thr_bits, int variant) {
    const bool want_u8 = (variant & 2) != 0, want_vec = (variant & 1) != 0;
    // Output channels are handled 64 at a time: blockIdx.y picks the group (its own code path).
    const int Oall = h.O, RS = h.R * h.S, OwAll = (Oall + 31) / 32, nhalf = (Oall + 63) / 64;
    std::string s;
    s.reserve(400 * 1024);
    s += "typedef unsigned int uint32_t;\n"
         "struct SpecArgs { const float* x; const unsigned char* x8; const float* lut; int B, H, W, OH, OW;\n"
         "  uint32_t* out; long long out_image_stride; void* res_out; int res_out_bytes, res_out_ld;\n"
         "  float* acc_out; unsigned total;\n"
         "  uint4* nxt; long long nxt_positions, nxt_front; int nxt_PW, nxt_VH; int res_out_chunked; };\n"
         // 32 packed bits -> 32 nibbles of +1 / -1 (e2m1), the order the conv kernels' filters use
         // (expand32_f4 in bconv_umma.cuh)
         "__device__ __forceinline__ uint32_t expand8_f4(uint32_t b) {\n"
         "  uint32_t x = b & 0xFFu; x = (x | (x << 12)) & 0x000F000Fu; x = (x | (x << 6)) & 0x03030303u;\n"
         "  x = (x | (x << 3)) & 0x11111111u; return 0xAAAAAAAAu ^ (x << 3); }\n"
         "__device__ __forceinline__ uint4 expand32_f4(uint32_t w) {\n"
         "  return make_uint4(expand8_f4(w >> 24), expand8_f4(w >> 16), expand8_f4(w >> 8), expand8_f4(w)); }\n";
    for (int half = 0; half < nhalf; half++) {
    const int OB = 64 * half, O = Oall - OB < 64 ? Oall - OB : 64;
    // VEC (stride 4 only, image rows a multiple of 4 pixels, aligned base): a thread's taps of one
    // image row are fetched with aligned 16-byte (fp32) / 4-byte (uint8) loads instead of one
    // load per tap; consecutive lanes then read consecutive 16 bytes.
    const bool vec_ok = h.sw == 4 && want_vec;
    const int OFF = (4 - h.pad_w % 4) % 4;          // x0 - OFF is a multiple of 4
    const int NQ4 = (OFF + h.S + 3) / 4;            // 4-column groups per row
    emit(s, "template <bool U8, bool VEC> __device__ __forceinline__ void body%d(const SpecArgs& c, const float* slut) {\n", half);
    emit(s, " constexpr int OBASE = %d;\n", OB);
    s += " const unsigned pix = blockIdx.x * blockDim.x + threadIdx.x;\n"
         " const bool live = pix < c.total;\n"
         " int n, y, x;\n";
    if (h.pool == 2) {
        // four consecutive indices are the four positions of one pooling window
        s += " { const unsigned pp = pix >> 2; const unsigned r = pp / (unsigned)c.OW; const int ox = (int)(pp - r * c.OW);\n"
             "   n = (int)(r / (unsigned)c.OH); const int oy = (int)(r - (unsigned)n * c.OH);\n"
             "   y = 2 * oy + ((int)(pix & 3) >> 1); x = 2 * ox + (int)(pix & 1); }\n";
    } else {
        s += " { const unsigned r = pix / (unsigned)c.OW; x = (int)(pix - r * c.OW);\n"
             "   n = (int)(r / (unsigned)c.OH); y = (int)(r - (unsigned)n * c.OH); }\n";
    }
    emit(s, " const int P = %d * c.OH, Q = %d * c.OW;\n", h.pool, h.pool);
    emit(s, " const int y0 = y * %d - %d, x0 = x * %d - %d;\n", h.sh, h.pad_h, h.sw, h.pad_w);
    s += " const size_t plane = (size_t)c.H * c.W;\n"
         " const float* img = c.x + (size_t)n * 3 * plane;\n"
         " const unsigned char* img8 = c.x8 + (size_t)n * 3 * plane;\n";
    s += " float ";
    for (int o = 0; o < O; o++) emit(s, "a%d = 0.f%s", o, o + 1 < O ? ", " : ";\n");
    for (int r = 0; r < h.R; r++) {
        s += " {\n";
        emit(s, "  float g0[%d], g1[%d], g2[%d];\n", 4 * NQ4, 4 * NQ4, 4 * NQ4);
        if (vec_ok) {
            emit(s, "  if (VEC) { const int ay = y0 + %d; const bool rok = live && (unsigned)ay < (unsigned)c.H; const int cx = x0 - %d;\n", r, OFF);
            for (int q = 0; q < NQ4; q++) {
                emit(s, "   { const bool ok = rok && cx + %d >= 0 && cx + %d < c.W; const size_t po = (size_t)ay * c.W + (cx + %d);\n",
                     4 * q, 4 * q + 3, 4 * q);
                s += "     if (U8) { unsigned b0 = 0, b1 = 0, b2 = 0;\n"
                     "       if (ok) { b0 = __ldg(reinterpret_cast<const unsigned*>(img8 + po)); b1 = __ldg(reinterpret_cast<const unsigned*>(img8 + po + plane)); b2 = __ldg(reinterpret_cast<const unsigned*>(img8 + po + 2 * plane)); }\n";
                for (int k = 0; k < 4; k++) {
                    const int gi = 4 * q + k;
                    if (gi < OFF || gi >= OFF + h.S) continue;          // column no tap uses
                    emit(s, "       g0[%d] = ok ? slut[(b0 >> %d) & 255u] : 0.f; g1[%d] = ok ? slut[256 + ((b1 >> %d) & 255u)] : 0.f; g2[%d] = ok ? slut[512 + ((b2 >> %d) & 255u)] : 0.f;\n",
                         gi, 8 * k, gi, 8 * k, gi, 8 * k);
                }
                s += "     } else { float4 t0 = make_float4(0.f, 0.f, 0.f, 0.f), t1 = t0, t2 = t0;\n"
                     "       if (ok) { t0 = __ldg(reinterpret_cast<const float4*>(img + po)); t1 = __ldg(reinterpret_cast<const float4*>(img + po + plane)); t2 = __ldg(reinterpret_cast<const float4*>(img + po + 2 * plane)); }\n";
                emit(s, "       g0[%d] = t0.x; g0[%d] = t0.y; g0[%d] = t0.z; g0[%d] = t0.w;\n", 4 * q, 4 * q + 1, 4 * q + 2, 4 * q + 3);
                emit(s, "       g1[%d] = t1.x; g1[%d] = t1.y; g1[%d] = t1.z; g1[%d] = t1.w;\n", 4 * q, 4 * q + 1, 4 * q + 2, 4 * q + 3);
                emit(s, "       g2[%d] = t2.x; g2[%d] = t2.y; g2[%d] = t2.z; g2[%d] = t2.w;\n", 4 * q, 4 * q + 1, 4 * q + 2, 4 * q + 3);
                s += "     } }\n";
            }
            s += "  }\n";
        }
        for (int sx = 0; sx < h.S; sx++) {
            const int t = r * h.S + sx;
            s += "  { float f0 = 0.f, f1 = 0.f, f2 = 0.f;\n";
            if (vec_ok) emit(s, "   if (VEC) { f0 = g0[%d]; f1 = g1[%d]; f2 = g2[%d]; } else\n", OFF + sx, OFF + sx, OFF + sx);
            emit(s, "   { const int ay = y0 + %d, ax = x0 + %d;\n", r, sx);
            s += "    if (live && (unsigned)ay < (unsigned)c.H && (unsigned)ax < (unsigned)c.W) {\n"
                 "     const size_t po = (size_t)ay * c.W + ax;\n"
                 "     if (U8) { f0 = slut[__ldg(img8 + po)]; f1 = slut[256 + __ldg(img8 + po + plane)]; f2 = slut[512 + __ldg(img8 + po + 2 * plane)]; }\n"
                 "     else { f0 = __ldg(img + po); f1 = __ldg(img + po + plane); f2 = __ldg(img + po + 2 * plane); }\n"
                 "    } }\n"
                 "   const float pp = __fadd_rn(f0, f1), pm = __fadd_rn(f0, -f1);\n"
                 "   const float v7 = __fadd_rn(pp, f2), v6 = __fadd_rn(pp, -f2), v5 = __fadd_rn(pm, f2), v4 = __fadd_rn(pm, -f2);\n";
            // The adds of one tap are independent of each other (one per channel), so their order is
            // free: they are emitted grouped by the magnitude they add, consecutive instructions then
            // share a source register and the assembler can serve it from the operand reuse cache
            // instead of the register file (fewer bank conflicts next to the accumulator reads).
            for (int mag = 4; mag < 8; mag++)
                for (int o = 0; o < O; o++) {
                    const int k = codes[(size_t)t * Oall + OB + o];
                    if ((k >= 4 ? k : 7 - k) != mag) continue;
                    if (k >= 4) emit(s, "   a%d = __fadd_rn(a%d, v%d);\n", o, o, k);
                    else emit(s, "   a%d = __fadd_rn(a%d, -v%d);\n", o, o, 7 - k);     // pattern k is minus pattern 7-k
                }
            s += "  }\n";
        }
        s += " }\n";
    }
    // threshold (kernel.cuh:655), pack, pool
    s += " uint32_t w0 = 0, w1 = 0;\n";
    for (int o = 0; o < O; o++)
        emit(s, " if (live && !(a%d < __uint_as_float(0x%08xu))) w%d |= 0x%08xu;\n", o, thr_bits[OB + o], o >> 5,
             0x80000000u >> (o & 31));
    if (h.pool == 2)
        s += " w0 |= __shfl_xor_sync(0xffffffffu, w0, 1); w0 |= __shfl_xor_sync(0xffffffffu, w0, 2);\n"
             " w1 |= __shfl_xor_sync(0xffffffffu, w1, 1); w1 |= __shfl_xor_sync(0xffffffffu, w1, 2);\n";
    s += " if (!live) return;\n";
    emit(s, " { uint32_t* dst = c.out + (size_t)n * c.out_image_stride + ((size_t)(y / %d) * c.OW + (x / %d)) * %d;\n",
         h.pool, h.pool, OwAll);
    if (h.pool == 2) s += "   if ((pix & 3) == 0)";
    emit(s, "   { dst[%d] = w0;", OB / 32);
    if (O > 32) emit(s, " dst[%d] = w1;", OB / 32 + 1);
    s += "\n";
    emit(s, "     if (c.nxt) { uint4* pl = c.nxt + c.nxt_front + ((long long)n * c.nxt_VH + (y / %d)) * c.nxt_PW + (x / %d);\n",
         h.pool, h.pool);
    for (int k = 0; k < (O + 31) / 32; k++)
        emit(s, "       pl[(size_t)%d * c.nxt_positions] = expand32_f4(w%d);\n", OB / 32 + k, k);
    s += "     }\n   } }\n";
    // residual = (int)acc (kernel.cuh:666-668), optional fp32 accumulators
    s += " const size_t opix = ((size_t)n * P + y) * Q + x;\n"
         " if (c.res_out) {\n"
         "  if (c.res_out_bytes == 2) {\n"
         "   short* r = reinterpret_cast<short*>(c.res_out) + opix * c.res_out_ld + OBASE;\n";
    if (O % 8 == 0) {
        // chunk-major layout [channel chunk of 8][pixel][8]: consecutive threads (pixels) store
        // consecutive 16 bytes, whole lines per warp
        emit(s, "   if (c.res_out_chunked) {\n    uint4* d4 = reinterpret_cast<uint4*>(c.res_out) + (size_t)%d * c.total + opix;\n", OB / 8);
        for (int j = 0; j < O / 8; j++) {
            emit(s, "    d4[(size_t)%d * c.total] = make_uint4(", j);
            for (int k = 0; k < 4; k++)
                emit(s, "((uint32_t)(int)a%d & 0xFFFFu) | ((uint32_t)(int)a%d << 16)%s", 8 * j + 2 * k, 8 * j + 2 * k + 1,
                     k < 3 ? ", " : ");\n");
        }
        s += "   } else\n";
        s += "   if ((c.res_out_ld & 7) == 0 && (reinterpret_cast<size_t>(c.res_out) & 15) == 0) {\n"
             "    uint4* d4 = reinterpret_cast<uint4*>(r);\n";
        for (int j = 0; j < O / 8; j++) {
            emit(s, "    d4[%d] = make_uint4(", j);
            for (int k = 0; k < 4; k++)
                emit(s, "((uint32_t)(int)a%d & 0xFFFFu) | ((uint32_t)(int)a%d << 16)%s", 8 * j + 2 * k, 8 * j + 2 * k + 1,
                     k < 3 ? ", " : ");\n");
        }
        s += "   } else\n";
    }
    s += "   {\n";
    for (int o = 0; o < O; o++) emit(s, "    r[%d] = (short)(int)a%d;\n", o, o);
    s += "   }\n  } else {\n   int* r = reinterpret_cast<int*>(c.res_out) + opix * c.res_out_ld + OBASE;\n";
    if (O % 4 == 0) {
        s += "   if ((c.res_out_ld & 3) == 0 && (reinterpret_cast<size_t>(c.res_out) & 15) == 0) {\n"
             "    int4* d4 = reinterpret_cast<int4*>(r);\n";
        for (int j = 0; j < O / 4; j++)
            emit(s, "    d4[%d] = make_int4((int)a%d, (int)a%d, (int)a%d, (int)a%d);\n", j, 4 * j, 4 * j + 1, 4 * j + 2, 4 * j + 3);
        s += "   } else\n";
    }
    s += "   {\n";
    for (int o = 0; o < O; o++) emit(s, "    r[%d] = (int)a%d;\n", o, o);
    s += "   }\n";
    s += "  }\n }\n if (c.acc_out) {\n";
    emit(s, "  float* q = c.acc_out + opix * %d + OBASE;\n", Oall);
    for (int o = 0; o < O; o++) emit(s, "  q[%d] = a%d;\n", o, o);
    s += " }\n}\n";
    }   // channel groups
    // two blocks per SM: at most 128 registers per thread (the sums take O of them)
    emit(s, "extern \"C\" __global__ void __launch_bounds__(%d, 2) tcbnn_spec(SpecArgs c) {\n", kSpecThreads);
    if (want_u8)
        s += " __shared__ float slut[768];\n"
             " for (int i = threadIdx.x; i < 768; i += blockDim.x) slut[i] = __ldg(c.lut + i);\n"
             " __syncthreads();\n";
    else
        s += " const float* slut = nullptr;\n";
    const bool vec_kernel = h.sw == 4 && want_vec;
    for (int half = 0; half < nhalf; half++)
        emit(s, " %sbody%d<%s, %s>(c, slut);\n", nhalf == 1 ? "" : (half == 0 ? "if (blockIdx.y == 0) " : "else "), half,
             want_u8 ? "true" : "false", vec_kernel ? "true" : "false");
    s += "}\n";
    return s;
}

// ---- NVRTC through dlopen ------------------------------------------------------------------
struct Nvrtc {
    void* so = nullptr;
    int (*createProgram)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    int (*compileProgram)(void*, int, const char* const*) = nullptr;
    int (*getCUBINSize)(void*, size_t*) = nullptr;
    int (*getCUBIN)(void*, char*) = nullptr;
    int (*getProgramLogSize)(void*, size_t*) = nullptr;
    int (*getProgramLog)(void*, char*) = nullptr;
    int (*destroyProgram)(void**) = nullptr;
    const char* (*getErrorString)(int) = nullptr;
    bool ok = false;
};

inline Nvrtc& nvrtc() {
    static Nvrtc n;
    static bool tried = false;
    if (tried) return n;
    tried = true;
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                           "/usr/local/cuda/lib64/libnvrtc.so"};
    const char* env = getenv("TCBNN_NVRTC");
    if (env) n.so = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    for (const char* nm : names) {
        if (n.so) break;
        n.so = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
    }
    if (!n.so) return n;
#define TCBNN_SYM(field, name) *(void**)(&n.field) = dlsym(n.so, name)
    TCBNN_SYM(createProgram, "nvrtcCreateProgram");
    TCBNN_SYM(compileProgram, "nvrtcCompileProgram");
    TCBNN_SYM(getCUBINSize, "nvrtcGetCUBINSize");
    TCBNN_SYM(getCUBIN, "nvrtcGetCUBIN");
    TCBNN_SYM(getProgramLogSize, "nvrtcGetProgramLogSize");
    TCBNN_SYM(getProgramLog, "nvrtcGetProgramLog");
    TCBNN_SYM(destroyProgram, "nvrtcDestroyProgram");
    TCBNN_SYM(getErrorString, "nvrtcGetErrorString");
#undef TCBNN_SYM
    n.ok = n.createProgram && n.compileProgram && n.getCUBINSize && n.getCUBIN && n.getProgramLogSize &&
           n.getProgramLog && n.destroyProgram;
    return n;
}

// Compiles `src` for sm_100a; on failure returns false with the reason in `err`.
inline bool compile_cubin(const std::string& src, std::vector<char>& cubin, std::string& err) {
    Nvrtc& n = nvrtc();
    if (!n.ok) { err = "libnvrtc could not be opened (set TCBNN_NVRTC to its path)"; return false; }
    void* prog = nullptr;
    int r = n.createProgram(&prog, src.c_str(), "tcbnn_inconv_spec.cu", 0, nullptr, nullptr);
    if (r) { err = "nvrtcCreateProgram failed"; return false; }
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo", "--fmad=false"};
    r = n.compileProgram(prog, 4, opts);
    if (r) {
        size_t ls = 0;
        n.getProgramLogSize(prog, &ls);
        std::string log(ls, '\0');
        if (ls) n.getProgramLog(prog, &log[0]);
        err = "nvrtc: " + log.substr(0, 600);
        n.destroyProgram(&prog);
        return false;
    }
    size_t cs = 0;
    n.getCUBINSize(prog, &cs);
    cubin.resize(cs);
    r = n.getCUBIN(prog, cubin.data());
    n.destroyProgram(&prog);
    if (r || !cs) { err = "nvrtcGetCUBIN failed"; return false; }
    return true;
}

}  // namespace spec
}  // namespace tcbnn
