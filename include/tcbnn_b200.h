/* C ABI of the B200 binarised-network library (libtcbnn_b200.so).
 *
 * Every entry point takes plain pointers and sizes.  Unless a name ends in _host, pointers
 * are DEVICE pointers on the current CUDA device and the work is queued on `stream`
 * (a cudaStream_t passed as void*; NULL = default stream) without synchronising.
 * Return value: 0 on success, non-zero on error (tcbnn_last_error() gives the text).
 * Nothing here falls back to the CPU: without a usable CUDA device the calls fail.
 *
 * Bit format, shared by all tensors: element e of a row sits in 32-bit word e/32 at bit
 * (31 - e%32) -- the order __brev(__ballot_sync()) produces in the reference packers
 * (param.h:60).  bit 1 = +1, bit 0 = -1, pad bits are 0.
 *   FC activations / weights : [rows][ld] words, ld a multiple of 4 (16-byte rows)
 *   conv activations         : NHWC [B][H][W][Cw] words, Cw = ceil(C/32)
 *   conv filters             : [O][R*S][Cw] words
 *   residuals / accumulators : NHWC int32 [B][P][Q][O]
 * Citations name the reference interface each entry point stands in for
 * (file:line inside pnnl/TCBNN).
 */
#ifndef TCBNN_B200_H
#define TCBNN_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int tcbnn_version(void);
const char* tcbnn_last_error(void);

/* fp32 [rows][cols] -> bit rows, bit = (x >= 0).  In128LayerFMT, kernel.cuh:153-172. */
int tcbnn_pack_rows(const float* x, int rows, int cols, int ld_words, uint32_t* out, void* stream);
/* bit rows -> +-1 fp32.  UnPackFcOutput128FMT param.h:87-104, UnpackConvOutput32FMT :661-688. */
int tcbnn_unpack_rows(const uint32_t* in, int rows, int cols, int ld_words, float* out,
                      void* stream);
/* fp32 W[K][N] -> bit rows [N][ld_words] over K.  PackFcWeight128FMT, param.h:44-63. */
int tcbnn_pack_fc_weight(const float* W, int K, int N, int ld_words, uint32_t* out, void* stream);
/* fp32 F[R*S][C][O] -> bits [O][R*S][Cw].  PackFiltersByInChannels128FMT, param.h:560-581. */
int tcbnn_pack_conv_filter(const float* F, int RS, int C, int O, uint32_t* out, void* stream);
/* fp32 F[R*S][3][O] -> [R*S][3][Ow] words over O.  PackFiltersByOutChannels32, param.h:613-632. */
int tcbnn_pack_inconv_filter(const float* F, int RS, int O, uint32_t* out, void* stream);

/* Scratch a GEMM-family call can use: partial sums to split K when M x N alone leaves SMs idle
 * and, for large problems (M >= 128, N >= 64, 512 <= K < 2^22, M*N*K >= 2^30), both operands
 * written out as +-1 4-bit values for the tcgen05 kernel (csrc/bgemm_umma.cuh), which is then used.
 * Passing NULL / 0 is always allowed (warp-level b1 MMA kernel, no split); the buffer must be
 * 256-byte aligned for the tcgen05 kernel to be taken. */
size_t tcbnn_gemm_workspace_bytes(int M, int N, int K);
/* Which kernel the GEMM family uses: 0 = automatic, 1 = always the warp-level b1 MMA kernel.
 * Process-wide; for tests and measurements.  tcbnn_gemm_status reads the tcgen05 GEMM kernel's
 * device-side status word (synchronises): 0 = fine, 1 = a bounded wait inside it gave up and the
 * results since the last reading are not valid; reading a non-zero status clears it.  No reference
 * counterparts. */
int tcbnn_set_gemm_path(int path);
int tcbnn_gemm_status(int* status);
/* Overrides what the tcgen05 GEMM derives from its cost model: `pair` 1 = CTAs own 256 x 128
 * tiles, 0 = 128 x 128, -1 = automatic; `splits` 1..32 = that many slices of K (1: the GEMM's own
 * epilogue finishes the layer; more: int32 partial sums and a finishing pass), -1 = automatic.
 * A forced plan also waives the M*N*K >= 2^30 rule.  A workspace sized by
 * tcbnn_gemm_workspace_bytes AFTER this call fits the forced plan.
 * Process-wide; for tests and measurements.  No reference counterpart. */
int tcbnn_set_gemm_plan(int pair, int splits);
/* How many kernels a GEMM-family call of this shape launches when given a workspace of that size
 * (warp-level kernel: 1, or 2 with split K; tcgen05 path: 2 = operand expansion and a GEMM that
 * finishes the layer, 3 with split K); for callers that account for their launches. */
int tcbnn_gemm_launches(int M, int N, int K, size_t workspace_bytes);

/* GEMM family (the next three entry points): the pad bits of every row of A and of B / W -- the
 * bits past element K up to the leading dimension -- must be zero, as tcbnn_pack_rows,
 * tcbnn_pack_fc_weight and the layer outputs leave them.  (The warp-level kernel counts whole
 * 64-bit words and relies on equal pads cancelling; the tcgen05 kernel masks them; which one runs
 * depends on shape and workspace, so non-zero pads give shape-dependent results.)
 * C[m][n] = K - 2*popc(A[m] xor B[n]), int32 [M][ldc].
 * BMMA / BMMAS_new, bmm/tensorcore_kernel.cu:138-356 (C = K - 2*acc at :331). */
int tcbnn_bgemm(const uint32_t* A, const uint32_t* B, int M, int N, int K, int lda, int ldb,
                int32_t* C, int ldc, void* workspace, size_t workspace_bytes, void* stream);
/* Hidden FC layer: bit[m][n] = ((float)K - 2*(float)popc >= thr[n]).
 * Fc128LayerFMT, kernel.cuh:174-226.  out: bit rows [M][ldo]; words past N/32 untouched. */
int tcbnn_fc_layer(const uint32_t* A, const uint32_t* W, const float* thr, int M, int K, int N,
                   int lda, int ldw, uint32_t* out, int ldo, void* workspace,
                   size_t workspace_bytes, void* stream);
/* Output layer: out[m][n] = fma((float)(K - 2*popc), scale[n], bias[n]), fp32 [M][ldo].
 * Out128LayerFMT, kernel.cuh:230-280. */
int tcbnn_out_layer(const uint32_t* A, const uint32_t* W, const float* scale, const float* bias,
                    int M, int K, int N, int lda, int ldw, float* out, int ldo, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Geometry of a conv layer.  Fill the input fields, call tcbnn_conv_shape() for the rest. */
typedef struct tcbnn_conv_desc {
    int B, H, W, C, O, R, S;
    int stride_h, stride_w;
    int padding;            /* 1: "same"-style padding with the reference's arithmetic */
    int pool;               /* 1 or 2 (non-overlapping pool x pool OR-pooling) */
    /* derived */
    int pad_h, pad_w, OH, OW;
} tcbnn_conv_desc;
/* pad / output-size arithmetic of InConv128LayerParam and Conv128LayerParam
 * (param.h:719-728, 897-906).  Host-only, no device needed. */
int tcbnn_conv_shape(tcbnn_conv_desc* d);

/* Bytes of the prepared-filter blob for a binary conv layer, and its construction from
 * filter bits [O][R*S][Cw] (tcbnn_pack_conv_filter output).  The blob is opaque device
 * memory owned by the caller; preparation happens once per layer, like the filter packing
 * in Conv128LayerParam::initialize (param.h:944-985). */
size_t tcbnn_conv_prepared_bytes(const tcbnn_conv_desc* d);
int tcbnn_conv_prepare(const tcbnn_conv_desc* d, const uint32_t* filter_bits, void* prepared,
                       void* stream);

/* Element formats of residual tensors: the res_in_bytes / res_out_bytes arguments below.
 * TCBNN_RES_INT16_CHUNKED is int16 laid out by 8-channel chunk, [ceil(ch/8)][pixels][8] with
 * pixels = B*P*Q of that tensor (element (pixel p, channel c) at ((c/8)*pixels + p)*8 + c%8): one
 * thread per pixel then reads and writes whole lines across a warp, which the residual layers with
 * narrow channel counts are bound by.  It is read and written only by the loader-fed tcgen05
 * kernel (layers with tcbnn_conv_planes_bytes != 0 called with their workspace, pool == 1, channel
 * counts in multiples of 8; other calls fail) and written by tcbnn_inconv_specialized_layer;
 * tcbnn_conv_prefers_chunked_residual says for which layers it is the faster choice (every layer
 * the loader-fed kernel takes: its tile-per-group epilogue handles no other residual layout, and
 * it reads a pooled chunk-major residual in place, without the pooling pass NHWC tensors get).
 * TCBNN_RES_PROVEN, ORed into the res_out_bytes of an int16 format, says that the caller has
 * proven the bound |value| <= 32767 (e.g. C*R*S + the bound of res_in, the way the drop-in classes
 * choose int16): the layer then skips the per-value range check that sets status 2, which costs
 * the residual layers' epilogues about a fifth of their instructions. */
#define TCBNN_RES_INT32 4
#define TCBNN_RES_INT16 2
#define TCBNN_RES_INT16_CHUNKED 18
#define TCBNN_RES_PROVEN 32
int tcbnn_conv_prefers_chunked_residual(const tcbnn_conv_desc* d);

/* Binary conv layer with threshold / OR-pool / residual / repack fused.
 * Conv128LayerFMT, kernel.cuh:676-827.
 *   in   [B][H][W][Cw]; out: image b at out + b*out_image_stride words, [OH][OW][Ow]
 *        (out_image_stride > OH*OW*Ow lets the next FC layer see padded rows: ahead_fc)
 *   res_in  (optional) [B][P or 2P][Q or 2Q][res_in_ch], int32 or int16 elements
 *           (res_in_bytes = 4 or 2, or TCBNN_RES_INT16_CHUNKED for the chunk-major layout);
 *           injected for o < residual_channels; residual_pool takes the max over the 2x2 window
 *   res_out (optional) [B][P][Q][O], int32 or int16 (res_out_bytes): value after injection
 *           (save_residual).  int16 halves the dominant HBM traffic of the residual layers;
 *           the caller picks it when the running sum is known to fit (|value| <= C*R*S +
 *           bound of res_in); a value that does not fit sets status 2 (tcbnn_conv_status).
 *   acc_out (optional) int32 [B][P][Q][O]: value before injection (for checking)       */
int tcbnn_conv_layer(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                     const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                     int residual_channels, int residual_pool, uint32_t* out,
                     long long out_image_stride, void* res_out, int res_out_bytes,
                     int32_t* acc_out, void* stream);

/* tcbnn_conv_layer with a scratch buffer.  Narrow stride-1 layers (at most 128 input channels)
 * run fastest when their input is first written out as +-1 bytes in the tensor cores' operand
 * layout by a streaming pass and the convolution kernel fetches it with bulk copies;
 * tcbnn_conv_workspace_bytes says how much device memory (256-byte aligned) that takes for a
 * descriptor, 0 when the layer has no use for it.  (Wide layers use the buffer for something
 * else: a pooled int16 residual is first reduced into it by a streaming pass.
 * tcbnn_conv_planes_bytes is the part that is the pre-expanded input: the size of the planes of
 * tcbnn_conv_layer_x, 0 for layers that take none.)  The buffer is only used during the call
 * (stream order); one buffer of the largest size serves all layers of a network on one stream.
 * With workspace == NULL this is tcbnn_conv_layer.  No reference counterpart. */
size_t tcbnn_conv_workspace_bytes(const tcbnn_conv_desc* d);
size_t tcbnn_conv_planes_bytes(const tcbnn_conv_desc* d);
int tcbnn_conv_layer_w(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                       const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                       int residual_channels, int residual_pool, uint32_t* out,
                       long long out_image_stride, void* res_out, int res_out_bytes,
                       int32_t* acc_out, void* workspace, size_t workspace_bytes, void* stream);

/* tcbnn_conv_layer_w plus the two halves of a producer -> consumer hand-over of the pre-expanded
 * input, which saves the consumer's expansion pass:
 *  - next / next_planes / next_planes_bytes (all NULL / 0 for none): `next` is the descriptor of
 *    the layer that consumes this layer's output (same batch, its H x W x C = this layer's
 *    OH x OW x O, and tcbnn_conv_planes_bytes(next) != 0); besides the packed bits the layer
 *    then also writes its output as +-1 bytes into next_planes in that layer's operand layout.
 *    The buffer (tcbnn_conv_planes_bytes(next) bytes, 256-byte aligned) must have been zeroed
 *    once and be used for this pair of layers only: the padding positions of the layout are never
 *    written.  out_image_stride must be dense.  Kernels that cannot write the planes themselves
 *    are followed by the expansion pass, so the result is the same for every layer.
 *  - workspace_ready != 0: `workspace` already holds this layer's input planes (its producer was
 *    called with next = this layer); the expansion pass is skipped.
 * No reference counterpart. */
int tcbnn_conv_layer_x(const tcbnn_conv_desc* d, const uint32_t* in, const void* prepared,
                       const float* thr, const void* res_in, int res_in_bytes, int res_in_ch,
                       int residual_channels, int residual_pool, uint32_t* out,
                       long long out_image_stride, void* res_out, int res_out_bytes,
                       int32_t* acc_out, void* workspace, size_t workspace_bytes, int workspace_ready,
                       const tcbnn_conv_desc* next, void* next_planes, size_t next_planes_bytes,
                       void* stream);

/* Which kernel tcbnn_conv_layer uses: 0 = automatic (tcgen05 int8 implicit GEMM where the layer
 * is eligible, else the warp-level b1 MMA), 1 = always the b1 MMA, 2 = tcgen05 or an error,
 * 3 = as 2 but only the filter-stationary tcgen05 kernel with its in-kernel bit expansion (wide
 * stride-1 layers otherwise take the activation-stationary kernel, narrow ones with a workspace the
 * kernel fed from a pre-expanded input), 4 = as 0 but the loader-fed kernel moves int16 residual
 * rows straight between registers and global memory, never staging them in shared memory, 5 = as 0
 * but staging them wherever the tensors allow (0 stages them where that measured faster), 6 = as
 * 0 but the loader-fed kernel always runs one CTA per SM (0 runs layers with an n-tile of 64 as
 * two smaller CTAs per SM when they fit), 7 = as 0 but without the loader-fed kernel's
 * tile-per-group epilogues (0 uses them for layers without residuals and for chunk-major int16
 * residuals), 8 = as 0 but two CTAs per SM also for the all-warps-per-tile residual epilogues at an
 * n-tile of 64, 9 = as 0 but the loader-fed kernel's stages hold one 64-channel block each (0
 * puts four or two in a stage where three such stages fit), 10 = as 0 but every n-tile of a layer
 * gets the same number of CTAs (0 gives the n-tiles that carry a pooled residual more).
 * Process-wide; meant for tests and measurements.  No reference counterpart (the reference has one
 * kernel per layer type). */
int tcbnn_set_conv_path(int path);
/* Tracing aid (the reference's counterpart is its in-kernel clock64 timer, utility.h:179-183):
 * while `device_buffer` (at least 16 int64, device memory) is set, CTA 0 of every tcgen05 conv
 * launch writes cycle counters: [0] expander total, [1] expander waiting for a free stage,
 * [2] stages, [3] MMA issuer total, [4] waiting for a free accumulator, [5] waiting for a full
 * stage, [6] epilogue total, [7] waiting for a full accumulator, [8] tiles; CTA 0 of every
 * tcgen05 GEMM launch writes [9] the CTA from entry to exit, [10] loader waiting for a free stage,
 * [11] MMA issuer total, [12] waiting for a full stage, [13] epilogue waiting for the accumulator,
 * [14] k-blocks, [15] epilogue after the accumulator arrived.
 * NULL turns it off. */
int tcbnn_conv_set_trace(void* device_buffer);
/* Reads the layer's device-side status word (synchronises): 0 = fine, 1 = a bounded wait inside
 * the tcgen05 kernel gave up and the layer's output is not valid, 2 = a residual value did not
 * fit the int16 element size the caller chose.  The word collects failures of every call since
 * tcbnn_conv_prepare or the last reading; reading a non-zero status clears it. */
int tcbnn_conv_status(const tcbnn_conv_desc* d, const void* prepared, int* status);

/* First layer on fp32 NCHW input [B][3][H][W] (d->C must be 3).
 * InConv128LayerFMT, kernel.cuh:578-672.  filter_bits from tcbnn_pack_inconv_filter.
 * res_out: (int)acc, truncated toward zero, stored as int32 or int16 (res_out_bytes = 4 or 2;
 * int16 only when the caller knows R*S*3*max|x| < 32768); acc_out (optional): fp32 sums. */
int tcbnn_inconv_layer(const tcbnn_conv_desc* d, const float* x, const uint32_t* filter_bits,
                       const float* thr, uint32_t* out, long long out_image_stride,
                       void* res_out, int res_out_bytes, float* acc_out, void* stream);

/* No counterpart in the reference.  Same result as tcbnn_fc_layer, for callers that must not
 * allocate device memory around the call: a process whose own arena already holds all of the
 * GPU's memory (so a cudaMalloc for a workspace would fail or fragment it), or a serving loop
 * that cannot afford the device-wide synchronisation an allocation implies.  The scratch the
 * layer needs (the split-K partial sums; for large problems, when they fit, the +-1 byte copies of
 * both operands that the tcgen05 kernel reads, as with a caller workspace) goes to a fixed array
 * inside the library (tcbnn_noalloc_scratch_bytes() bytes, 8 MiB; resident on every GPU that
 * loads the library until the process exits) instead of a caller workspace.  The call itself
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *   - The array is part of the library's device code: the CUDA runtime places it on a device
 *     when the library's code is first used there.  A caller whose arena takes all of the GPU's
 *     memory must make one call into the library on that device (any entry point that launches,
 *     or this one) BEFORE the arena is created, or the 8 MiB will not be there to place.
 *   - Shapes whose split-K partials (splits * M * N * 4 bytes) exceed the array are rejected
 *     with an error.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents.  Nothing in
 *     it needs to start at zero (every partial a call reads was stored by that same call),
 *     but two calls that overlap on the GPU (different streams, or different host threads
 *     without ordering) race on it: order them on one stream or with events. */
size_t tcbnn_noalloc_scratch_bytes(void);
int tcbnn_fc_layer_noalloc(const uint32_t* A, const uint32_t* W, const float* thr, int M, int K,
                           int N, int lda, int ldw, uint32_t* out, int ldo, void* stream);

/* The same first layer fed with the images as bytes: x is uint8 NCHW [B][3][H][W] and lut[c][v]
 * (fp32 [3][256]) is the value the caller's reader would have produced for byte v of channel c
 * -- e.g. (v/255.0f)*4.3668f-2.1179f for the reference's ImageNet reader (data.cpp:534-542).
 * The kernel replaces every byte by its table entry and then runs exactly the arithmetic of
 * tcbnn_inconv_layer, so results are identical to feeding the fp32 images; the host->device copy
 * is a quarter of the size.  The reference normalises on the host (data.cpp) and has no such
 * entry point. */
int tcbnn_inconv_layer_u8(const tcbnn_conv_desc* d, const uint8_t* x, const float* lut,
                          const uint32_t* filter_bits, const float* thr, uint32_t* out,
                          long long out_image_stride, void* res_out, int res_out_bytes,
                          float* acc_out, void* stream);

/* First layer compiled for one filter.  No reference counterpart: InConv128LayerFMT
 * (kernel.cuh:578-672) reads the filter bits at run time, as tcbnn_inconv_layer does.  A model's
 * first-layer filter and thresholds never change, so tcbnn_inconv_specialize reads them back
 * (filter_bits and thr are device pointers, laid out as for tcbnn_inconv_layer; synchronises the
 * stream) and keeps them; the layer calls then run a generated kernel whose instruction stream
 * contains the filter -- one register-to-register fp32 add per (tap, output channel), same
 * operands, order and roundings as the reference -- compiled with NVRTC (libnvrtc.so.12 is looked
 * up with dlopen; the environment variable TCBNN_NVRTC may name it).  There are four variants
 * (fp32 or uint8 images; aligned row loads for stride 4 and rows of a multiple of 4 pixels, or one
 * load per tap); each is compiled and loaded by the first call that needs it (1-4 s), so run one
 * call before timing or capturing a graph.  d->O <= 128 (64 channels per thread; a second
 * group of threads takes channels 64 and up).  The kernel does not
 * depend on d->B, d->H or d->W.  tcbnn_inconv_specialized_layer then runs the layer on fp32 images
 * (x, x8 = lut = NULL) or on uint8 images with their value table (x = NULL), with the outputs of
 * tcbnn_inconv_layer; d must agree with the descriptor used to specialise in everything but
 * B, H, W.  tcbnn_inconv_release unloads the kernel. */
int tcbnn_inconv_specialize(const tcbnn_conv_desc* d, const uint32_t* filter_bits, const float* thr,
                            void* stream, void** handle);
int tcbnn_inconv_specialized_layer(void* handle, const tcbnn_conv_desc* d, const float* x,
                                   const uint8_t* x8, const float* lut, uint32_t* out,
                                   long long out_image_stride, void* res_out, int res_out_bytes,
                                   float* acc_out, void* stream);
/* The same with the hand-over to the next layer of tcbnn_conv_layer_x. */
int tcbnn_inconv_specialized_layer_x(void* handle, const tcbnn_conv_desc* d, const float* x,
                                     const uint8_t* x8, const float* lut, uint32_t* out,
                                     long long out_image_stride, void* res_out, int res_out_bytes,
                                     float* acc_out, const tcbnn_conv_desc* next, void* next_planes,
                                     size_t next_planes_bytes, void* stream);
int tcbnn_inconv_release(void* handle);
/* Generates the kernel above for pseudo-random filter bits and compiles it, without loading it:
 * needs NVRTC but no GPU.  *source_bytes (optional) receives the size of the generated source. */
int tcbnn_inconv_specialize_selftest(const tcbnn_conv_desc* d, unsigned seed, long long* source_bytes);

/* Issue-rate probe of the MMA forms on all SMs: kind 0 = b1 and.popc m16n8k256 (mma.sync),
 * 1 = b1 xor.popc m16n8k256, 2 = s8 m16n8k32, 3 = tcgen05.mma kind::i8 128x256x32 (warps_per_sm
 * ignored).  Kinds 4-6 measure what the issuing thread's bookkeeping costs a tcgen05 stream of
 * 128x128x32 MMAs issued in groups of warps_per_sm: 4 = nothing between the groups, 5 = a lone
 * lane doing mbarrier.try_wait + tcgen05.commit per group, 6 = the converged warp doing
 * mbarrier.test_wait and the elect.sync lane issuing and committing.  Kind 7 = tcgen05.mma
 * kind::mxf4 128x256x64 (e2m1 operands +-1.0, unit ue8m0 block scales, fp32 accumulators), with the
 * accumulators checked against the exact sum; at most 2^18 iterations.  Returns tera-ops/s
 * (2*m*n*k per MMA) in *tops.
 * Synchronises the device.  The reference's counterpart is the WMMA latency probe
 * bmm/bmma_op_test/main_test.cu:35-220 and its TOPS formula at :368. */
int tcbnn_mma_peak(int kind, int warps_per_sm, int iters, double* tops);

/* Failure-handling probe.  Every wait inside the tcgen05 kernels is bounded: a role that waits
 * for a partner which never arrives gives up after a fixed number of polls, records status 1
 * (tcbnn_conv_status / tcbnn_gemm_status), the kernel drains, frees its tensor memory and returns.
 * This call runs that path in isolation: one CTA allocates tensor memory, waits `polls` times on an
 * mbarrier nobody arrives at, gives up, records *status = 1, frees its tensor memory and returns.
 * Synchronises.  The device context stays usable (the next call works as usual).  The reference has
 * no counterpart: its error handling is exit() on a failed CUDA call (utility.h:57-101). */
int tcbnn_wait_probe(int polls, int* status);
/* Measurement aid: clocks per tcgen05.mma kind::mxf4 of 128 x n x 64 (operands resident in shared
 * memory, K-major without swizzle, issued back to back on every SM) when the A operand's
 * descriptor starts `a_off16` 16-byte rows into its buffer -- the conv kernels address a filter
 * tap by such an offset.  No reference counterpart. */
int tcbnn_mma_operand_probe(int n, int a_off16, int iters, double* clocks_per_mma);
/* Measurement aid: `ctas` CTAs (one per SM up to the SM count) each run `iters` rounds in which
 * one thread of each of `warps` warps issues `depth` bulk copies (cp.async.bulk, global -> shared,
 * completion on an mbarrier) of `bytes` back to back over an L2-resident buffer and then waits for
 * them.  Returns, for the slowest CTA, the clocks an issuing thread spent per copy and the bytes
 * per SM clock over issue + wait -- what the loaders of the tcgen05 kernels can be fed with.
 * Allocates and frees its buffer; every wait is bounded.  No reference counterpart. */
int tcbnn_bulk_copy_rate(int bytes, int depth, int warps, int ctas, int iters, double* issue_clocks_per_copy,
                         double* bytes_per_clock);

#ifdef __cplusplus
}
#endif
#endif
