// C++ host side of the fast path: the reference's five layer-parameter classes (param.h:115-1065)
// -- same names, constructor arguments, initialize() / get_output_gpu() /
// get_output_residual_gpu() / download_output() / download_full_output() -- on top of the C ABI
// of libtcbnn_b200.so (include/tcbnn_b200.h).  Where the reference's objects are handed to the
// driver's cooperative kernel, these have a forward(stream) that queues the library's kernels
// (tcgen05 convolutions and GEMM, the first layer compiled for its filter), so a driver replaces
//
//     cudaLaunchCooperativeKernel(resnet128, ...)        by        for (layer : net) layer->forward(stream);
//
// Host-only C++14: needs cuda_runtime.h and the library, no nvcc.  Errors follow the reference's
// convention (utility.h:57-92): message on stderr, exit(-1).
//
// Differences from the reference a caller sees: packed layouts are the library's (NHWC words;
// the unpacked +-1 values, residuals and logits are the reference's); layers store their outputs,
// so the same objects run any number of passes; weights come from a text file in launch_array
// order (initialize(FILE*, ...), the reference's own signatures, so that a driver's layer lines
// stay as they are), a raw fp32 file or a host array (Weights); the batch given to a constructor
// is the largest the object will see and set_batch(n) makes the following passes process the first
// n images in the same buffers.
#ifndef TCBNN_HOST_HPP
#define TCBNN_HOST_HPP

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>
#include <cuda_runtime.h>
#include "tcbnn_b200.h"

namespace tcbnn_host {

typedef unsigned int uin32;

#define TCBNN_HOST_CUDA(call)                                                                      \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            fprintf(stderr, "cudaSafeCall() failed at %s:%i : %s\n", __FILE__, __LINE__,           \
                    cudaGetErrorString(e_));                                                       \
            exit(-1);                                                                              \
        }                                                                                          \
    } while (0)
#define TCBNN_HOST_CALL(call)                                                                      \
    do {                                                                                           \
        if ((call) != 0) {                                                                         \
            fprintf(stderr, "%s failed at %s:%i : %s\n", #call, __FILE__, __LINE__,                \
                    tcbnn_last_error());                                                           \
            exit(-1);                                                                              \
        }                                                                                          \
    } while (0)

inline int step128_words(long long k) { return (int)(((k + 127) / 128) * 4); }   // STEP128(k) * 4, utility.h:38

template <class T>
inline T* dev_alloc(size_t count, bool zero = true) {
    T* p = NULL;
    TCBNN_HOST_CUDA(cudaMalloc((void**)&p, (count ? count : 1) * sizeof(T)));
    if (zero) TCBNN_HOST_CUDA(cudaMemset(p, 0, (count ? count : 1) * sizeof(T)));
    return p;
}

// set_residual_bytes takes a residual format of the C header: 4 (int32, the reference's), 2 (int16)
// or TCBNN_RES_INT16_CHUNKED (int16 by 8-channel chunk, the layout the tcgen05 conv kernel's
// epilogue is fastest on; every layer that injects the tensor must then run that kernel, i.e. have
// its workspace, or its call fails).  Anything else means int32.
inline int residual_code(int code) { return (code == 2 || code == TCBNN_RES_INT16_CHUNKED) ? code : 4; }
inline int residual_elem_bytes(int code) { return code == 4 ? 4 : 2; }

// What a layer that saves its residual tells the layers that inject it: the reference hands over
// a bare int* (param.h:944), so channel count and element size travel through this table.
struct ResidualInfo { const void* ptr; int channels; int bytes; };
inline std::vector<ResidualInfo>& residual_table() { static std::vector<ResidualInfo> t; return t; }
inline std::mutex& residual_mutex() { static std::mutex m; return m; }
inline void publish_residual(const void* ptr, int channels, int bytes) {
    std::lock_guard<std::mutex> lock(residual_mutex());
    ResidualInfo r = {ptr, channels, bytes};
    residual_table().push_back(r);
}
inline void retract_residual(const void* ptr) {
    std::lock_guard<std::mutex> lock(residual_mutex());
    std::vector<ResidualInfo>& t = residual_table();
    for (size_t i = 0; i < t.size(); i++)
        if (t[i].ptr == ptr) { t.erase(t.begin() + i); return; }
}
inline bool lookup_residual(const void* ptr, int* channels, int* bytes) {
    std::lock_guard<std::mutex> lock(residual_mutex());
    const std::vector<ResidualInfo>& t = residual_table();
    for (size_t i = t.size(); i-- > 0;)
        if (t[i].ptr == ptr) { *channels = t[i].channels; *bytes = t[i].bytes; return true; }
    return false;
}

// Where initialize() takes its numbers from: the reference's text file (launch_array,
// utility.h:188-196), a raw fp32 file, or a host array -- same values, same order.
struct Weights {
    FILE* text;
    FILE* binary;
    const float* memory;
    size_t left;
    static Weights from_text(FILE* f) {
        if (!f) { fprintf(stderr, "NULL pointer to the network configuration file.\n"); exit(1); }
        Weights w = {f, NULL, NULL, 0};
        return w;
    }
    static Weights from_binary(FILE* f) {
        if (!f) { fprintf(stderr, "NULL pointer to the network configuration file.\n"); exit(1); }
        Weights w = {NULL, f, NULL, 0};
        return w;
    }
    static Weights from_memory(const float* p, size_t count) {
        if (!p) { fprintf(stderr, "NULL pointer to the network weights.\n"); exit(1); }
        Weights w = {NULL, NULL, p, count};
        return w;
    }
    void read(float* dst, size_t n) {
        size_t got = 0;
        if (binary) {
            got = fread(dst, sizeof(float), n, binary);
        } else if (memory) {
            got = left < n ? left : n;
            memcpy(dst, memory, got * sizeof(float));
            memory += got;
            left -= got;
        } else {
            for (; got < n; got++)
                if (fscanf(text, "%f", &dst[got]) != 1) break;
        }
        if (got != n) { fprintf(stderr, "network weights ended after %zu of %zu values.\n", got, n); exit(1); }
    }
    // n floats from the source in a fresh device buffer
    float* upload(size_t n) {
        std::vector<float> h(n);
        read(h.data(), n);
        float* d = dev_alloc<float>(n, false);
        TCBNN_HOST_CUDA(cudaMemcpy(d, h.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        return d;
    }
};

// Scratch memory the GEMM and conv entry points may use during a call (stream order): one buffer
// of the largest size serves every layer of a network that runs on one stream.
struct Workspace {
    void* ptr;
    size_t bytes;
    Workspace() : ptr(NULL), bytes(0) {}
    void reserve(size_t n) {
        if (n <= bytes) return;
        if (ptr) TCBNN_HOST_CUDA(cudaFree(ptr));
        TCBNN_HOST_CUDA(cudaMalloc(&ptr, n));
        TCBNN_HOST_CUDA(cudaMemset(ptr, 0, n));
        bytes = n;
    }
    ~Workspace() { if (ptr) cudaFree(ptr); }
};

// +-1 floats of bit rows [rows][ld_words] in a fresh pinned host buffer (the reference's
// download_full_output(), param.h:176-199)
inline float* unpack_to_host(const uin32* bits, int images, long long image_stride_words, int rows_per_image,
                             int cols, int ld_words) {
    const size_t per = (size_t)rows_per_image * cols;
    float* dev = dev_alloc<float>(per * images, false);
    for (int b = 0; b < images; b++)
        TCBNN_HOST_CALL(tcbnn_unpack_rows(bits + (size_t)b * image_stride_words, rows_per_image, cols, ld_words,
                                          dev + (size_t)b * per, NULL));
    float* host = NULL;
    TCBNN_HOST_CUDA(cudaMallocHost((void**)&host, per * images * sizeof(float)));
    TCBNN_HOST_CUDA(cudaMemcpy(host, dev, per * images * sizeof(float), cudaMemcpyDeviceToHost));
    TCBNN_HOST_CUDA(cudaFree(dev));
    return host;
}

// ---- input layer (param.h:115-222, In128LayerFMT kernel.cuh:153-172) ---------------------------
class In128LayerParam {
public:
    In128LayerParam(const char* _name, int _input_height, int _input_width)
        : input_height(_input_height), input_width(_input_width), output_height(_input_height),
          output_width(_input_width), input_gpu(NULL), output_gpu(NULL), live(_input_height) {
        strncpy(name, _name, 7); name[7] = 0;
    }
    // the following passes process the first n rows (n <= the constructor's input_height)
    void set_batch(int n) {
        if (n <= 0 || n > input_height) { fprintf(stderr, "%s: batch %d outside 1..%d.\n", name, n, input_height); exit(-1); }
        live = n;
    }
    void set_input(const float* input, int rows) {
        TCBNN_HOST_CUDA(cudaMemcpy(input_gpu, input, (size_t)rows * input_width * sizeof(float), cudaMemcpyHostToDevice));
    }
    int ld() const { return step128_words(output_width); }
    size_t output_size() const { return (size_t)output_height * output_width; }
    In128LayerParam* initialize(const float* input) {
        if (!input) { fprintf(stderr, "NULL pointer.\n"); exit(-1); }
        input_gpu = dev_alloc<float>(output_size(), false);
        TCBNN_HOST_CUDA(cudaMemcpy(input_gpu, input, output_size() * sizeof(float), cudaMemcpyHostToDevice));
        output_gpu = dev_alloc<uin32>((size_t)output_height * ld());
        return this;
    }
    void forward(cudaStream_t stream = 0) {
        TCBNN_HOST_CALL(tcbnn_pack_rows(input_gpu, live, input_width, ld(), output_gpu, stream));
    }
    float* get_input_gpu() { return input_gpu; }
    uin32* get_output_gpu() { return output_gpu; }
    float* download_full_output() { return unpack_to_host(output_gpu, 1, 0, live, output_width, ld()); }
    ~In128LayerParam() { cudaFree(input_gpu); cudaFree(output_gpu); }
    int input_height, input_width, output_height, output_width;
    float* input_gpu;
    uin32* output_gpu;
    int live;
    char name[8];
};

// ---- hidden FC layer (param.h:224-385, Fc128LayerFMT kernel.cuh:174-226) -----------------------
class Fc128LayerParam {
public:
    Fc128LayerParam(const char* _name, int _input_height, int _input_width, int _weight_width)
        : input_height(_input_height), input_width(_input_width), weight_height(_input_width),
          weight_width(_weight_width), output_height(_input_height), output_width(_weight_width),
          weight_gpu(NULL), bn_gpu(NULL), input_gpu(NULL), output_gpu(NULL), workspace(NULL), live(_input_height) {
        strncpy(name, _name, 7); name[7] = 0;
    }
    int ld() const { return step128_words(output_width); }
    int ldw() const { return step128_words(weight_height); }
    size_t output_size() const { return (size_t)output_height * output_width; }
    size_t workspace_bytes() const { return tcbnn_gemm_workspace_bytes(input_height, weight_width, input_width); }
    void set_batch(int n) {
        if (n <= 0 || n > input_height) { fprintf(stderr, "%s: batch %d outside 1..%d.\n", name, n, input_height); exit(-1); }
        live = n;
    }
    // the reference's signature (param.h:270): weights from its text file
    Fc128LayerParam* initialize(FILE* config_file, uin32* prev_layer_gpu) {
        Weights w = Weights::from_text(config_file);
        return initialize(w, prev_layer_gpu);
    }
    Fc128LayerParam* initialize(Weights& config, uin32* prev_layer_gpu) {
        float* w = config.upload((size_t)weight_height * weight_width);          // [K][N]
        weight_gpu = dev_alloc<uin32>((size_t)weight_width * ldw());
        TCBNN_HOST_CALL(tcbnn_pack_fc_weight(w, weight_height, weight_width, ldw(), weight_gpu, NULL));
        TCBNN_HOST_CUDA(cudaDeviceSynchronize());
        TCBNN_HOST_CUDA(cudaFree(w));
        bn_gpu = config.upload(weight_width);
        output_gpu = dev_alloc<uin32>((size_t)output_height * ld());
        input_gpu = prev_layer_gpu;
        return this;
    }
    void set_workspace(Workspace* w) { workspace = w; }
    void forward(cudaStream_t stream = 0) {
        TCBNN_HOST_CALL(tcbnn_fc_layer(input_gpu, weight_gpu, bn_gpu, live, input_width, weight_width,
                                       step128_words(input_width), ldw(), output_gpu, ld(),
                                       workspace ? workspace->ptr : NULL, workspace ? workspace->bytes : 0, stream));
    }
    uin32* get_output_gpu() { return output_gpu; }
    float* download_full_output() { return unpack_to_host(output_gpu, 1, 0, live, output_width, ld()); }
    ~Fc128LayerParam() { cudaFree(weight_gpu); cudaFree(bn_gpu); cudaFree(output_gpu); }
    int input_height, input_width, weight_height, weight_width, output_height, output_width;
    uin32* weight_gpu; float* bn_gpu; uin32* input_gpu; uin32* output_gpu;
    Workspace* workspace;
    int live;
    char name[8];
};

// ---- output layer (param.h:388-531, Out128LayerFMT kernel.cuh:230-280) -------------------------
class Out128LayerParam {
public:
    Out128LayerParam(const char* _name, int _input_height, int _input_width, int _weight_width)
        : input_height(_input_height), input_width(_input_width), weight_height(_input_width),
          weight_width(_weight_width), output_height(_input_height), output_width(_weight_width),
          weight_gpu(NULL), bn_scale_gpu(NULL), bn_bias_gpu(NULL), input_gpu(NULL), output_gpu(NULL),
          output(NULL), workspace(NULL), live(_input_height) {
        strncpy(name, _name, 7); name[7] = 0;
    }
    int ldw() const { return step128_words(weight_height); }
    size_t output_size() const { return (size_t)output_height * output_width; }
    size_t workspace_bytes() const { return tcbnn_gemm_workspace_bytes(input_height, weight_width, input_width); }
    void set_batch(int n) {
        if (n <= 0 || n > input_height) { fprintf(stderr, "%s: batch %d outside 1..%d.\n", name, n, input_height); exit(-1); }
        live = n;
    }
    // the reference's signature (param.h:439)
    Out128LayerParam* initialize(FILE* config_file, uin32* prev_layer_gpu) {
        Weights w = Weights::from_text(config_file);
        return initialize(w, prev_layer_gpu);
    }
    Out128LayerParam* initialize(Weights& config, uin32* prev_layer_gpu) {
        float* w = config.upload((size_t)weight_height * weight_width);
        weight_gpu = dev_alloc<uin32>((size_t)weight_width * ldw());
        TCBNN_HOST_CALL(tcbnn_pack_fc_weight(w, weight_height, weight_width, ldw(), weight_gpu, NULL));
        TCBNN_HOST_CUDA(cudaDeviceSynchronize());
        TCBNN_HOST_CUDA(cudaFree(w));
        bn_scale_gpu = config.upload(weight_width);
        bn_bias_gpu = config.upload(weight_width);
        output_gpu = dev_alloc<float>(output_size());
        input_gpu = prev_layer_gpu;
        return this;
    }
    void set_workspace(Workspace* w) { workspace = w; }
    void forward(cudaStream_t stream = 0) {
        TCBNN_HOST_CALL(tcbnn_out_layer(input_gpu, weight_gpu, bn_scale_gpu, bn_bias_gpu, live, input_width,
                                        weight_width, step128_words(input_width), ldw(), output_gpu, weight_width,
                                        workspace ? workspace->ptr : NULL, workspace ? workspace->bytes : 0, stream));
    }
    float* get_output_gpu() { return output_gpu; }
    float* download_output() {
        if (!output) TCBNN_HOST_CUDA(cudaMallocHost((void**)&output, output_size() * sizeof(float)));
        TCBNN_HOST_CUDA(cudaMemcpy(output, output_gpu, output_size() * sizeof(float), cudaMemcpyDeviceToHost));
        return output;
    }
    ~Out128LayerParam() {
        cudaFree(weight_gpu); cudaFree(bn_scale_gpu); cudaFree(bn_bias_gpu); cudaFree(output_gpu);
        if (output) cudaFreeHost(output);
    }
    int input_height, input_width, weight_height, weight_width, output_height, output_width;
    uin32* weight_gpu; float* bn_scale_gpu; float* bn_bias_gpu; uin32* input_gpu; float* output_gpu; float* output;
    Workspace* workspace;
    int live;                  // rows of the live batch: the first `live` rows of the output are current
    char name[8];
};

// The planes of a producer -> consumer hand-over (tcbnn_conv_layer_x): the consumer's input as
// +-1 bytes, written by the producer's epilogue.  Sized for the consumer's other scratch needs too
// (a pooled consumer reduces into the same buffer), zeroed once.
struct Planes {
    void* ptr;
    size_t bytes;
    Planes() : ptr(NULL), bytes(0) {}
    bool create(const tcbnn_conv_desc* consumer) {
        if (tcbnn_conv_planes_bytes(consumer) == 0) return false;
        const size_t a = tcbnn_conv_planes_bytes(consumer), b = tcbnn_conv_workspace_bytes(consumer);
        bytes = a > b ? a : b;
        TCBNN_HOST_CUDA(cudaMalloc(&ptr, bytes));
        TCBNN_HOST_CUDA(cudaMemset(ptr, 0, bytes));
        return true;
    }
    ~Planes() { if (ptr) cudaFree(ptr); }
};

class Conv128LayerParam;

// ---- first layer (param.h:701-870, InConv128LayerFMT kernel.cuh:578-672) -----------------------
class InConv128LayerParam {
public:
    InConv128LayerParam(const char* _name, int _input_height, int _input_width, int _filter_height,
                        int _filter_width, int _input_channels, int _output_channels, int _batch,
                        int _stride_height = 1, int _stride_width = 1, bool _padding = true,
                        int _pool_height = 1, int _pool_width = 1, bool _save_residual = false)
        : save_residual(_save_residual), residual_bytes(4), input_gpu(NULL), filter_gpu(NULL), bn_gpu(NULL),
          output_gpu(NULL), output_residual_gpu(NULL), handle(NULL), next(NULL), next_planes(NULL) {
        strncpy(name, _name, 7); name[7] = 0;
        if (_pool_height != _pool_width || _input_channels != 3) {
            fprintf(stderr, "%s: square pooling windows and 3 input channels only.\n", name);
            exit(-1);
        }
        memset(&desc, 0, sizeof desc);
        desc.B = _batch; desc.H = _input_height; desc.W = _input_width; desc.C = 3; desc.O = _output_channels;
        desc.R = _filter_height; desc.S = _filter_width; desc.stride_h = _stride_height; desc.stride_w = _stride_width;
        desc.padding = _padding ? 1 : 0; desc.pool = _pool_height;
        TCBNN_HOST_CALL(tcbnn_conv_shape(&desc));
        output_height = desc.OH; output_width = desc.OW; output_channels = desc.O; batch = desc.B;
    }
    int Ow() const { return (desc.O + 31) / 32; }
    // Extension: keep the saved residual as int16 instead of the reference's int (call before
    // initialize()).  The caller vouches that R*S*3*max|pixel| < 32768; the residual layers are
    // bound by this tensor's traffic, which it halves.
    void set_residual_bytes(int bytes) { residual_bytes = residual_code(bytes); }
    size_t input_size() const { return (size_t)desc.B * 3 * desc.H * desc.W; }
    size_t output_size() const { return (size_t)batch * desc.OH * desc.OW * desc.O; }   // at the constructor's batch
    // the following passes process the first n images (n <= the constructor's batch)
    void set_batch(int n) {
        if (n <= 0 || n > batch) { fprintf(stderr, "%s: batch %d outside 1..%d.\n", name, n, batch); exit(-1); }
        desc.B = n;
    }
    void set_input(const float* input, int images) {
        TCBNN_HOST_CUDA(cudaMemcpy(input_gpu, input, (size_t)images * 3 * desc.H * desc.W * sizeof(float), cudaMemcpyHostToDevice));
    }
    // the reference's signature (param.h:760)
    InConv128LayerParam* initialize(const float* input, FILE* config_file) {
        Weights w = Weights::from_text(config_file);
        return initialize(input, w);
    }
    InConv128LayerParam* initialize(const float* input, Weights& config) {
        if (!input) { fprintf(stderr, "NULL pointer.\n"); exit(-1); }
        input_gpu = dev_alloc<float>(input_size(), false);
        TCBNN_HOST_CUDA(cudaMemcpy(input_gpu, input, input_size() * sizeof(float), cudaMemcpyHostToDevice));
        const int RS = desc.R * desc.S;
        float* f = config.upload((size_t)RS * 3 * desc.O);                    // [R*S][3][O]
        filter_gpu = dev_alloc<uin32>((size_t)RS * 3 * Ow());
        TCBNN_HOST_CALL(tcbnn_pack_inconv_filter(f, RS, desc.O, filter_gpu, NULL));
        TCBNN_HOST_CUDA(cudaDeviceSynchronize());
        TCBNN_HOST_CUDA(cudaFree(f));
        bn_gpu = config.upload(desc.O);
        output_gpu = dev_alloc<uin32>((size_t)desc.B * desc.OH * desc.OW * Ow());
        if (save_residual) {
            output_residual_gpu = (int*)dev_alloc<char>((size_t)desc.B * desc.pool * desc.OH * desc.pool * desc.OW * desc.O *
                                                        residual_elem_bytes(residual_bytes));
            publish_residual(output_residual_gpu, desc.O, residual_bytes);
        }
        // the layer compiled for its filter, where the library offers it (at most 128 output channels)
        if (desc.O <= 128) TCBNN_HOST_CALL(tcbnn_inconv_specialize(&desc, filter_gpu, bn_gpu, NULL, &handle));
        return this;
    }
    inline void hand_over_to(Conv128LayerParam* consumer);
    void forward(cudaStream_t stream = 0) {
        const long long stride = (long long)desc.OH * desc.OW * Ow();
        if (handle)
            TCBNN_HOST_CALL(tcbnn_inconv_specialized_layer_x(handle, &desc, input_gpu, NULL, NULL, output_gpu, stride,
                                                             output_residual_gpu, residual_bytes, NULL, next,
                                                             next_planes ? next_planes->ptr : NULL,
                                                             next_planes ? next_planes->bytes : 0, stream));
        else
            TCBNN_HOST_CALL(tcbnn_inconv_layer(&desc, input_gpu, filter_gpu, bn_gpu, output_gpu, stride,
                                               output_residual_gpu, residual_bytes, NULL, stream));
    }
    float* get_input_gpu() { return input_gpu; }
    uin32* get_output_gpu() { return output_gpu; }
    int* get_output_residual_gpu() { return output_residual_gpu; }
    float* download_full_output() {
        return unpack_to_host(output_gpu, 1, 0, desc.B * desc.OH * desc.OW, desc.O, Ow());
    }
    ~InConv128LayerParam() {
        if (output_residual_gpu) retract_residual(output_residual_gpu);
        cudaFree(input_gpu); cudaFree(filter_gpu); cudaFree(bn_gpu); cudaFree(output_gpu); cudaFree(output_residual_gpu);
        if (handle) tcbnn_inconv_release(handle);
        delete next_planes;
    }
    tcbnn_conv_desc desc;
    int output_height, output_width, output_channels, batch;
    bool save_residual;
    int residual_bytes;
    float* input_gpu; uin32* filter_gpu; float* bn_gpu; uin32* output_gpu; int* output_residual_gpu;
    void* handle;
    const tcbnn_conv_desc* next;
    Planes* next_planes;
    char name[8];
};

// ---- binary conv layer (param.h:872-1065, Conv128LayerFMT kernel.cuh:676-827) ------------------
class Conv128LayerParam {
public:
    Conv128LayerParam(const char* _name, int _input_height, int _input_width, int _filter_height,
                      int _filter_width, int _input_channels, int _output_channels, int _batch,
                      int _stride_height = 1, int _stride_width = 1, bool _padding = true,
                      int _pool_height = 1, int _pool_width = 1, bool _ahead_fc = false,
                      bool _save_residual = false, bool _inject_residual = false,
                      int _residual_channels = 0, bool _residual_pool = false)
        : ahead_fc(_ahead_fc), save_residual(_save_residual), inject_residual(_inject_residual),
          residual_channels(_residual_channels), residual_pool(_residual_pool), filter_gpu(NULL), prepared_gpu(NULL),
          bn_gpu(NULL), input_gpu(NULL), output_gpu(NULL), input_residual_gpu(NULL), output_residual_gpu(NULL),
          input_residual_channels(0), residual_bytes(4), input_residual_bytes(4), workspace(NULL), next(NULL),
          next_planes(NULL) {
        strncpy(name, _name, 7); name[7] = 0;
        if (_pool_height != _pool_width) { fprintf(stderr, "%s: square pooling windows only.\n", name); exit(-1); }
        memset(&desc, 0, sizeof desc);
        desc.B = _batch; desc.H = _input_height; desc.W = _input_width; desc.C = _input_channels;
        desc.O = _output_channels; desc.R = _filter_height; desc.S = _filter_width;
        desc.stride_h = _stride_height; desc.stride_w = _stride_width; desc.padding = _padding ? 1 : 0;
        desc.pool = _pool_height;
        TCBNN_HOST_CALL(tcbnn_conv_shape(&desc));
        output_height = desc.OH; output_width = desc.OW; output_channels = desc.O; batch = desc.B;
        const long long words = (long long)desc.OH * desc.OW * Ow();
        // a layer feeding an FC layer pads each image to a whole number of 128-bit rows
        out_image_stride = ahead_fc ? step128_words(words * 32) : words;
    }
    int Ow() const { return (desc.O + 31) / 32; }
    size_t output_size() const { return (size_t)batch * desc.OH * desc.OW * desc.O; }   // at the constructor's batch
    size_t workspace_bytes() const { return tcbnn_conv_workspace_bytes(&desc); }
    // Extension: save this layer's residual as int16 (call before initialize()).  The caller vouches
    // that the running sum fits: |value| <= C*R*S + bound of the injected residual.  A value that
    // does not fit raises status 2 (overflowed()).
    void set_residual_bytes(int bytes) { residual_bytes = residual_code(bytes); }
    bool overflowed() {
        int st = 0;
        TCBNN_HOST_CALL(tcbnn_conv_status(&desc, prepared_gpu, &st));
        return st == 2;
    }
    // the following passes process the first n images (n <= the constructor's batch); planes a
    // producer fills are cleared, because their layout depends on the batch and their padding
    // positions must read as zero
    void set_batch(int n) {
        if (n <= 0 || n > batch) { fprintf(stderr, "%s: batch %d outside 1..%d.\n", name, n, batch); exit(-1); }
        if (n != desc.B && input_planes.p) TCBNN_HOST_CUDA(cudaMemset(input_planes.p->ptr, 0, input_planes.p->bytes));
        desc.B = n;
    }
    // the reference's signature (param.h:944): weights from its text file; channel count and element
    // size of the injected residual are those its producer published
    Conv128LayerParam* initialize(FILE* config_file, uin32* prev_layer_gpu, int* _input_residual_gpu = NULL) {
        Weights w = Weights::from_text(config_file);
        int ch = 0, bytes = 4;
        if (inject_residual && !lookup_residual(_input_residual_gpu, &ch, &bytes)) {
            fprintf(stderr, "%s: the injected residual is not the saved residual of an initialised layer.\n", name);
            exit(-1);
        }
        return initialize(w, prev_layer_gpu, _input_residual_gpu, ch, bytes);
    }
    // input_residual_channels_: channels per pixel of the injected tensor (the producer's O)
    // input_residual_bytes_: element size of the injected tensor (its producer's set_residual_bytes)
    Conv128LayerParam* initialize(Weights& config, uin32* prev_layer_gpu, int* _input_residual_gpu = NULL,
                                  int input_residual_channels_ = 0, int input_residual_bytes_ = 4) {
        const int RS = desc.R * desc.S;
        float* f = config.upload((size_t)RS * desc.C * desc.O);               // [R*S][C][O]
        filter_gpu = dev_alloc<uin32>((size_t)desc.O * RS * ((desc.C + 31) / 32));
        TCBNN_HOST_CALL(tcbnn_pack_conv_filter(f, RS, desc.C, desc.O, filter_gpu, NULL));
        TCBNN_HOST_CUDA(cudaDeviceSynchronize());
        TCBNN_HOST_CUDA(cudaFree(f));
        const size_t pb = tcbnn_conv_prepared_bytes(&desc);
        TCBNN_HOST_CUDA(cudaMalloc(&prepared_gpu, pb ? pb : 1));
        TCBNN_HOST_CALL(tcbnn_conv_prepare(&desc, filter_gpu, prepared_gpu, NULL));
        TCBNN_HOST_CUDA(cudaDeviceSynchronize());
        bn_gpu = config.upload(desc.O);
        output_gpu = dev_alloc<uin32>((size_t)desc.B * out_image_stride);
        if (save_residual) {
            output_residual_gpu = (int*)dev_alloc<char>((size_t)desc.B * desc.pool * desc.OH * desc.pool * desc.OW * desc.O *
                                                        residual_elem_bytes(residual_bytes));
            publish_residual(output_residual_gpu, desc.O, residual_bytes);
        }
        input_gpu = prev_layer_gpu;
        if (inject_residual) {
            if (!_input_residual_gpu || input_residual_channels_ <= 0) {
                fprintf(stderr, "%s: inject_residual needs the residual tensor and its channel count.\n", name);
                exit(-1);
            }
            input_residual_gpu = _input_residual_gpu;
            input_residual_channels = input_residual_channels_;
            input_residual_bytes = residual_code(input_residual_bytes_);
        }
        return this;
    }
    void set_workspace(Workspace* w) { workspace = w; }
    // this layer also writes its output as the consumer's pre-expanded input
    void hand_over_to(Conv128LayerParam* consumer) {
        const bool dense = out_image_stride == (long long)desc.OH * desc.OW * Ow();
        if (desc.pool != 1 || !dense) return;
        Planes* p = new Planes();
        if (!p->create(&consumer->desc)) { delete p; return; }
        next = &consumer->desc; next_planes = p; consumer->input_planes.reset_to(p);
    }
    void forward(cudaStream_t stream = 0) {
        void* ws = input_planes.p ? input_planes.p->ptr : (workspace ? workspace->ptr : NULL);
        const size_t wsb = input_planes.p ? input_planes.p->bytes : (workspace ? workspace->bytes : 0);
        TCBNN_HOST_CALL(tcbnn_conv_layer_x(&desc, input_gpu, prepared_gpu, bn_gpu,
                                           inject_residual ? input_residual_gpu : NULL, input_residual_bytes,
                                           input_residual_channels,
                                           residual_channels, residual_pool ? 1 : 0, output_gpu, out_image_stride,
                                           output_residual_gpu, residual_bytes, NULL, ws, wsb, input_planes.p ? 1 : 0, next,
                                           next_planes ? next_planes->ptr : NULL, next_planes ? next_planes->bytes : 0,
                                           stream));
    }
    uin32* get_output_gpu() { return output_gpu; }
    int* get_output_residual_gpu() { return output_residual_gpu; }
    float* download_full_output() {
        return unpack_to_host(output_gpu, desc.B, out_image_stride, desc.OH * desc.OW, desc.O, Ow());
    }
    ~Conv128LayerParam() {
        if (output_residual_gpu) retract_residual(output_residual_gpu);
        cudaFree(filter_gpu); cudaFree(prepared_gpu); cudaFree(bn_gpu); cudaFree(output_gpu); cudaFree(output_residual_gpu);
        delete next_planes;
    }
    // the planes this layer reads, owned by its producer
    struct PlanesRef { Planes* p; PlanesRef() : p(NULL) {} void reset_to(Planes* q) { p = q; } };
    tcbnn_conv_desc desc;
    int output_height, output_width, output_channels, batch;
    long long out_image_stride;
    bool ahead_fc, save_residual, inject_residual;
    int residual_channels;
    bool residual_pool;
    uin32* filter_gpu; void* prepared_gpu; float* bn_gpu; uin32* input_gpu; uin32* output_gpu;
    int* input_residual_gpu; int* output_residual_gpu;
    int input_residual_channels, residual_bytes, input_residual_bytes;
    Workspace* workspace;
    const tcbnn_conv_desc* next;
    Planes* next_planes;
    PlanesRef input_planes;
    char name[8];
};

inline void InConv128LayerParam::hand_over_to(Conv128LayerParam* consumer) {
    if (!handle) return;                         // only the specialised first layer writes planes
    Planes* p = new Planes();
    if (!p->create(&consumer->desc)) { delete p; return; }
    next = &consumer->desc; next_planes = p; consumer->input_planes.reset_to(p);
}

}  // namespace tcbnn_host
#endif
