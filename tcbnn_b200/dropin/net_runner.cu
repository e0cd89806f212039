// Generic driver on the drop-in layer API: builds a network from a small text description with
// the reference's classes (param.h), runs it as ONE cooperative kernel that calls the layer
// functions with grid.sync() between them -- the structure of the reference drivers
// (imagenet_resnet.cu:34-125, 328-363) -- and writes the fp32 logits to a file.
//
//   net_runner <spec.txt> <weights.txt> <input.bin> <logits.bin> [device]
//
// spec.txt : first line "batch B", then one layer per line
//   in K
//   inconv H W R S C O stride pool save_residual
//   conv R S C O stride pool ahead_fc save_residual inject(-1 or layer index) residual_channels residual_pool
//   fc N
//   out N
// weights.txt : whitespace-separated floats in launch_array order (utility.h).  With the drop-in
//   headers a name ending in ".bin" is read as raw fp32 in the same order (from the file, or, with
//   TCBNN_WEIGHTS_IN_MEMORY set, loaded first and handed over as a host array).
// TCBNN_RUNS=n launches the forward kernel n times on the same objects (layers store their
//   outputs, so every run gives the same result); the last one is timed.
// TCBNN_LIVE_BATCH=n (drop-in headers only): after the first runs on the full batch the same objects
//   are switched to the first n images (set_batch) for the last, timed run; logits and dumps then
//   hold n images.
// TCBNN_RUNNER_FAST (drop-in headers only): instead of the cooperative kernel, queue every layer
//   through the C ABI of libtcbnn_b200.so, the way the drop-in does for a driver whose kernel
//   takes its layer objects as arguments (tcbnn_dropin::launch_network in param.h).
// input.bin   : fp32, [B][K] for "in" networks, NCHW [B][3][H][W] otherwise.
#include <cooperative_groups.h>
#include <vector>
#include <string>
#include "utility.h"
#include "param.h"
#include "kernel.cuh"

using namespace cooperative_groups;

enum LayerKind { K_IN = 0, K_INCONV = 1, K_CONV = 2, K_FC = 3, K_OUT = 4 };
struct LayerRef { int kind; void* gpu; };

__global__ void run_network(const LayerRef* layers, int n) {
    grid_group grid = this_grid();
    for (int i = 0; i < n; i++) {
        switch (layers[i].kind) {
            case K_IN: In128LayerFMT((In128LayerParam*)layers[i].gpu); break;
            case K_INCONV: InConv128LayerFMT((InConv128LayerParam*)layers[i].gpu); break;
            case K_CONV: Conv128LayerFMT((Conv128LayerParam*)layers[i].gpu); break;
            case K_FC: Fc128LayerFMT((Fc128LayerParam*)layers[i].gpu); break;
            default: Out128LayerFMT((Out128LayerParam*)layers[i].gpu); break;
        }
        if (i + 1 < n) grid.sync();
    }
}

struct Built {
    int kind;
    In128LayerParam* in; InConv128LayerParam* inconv; Conv128LayerParam* conv;
    Fc128LayerParam* fc; Out128LayerParam* out;
};

int main(int argc, char** argv) {
    if (argc < 5) { fprintf(stderr, "usage: net_runner spec weights input logits [device]\n"); return 2; }
    const int device = argc > 5 ? atoi(argv[5]) : 0;
    CUDA_SAFE_CALL(cudaSetDevice(device));
    FILE* spec = fopen(argv[1], "r");
    FILE* fin = fopen(argv[3], "rb");
#ifdef TCBNN_DROPIN
    const size_t len = strlen(argv[2]);
    const bool binary = len > 4 && strcmp(argv[2] + len - 4, ".bin") == 0;
    FILE* wfile = fopen(argv[2], binary ? "rb" : "r");
    if (!spec || !wfile || !fin) { fprintf(stderr, "cannot open an input file\n"); return 2; }
    std::vector<float> held;
    if (binary && getenv("TCBNN_WEIGHTS_IN_MEMORY")) {
        fseek(wfile, 0, SEEK_END);
        held.resize((size_t)ftell(wfile) / sizeof(float));
        fseek(wfile, 0, SEEK_SET);
        if (fread(held.data(), sizeof(float), held.size(), wfile) != held.size()) return 2;
    }
    tcbnn_dropin::Weights config_file = !binary ? tcbnn_dropin::Weights::from_text(wfile)
                                        : held.empty() ? tcbnn_dropin::Weights::from_binary(wfile)
                                                       : tcbnn_dropin::Weights::from_memory(held.data(), held.size());
#else
    FILE* config_file = fopen(argv[2], "r");
    if (!spec || !config_file || !fin) { fprintf(stderr, "cannot open an input file\n"); return 2; }
#endif
    int batch = 0;
    char word[64];
    if (fscanf(spec, "%63s %d", word, &batch) != 2 || std::string(word) != "batch") return 2;

    std::vector<Built> net;
    std::vector<LayerRef> refs;
    float* images = NULL;
    uin32* prev = NULL;
    int H = 0, W = 0, K = 0;
    while (fscanf(spec, "%63s", word) == 1) {
        const std::string t(word);
        Built b = {};
        LayerRef r = {};
        if (t == "in") {
            fscanf(spec, "%d", &K);
            images = (float*)malloc((size_t)batch * K * sizeof(float));
            if (fread(images, sizeof(float), (size_t)batch * K, fin) != (size_t)batch * K) return 2;
            b.kind = K_IN; b.in = new In128LayerParam("Fin", batch, K);
            r.gpu = b.in->initialize(images); prev = b.in->get_output_gpu();
        } else if (t == "inconv") {
            int R, S, C, O, st, pool, save;
            fscanf(spec, "%d %d %d %d %d %d %d %d %d", &H, &W, &R, &S, &C, &O, &st, &pool, &save);
            const size_t n = (size_t)batch * C * H * W;
            images = (float*)malloc(n * sizeof(float));
            if (fread(images, sizeof(float), n, fin) != n) return 2;
            b.kind = K_INCONV;
            b.inconv = new InConv128LayerParam("Conv1", H, W, R, S, C, O, batch, st, st, true, pool, pool, save != 0);
            r.gpu = b.inconv->initialize(images, config_file);
            prev = b.inconv->get_output_gpu(); H = b.inconv->output_height; W = b.inconv->output_width;
            K = H * W * O;
        } else if (t == "conv") {
            int R, S, C, O, st, pool, afc, save, inj, rc, rpool;
            fscanf(spec, "%d %d %d %d %d %d %d %d %d %d %d", &R, &S, &C, &O, &st, &pool, &afc, &save, &inj, &rc, &rpool);
            b.kind = K_CONV;
            b.conv = new Conv128LayerParam("Conv", H, W, R, S, C, O, batch, st, st, true, pool, pool, afc != 0,
                                           save != 0, inj >= 0, rc, rpool != 0);
            int* res = NULL;
            if (inj >= 0) res = net[inj].kind == K_INCONV ? net[inj].inconv->get_output_residual_gpu()
                                                          : net[inj].conv->get_output_residual_gpu();
            r.gpu = b.conv->initialize(config_file, prev, res);
            prev = b.conv->get_output_gpu(); H = b.conv->output_height; W = b.conv->output_width;
            K = H * W * O;
        } else if (t == "fc") {
            int N; fscanf(spec, "%d", &N);
            b.kind = K_FC; b.fc = new Fc128LayerParam("Fc", batch, K, N);
            r.gpu = b.fc->initialize(config_file, prev); prev = b.fc->get_output_gpu(); K = N;
        } else if (t == "out") {
            int N; fscanf(spec, "%d", &N);
            b.kind = K_OUT; b.out = new Out128LayerParam("Fout", batch, K, N);
            r.gpu = b.out->initialize(config_file, prev); K = N;
        } else { fprintf(stderr, "unknown layer %s\n", word); return 2; }
        r.kind = b.kind;
        net.push_back(b);
        refs.push_back(r);
    }
    if (net.empty() || net.back().kind != K_OUT) { fprintf(stderr, "network must end with an out layer\n"); return 2; }

    LayerRef* refs_gpu = NULL;
    SAFE_ALOC_GPU(refs_gpu, refs.size() * sizeof(LayerRef));
    CUDA_SAFE_CALL(cudaMemcpy(refs_gpu, refs.data(), refs.size() * sizeof(LayerRef), cudaMemcpyHostToDevice));

    // launch exactly like the reference drivers: 1024 threads, occupancy x SMs blocks, cooperative
    int numThreads = 1024, numBlocksPerSm = 0, n = (int)refs.size();
    cudaDeviceProp deviceProp;
    cudaGetDeviceProperties(&deviceProp, device);
    int shared_memory = 512 * sizeof(int) * 32;
    cudaFuncSetAttribute(run_network, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_memory);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&numBlocksPerSm, run_network, numThreads, shared_memory);
    void* args[] = {&refs_gpu, &n};
    const int runs = getenv("TCBNN_RUNS") ? atoi(getenv("TCBNN_RUNS")) : 1;
    bool fast = false;
#ifdef TCBNN_DROPIN
    fast = getenv("TCBNN_RUNNER_FAST") != NULL;
#endif
    auto forward = [&]() {
#ifdef TCBNN_DROPIN
        if (fast) {
            for (size_t i = 0; i < refs.size(); i++)
                if (!tcbnn_dropin::forward_registered(refs[i].gpu, 0, false)) {
                    fprintf(stderr, "layer %zu cannot take the fast path\n", i);
                    exit(2);
                }
            return;
        }
#endif
        CUDA_SAFE_CALL(cudaLaunchCooperativeKernel((void*)run_network, numBlocksPerSm * deviceProp.multiProcessorCount,
                                                   numThreads, args, shared_memory));
    };
    for (int i = 1; i < runs; i++) forward();
    int live = batch;
#ifdef TCBNN_DROPIN
    if (getenv("TCBNN_LIVE_BATCH")) {
        live = atoi(getenv("TCBNN_LIVE_BATCH"));
        CUDA_SAFE_CALL(cudaDeviceSynchronize());
        for (size_t i = 0; i < net.size(); i++) {
            if (net[i].in) net[i].in->set_batch(live);
            if (net[i].inconv) net[i].inconv->set_batch(live);
            if (net[i].conv) net[i].conv->set_batch(live);
            if (net[i].fc) net[i].fc->set_batch(live);
            if (net[i].out) net[i].out->set_batch(live);
        }
    }
#endif
    START_TIMER;
    forward();
    STOP_TIMER;
    CUDA_CHECK_KERNEL();
    CUDA_SAFE_CALL(cudaDeviceSynchronize());
    printf("{\"forward_ms\": %.4f, \"batch\": %d, \"layers\": %d, \"blocks\": %d, \"fast\": %d}\n", milliseconds, batch, n,
           numBlocksPerSm * deviceProp.multiProcessorCount, fast ? 1 : 0);

    float* logits = net.back().out->download_output();
    FILE* fo = fopen(argv[4], "wb");
    fwrite(logits, sizeof(float), (size_t)live * K, fo);
    fclose(fo);
    // also dump every layer's +-1 activations when asked (parity checks)
    if (getenv("TCBNN_DUMP_DIR")) {
        for (size_t i = 0; i + 1 < net.size(); i++) {
            float* full = NULL; size_t cnt = 0;
            if (net[i].kind == K_IN) { full = net[i].in->download_full_output(); cnt = net[i].in->output_size(); }
            if (net[i].kind == K_FC) { full = net[i].fc->download_full_output(); cnt = net[i].fc->output_size(); }
            if (net[i].kind == K_INCONV) { full = net[i].inconv->download_full_output(); cnt = net[i].inconv->output_size(); }
            if (net[i].kind == K_CONV) { full = net[i].conv->download_full_output(); cnt = net[i].conv->output_size(); }
            char path[512];
            snprintf(path, sizeof(path), "%s/layer%02zu.bin", getenv("TCBNN_DUMP_DIR"), i);
            FILE* f = fopen(path, "wb");
            fwrite(full, sizeof(float), cnt, f);
            fclose(f);
            cudaFreeHost(full);
        }
    }
    for (size_t i = 0; i < net.size(); i++) {
        delete net[i].in; delete net[i].inconv; delete net[i].conv; delete net[i].fc; delete net[i].out;
    }
    return 0;
}
