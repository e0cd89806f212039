// Generic driver on the C++ host classes of tcbnn_host.hpp: builds a network from the text
// description tcbnn_b200/dropin/net_runner.cu reads (same command line, same files), runs it layer
// by layer through the C ABI -- the tcgen05 kernels, the first layer compiled for its filter,
// producer -> consumer hand-over of the pre-expanded inputs -- and writes the fp32 logits.
//
//   fast_runner <spec.txt> <weights.txt | weights.bin> <input.bin> <logits.bin> [device]
//
// spec.txt : first line "batch B", then one layer per line
//   in K
//   inconv H W R S C O stride pool save_residual
//   conv R S C O stride pool ahead_fc save_residual inject(-1 or layer index) residual_channels residual_pool
//   fc N
//   out N
// A weights name ending in ".bin" is raw fp32 in launch_array order, anything else the
// reference's text format.  TCBNN_RESIDUAL16=1 (or =chunked, the chunk-major layout) keeps the saved residuals as int16 (the caller's
// promise that they fit; an overflow is reported and fails the run).  TCBNN_RUNS=n runs the forward pass n times (the last one is timed);
// TCBNN_DUMP_DIR=<dir> also writes every layer's download_full_output() as layerNN.bin.
// TCBNN_TEXT_SIGNATURES=1 (text weights) builds the layers through the reference's own
// initialize(FILE*, ...) signatures.  TCBNN_LIVE_BATCH=n: after the first runs on the full batch the
// same objects are switched to the first n images (set_batch) for the last, timed run; logits and
// dumps then hold n images.
#include <cstring>
#include <string>
#include <vector>
#include "tcbnn_host.hpp"

using namespace tcbnn_host;

enum LayerKind { K_IN = 0, K_INCONV = 1, K_CONV = 2, K_FC = 3, K_OUT = 4 };
struct Built {
    int kind;
    In128LayerParam* in; InConv128LayerParam* inconv; Conv128LayerParam* conv;
    Fc128LayerParam* fc; Out128LayerParam* out;
};

static void forward(std::vector<Built>& net, cudaStream_t st) {
    for (size_t i = 0; i < net.size(); i++) {
        switch (net[i].kind) {
            case K_IN: net[i].in->forward(st); break;
            case K_INCONV: net[i].inconv->forward(st); break;
            case K_CONV: net[i].conv->forward(st); break;
            case K_FC: net[i].fc->forward(st); break;
            default: net[i].out->forward(st); break;
        }
    }
}

int main(int argc, char** argv) {
    if (argc < 5) { fprintf(stderr, "usage: fast_runner spec weights input logits [device]\n"); return 2; }
    TCBNN_HOST_CUDA(cudaSetDevice(argc > 5 ? atoi(argv[5]) : 0));
    FILE* spec = fopen(argv[1], "r");
    const size_t len = strlen(argv[2]);
    const bool binary = len > 4 && strcmp(argv[2] + len - 4, ".bin") == 0;
    FILE* wfile = fopen(argv[2], binary ? "rb" : "r");
    FILE* fin = fopen(argv[3], "rb");
    if (!spec || !wfile || !fin) { fprintf(stderr, "cannot open an input file\n"); return 2; }
    Weights config = binary ? Weights::from_binary(wfile) : Weights::from_text(wfile);
    int batch = 0;
    char word[64];
    if (fscanf(spec, "%63s %d", word, &batch) != 2 || std::string(word) != "batch") return 2;

    std::vector<Built> net;
    std::vector<float> images;
    uin32* prev = NULL;
    int H = 0, W = 0, K = 0;
    // TCBNN_RESIDUAL16=1: int16 residual tensors; =chunked: int16 in the chunk-major layout the
    // tcgen05 conv kernel's epilogue is fastest on (every conv layer has its workspace here)
    const char* r16 = getenv("TCBNN_RESIDUAL16");
    const int res_bytes = !r16 ? 4 : (strcmp(r16, "chunked") == 0 ? TCBNN_RES_INT16_CHUNKED : 2);
    const bool text_sig = getenv("TCBNN_TEXT_SIGNATURES") != NULL && !binary;
    while (fscanf(spec, "%63s", word) == 1) {
        const std::string t(word);
        Built b = {};
        if (t == "in") {
            if (fscanf(spec, "%d", &K) != 1) return 2;
            images.resize((size_t)batch * K);
            if (fread(images.data(), sizeof(float), images.size(), fin) != images.size()) return 2;
            b.kind = K_IN; b.in = new In128LayerParam("Fin", batch, K);
            b.in->initialize(images.data()); prev = b.in->get_output_gpu();
        } else if (t == "inconv") {
            int R, S, C, O, st, pool, save;
            if (fscanf(spec, "%d %d %d %d %d %d %d %d %d", &H, &W, &R, &S, &C, &O, &st, &pool, &save) != 9) return 2;
            images.resize((size_t)batch * C * H * W);
            if (fread(images.data(), sizeof(float), images.size(), fin) != images.size()) return 2;
            b.kind = K_INCONV;
            b.inconv = new InConv128LayerParam("Conv1", H, W, R, S, C, O, batch, st, st, true, pool, pool, save != 0);
            b.inconv->set_residual_bytes(res_bytes);
            if (text_sig) b.inconv->initialize(images.data(), wfile); else b.inconv->initialize(images.data(), config);
            prev = b.inconv->get_output_gpu(); H = b.inconv->output_height; W = b.inconv->output_width;
            K = H * W * O;
        } else if (t == "conv") {
            int R, S, C, O, st, pool, afc, save, inj, rc, rpool;
            if (fscanf(spec, "%d %d %d %d %d %d %d %d %d %d %d", &R, &S, &C, &O, &st, &pool, &afc, &save, &inj, &rc, &rpool) != 11) return 2;
            b.kind = K_CONV;
            b.conv = new Conv128LayerParam("Conv", H, W, R, S, C, O, batch, st, st, true, pool, pool, afc != 0,
                                           save != 0, inj >= 0, rc, rpool != 0);
            int* res = NULL;
            int res_ch = 0;
            if (inj >= 0) {
                if (net[inj].kind == K_INCONV) { res = net[inj].inconv->get_output_residual_gpu(); res_ch = net[inj].inconv->output_channels; }
                else { res = net[inj].conv->get_output_residual_gpu(); res_ch = net[inj].conv->output_channels; }
            }
            b.conv->set_residual_bytes(res_bytes);
            if (text_sig) b.conv->initialize(wfile, prev, res); else b.conv->initialize(config, prev, res, res_ch, res_bytes);
            prev = b.conv->get_output_gpu(); H = b.conv->output_height; W = b.conv->output_width;
            K = H * W * O;
        } else if (t == "fc") {
            int N; if (fscanf(spec, "%d", &N) != 1) return 2;
            b.kind = K_FC; b.fc = new Fc128LayerParam("Fc", batch, K, N);
            if (text_sig) b.fc->initialize(wfile, prev); else b.fc->initialize(config, prev);
            prev = b.fc->get_output_gpu(); K = N;
        } else if (t == "out") {
            int N; if (fscanf(spec, "%d", &N) != 1) return 2;
            b.kind = K_OUT; b.out = new Out128LayerParam("Fout", batch, K, N);
            if (text_sig) b.out->initialize(wfile, prev); else b.out->initialize(config, prev);
            K = N;
        } else { fprintf(stderr, "unknown layer %s\n", word); return 2; }
        net.push_back(b);
    }
    if (net.empty() || net.back().kind != K_OUT) { fprintf(stderr, "network must end with an out layer\n"); return 2; }

    // one scratch buffer for the whole network; hand-over between consecutive conv layers
    Workspace ws;
    for (size_t i = 0; i < net.size(); i++) {
        if (net[i].kind == K_CONV) ws.reserve(net[i].conv->workspace_bytes());
        if (net[i].kind == K_FC) ws.reserve(net[i].fc->workspace_bytes());
        if (net[i].kind == K_OUT) ws.reserve(net[i].out->workspace_bytes());
    }
    for (size_t i = 0; i < net.size(); i++) {
        if (net[i].kind == K_CONV) net[i].conv->set_workspace(&ws);
        if (net[i].kind == K_FC) net[i].fc->set_workspace(&ws);
        if (net[i].kind == K_OUT) net[i].out->set_workspace(&ws);
        if (i + 1 < net.size() && net[i + 1].kind == K_CONV && !getenv("TCBNN_NO_HANDOVER")) {
            if (net[i].kind == K_CONV) net[i].conv->hand_over_to(net[i + 1].conv);
            if (net[i].kind == K_INCONV) net[i].inconv->hand_over_to(net[i + 1].conv);
        }
    }

    cudaStream_t st;
    TCBNN_HOST_CUDA(cudaStreamCreate(&st));
    const int runs = getenv("TCBNN_RUNS") ? atoi(getenv("TCBNN_RUNS")) : 1;
    for (int i = 1; i < runs; i++) forward(net, st);
    int live = batch;
    if (getenv("TCBNN_LIVE_BATCH")) {
        live = atoi(getenv("TCBNN_LIVE_BATCH"));
        TCBNN_HOST_CUDA(cudaStreamSynchronize(st));
        for (size_t i = 0; i < net.size(); i++) {
            if (net[i].in) net[i].in->set_batch(live);
            if (net[i].inconv) net[i].inconv->set_batch(live);
            if (net[i].conv) net[i].conv->set_batch(live);
            if (net[i].fc) net[i].fc->set_batch(live);
            if (net[i].out) net[i].out->set_batch(live);
        }
    }
    cudaEvent_t e0, e1;
    TCBNN_HOST_CUDA(cudaEventCreate(&e0));
    TCBNN_HOST_CUDA(cudaEventCreate(&e1));
    TCBNN_HOST_CUDA(cudaEventRecord(e0, st));
    forward(net, st);
    TCBNN_HOST_CUDA(cudaEventRecord(e1, st));
    TCBNN_HOST_CUDA(cudaStreamSynchronize(st));
    float ms = 0;
    TCBNN_HOST_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    printf("{\"forward_ms\": %.4f, \"batch\": %d, \"layers\": %d, \"live\": %d}\n", ms, batch, (int)net.size(), live);

    for (size_t i = 0; i < net.size(); i++)
        if (net[i].kind == K_CONV && net[i].conv->overflowed()) {
            fprintf(stderr, "layer %zu: a residual does not fit in int16\n", i);
            return 3;
        }
    float* logits = net.back().out->download_output();
    FILE* fo = fopen(argv[4], "wb");
    if (!fo) return 2;
    fwrite(logits, sizeof(float), (size_t)live * K, fo);
    fclose(fo);
    if (getenv("TCBNN_DUMP_DIR")) {
        for (size_t i = 0; i + 1 < net.size(); i++) {
            float* full = NULL; size_t cnt = 0;
            if (net[i].kind == K_IN) { full = net[i].in->download_full_output(); cnt = net[i].in->output_size(); }
            if (net[i].kind == K_FC) { full = net[i].fc->download_full_output(); cnt = net[i].fc->output_size(); }
            if (net[i].kind == K_INCONV) { full = net[i].inconv->download_full_output(); cnt = net[i].inconv->output_size(); }
            if (net[i].kind == K_CONV) { full = net[i].conv->download_full_output(); cnt = net[i].conv->output_size(); }
            cnt = cnt / batch * live;
            char path[512];
            snprintf(path, sizeof(path), "%s/layer%02zu.bin", getenv("TCBNN_DUMP_DIR"), i);
            FILE* f = fopen(path, "wb");
            if (!f) return 2;
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
