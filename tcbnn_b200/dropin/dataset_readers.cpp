// Dataset readers behind the reference's data.h interface (data.h:47-118): MNIST idx files and
// the CIFAR-10 binary batches, raw and normalised, with the reference's output layouts and
// normalisation arithmetic (data.cpp:116-315).  Link this file instead of synthetic_data.cpp to
// run a driver on real data.  Whole records are read at once (the reference reads byte by byte);
// a file that is missing or too short is fatal, as there.
//
// The ImageNet readers (data.cpp:317-591) decode JPEG files with libjpeg, which this build does
// not have: they stop with a message.  Feed ImageNet through the uint8 first-layer entry point
// (tcbnn_inconv_layer_u8) from whatever decoder the application already has.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

typedef unsigned char uchar;
using std::string;

void read_MNIST_raw(string filename, string labelname, uchar* images, unsigned* labels, const unsigned batch);
void read_MNIST_normalized(string filename, string labelname, float* images, unsigned* labels, const unsigned batch);
void read_CIFAR10_raw(string filename, unsigned* images, unsigned* labels, const unsigned batch);
void read_CIFAR10_normalized(string filename, float* images, unsigned* labels, const unsigned batch);
void read_ImageNet_raw(const char* descfilename, unsigned* images, unsigned* labels, int batch);
void read_ImageNet_normalized(const char* descfilename, float* images, unsigned* labels, int batch);

namespace {

void need(const void* p, const char* what, const char* set) {
    if (p == NULL) {
        fprintf(stderr, "NULL %s pointer in reading %s.\n", what, set);
        exit(1);
    }
}

FILE* open_or_die(const string& path, const char* what) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) {
        fprintf(stderr, "Error in reading %s file '%s'.\n", what, path.c_str());
        exit(1);
    }
    return f;
}

void read_or_die(FILE* f, void* dst, size_t bytes, const string& path) {
    if (fread(dst, 1, bytes, f) != bytes) {
        fprintf(stderr, "File '%s' ended before %zu bytes could be read.\n", path.c_str(), bytes);
        exit(1);
    }
}

// idx header: big-endian 32-bit magic, item count and (for images) rows and columns
unsigned be32(const uchar* p) { return ((unsigned)p[0] << 24) | ((unsigned)p[1] << 16) | ((unsigned)p[2] << 8) | p[3]; }

// the first `batch` images (28 x 28 bytes each) and labels of an MNIST idx pair
void mnist_bytes(const string& filename, const string& labelname, unsigned batch, std::vector<uchar>& pixels,
                 unsigned* labels) {
    uchar head[16];
    FILE* f = open_or_die(filename, "MNIST image");
    read_or_die(f, head, 16, filename);
    if (be32(head) != 2051 || be32(head + 8) != 28 || be32(head + 12) != 28 || be32(head + 4) < batch) {
        fprintf(stderr, "'%s' is not an idx3 file of at least %u 28x28 images.\n", filename.c_str(), batch);
        exit(1);
    }
    pixels.resize((size_t)batch * 784);
    read_or_die(f, pixels.data(), pixels.size(), filename);
    fclose(f);
    FILE* l = open_or_die(labelname, "MNIST label");
    read_or_die(l, head, 8, labelname);
    if (be32(head) != 2049 || be32(head + 4) < batch) {
        fprintf(stderr, "'%s' is not an idx1 file of at least %u labels.\n", labelname.c_str(), batch);
        exit(1);
    }
    std::vector<uchar> lab(batch);
    read_or_die(l, lab.data(), batch, labelname);
    fclose(l);
    for (unsigned i = 0; i < batch; i++) labels[i] = lab[i];
}

// the first `batch` records of a CIFAR-10 batch file: <label><1024 R><1024 G><1024 B>
void cifar_records(const string& filename, unsigned batch, std::vector<uchar>& rec) {
    FILE* f = open_or_die(filename, "Cifar-10 bin");
    rec.resize((size_t)batch * 3073);
    read_or_die(f, rec.data(), rec.size(), filename);
    fclose(f);
}

}  // namespace

// [batch][28][28] bytes (data.cpp:52-114)
void read_MNIST_raw(string filename, string labelname, uchar* images, unsigned* labels, const unsigned batch) {
    need(images, "images", "MNIST");
    need(labels, "labels", "MNIST");
    std::vector<uchar> px;
    mnist_bytes(filename, labelname, batch, px, labels);
    memcpy(images, px.data(), px.size());
}

// [batch][1][28][28] floats, (v/255 - 0.1307) / 0.3081 (data.cpp:116-199)
void read_MNIST_normalized(string filename, string labelname, float* images, unsigned* labels, const unsigned batch) {
    need(images, "images", "MNIST");
    need(labels, "labels", "MNIST");
    std::vector<uchar> px;
    mnist_bytes(filename, labelname, batch, px, labels);
    for (size_t i = 0; i < px.size(); i++) images[i] = (((float)px[i] / 255.f) - 0.1307f) / 0.3081f;
}

// [batch][32][32] words, byte c of a word = channel c (R, G, B), fourth byte 0 (data.cpp:203-254)
void read_CIFAR10_raw(string filename, unsigned* images, unsigned* labels, const unsigned batch) {
    need(images, "images", "Cifar-10");
    need(labels, "labels", "Cifar-10");
    std::vector<uchar> rec;
    cifar_records(filename, batch, rec);
    uchar* out = (uchar*)images;
    for (unsigned l = 0; l < batch; l++) {
        const uchar* r = rec.data() + (size_t)l * 3073;
        labels[l] = r[0];
        for (int p = 0; p < 1024; p++) {
            uchar* w = out + ((size_t)l * 1024 + p) * 4;
            w[0] = r[1 + p]; w[1] = r[1 + 1024 + p]; w[2] = r[1 + 2048 + p]; w[3] = 0;
        }
    }
}

// [batch][3][32][32] floats, (v/255 - mean[c]) / std[c] (data.cpp:257-315)
void read_CIFAR10_normalized(string filename, float* images, unsigned* labels, const unsigned batch) {
    need(images, "images", "Cifar-10");
    need(labels, "labels", "Cifar-10");
    static const float mean[3] = {0.4914f, 0.4822f, 0.4465f}, sd[3] = {0.2470f, 0.2435f, 0.2616f};
    std::vector<uchar> rec;
    cifar_records(filename, batch, rec);
    for (unsigned l = 0; l < batch; l++) {
        const uchar* r = rec.data() + (size_t)l * 3073;
        labels[l] = r[0];
        for (int c = 0; c < 3; c++)
            for (int p = 0; p < 1024; p++)
                images[((size_t)l * 3 + c) * 1024 + p] = ((float)r[1 + c * 1024 + p] / 255.0f - mean[c]) / sd[c];
    }
}

void read_ImageNet_raw(const char*, unsigned*, unsigned*, int) {
    fprintf(stderr, "read_ImageNet_raw: this build has no JPEG decoder (libjpeg is not installed).\n");
    exit(1);
}
void read_ImageNet_normalized(const char*, float*, unsigned*, int) {
    fprintf(stderr, "read_ImageNet_normalized: this build has no JPEG decoder (libjpeg is not installed).\n");
    exit(1);
}
