// Seeded synthetic stand-ins for the reference's dataset readers (data.h:47-118), so that the
// unchanged drivers link and run without MNIST / CIFAR-10 / ImageNet files or libjpeg.
// Pixels are a counter hash -> uint8 -> the same scale-and-normalise arithmetic the real readers
// apply (data.cpp:161, 295-315, 534-542); labels are hash % classes.  No dataset item is
// reproduced.
#include "data.h"
#include <stdint.h>

static inline uint32_t mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (uint32_t)((z ^ (z >> 31)) >> 32);
}

void read_MNIST_raw(string, string, uchar* images, unsigned* labels, const unsigned batch) {
    for (size_t i = 0; i < (size_t)batch * 28 * 28; i++) images[i] = (uchar)(mix(i) & 0xFF);
    for (unsigned i = 0; i < batch; i++) labels[i] = mix(0x1000000000ull + i) % 10;
}
void read_MNIST_normalized(string, string, float* images, unsigned* labels, const unsigned batch) {
    for (size_t i = 0; i < (size_t)batch * 28 * 28; i++)
        images[i] = ((mix(i) & 0xFF) / 255.0f - 0.1307f) / 0.3081f;
    for (unsigned i = 0; i < batch; i++) labels[i] = mix(0x1000000000ull + i) % 10;
}
void read_CIFAR10_raw(string, unsigned* images, unsigned* labels, const unsigned batch) {
    for (size_t i = 0; i < (size_t)batch * 32 * 32; i++) images[i] = mix(i) & 0xFFFFFFu;
    for (unsigned i = 0; i < batch; i++) labels[i] = mix(0x2000000000ull + i) % 10;
}
void read_CIFAR10_normalized(string, float* images, unsigned* labels, const unsigned batch) {
    const float mean[3] = {0.4914f, 0.4822f, 0.4465f}, sd[3] = {0.2470f, 0.2435f, 0.2616f};
    for (size_t b = 0; b < batch; b++)
        for (int c = 0; c < 3; c++)
            for (int p = 0; p < 32 * 32; p++) {
                const size_t i = (b * 3 + c) * 32 * 32 + p;
                images[i] = ((mix(i) & 0xFF) / 255.0f - mean[c]) / sd[c];
            }
    for (unsigned i = 0; i < batch; i++) labels[i] = mix(0x2000000000ull + i) % 10;
}
void read_ImageNet_raw(const char*, unsigned* images, unsigned* labels, int batch) {
    for (size_t i = 0; i < (size_t)batch * 224 * 224; i++) images[i] = mix(i) & 0xFFFFFFu;
    for (int i = 0; i < batch; i++) labels[i] = mix(0x3000000000ull + i) % 1000;
}
void read_ImageNet_normalized(const char*, float* images, unsigned* labels, int batch) {
    const float mean[3] = {0.485f, 0.456f, 0.406f}, sd[3] = {0.229f, 0.224f, 0.225f};
    for (size_t b = 0; b < (size_t)batch; b++)
        for (int c = 0; c < 3; c++)
            for (int p = 0; p < 224 * 224; p++) {
                const size_t i = (b * 3 + c) * 224 * 224 + p;
                images[i] = ((mix(i) & 0xFF) / 255.0f - mean[c]) / sd[c];
            }
    for (int i = 0; i < batch; i++) labels[i] = mix(0x3000000000ull + i) % 1000;
}
