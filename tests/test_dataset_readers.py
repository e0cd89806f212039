"""The dataset readers (tcbnn_b200/dropin/dataset_readers.cpp behind the reference's data.h
signatures, and their numpy twins in tcbnn_b200/data.py) on files this test writes in the MNIST idx
and CIFAR-10 binary formats: layouts and normalisation arithmetic of data.cpp:52-315, and the
byte -> fp32 tables that reproduce the normalised values bit for bit.  No dataset item is used:
the pixels are seeded noise."""
import os
import subprocess

import numpy as np
import pytest

import util
from tcbnn_b200 import data

HERE = os.path.dirname(os.path.abspath(__file__))
READERS = os.path.join(os.path.dirname(HERE), "tcbnn_b200", "dropin", "dataset_readers.cpp")

HARNESS = r'''
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>
typedef unsigned char uchar;
using std::string;
void read_MNIST_raw(string, string, uchar*, unsigned*, const unsigned);
void read_MNIST_normalized(string, string, float*, unsigned*, const unsigned);
void read_CIFAR10_raw(string, unsigned*, unsigned*, const unsigned);
void read_CIFAR10_normalized(string, float*, unsigned*, const unsigned);
void read_ImageNet_normalized(const char*, float*, unsigned*, int);
static void dump(const char* path, const void* p, size_t n) { FILE* f = fopen(path, "wb"); fwrite(p, 1, n, f); fclose(f); }
int main(int argc, char** argv) {
    const string dir = argv[1];
    const unsigned batch = (unsigned)atoi(argv[2]);
    if (argc > 3) { read_ImageNet_normalized("x", NULL, NULL, 1); return 0; }
    std::vector<unsigned> lab(batch);
    std::vector<uchar> m8((size_t)batch * 784);
    read_MNIST_raw(dir + "/img.idx", dir + "/lab.idx", m8.data(), lab.data(), batch);
    dump((dir + "/mnist_raw.bin").c_str(), m8.data(), m8.size());
    dump((dir + "/mnist_lab.bin").c_str(), lab.data(), batch * 4);
    std::vector<float> mf((size_t)batch * 784);
    read_MNIST_normalized(dir + "/img.idx", dir + "/lab.idx", mf.data(), lab.data(), batch);
    dump((dir + "/mnist_norm.bin").c_str(), mf.data(), mf.size() * 4);
    std::vector<unsigned> cw((size_t)batch * 1024);
    read_CIFAR10_raw(dir + "/cifar.bin", cw.data(), lab.data(), batch);
    dump((dir + "/cifar_raw.bin").c_str(), cw.data(), cw.size() * 4);
    dump((dir + "/cifar_lab.bin").c_str(), lab.data(), batch * 4);
    std::vector<float> cf((size_t)batch * 3072);
    read_CIFAR10_normalized(dir + "/cifar.bin", cf.data(), lab.data(), batch);
    dump((dir + "/cifar_norm.bin").c_str(), cf.data(), cf.size() * 4);
    return 0;
}
'''


def _files(tmp_path, n_file, seed):
    g = util.rng(seed)
    m = g.integers(0, 256, size=(n_file, 28, 28), dtype=np.uint8)
    ml = g.integers(0, 10, size=n_file, dtype=np.uint8)
    c = g.integers(0, 256, size=(n_file, 3, 32, 32), dtype=np.uint8)
    cl = g.integers(0, 10, size=n_file, dtype=np.uint8)
    d = str(tmp_path)
    data.write_mnist(os.path.join(d, "img.idx"), os.path.join(d, "lab.idx"), m, ml)
    data.write_cifar10(os.path.join(d, "cifar.bin"), c, cl)
    return d, m, ml, c, cl


def test_numpy_readers_layout_and_normalisation(tmp_path):
    d, m, ml, c, cl = _files(tmp_path, 12, 1)
    raw, lab = data.read_mnist_raw(os.path.join(d, "img.idx"), os.path.join(d, "lab.idx"), 9)
    assert np.array_equal(raw, m[:9]) and np.array_equal(lab, ml[:9])
    x, _ = data.read_mnist_normalized(os.path.join(d, "img.idx"), os.path.join(d, "lab.idx"), 9)
    exp = ((m[:9].astype(np.float32) / np.float32(255)) - np.float32(0.1307)) / np.float32(0.3081)
    assert x.dtype == np.float32 and np.array_equal(x, exp.reshape(9, 784))
    u8, lab = data.read_cifar10_raw(os.path.join(d, "cifar.bin"), 12)
    assert np.array_equal(u8, c) and np.array_equal(lab, cl)
    xf, _ = data.read_cifar10_normalized(os.path.join(d, "cifar.bin"), 12)
    lut = data.cifar10_lut()
    via_table = np.stack([lut[ch][c[:, ch]] for ch in range(3)], axis=1)
    assert np.array_equal(xf, via_table)                 # the table reproduces the reader bit for bit
    with pytest.raises(ValueError):
        data.read_cifar10_raw(os.path.join(d, "cifar.bin"), 13)          # ragged: more than the file holds
    with pytest.raises(ValueError):
        data.read_mnist_raw(os.path.join(d, "lab.idx"), os.path.join(d, "lab.idx"), 1)   # wrong magic


def test_cpp_readers_match_numpy(tmp_path):
    d, m, ml, c, cl = _files(tmp_path, 7, 2)
    src = os.path.join(d, "harness.cpp")
    with open(src, "w") as f:
        f.write(HARNESS)
    exe = os.path.join(d, "harness")
    subprocess.run(["g++", "-O2", "-std=c++14", "-o", exe, src, READERS], check=True)
    subprocess.run([exe, d, "5"], check=True)
    rd = lambda name, dt: np.fromfile(os.path.join(d, name), dtype=dt)
    assert np.array_equal(rd("mnist_raw.bin", np.uint8).reshape(5, 28, 28), m[:5])
    assert np.array_equal(rd("mnist_lab.bin", np.uint32), ml[:5])
    xn, _ = data.read_mnist_normalized(os.path.join(d, "img.idx"), os.path.join(d, "lab.idx"), 5)
    assert np.array_equal(rd("mnist_norm.bin", np.float32).reshape(5, 784), xn)
    words = rd("cifar_raw.bin", np.uint32).reshape(5, 32, 32)
    for ch in range(3):                                  # byte ch of a pixel's word = channel ch
        assert np.array_equal((words >> (8 * ch)) & 0xFF, c[:5, ch])
    assert np.all(words >> 24 == 0)
    assert np.array_equal(rd("cifar_lab.bin", np.uint32), cl[:5])
    cn, _ = data.read_cifar10_normalized(os.path.join(d, "cifar.bin"), 5)
    assert np.array_equal(rd("cifar_norm.bin", np.float32).reshape(5, 3, 32, 32), cn)
    # more images than the file holds, and the ImageNet reader without a JPEG decoder: fatal, with a message
    r = subprocess.run([exe, d, "8"], capture_output=True, text=True)
    assert r.returncode == 1 and "at least 8" in r.stderr
    r = subprocess.run([exe, d, "1", "imagenet"], capture_output=True, text=True)
    assert r.returncode == 1 and "JPEG" in r.stderr


def test_validate_prediction_counts(tmp_path):
    """validate_prediction of the drop-in utility.h (the reference's is utility.h:198-232):
    top-1 / top-5 percentages on logits with known ranks."""
    src = os.path.join(str(tmp_path), "vp.cpp")
    inc = os.path.join(os.path.dirname(HERE), "tcbnn_b200", "dropin")
    with open(src, "w") as f:
        f.write('#include "utility.h"\nint main(){ float p[3*8]; unsigned lab[3]={2,0,7};\n'
                ' for(int i=0;i<3;i++) for(int j=0;j<8;j++) p[i*8+j]=(float)j;\n'
                ' validate_prediction(p, lab, 8, 3); return 0; }\n')
    cuda_inc = "/usr/local/cuda/include"
    if not os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")):
        pytest.skip("CUDA headers not found")
    exe = os.path.join(str(tmp_path), "vp")
    subprocess.run(["g++", "-std=c++14", "-I", inc, "-I", cuda_inc, "-o", exe, src, "-L/usr/local/cuda/lib64", "-lcudart"],
                   check=True)
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout
    # label 7 is the arg-max (top-1 and top-5); label 2 has five classes above it; label 0 seven
    assert "Top-1:33.3" in out and "Top-5:33.3" in out
