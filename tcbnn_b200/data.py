"""Dataset file formats of the reference's readers (data.cpp:52-315) in numpy: MNIST idx files and
CIFAR-10 binary batches, raw bytes or normalised fp32 with the reference's arithmetic, and the
per-channel byte -> fp32 tables that let the first layer take the raw bytes
(tcbnn_inconv_layer_u8: a quarter of the host-to-device traffic, identical results).
The C++ twins behind the reference's data.h interface are in dropin/dataset_readers.cpp.
ImageNet needs a JPEG decoder, which this build does not have; `imagenet_lut` is the table for
bytes decoded elsewhere (data.cpp:534-542)."""
import numpy as np

MNIST_MEAN, MNIST_STD = np.float32(0.1307), np.float32(0.3081)
CIFAR_MEAN = np.array([0.4914, 0.4822, 0.4465], dtype=np.float32)
CIFAR_STD = np.array([0.2470, 0.2435, 0.2616], dtype=np.float32)
IMAGENET_MEAN = np.array([0.485, 0.456, 0.406], dtype=np.float32)
IMAGENET_STD = np.array([0.229, 0.224, 0.225], dtype=np.float32)


def _idx(path, magic, dims):
    raw = np.fromfile(path, dtype=np.uint8)
    head = raw[:4 * (1 + dims)].view(">u4")
    if raw.size < 4 * (1 + dims) or int(head[0]) != magic:
        raise ValueError("%s is not an idx file with magic %d" % (path, magic))
    shape = tuple(int(v) for v in head[1:])
    body = raw[4 * (1 + dims):]
    if body.size < int(np.prod(shape)):
        raise ValueError("%s ends before its %s items" % (path, shape))
    return body[:int(np.prod(shape))].reshape(shape)


def read_mnist_raw(image_path, label_path, batch):
    """uint8 [batch][28][28], uint32 labels [batch] (read_MNIST_raw, data.cpp:52-114)."""
    img, lab = _idx(image_path, 2051, 3), _idx(label_path, 2049, 1)
    if img.shape[0] < batch or lab.shape[0] < batch or img.shape[1:] != (28, 28):
        raise ValueError("MNIST files hold fewer than %d 28x28 images" % batch)
    return img[:batch].copy(), lab[:batch].astype(np.uint32)


def read_mnist_normalized(image_path, label_path, batch):
    """fp32 [batch][784] = (v/255 - 0.1307) / 0.3081 (read_MNIST_normalized, data.cpp:116-199)."""
    img, lab = read_mnist_raw(image_path, label_path, batch)
    x = (img.astype(np.float32) / np.float32(255.0) - MNIST_MEAN) / MNIST_STD
    return x.reshape(batch, 784), lab


def read_cifar10_raw(path, batch):
    """uint8 NCHW [batch][3][32][32] and uint32 labels from a CIFAR-10 binary batch
    (<label><1024 R><1024 G><1024 B> per record, data.cpp:203-254; the reference packs the three
    channel bytes of a pixel into one word, the planes here are what the first layer reads)."""
    raw = np.fromfile(path, dtype=np.uint8)
    if raw.size < batch * 3073:
        raise ValueError("%s holds fewer than %d CIFAR-10 records" % (path, batch))
    rec = raw[:batch * 3073].reshape(batch, 3073)
    return rec[:, 1:].reshape(batch, 3, 32, 32).copy(), rec[:, 0].astype(np.uint32)


def read_cifar10_normalized(path, batch):
    """fp32 NCHW [batch][3][32][32] = (v/255 - mean[c]) / std[c] (data.cpp:257-315)."""
    u8, lab = read_cifar10_raw(path, batch)
    return u8_to_fp32(u8, CIFAR_MEAN, CIFAR_STD), lab


def u8_to_fp32(u8, mean, std):
    m = np.asarray(mean, np.float32).reshape(1, -1, 1, 1)
    s = np.asarray(std, np.float32).reshape(1, -1, 1, 1)
    return (u8.astype(np.float32) / np.float32(255.0) - m) / s


def value_table(mean, std):
    """fp32 [3][256]: table[c][v] is the fp32 value the readers give byte v of channel c."""
    v = np.arange(256, dtype=np.float32).reshape(1, 256)
    m = np.asarray(mean, np.float32).reshape(3, 1)
    s = np.asarray(std, np.float32).reshape(3, 1)
    return ((v / np.float32(255.0) - m) / s).astype(np.float32)


def cifar10_lut():
    return value_table(CIFAR_MEAN, CIFAR_STD)


def imagenet_lut():
    return value_table(IMAGENET_MEAN, IMAGENET_STD)


def write_mnist(image_path, label_path, images_u8, labels):
    """Writes an idx3 / idx1 pair (for tests and for exporting synthetic batches)."""
    images_u8 = np.ascontiguousarray(images_u8, dtype=np.uint8)
    n = images_u8.shape[0]
    with open(image_path, "wb") as f:
        np.array([2051, n, 28, 28], dtype=">u4").tofile(f)
        images_u8.reshape(n, 28, 28).tofile(f)
    with open(label_path, "wb") as f:
        np.array([2049, n], dtype=">u4").tofile(f)
        np.asarray(labels, dtype=np.uint8).tofile(f)


def write_cifar10(path, images_u8_nchw, labels):
    images_u8_nchw = np.ascontiguousarray(images_u8_nchw, dtype=np.uint8)
    n = images_u8_nchw.shape[0]
    rec = np.empty((n, 3073), dtype=np.uint8)
    rec[:, 0] = np.asarray(labels, dtype=np.uint8)
    rec[:, 1:] = images_u8_nchw.reshape(n, 3072)
    rec.tofile(path)
