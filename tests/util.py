"""Shared helpers for the tests: seeded inputs and an independent +-1 restatement of the
layers in numpy (dot products of +-1 values, zeros outside the frame) used to cross-check the
popcount oracle on small cases."""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def rand_words(g, shape):
    return g.integers(0, 2**32, size=shape, dtype=np.uint64).astype(np.uint32)


def rand_pm1(g, shape):
    return (g.integers(0, 2, size=shape).astype(np.float32) * 2 - 1)


def mask_row_pad(words, k):
    """Zero the pad bits past element k of each row (MSB-first bit order)."""
    words = words.copy()
    ld = words.shape[-1]
    for w in range(ld):
        lo = w * 32
        if lo >= k:
            words[..., w] = 0
        elif lo + 32 > k:
            keep = k - lo
            words[..., w] &= np.uint32((0xFFFFFFFF << (32 - keep)) & 0xFFFFFFFF)
    return words


def bits_to_pm1(words, n):
    """[..., ld] words -> [..., n] float +-1 (bit e at word e//32, bit 31-e%32)."""
    words = np.asarray(words, dtype=np.uint32)
    e = np.arange(n)
    b = (words[..., e // 32] >> (31 - (e % 32)).astype(np.uint32)) & 1
    return b.astype(np.float32) * 2 - 1


def pm1_to_bits(x, ld=None):
    n = x.shape[-1]
    ld = ld or (n + 31) // 32
    out = np.zeros(x.shape[:-1] + (ld,), dtype=np.uint32)
    for e in range(n):
        out[..., e // 32] |= ((x[..., e] >= 0).astype(np.uint32) << np.uint32(31 - e % 32))
    return out


def conv_shape(H, W, R, S, sh, sw, padding, pool):
    """param.h:897-906."""
    pad_h = (((H + sh - (H % sh)) // sh - 1) * sh + R - H) // 2 if padding else 0
    pad_w = (((W + sw - (W % sw)) // sw - 1) * sw + S - W) // 2 if padding else 0
    bh = (H + sh - 1) // sh if padding else (H - R) // sh + 1
    bw = (W + sw - 1) // sw if padding else (W - S) // sw + 1
    OH, OW = (bh + pool - 1) // pool, (bw + pool - 1) // pool
    return pad_h, pad_w, OH, OW


def conv_pm1_reference(x_pm1, f_pm1, thr, sh, sw, padding, pool, res_in=None,
                       residual_channels=0, residual_pool=False):
    """+-1 restatement of Conv128LayerFMT (kernel.cuh:676-827).
    x_pm1 [B][H][W][C], f_pm1 [R][S][C][O].  Returns (bits_pm [B][OH][OW][O] in {0,1},
    res [B][P][Q][O] after injection, acc before injection)."""
    B, H, W, C = x_pm1.shape
    R, S, _, O = f_pm1.shape
    pad_h, pad_w, OH, OW = conv_shape(H, W, R, S, sh, sw, padding, pool)
    P, Q = pool * OH, pool * OW
    acc = np.zeros((B, P, Q, O), dtype=np.int64)
    for y in range(P):
        for x in range(Q):
            for r in range(R):
                for s in range(S):
                    ay, ax = y * sh - pad_h + r, x * sw - pad_w + s
                    if 0 <= ay < H and 0 <= ax < W:
                        acc[:, y, x, :] += (x_pm1[:, ay, ax, :] @ f_pm1[r, s]).astype(np.int64)
    res = acc.copy()
    if res_in is not None:
        rc = min(residual_channels, O)
        rin = np.zeros(res_in.shape[:-1] + (max(O, res_in.shape[-1]),), dtype=np.int64)
        rin[..., :res_in.shape[-1]] = res_in
        if residual_pool:
            rp = rin.reshape(B, P, 2, Q, 2, -1).max(axis=(2, 4))
            res[..., :rc] += rp[..., :rc]
        else:
            res[..., :rc] += rin[..., :rc]
    bit = ~(res.astype(np.float32) < thr.astype(np.float32)[None, None, None, :])
    pooled = bit.reshape(B, OH, pool, OW, pool, O).any(axis=(2, 4))
    return pooled.astype(np.uint8), res.astype(np.int32), acc.astype(np.int32)


def _mix(i):
    """The counter hash of tcbnn_b200/dropin/synthetic_data.cpp (the stand-in dataset readers the
    reference's drivers are linked with), vectorised: uint64 index array -> uint32."""
    z = i.astype(np.uint64) + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return ((z ^ (z >> np.uint64(31))) >> np.uint64(32)).astype(np.uint32)


def reader_images(kind, batch):
    """The fp32 images those readers hand to the drivers: 'mnist' [B][784], 'cifar' [B][3][32][32],
    'imagenet' [B][3][224][224], same float32 arithmetic as the C++ code."""
    if kind == "mnist":
        n = batch * 784
        v = (_mix(np.arange(n, dtype=np.uint64)) & 0xFF).astype(np.float32)
        return ((v / np.float32(255.0) - np.float32(0.1307)) / np.float32(0.3081)).reshape(batch, 784)
    hw, mean, sd = {"cifar": (32, (0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616)),
                    "imagenet": (224, (0.485, 0.456, 0.406), (0.229, 0.224, 0.225))}[kind]
    n = batch * 3 * hw * hw
    v = (_mix(np.arange(n, dtype=np.uint64)) & 0xFF).astype(np.float32).reshape(batch, 3, hw, hw)
    m = np.array(mean, np.float32).reshape(1, 3, 1, 1)
    s_ = np.array(sd, np.float32).reshape(1, 3, 1, 1)
    return (v / np.float32(255.0) - m) / s_
