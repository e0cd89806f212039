"""CPU-only: pin the oracle against the reference's golden vectors and cross-check the layer
restatements against an independent +-1 formulation."""
import os

import numpy as np
import pytest

import oracle as orc
import util

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _tags(npz, prefix):
    return sorted(k[len(prefix):] for k in npz.files if k.startswith(prefix))


def test_kat_srand4_matches_reference_recipe():
    """srand(4)+rand() inputs, D from the reference's WMMABOOLCPU (main_test.cu:293-299, 350)."""
    z = np.load(os.path.join(GOLD, "wmma_kat_srand4.npz"))
    tags = _tags(z, "A_")
    assert "8x8x128" in tags
    for t in tags:
        k = int(t.split("x")[2])
        got = orc.bgemm_popc(z["A_" + t], z["B_" + t], k) + z["C_" + t]
        assert np.array_equal(got, z["D_" + t]), t


def test_bmma_cpu_reference_outputs():
    z = np.load(os.path.join(GOLD, "bmma_cpu_ref.npz"))
    for t in _tags(z, "A_"):
        k = int(t.split("x")[2])
        assert np.array_equal(orc.bgemm_popc(z["A_" + t], z["B_" + t], k), z["popc_" + t]), t
        # C = K - 2*acc (tensorcore_kernel.cu:331)
        assert np.array_equal(orc.bgemm(z["A_" + t], z["B_" + t], k), k - 2 * z["popc_" + t]), t


def test_live_reference_host_functions_when_available():
    """Where oracle/_ref was built (reference tree present) compare directly, fresh seeds."""
    if orc.ref_lib() is None:
        pytest.skip("reference tree not present on this machine")
    g = util.rng(99)
    for (m, n, k) in [(8, 8, 128), (33, 17, 256), (5, 70, 2048)]:
        A, B = util.rand_words(g, (m, k // 32)), util.rand_words(g, (n, k // 32))
        assert np.array_equal(orc.bgemm_popc(A, B, k), orc.ref_bmma_cpu(A, B, k))


def test_pack_rows_bit_order_and_padding():
    g = util.rng(1)
    x = g.standard_normal((5, 70)).astype(np.float32)
    x[0, 3] = 0.0          # >= 0 -> bit 1 (kernel.cuh:168)
    x[1, 4] = -0.0
    bits = orc.pack_rows(x)
    assert bits.shape == (5, 4)
    exp = util.pm1_to_bits(np.where(x >= 0, 1.0, -1.0).astype(np.float32), 4)
    assert np.array_equal(bits, exp)
    assert np.array_equal(orc.unpack_rows(bits, 70), np.where(x >= 0, 1.0, -1.0))


def test_pack_fc_weight_and_conv_filter():
    g = util.rng(2)
    W = g.standard_normal((100, 12)).astype(np.float32)
    wb = orc.pack_fc_weight(W)
    assert np.array_equal(util.bits_to_pm1(wb, 100), np.where(W.T >= 0, 1.0, -1.0))
    F = g.standard_normal((9, 64, 40)).astype(np.float32)
    fb = orc.pack_conv_filter(F)                       # [O][RS][Cw]
    assert fb.shape == (40, 9, 2)
    assert np.array_equal(util.bits_to_pm1(fb, 64), np.where(F.transpose(2, 0, 1) >= 0, 1.0, -1.0))


@pytest.mark.parametrize("M,K,N", [(8, 128, 8), (19, 200, 37), (64, 784, 100)])
def test_fc_and_out_layer_against_pm1(M, K, N):
    g = util.rng(M * 1000 + K)
    a = util.rand_pm1(g, (M, K))
    w = util.rand_pm1(g, (K, N))
    thr = (g.standard_normal(N) * np.sqrt(K)).astype(np.float32)
    thr[0] = 0.0
    A, Wb = orc.pack_rows(a), orc.pack_fc_weight(w)
    dot = (a @ w).astype(np.int32)
    assert np.array_equal(orc.bgemm(A, Wb, K), dot)
    bits = orc.fc_layer(A, Wb, thr, K)
    exp = (dot.astype(np.float32) >= thr[None, :])
    assert np.array_equal(util.bits_to_pm1(bits, N) > 0, exp)
    assert not np.any(util.mask_row_pad(bits, N) != bits)        # pad bits stay 0
    scale = g.standard_normal(N).astype(np.float32)
    bias = g.standard_normal(N).astype(np.float32)
    out = orc.out_layer(A, Wb, scale, bias, K)
    ref = dot.astype(np.float64) * scale.astype(np.float64) + bias.astype(np.float64)
    np.testing.assert_allclose(out, ref, rtol=1e-6, atol=1e-6)


CONV_CASES = [
    # B, H, W, C, O, R, S, sh, sw, padding, pool, residual mode
    (2, 6, 6, 64, 32, 3, 3, 1, 1, True, 1, None),
    (2, 8, 8, 64, 64, 3, 3, 1, 1, True, 2, None),
    (1, 9, 7, 128, 40, 3, 3, 2, 2, True, 1, None),
    (2, 6, 6, 64, 64, 3, 3, 1, 1, True, 1, "plain"),
    (2, 4, 4, 64, 128, 3, 3, 1, 1, True, 1, "pool"),
    (1, 7, 7, 64, 32, 5, 5, 1, 1, True, 1, None),
    (1, 8, 8, 64, 32, 3, 3, 1, 1, False, 1, None),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_layer_against_pm1(case):
    B, H, W, C, O, R, S, sh, sw, padding, pool, resmode = case
    g = util.rng(hash(case[:9]) & 0xFFFF)
    x = util.rand_pm1(g, (B, H, W, C))
    f = util.rand_pm1(g, (R, S, C, O))
    thr = (g.standard_normal(O) * np.sqrt(C * R * S) * 0.5).astype(np.float32)
    xb = util.pm1_to_bits(x)
    fb = orc.pack_conv_filter(f.reshape(R * S, C, O))
    pad_h, pad_w, OH, OW = util.conv_shape(H, W, R, S, sh, sw, padding, pool)
    res_in, rc, rpool = None, 0, False
    if resmode == "plain":
        res_in = g.integers(-300, 300, size=(B, OH, OW, 48)).astype(np.int32)
        rc = 64
    elif resmode == "pool":
        res_in = g.integers(-300, 300, size=(B, 2 * OH, 2 * OW, 64)).astype(np.int32)
        rc, rpool = 64, True
    out, res, acc = orc.conv_layer(xb, fb, thr, C, R, S, sh, sw, padding, pool, res_in=res_in,
                                   residual_channels=rc, residual_pool=rpool,
                                   save_residual=True, want_acc=True)
    ebits, eres, eacc = util.conv_pm1_reference(x, f, thr, sh, sw, padding, pool, res_in, rc, rpool)
    assert np.array_equal(acc, eacc)
    assert np.array_equal(res, eres)
    Ow = (O + 31) // 32
    got = util.bits_to_pm1(out.reshape(B, OH, OW, Ow), O) > 0
    assert np.array_equal(got, ebits.astype(bool))


def test_conv_shape_matches_reference_arithmetic():
    # ResNet stem 224 / 7x7 / stride 4 -> pad 3, 56x56 (imagenet_resnet.cu:223-224)
    g = orc.conv_shape(224, 224, 7, 7, 4, 4, True, 1)
    assert (g["pad_h"], g["OH"], g["OW"]) == (3, 56, 56)
    g = orc.conv_shape(56, 56, 3, 3, 2, 2, True, 1)
    assert (g["pad_h"], g["OH"]) == (1, 28)
    g = orc.conv_shape(32, 32, 3, 3, 1, 1, True, 2)
    assert (g["pad_h"], g["OH"], g["P"]) == (1, 16, 32)
    for a in [(13, 11, 3, 3, 2, 2, True, 2), (8, 8, 5, 5, 1, 1, False, 1)]:
        pad_h, pad_w, OH, OW = util.conv_shape(*a)
        g = orc.conv_shape(*a)
        assert (g["pad_h"], g["pad_w"], g["OH"], g["OW"]) == (pad_h, pad_w, OH, OW)


def test_inconv_layer_order_and_truncation():
    """fp32 first layer: same add order as kernel.cuh:636-638, residual truncated (:666-668)."""
    g = util.rng(5)
    B, H, W, O, R, S = 2, 9, 9, 40, 3, 3
    x = g.standard_normal((B, 3, H, W)).astype(np.float32)
    F = g.standard_normal((R * S, 3, O)).astype(np.float32)
    thr = g.standard_normal(O).astype(np.float32)
    out, res, acc = orc.inconv_layer(x, F, thr, R, S, 2, 2, True, 1, save_residual=True, want_acc=True)
    pad_h, pad_w, OH, OW = util.conv_shape(H, W, R, S, 2, 2, True, 1)
    sg = np.where(F >= 0, np.float32(1), np.float32(-1))
    exp = np.zeros((B, OH, OW, O), dtype=np.float32)
    for y in range(OH):
        for xq in range(OW):
            a = np.zeros((B, O), dtype=np.float32)
            for r in range(R):
                for s in range(S):
                    ay, ax = y * 2 - pad_h + r, xq * 2 - pad_w + s
                    if 0 <= ay < H and 0 <= ax < W:
                        t = (sg[r * S + s, 0][None] * x[:, 0, ay, ax][:, None]
                             + sg[r * S + s, 1][None] * x[:, 1, ay, ax][:, None])
                        t = t + sg[r * S + s, 2][None] * x[:, 2, ay, ax][:, None]
                        a = a + t
            exp[:, y, xq] = a
    assert np.array_equal(acc, exp)
    assert np.array_equal(res, np.trunc(exp).astype(np.int32))
    Ow = (O + 31) // 32
    got = util.bits_to_pm1(out.reshape(B, OH, OW, Ow), O) > 0
    assert np.array_equal(got, ~(exp < thr[None, None, None, :]))
