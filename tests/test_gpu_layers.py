"""GPU parity: every C-ABI entry point against the CPU oracle on the same seeded inputs.
Bit-exact for packed tensors and int32 values; fp32 logits within 1e-5 relative."""
import numpy as np
import pytest
import torch

import oracle as orc
import util
from tcbnn_b200 import ops

pytestmark = pytest.mark.gpu


def dev(a, cuda):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).to(cuda)


def host_u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 70), (64, 784), (33, 1000), (8, 4096), (20000, 260), (777, 130)])
def test_pack_unpack_rows(cuda, rows, cols):
    g = util.rng(rows * 7 + cols)
    x = g.standard_normal((rows, cols)).astype(np.float32)
    x[0, 0] = 0.0
    bits = ops.pack_rows(dev(x, cuda))
    assert np.array_equal(host_u32(bits), orc.pack_rows(x))
    back = ops.unpack_rows(bits, cols).cpu().numpy()
    assert np.array_equal(back, orc.unpack_rows(orc.pack_rows(x), cols))


def test_pack_weights_and_filters(cuda):
    g = util.rng(3)
    W = g.standard_normal((200, 37)).astype(np.float32)
    assert np.array_equal(host_u32(ops.pack_fc_weight(dev(W, cuda))), orc.pack_fc_weight(W))
    F = g.standard_normal((9, 192, 40)).astype(np.float32)
    assert np.array_equal(host_u32(ops.pack_conv_filter(dev(F, cuda))), orc.pack_conv_filter(F))


GEMM_SHAPES = [(8, 8, 128), (32, 32, 256), (33, 17, 200), (100, 70, 784), (256, 128, 4096),
               (64, 10, 1024), (40, 1000, 512), (1024, 1024, 4096)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("split", [False, True])
def test_bgemm_fc_out(cuda, M, N, K, split):
    g = util.rng(M + 3 * N + 7 * K)
    ld = orc.step128_words(K)
    A = util.mask_row_pad(util.rand_words(g, (M, ld)), K)
    W = util.mask_row_pad(util.rand_words(g, (N, ld)), K)
    thr = (g.standard_normal(N) * np.sqrt(K)).astype(np.float32)
    scale = g.standard_normal(N).astype(np.float32)
    bias = g.standard_normal(N).astype(np.float32)
    dA, dW = dev(A, cuda), dev(W, cuda)
    ws = None
    if split:
        # force a split by handing over a generous workspace; small shapes may still not split
        ws = torch.empty((32 * M * N,), dtype=torch.int32, device=cuda)
    Cg = ops.bgemm(dA, dW, K, workspace=ws).cpu().numpy()
    assert np.array_equal(Cg, orc.bgemm(A, W, K))
    bits = ops.fc_layer(dA, dW, dev(thr, cuda), K, workspace=ws)
    assert np.array_equal(host_u32(bits), orc.fc_layer(A, W, thr, K))
    out = ops.out_layer(dA, dW, dev(scale, cuda), dev(bias, cuda), K, workspace=ws).cpu().numpy()
    ref = orc.out_layer(A, W, scale, bias, K)
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5)


UMMA_GEMM_CASES = [
    # M, N, K, pair, splits: large enough for the tcgen05 GEMM (M*N*K >= 2^30, less with a forced
    # plan), ragged on purpose.
    # pair / splits force the tile shape (1: 256 x 128, 0: 128 x 128) and the number of K slices
    # (1: the GEMM's own epilogue finishes the layer; more: partial sums and a finishing pass);
    # -1 leaves the choice to the library's cost model.
    (300, 200, 40010, -1, -1),      # partial row tiles, K not a multiple of 32
    (300, 200, 40010, 1, 1),
    (300, 200, 40010, 0, 7),
    (1024, 512, 25088, -1, -1),     # the ResNet-18 FC layer
    (129, 64, 300000, -1, -1),      # one full + one almost empty row tile, very long K
    (129, 64, 300000, 1, 32),
    (512, 1000, 4200, -1, -1),      # N not a multiple of 128
    (256, 130, 65536, -1, -1),      # N not a multiple of 4: scalar stores
    (256, 130, 65536, 0, 1),
    (256, 130, 65536, 1, 5),
    (1024, 1024, 4096, -1, -1),     # the standalone bit-GEMM benchmark shape
    (8192, 1024, 1024, -1, -1),     # an MLP hidden layer
    (2100, 1000, 1030, 0, 1),       # ragged in M, N (not a multiple of 32) and K
    (2100, 1000, 1030, 1, 1),
    (2100, 1000, 1030, 1, 2),
    (2050, 130, 1500, 0, 1),
    (140, 66, 30000, 1, 1),         # a 256-row tile whose second half is nearly empty
    (128, 64, 32768, 0, 3),         # a single tile
    (128, 64, 32768, 1, 1),         # a pair tile without a second half
    (1000, 520, 576, 0, 1),         # K = 9 k-blocks: stages of 4, 4 and 1
    (1000, 520, 576, 1, 2),         # splits of 5 and 4 k-blocks
]


@pytest.mark.parametrize("M,N,K,pair,splits", UMMA_GEMM_CASES)
def test_gemm_family_on_tcgen05_matches_oracle_and_b1_kernel(cuda, M, N, K, pair, splits):
    g = util.rng(M + 3 * N + 7 * K)
    ld = orc.step128_words(K)
    A = util.mask_row_pad(util.rand_words(g, (M, ld)), K)
    W = util.mask_row_pad(util.rand_words(g, (N, ld)), K)
    thr = (g.standard_normal(N) * np.sqrt(K)).astype(np.float32)
    scale = g.standard_normal(N).astype(np.float32)
    bias = g.standard_normal(N).astype(np.float32)
    dA, dW = dev(A, cuda), dev(W, cuda)
    ref = orc.bgemm(A, W, K)
    try:
        ops.set_gemm_plan(pair, splits)
        ws = ops.gemm_workspace(M, N, K, cuda)
        assert ws is not None and ws.numel() * 4 >= (M + N) * K // 2     # room for both operands as nibbles
        launches = ops.gemm_launches(M, N, K, ws)
        assert launches in (2, 3)                                        # i.e. the tcgen05 path
        if splits > 0:
            assert launches == (2 if splits == 1 else 3)
        for path in (0, 1):
            ops.set_gemm_path(path)
            assert np.array_equal(ops.bgemm(dA, dW, K, workspace=ws).cpu().numpy(), ref), path
            bits = ops.fc_layer(dA, dW, dev(thr, cuda), K, workspace=ws)
            assert np.array_equal(host_u32(bits), orc.fc_layer(A, W, thr, K)), path
            out = ops.out_layer(dA, dW, dev(scale, cuda), dev(bias, cuda), K, workspace=ws).cpu().numpy()
            np.testing.assert_allclose(out, orc.out_layer(A, W, scale, bias, K), rtol=1e-5, atol=1e-5)
            assert ops.gemm_status() == 0
    finally:
        ops.set_gemm_path(0)
        ops.set_gemm_plan(-1, -1)


def test_gemm_kat_srand4(cuda):
    """The reference's seeded known-answer recipe, through the GPU path."""
    import os
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "wmma_kat_srand4.npz"))
    for t in sorted(k[2:] for k in z.files if k.startswith("A_")):
        m, n, k = (int(v) for v in t.split("x"))
        ld = orc.step128_words(k)
        A = np.zeros((m, ld), np.uint32); A[:, :k // 32] = z["A_" + t]
        B = np.zeros((n, ld), np.uint32); B[:, :k // 32] = z["B_" + t]
        Cg = ops.bgemm(dev(A, cuda), dev(B, cuda), k).cpu().numpy()      # K - 2*popc
        popc = (k - Cg) // 2
        assert np.array_equal(popc + z["C_" + t], z["D_" + t]), t


CONV_CASES = [
    # B, H, W, C, O, R, S, sh, sw, padding, pool, residual
    (2, 6, 6, 64, 32, 3, 3, 1, 1, True, 1, None),
    (3, 8, 8, 64, 64, 3, 3, 1, 1, True, 2, None),
    (1, 9, 7, 128, 40, 3, 3, 2, 2, True, 1, None),
    (2, 6, 6, 64, 64, 3, 3, 1, 1, True, 1, "plain"),
    (2, 4, 4, 64, 128, 3, 3, 1, 1, True, 1, "pool"),
    (1, 7, 7, 64, 32, 5, 5, 1, 1, True, 1, None),
    (1, 8, 8, 64, 32, 3, 3, 1, 1, False, 1, None),
    (5, 14, 14, 256, 256, 3, 3, 1, 1, True, 1, "plain"),
    (4, 14, 14, 128, 256, 3, 3, 2, 2, True, 1, None),
    (3, 7, 7, 512, 512, 3, 3, 1, 1, True, 1, "plain"),
    (2, 13, 13, 192, 384, 3, 3, 1, 1, True, 1, None),
    (2, 28, 28, 64, 192, 5, 5, 1, 1, True, 2, None),
    (2, 9, 9, 64, 64, 3, 3, 1, 1, True, 2, None),
    (8, 56, 56, 64, 64, 3, 3, 1, 1, True, 1, "plain"),
    (4, 32, 32, 128, 128, 3, 3, 1, 1, True, 2, None),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_layer(cuda, case):
    B, H, W, C, O, R, S, sh, sw, padding, pool, resmode = case
    g = util.rng(hash(case[:9]) & 0xFFFF)
    Cw = (C + 31) // 32
    x = util.rand_words(g, (B, H, W, Cw))
    f = util.rand_words(g, (O, R * S, Cw))
    thr = (g.standard_normal(O) * np.sqrt(C * R * S) * 0.5).astype(np.float32)
    pad_h, pad_w, OH, OW = util.conv_shape(H, W, R, S, sh, sw, padding, pool)
    res_in, rc, rpool = None, 0, False
    if resmode == "plain":
        res_in = g.integers(-300, 300, size=(B, OH, OW, max(32, O // 2))).astype(np.int32)
        rc = O
    elif resmode == "pool":
        res_in = g.integers(-300, 300, size=(B, 2 * OH, 2 * OW, O // 2)).astype(np.int32)
        rc, rpool = O // 2, True
    Ow = (O + 31) // 32
    stride = OH * OW * Ow + 4            # padded image stride, like an ahead_fc layer
    eo, er, ea = orc.conv_layer(x, f, thr, C, R, S, sh, sw, padding, pool, res_in=res_in,
                                residual_channels=rc, residual_pool=rpool, out_image_stride=stride,
                                save_residual=(pool == 1), want_acc=True)
    d = ops.conv_desc(B, H, W, C, O, R, S, sh, sw, padding, pool)
    assert (d.pad_h, d.pad_w, d.OH, d.OW) == (pad_h, pad_w, OH, OW)
    prep = ops.conv_prepare(d, dev(f, cuda))
    go, gr, ga = ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda),
                                res_in=dev(res_in, cuda) if res_in is not None else None,
                                residual_channels=rc, residual_pool=rpool, out_image_stride=stride,
                                save_residual=(pool == 1), want_acc=True)
    assert np.array_equal(ga.cpu().numpy(), ea)
    if pool == 1:
        assert np.array_equal(gr.cpu().numpy(), er)
    assert np.array_equal(host_u32(go), eo)
    # running the layer again on the same buffers gives the same bits (stores, not ORs)
    go2, _, _ = ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda),
                               res_in=dev(res_in, cuda) if res_in is not None else None,
                               residual_channels=rc, residual_pool=rpool, out=go,
                               out_image_stride=stride)
    assert np.array_equal(host_u32(go2), eo)


INCONV_CASES = [
    (2, 9, 9, 40, 3, 3, 2, 2, 1),
    (2, 32, 32, 128, 3, 3, 1, 1, 1),
    (2, 64, 64, 64, 7, 7, 4, 4, 1),
    (1, 48, 48, 64, 11, 11, 4, 4, 2),
]


@pytest.mark.parametrize("case", INCONV_CASES)
def test_inconv_layer(cuda, case):
    B, H, W, O, R, S, sh, sw, pool = case
    g = util.rng(sum(case))
    x = g.standard_normal((B, 3, H, W)).astype(np.float32)
    F = g.standard_normal((R * S, 3, O)).astype(np.float32)
    thr = (g.standard_normal(O) * 3).astype(np.float32)
    eo, er, ea = orc.inconv_layer(x, F, thr, R, S, sh, sw, True, pool, save_residual=True, want_acc=True)
    d = ops.conv_desc(B, H, W, 3, O, R, S, sh, sw, True, pool)
    fb = ops.pack_inconv_filter(dev(F, cuda))
    go, gr, ga = ops.inconv_layer(d, dev(x, cuda), fb, dev(thr, cuda), save_residual=True, want_acc=True)
    assert np.array_equal(ga.cpu().numpy(), ea)          # fp32 sums bit-exact (same add order)
    assert np.array_equal(gr.cpu().numpy(), er)
    assert np.array_equal(host_u32(go), eo)


SPEC_CASES = INCONV_CASES + [
    (3, 20, 20, 16, 5, 5, 1, 1, 2),
    (2, 16, 16, 96, 3, 3, 1, 1, 2),      # two channel groups, the second one half full; pooled
    (5, 30, 28, 64, 7, 7, 4, 4, 1),      # odd output sizes, several blocks of pixels
]


@pytest.mark.parametrize("case", SPEC_CASES)
def test_inconv_layer_specialized_kernel(cuda, case):
    """The first-layer kernel compiled for one filter against the oracle: fp32 images, uint8
    images with their value table, int32 and int16 residuals, and a batch size other than the
    one it was built with."""
    B, H, W, O, R, S, sh, sw, pool = case
    g = util.rng(sum(case) + 5)
    F = g.standard_normal((R * S, 3, O)).astype(np.float32)
    thr = (g.standard_normal(O) * 3).astype(np.float32)
    thr[0] = np.nan                                                   # never "less than": bit always set
    fb = ops.pack_inconv_filter(dev(F, cuda))
    d = ops.conv_desc(B, H, W, 3, O, R, S, sh, sw, True, pool)
    spec = ops.inconv_specialize(d, fb, dev(thr, cuda))
    for batch in (B, B + 3):
        x = g.standard_normal((batch, 3, H, W)).astype(np.float32)
        eo, er, ea = orc.inconv_layer(x, F, thr, R, S, sh, sw, True, pool, save_residual=True, want_acc=True)
        db = ops.conv_desc(batch, H, W, 3, O, R, S, sh, sw, True, pool)
        go, gr, ga = ops.inconv_layer(db, dev(x, cuda), fb, dev(thr, cuda), save_residual=True, want_acc=True,
                                      specialized=spec)
        assert np.array_equal(ga.cpu().numpy(), ea)
        assert np.array_equal(gr.cpu().numpy(), er)
        assert np.array_equal(host_u32(go), eo)
        go, gr, _ = ops.inconv_layer(db, dev(x, cuda), fb, dev(thr, cuda), save_residual=True,
                                     residual_dtype=torch.int16, specialized=spec)
        assert np.array_equal(gr.cpu().numpy().astype(np.int32), er)
        assert np.array_equal(host_u32(go), eo)
    # uint8 images: the table plays the reader's normalisation
    x8 = g.integers(0, 256, size=(B, 3, H, W)).astype(np.uint8)
    lut = ((np.arange(256, dtype=np.float32)[None, :] / 255.0 - np.array([[0.4], [0.5], [0.45]], np.float32))
           / np.array([[0.2], [0.25], [0.22]], np.float32)).astype(np.float32)
    xf = np.stack([lut[c][x8[:, c]] for c in range(3)], axis=1)
    eo, er, ea = orc.inconv_layer(xf, F, thr, R, S, sh, sw, True, pool, save_residual=True, want_acc=True)
    go, gr, ga = ops.inconv_layer(d, dev(x8, cuda), fb, dev(thr, cuda), save_residual=True, want_acc=True,
                                  lut=dev(lut, cuda), specialized=spec)
    assert np.array_equal(ga.cpu().numpy(), ea)
    assert np.array_equal(gr.cpu().numpy(), er)
    assert np.array_equal(host_u32(go), eo)
    spec.release()


def test_inconv_specialize_rejects_wide_layers_and_mismatched_descriptors(cuda):
    from tcbnn_b200.lib import TcbnnError
    d = ops.conv_desc(1, 8, 8, 3, 160, 3, 3)
    fb = torch.zeros((9, 3, 5), dtype=torch.int32, device=cuda)
    thr = torch.zeros((160,), device=cuda)
    with pytest.raises(TcbnnError):
        ops.inconv_specialize(d, fb, thr)
    d = ops.conv_desc(1, 8, 8, 3, 32, 3, 3)
    spec = ops.inconv_specialize(d, torch.zeros((9, 3, 1), dtype=torch.int32, device=cuda), thr[:32].contiguous())
    other = ops.conv_desc(1, 8, 8, 3, 32, 5, 5)
    with pytest.raises(TcbnnError):
        ops.inconv_layer(other, torch.zeros((1, 3, 8, 8), device=cuda), None, None, specialized=spec)


def test_int16_residual_overflow_is_flagged(cuda):
    """A residual that does not fit the int16 element size the caller chose sets status 2."""
    g = util.rng(77)
    B, H, W, C, O = 1, 4, 4, 64, 64
    x = util.rand_words(g, (B, H, W, 2))
    f = util.rand_words(g, (O, 9, 2))
    thr = np.zeros(O, np.float32)
    res_in = np.full((B, H, W, O), 40000, np.int32)
    d = ops.conv_desc(B, H, W, C, O, 3, 3)
    prep = ops.conv_prepare(d, dev(f, cuda))
    ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda), res_in=dev(res_in, cuda),
                   residual_channels=O, save_residual=True, residual_dtype=torch.int16)
    assert ops.conv_status(d, prep) == 2


def test_bad_arguments_are_rejected(cuda):
    from tcbnn_b200.lib import TcbnnError
    A = torch.zeros((8, 3), dtype=torch.int32, device=cuda)      # odd leading dimension
    with pytest.raises(TcbnnError):
        ops.bgemm(A, A, 96)
    with pytest.raises(TcbnnError):
        ops.conv_desc(1, 8, 8, 64, 64, 3, 3, pool=0)
    d = ops.conv_desc(1, 8, 8, 32, 64, 3, 3)                     # odd word count per pixel
    with pytest.raises(TcbnnError):
        ops.conv_prepare(d, torch.zeros((64, 9, 1), dtype=torch.int32, device=cuda))


UMMA_CASES = [
    # B, H, W, C, O, R, residual[, stride]   ("same" padding, no pooling: tcgen05-eligible)
    (2, 8, 8, 64, 128, 3, None, 2),
    (3, 14, 14, 128, 256, 3, None, 2),
    (2, 7, 9, 64, 64, 3, None, 2),           # odd sizes under stride 2
    (9, 14, 14, 256, 512, 3, None, 2),
    (300, 7, 7, 512, 64, 3, None),           # 8 channel blocks per tile, many tiles per CTA
    (1, 4, 4, 64, 64, 3, None),
    (2, 6, 6, 64, 64, 3, "plain"),
    (2, 4, 4, 64, 128, 3, "pool"),
    (3, 10, 12, 128, 128, 3, None),
    (2, 9, 9, 64, 64, 5, None),
    (5, 7, 7, 128, 64, 3, "plain"),
    (4, 56, 56, 64, 64, 3, "plain"),
    (8, 28, 28, 128, 128, 3, "pool"),
    (130, 3, 5, 64, 64, 3, None),          # many tiny images per tile
    (6, 14, 14, 256, 256, 3, "plain"),
    (5, 7, 7, 512, 512, 3, "pool"),
    (3, 7, 7, 512, 64, 3, None),
    (2, 8, 8, 256, 96, 3, None),
    # wide stride-1 layers: the activation-stationary tcgen05 kernel (path 2) and the
    # filter-stationary one (path 3)
    (40, 14, 14, 256, 256, 3, "plain"),     # many 256-position tasks
    (70, 7, 7, 512, 512, 3, "plain"),       # 8 channel blocks, 4 n-tiles
    (3, 9, 9, 256, 128, 5, None),           # 5x5 filter, one n-tile
    (2, 14, 14, 384, 256, 3, "pool"),       # 6 channel blocks
    (1, 3, 3, 256, 128, 3, None),           # a single partial task
    (2, 28, 28, 512, 128, 3, None),         # 512 channels at 28 x 28: patch leaves room for a 2-group filter ring only
    (1, 40, 200, 64, 64, 3, "plain"),       # rows too wide for the in-CTA expansion: loader-fed kernel only
]


@pytest.mark.parametrize("case", UMMA_CASES)
def test_conv_layer_tcgen05_and_b1_paths_agree_with_oracle(cuda, case):
    """The conv kernels (tcgen05 implicit GEMM on 4-bit and on int8 operands, warp-level b1 MMA) and
    the epilogue variants of the loader-fed one against the oracle."""
    B, H, W, C, O, R, resmode = case[:7]
    st = case[7] if len(case) > 7 else 1
    g = util.rng(sum(case[:6]))
    Cw = C // 32
    x = util.rand_words(g, (B, H, W, Cw))
    f = util.rand_words(g, (O, R * R, Cw))
    thr = (g.standard_normal(O) * np.sqrt(C * R * R) * 0.5).astype(np.float32)
    res_in, rc, rpool = None, 0, False
    if resmode == "plain":
        res_in = g.integers(-300, 300, size=(B, H, W, O)).astype(np.int32)
        rc = O
    elif resmode == "pool":
        res_in = g.integers(-300, 300, size=(B, 2 * H, 2 * W, O // 2)).astype(np.int32)
        rc, rpool = O // 2, True
    eo, er, ea = orc.conv_layer(x, f, thr, C, R, R, st, st, True, 1, res_in=res_in,
                                residual_channels=rc, residual_pool=rpool,
                                save_residual=True, want_acc=True)
    d = ops.conv_desc(B, H, W, C, O, R, R, st, st)
    prep = ops.conv_prepare(d, dev(f, cuda))
    try:
        # 5x5 filters over 256 channels do not fit the filter-stationary kernel's shared memory
        # ... and 200-pixel rows do not fit its patch
        # path 5: automatic choice with the int16 residual rows staged in shared memory wherever possible
        for path in ((2, 5, 1) if ((R == 5 and C >= 256) or W >= 160) else (2, 5, 3, 1)):
            ops.set_conv_path(path)
            go, gr, ga = ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda),
                                        res_in=dev(res_in, cuda) if res_in is not None else None,
                                        residual_channels=rc, residual_pool=rpool,
                                        save_residual=True, want_acc=True)
            assert ops.conv_status(d, prep) == 0
            assert np.array_equal(ga.cpu().numpy(), ea), path
            assert np.array_equal(gr.cpu().numpy(), er), path
            assert np.array_equal(host_u32(go), eo), path
            # int16 residual tensors in and out: same values
            r16 = dev(res_in.astype(np.int16), cuda) if res_in is not None else None
            go, gr, _ = ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda), res_in=r16,
                                       residual_channels=rc, residual_pool=rpool,
                                       save_residual=True, residual_dtype=torch.int16)
            assert gr.dtype == torch.int16 and ops.conv_status(d, prep) == 0
            assert np.array_equal(gr.cpu().numpy().astype(np.int32), er), path
            assert np.array_equal(host_u32(go), eo), path
    finally:
        ops.set_conv_path(0)


HANDOVER_CASES = [
    # producer (C, O, stride), consumer O: the consumer has C = producer's O and at most 128 of them
    (64, 64, 1, 64),        # loader-fed kernel writes the planes (16 columns per thread)
    (128, 128, 1, 128),     # the same, 32 columns per thread
    (64, 128, 2, 128),      # stride-2 filter-stationary kernel writes them
    (256, 128, 1, 64),      # activation-stationary kernel cannot: followed by the expansion pass
]


@pytest.mark.parametrize("case", HANDOVER_CASES)
def test_conv_layer_hands_its_output_to_the_next_layer(cuda, case):
    """tcbnn_conv_layer_x: the producer writes the consumer's pre-expanded input, the consumer
    skips its expansion pass; both layers against the oracle."""
    C1, O1, st, O2 = case
    B, H = 3, 12
    g = util.rng(sum(case) + 11)
    x = util.rand_words(g, (B, H, H, C1 // 32))
    f1 = util.rand_words(g, (O1, 9, C1 // 32))
    f2 = util.rand_words(g, (O2, 9, O1 // 32))
    t1 = (g.standard_normal(O1) * np.sqrt(C1 * 9) * 0.5).astype(np.float32)
    t2 = (g.standard_normal(O2) * np.sqrt(O1 * 9) * 0.5).astype(np.float32)
    e1, _, _ = orc.conv_layer(x, f1, t1, C1, 3, 3, st, st, True, 1)
    H2 = H // st
    e2, _, _ = orc.conv_layer(e1.reshape(B, H2, H2, O1 // 32), f2, t2, O1, 3, 3, 1, 1, True, 1)
    d1 = ops.conv_desc(B, H, H, C1, O1, 3, 3, st, st)
    d2 = ops.conv_desc(B, H2, H2, O1, O2, 3, 3)
    p1, p2 = ops.conv_prepare(d1, dev(f1, cuda)), ops.conv_prepare(d2, dev(f2, cuda))
    planes = ops.new_planes(d2, cuda)
    assert planes is not None
    for _ in range(2):                      # a second pass over the same planes gives the same result
        o1, _, _ = ops.conv_layer(d1, dev(x, cuda), p1, dev(t1, cuda), next_layer=(d2, planes))
        o2, _, _ = ops.conv_layer(d2, o1.view(B, H2, H2, O1 // 32), p2, dev(t2, cuda),
                                  workspace=planes, workspace_ready=True)
        assert ops.conv_status(d1, p1) == 0 and ops.conv_status(d2, p2) == 0
        assert np.array_equal(host_u32(o1), e1)
        assert np.array_equal(host_u32(o2), e2)


def test_specialized_first_layer_hands_its_output_to_the_next_layer(cuda):
    g = util.rng(4711)
    B, H, O1, O2 = 3, 32, 64, 64
    x = g.standard_normal((B, 3, H, H)).astype(np.float32)
    F = g.standard_normal((49, 3, O1)).astype(np.float32)
    t1 = (g.standard_normal(O1) * 3).astype(np.float32)
    f2 = util.rand_words(g, (O2, 9, O1 // 32))
    t2 = (g.standard_normal(O2) * np.sqrt(O1 * 9) * 0.5).astype(np.float32)
    e1, _, _ = orc.inconv_layer(x, F, t1, 7, 7, 4, 4, True, 1)
    e2, _, _ = orc.conv_layer(e1.reshape(B, 8, 8, O1 // 32), f2, t2, O1, 3, 3, 1, 1, True, 1)
    d1 = ops.conv_desc(B, H, H, 3, O1, 7, 7, 4, 4)
    d2 = ops.conv_desc(B, 8, 8, O1, O2, 3, 3)
    fb = ops.pack_inconv_filter(dev(F, cuda))
    spec = ops.inconv_specialize(d1, fb, dev(t1, cuda))
    p2 = ops.conv_prepare(d2, dev(f2, cuda))
    planes = ops.new_planes(d2, cuda)
    o1, _, _ = ops.inconv_layer(d1, dev(x, cuda), fb, dev(t1, cuda), specialized=spec, next_layer=(d2, planes))
    o2, _, _ = ops.conv_layer(d2, o1.view(B, 8, 8, O1 // 32), p2, dev(t2, cuda), workspace=planes, workspace_ready=True)
    assert np.array_equal(host_u32(o1), e1)
    assert np.array_equal(host_u32(o2), e2)
    from tcbnn_b200.lib import TcbnnError
    with pytest.raises(TcbnnError):         # a consumer of another shape is refused
        ops.inconv_layer(d1, dev(x, cuda), fb, dev(t1, cuda), specialized=spec,
                         next_layer=(ops.conv_desc(B, 16, 16, O1, O2, 3, 3), planes))


POOLED_UMMA_CASES = [
    # B, H, W, C, O, stride: 2x2 OR-pooled layers on the tcgen05 kernels (pre-pool grid + pooling pass)
    (4, 16, 16, 128, 128, 1),      # loader-fed kernel
    (3, 8, 8, 256, 256, 1),        # activation-stationary kernel
    (2, 16, 12, 64, 128, 2),       # stride-2 filter-stationary kernel
    (5, 6, 10, 64, 64, 1),
    (1, 24, 224, 64, 64, 1),       # VGG-16's second layer: 224-pixel rows, loader-fed kernel only
]


@pytest.mark.parametrize("case", POOLED_UMMA_CASES)
def test_pooled_conv_layer_on_tcgen05_matches_oracle(cuda, case):
    B, H, W, C, O, st = case
    g = util.rng(sum(case) + 3)
    x = util.rand_words(g, (B, H, W, C // 32))
    f = util.rand_words(g, (O, 9, C // 32))
    thr = (g.standard_normal(O) * np.sqrt(C * 9) * 0.5).astype(np.float32)
    eo, _, ea = orc.conv_layer(x, f, thr, C, 3, 3, st, st, True, 2, want_acc=True)
    d = ops.conv_desc(B, H, W, C, O, 3, 3, st, st, True, 2)
    prep = ops.conv_prepare(d, dev(f, cuda))
    try:
        for path in ((2, 1, 0) if W >= 160 else (2, 3, 1, 0)):
            ops.set_conv_path(path)
            go, _, ga = ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda), want_acc=True)
            assert ops.conv_status(d, prep) == 0
            assert np.array_equal(ga.cpu().numpy(), ea), path
            assert np.array_equal(host_u32(go), eo), path
        ops.set_conv_path(2)
        from tcbnn_b200.lib import TcbnnError
        with pytest.raises(TcbnnError):          # no room for the pre-pool bits: not on this path
            ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda), workspace=False)
    finally:
        ops.set_conv_path(0)


def test_tcgen05_path_refuses_ineligible_layer(cuda):
    from tcbnn_b200.lib import TcbnnError
    d = ops.conv_desc(1, 8, 8, 64, 64, 3, 3, padding=False)    # "valid" padding stays on the b1 MMA kernel
    f = torch.zeros((64, 9, 2), dtype=torch.int32, device=cuda)
    prep = ops.conv_prepare(d, f)
    x = torch.zeros((1, 8, 8, 2), dtype=torch.int32, device=cuda)
    thr = torch.zeros((64,), device=cuda)
    try:
        ops.set_conv_path(2)
        with pytest.raises(TcbnnError):
            ops.conv_layer(d, x, prep, thr)
    finally:
        ops.set_conv_path(0)


def test_bounded_wait_gives_up_and_the_context_stays_usable(cuda):
    """A wait on a barrier nobody arrives at runs out after its poll limit, the kernel records
    status 1, frees its tensor memory and returns (tcbnn_wait_probe runs that path of the tcgen05
    kernels in isolation); the next tcgen05 convolution on the same context is bit-exact and
    reports status 0."""
    import ctypes as C
    from tcbnn_b200 import lib
    st = C.c_int(-1)
    lib.call("tcbnn_wait_probe", 1 << 16, C.byref(st))
    assert st.value == 1
    g = util.rng(99)
    B, H, Cc, O = 2, 12, 64, 64
    x = util.rand_words(g, (B, H, H, Cc // 32))
    f = util.rand_words(g, (O, 9, Cc // 32))
    thr = (g.standard_normal(O) * 24).astype(np.float32)
    d = ops.conv_desc(B, H, H, Cc, O, 3, 3)
    prep = ops.conv_prepare(d, dev(f, cuda))
    try:
        ops.set_conv_path(2)
        out, _, _ = ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda))
    finally:
        ops.set_conv_path(0)
    eb, _, _ = orc.conv_layer(x, f, thr, Cc, 3, 3)
    assert np.array_equal(host_u32(out).reshape(eb.shape), eb)
    assert ops.conv_status(d, prep) == 0
    lib.call("tcbnn_wait_probe", 1 << 10, C.byref(st))       # and once more after real work
    assert st.value == 1


CHUNKED_CASES = [
    # B, H, W, C, O, residual: "plain" (same grid), "pool" (2x2 max of a [2H][2W][O/2] tensor) or
    # "none" (no residual in; the layer still saves one)
    (3, 9, 11, 64, 64, "plain"),        # n-tile 64, two images straddle tiles
    (2, 56, 56, 64, 64, "plain"),
    (5, 6, 6, 128, 64, "plain"),
    (2, 8, 8, 128, 128, "pool"),        # n-tile 128: groups of 8 warps, half of the columns injected
    (2, 7, 9, 64, 64, "pool"),
    (130, 3, 5, 64, 64, "plain"),       # many tiny images per tile
    (9, 28, 28, 128, 128, "plain"),     # n-tile 128, several tiles per group
    (7, 14, 14, 256, 256, "pool"),      # two n-tiles of 128, four channel blocks
    (40, 7, 7, 512, 512, "plain"),      # n-tile 64 of a wide layer: eight n-tiles, eight channel blocks
    (3, 7, 7, 512, 64, "none"),
    (2, 8, 8, 256, 96, "plain"),        # n-tile 32: one pass per thread
    (4, 12, 10, 64, 128, "none"),
]


@pytest.mark.parametrize("case", CHUNKED_CASES)
def test_conv_layer_chunked_int16_residuals(cuda, case):
    """int16 residual tensors laid out by 8-channel chunk (TCBNN_RES_INT16_CHUNKED) in and out of
    the loader-fed kernel -- its tile-per-group epilogue (one or two CTAs per SM) and, with an
    NHWC tensor on the other side or path 7, the all-warps-per-tile epilogues: same values as the
    oracle's NHWC tensors; calls that cannot honour the layout fail instead of misreading it."""
    B, H, W, C, O, mode = case
    g = util.rng(sum(case[:5]) + 5)
    Cw = C // 32
    x = util.rand_words(g, (B, H, W, Cw))
    f = util.rand_words(g, (O, 9, Cw))
    thr = (g.standard_normal(O) * np.sqrt(C * 9) * 0.5).astype(np.float32)
    res_in, rc, rpool = None, 0, False
    if mode == "plain":
        res_in = g.integers(-300, 300, size=(B, H, W, O)).astype(np.int32)
        rc = O
    elif mode == "pool":
        res_in = g.integers(-300, 300, size=(B, 2 * H, 2 * W, O // 2)).astype(np.int32)
        rc, rpool = O // 2, True
    eo, er, _ = orc.conv_layer(x, f, thr, C, 3, 3, 1, 1, True, 1, res_in=res_in, residual_channels=rc,
                               residual_pool=rpool, save_residual=True)
    eo_plain, _, _ = orc.conv_layer(x, f, thr, C, 3, 3, 1, 1, True, 1)
    d = ops.conv_desc(B, H, W, C, O, 3, 3)
    assert ops.conv_prefers_chunked_residual(d)
    prep = ops.conv_prepare(d, dev(f, cuda))
    r16 = ops.nhwc_to_chunked(dev(res_in.astype(np.int16), cuda)) if res_in is not None else None
    dx, dthr = dev(x, cuda), dev(thr, cuda)
    try:
        for path in (0, 6, 8, 7, 9, 10):
            ops.set_conv_path(path)
            for out_chunked in (True, False):
                for proven in (False, True):
                    go, gr, _ = ops.conv_layer(d, dx, prep, dthr, res_in=r16, residual_channels=rc,
                                               residual_pool=rpool, save_residual=True, residual_dtype=torch.int16,
                                               res_in_chunked=r16 is not None, res_out_chunked=out_chunked,
                                               res_out_proven=proven)
                    assert ops.conv_status(d, prep) == 0
                    if out_chunked:
                        gr = ops.chunked_to_nhwc(gr)
                    assert np.array_equal(gr.cpu().numpy().astype(np.int32), er), (path, out_chunked, proven)
                    assert np.array_equal(host_u32(go), eo), (path, out_chunked, proven)
            # no residual saved: chunked in only
            if r16 is not None:
                go, _, _ = ops.conv_layer(d, dx, prep, dthr, res_in=r16, residual_channels=rc, residual_pool=rpool,
                                          res_in_chunked=True)
                assert np.array_equal(host_u32(go), eo), path
            # no residual at all: the fp32 comparison of the plain epilogues
            go, _, _ = ops.conv_layer(d, dx, prep, dthr)
            assert np.array_equal(host_u32(go), eo_plain), path
            assert ops.conv_status(d, prep) == 0
    finally:
        ops.set_conv_path(0)
    if rpool:
        # a workspace with room for the planes only (no pooling pass possible on any path)
        ws = torch.zeros((ops.new_planes_bytes(d),), dtype=torch.uint8, device=cuda)
        go, gr, _ = ops.conv_layer(d, dx, prep, dthr, res_in=r16, residual_channels=rc,
                                   residual_pool=True, save_residual=True, residual_dtype=torch.int16,
                                   res_in_chunked=True, workspace=ws)
        assert np.array_equal(gr.cpu().numpy().astype(np.int32), er) and np.array_equal(host_u32(go), eo)
    if r16 is not None:
        # without its workspace the layer runs on a kernel that does not know the layout: refused
        with pytest.raises(Exception):
            ops.conv_layer(d, dx, prep, dthr, res_in=r16, residual_channels=rc, residual_pool=rpool,
                           workspace=False, res_in_chunked=True)


def test_conv_layer_reports_int16_overflow_on_tile_epilogue(cuda):
    """A saved int16 residual that does not fit sets status 2 on the tile-per-group epilogue too,
    unless the caller claimed to have proven the bound."""
    g = util.rng(77)
    B, H, W, C, O = 2, 6, 6, 64, 64
    x = util.rand_words(g, (B, H, W, 2))
    f = util.rand_words(g, (O, 9, 2))
    thr = np.zeros(O, np.float32)
    res_in = np.full((B, H, W, O), 32700, np.int16)
    res_in[:, :, :, 1::2] = -32700
    d = ops.conv_desc(B, H, W, C, O, 3, 3)
    prep = ops.conv_prepare(d, dev(f, cuda))
    r16 = ops.nhwc_to_chunked(dev(res_in, cuda))
    ops.conv_layer(d, dev(x, cuda), prep, dev(thr, cuda), res_in=r16, residual_channels=O, save_residual=True,
                   residual_dtype=torch.int16, res_in_chunked=True, res_out_chunked=True)
    assert ops.conv_status(d, prep) == 2
    assert ops.conv_status(d, prep) == 0          # reading clears it


def test_specialized_first_layer_writes_chunked_residual(cuda):
    g = util.rng(123)
    B, H = 3, 36
    d = ops.conv_desc(B, H, H, 3, 64, 7, 7, 4, 4)
    x = g.standard_normal((B, 3, H, H)).astype(np.float32)
    F = util.rand_pm1(g, (49, 3, 64))
    thr = (g.standard_normal(64) * 6).astype(np.float32)
    fb = ops.pack_inconv_filter(dev(F, cuda))
    spec = ops.inconv_specialize(d, fb, dev(thr, cuda))
    _, r_nhwc, _ = ops.inconv_layer(d, dev(x, cuda), fb, dev(thr, cuda), save_residual=True,
                                    residual_dtype=torch.int16, specialized=spec)
    _, r_chunk, _ = ops.inconv_layer(d, dev(x, cuda), fb, dev(thr, cuda), save_residual=True,
                                     residual_dtype=torch.int16, specialized=spec, res_out_chunked=True)
    assert torch.equal(ops.chunked_to_nhwc(r_chunk), r_nhwc)
