"""numpy/ctypes front end of the CPU oracle (liboracle.so, built from tcbnn_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the cpu_baseline /
reference legs of bench.py -- never by the tcbnn_b200 package."""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import build as _build  # noqa: E402

_lib = None
_ref = None


def lib(native=False):
    global _lib
    if _lib is None or native:
        path = _build.build_oracle(native=native)
        L = C.CDLL(path)
        L.orc_num_threads.restype = C.c_int
        if native:
            return L
        _lib = L
    return _lib


def ref_lib():
    """The reference's own host popcount loops (oracle/_ref/libref_bmm.so) or None."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libref_bmm.so")
        if not os.path.exists(path):
            path = _build.build_ref()
        if path is None:
            return None
        _ref = C.CDLL(path)
    return _ref


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else C.c_void_p(0)


def _u32(a):
    return np.ascontiguousarray(a).view(np.uint32)


def step128_words(k):
    return ((k + 127) // 128) * 4


def pack_rows(x, ld_words=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    ld = ld_words or step128_words(cols)
    out = np.zeros((rows, ld), dtype=np.uint32)
    lib().orc_pack_rows(_p(x), rows, cols, ld, _p(out))
    return out


def pack_fc_weight(W, ld_words=None):
    W = np.ascontiguousarray(W, dtype=np.float32)
    K, N = W.shape
    ld = ld_words or step128_words(K)
    out = np.zeros((N, ld), dtype=np.uint32)
    lib().orc_pack_fc_weight(_p(W), K, N, ld, _p(out))
    return out


def pack_conv_filter(F):
    F = np.ascontiguousarray(F, dtype=np.float32)
    RS, Cc, O = F.shape
    out = np.zeros((O, RS, (Cc + 31) // 32), dtype=np.uint32)
    lib().orc_pack_conv_filter(_p(F), RS, Cc, O, _p(out))
    return out


def unpack_rows(bits, cols):
    bits = _u32(bits)
    rows, ld = bits.shape
    out = np.zeros((rows, cols), dtype=np.float32)
    lib().orc_unpack_rows(_p(bits), rows, cols, ld, _p(out))
    return out


def bgemm_popc(A, B, K):
    A, B = _u32(A), _u32(B)
    out = np.zeros((A.shape[0], B.shape[0]), dtype=np.int32)
    lib().orc_bgemm_popc(_p(A), _p(B), A.shape[0], B.shape[0], K, A.shape[1], B.shape[1], _p(out))
    return out


def bgemm(A, B, K, L=None):
    A, B = _u32(A), _u32(B)
    out = np.zeros((A.shape[0], B.shape[0]), dtype=np.int32)
    (L or lib()).orc_bgemm(_p(A), _p(B), A.shape[0], B.shape[0], K, A.shape[1], B.shape[1], _p(out))
    return out


def fc_layer(A, W, thr, K, ldo=None):
    A, W = _u32(A), _u32(W)
    thr = np.ascontiguousarray(thr, dtype=np.float32)
    M, N = A.shape[0], W.shape[0]
    ldo = ldo or step128_words(N)
    out = np.zeros((M, ldo), dtype=np.uint32)
    lib().orc_fc_layer(_p(A), _p(W), _p(thr), M, K, N, A.shape[1], W.shape[1], ldo, _p(out))
    return out


def out_layer(A, W, scale, bias, K):
    A, W = _u32(A), _u32(W)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    M, N = A.shape[0], W.shape[0]
    out = np.zeros((M, N), dtype=np.float32)
    lib().orc_out_layer(_p(A), _p(W), _p(scale), _p(bias), M, K, N, A.shape[1], W.shape[1], _p(out))
    return out


def conv_shape(H, W, R, S, sh=1, sw=1, padding=True, pool=1):
    v = [C.c_int(0) for _ in range(6)]
    lib().orc_conv_shape(H, W, R, S, sh, sw, int(bool(padding)), pool, pool, *[C.byref(x) for x in v])
    pad_h, pad_w, P, Q, OH, OW = [x.value for x in v]
    return dict(pad_h=pad_h, pad_w=pad_w, P=P, Q=Q, OH=OH, OW=OW)


def conv_layer(x, filt, thr, Cc, R, S, sh=1, sw=1, padding=True, pool=1, res_in=None,
               residual_channels=0, residual_pool=False, out_image_stride=None,
               save_residual=False, want_acc=False, L=None):
    """x [B][H][W][Cw] words, filt [O][R*S][Cw] words -> (out [B][stride], res_out, acc_out)."""
    x, filt = _u32(x), _u32(filt)
    thr = np.ascontiguousarray(thr, dtype=np.float32)
    B, H, W, Cw = x.shape
    O = filt.shape[0]
    g = conv_shape(H, W, R, S, sh, sw, padding, pool)
    Ow = (O + 31) // 32
    stride = out_image_stride or g["OH"] * g["OW"] * Ow
    out = np.zeros((B, stride), dtype=np.uint32)
    res_out = np.zeros((B, g["P"], g["Q"], O), dtype=np.int32) if save_residual else None
    acc_out = np.zeros((B, g["P"], g["Q"], O), dtype=np.int32) if want_acc else None
    if res_in is not None:
        res_in = np.ascontiguousarray(res_in, dtype=np.int32)
    (L or lib()).orc_conv_layer(
        _p(x), _p(filt), _p(thr), B, H, W, Cc, O, R, S, sh, sw, g["pad_h"], g["pad_w"], pool, pool,
        g["OH"], g["OW"], _p(res_in), res_in.shape[-1] if res_in is not None else 0,
        residual_channels, int(bool(residual_pool)), _p(out), C.c_long(stride), _p(res_out),
        _p(acc_out))
    return out, res_out, acc_out


def inconv_layer(x, F, thr, R, S, sh=1, sw=1, padding=True, pool=1, out_image_stride=None,
                 save_residual=False, want_acc=False, L=None):
    """x fp32 [B][3][H][W], F fp32 [R*S][3][O] -> (out bits, res_out int32, acc fp32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    F = np.ascontiguousarray(F, dtype=np.float32)
    thr = np.ascontiguousarray(thr, dtype=np.float32)
    B, _, H, W = x.shape
    O = F.shape[2]
    g = conv_shape(H, W, R, S, sh, sw, padding, pool)
    Ow = (O + 31) // 32
    stride = out_image_stride or g["OH"] * g["OW"] * Ow
    out = np.zeros((B, stride), dtype=np.uint32)
    res_out = np.zeros((B, g["P"], g["Q"], O), dtype=np.int32) if save_residual else None
    acc_out = np.zeros((B, g["P"], g["Q"], O), dtype=np.float32) if want_acc else None
    (L or lib()).orc_inconv_layer(
        _p(x), _p(F), _p(thr), B, H, W, O, R, S, sh, sw, g["pad_h"], g["pad_w"], pool, pool,
        g["OH"], g["OW"], _p(out), C.c_long(stride), _p(res_out), _p(acc_out))
    return out, res_out, acc_out


def use_all_cores(L=None):
    """Make the oracle use every host core (a launcher may have exported OMP_NUM_THREADS=1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    (L or lib()).orc_set_num_threads(n)
    return n


def num_threads(L=None):
    return (L or lib()).orc_num_threads()


# --- the reference's own host loops (pin for the oracle) -----------------------------------
def ref_bmma_cpu(A, B, k):
    """BMMAcpu(A, B, C, m, n, k): C += popc(A^B) (bmm/tensorcore_kernel.cu:38-57)."""
    R = ref_lib()
    A, B = _u32(A), _u32(B)
    out = np.zeros((A.shape[0], B.shape[0]), dtype=np.int32)
    R.ref_BMMAcpu(_p(A), _p(B), _p(out), A.shape[0], B.shape[0], k)
    return out


def ref_wmma_bool_cpu(A, B, Cin, k):
    """WMMABOOLCPU: D = popc(A^B) + C (bmm/bmma_op_test/main_test.cu:232-254)."""
    R = ref_lib()
    A, B = _u32(A), _u32(B)
    Cin = np.ascontiguousarray(Cin, dtype=np.int32)
    D = np.zeros_like(Cin)
    R.ref_WMMABOOLCPU(_p(A), _p(B), _p(Cin), _p(D), A.shape[0], B.shape[0], k)
    return D
