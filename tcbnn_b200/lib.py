"""ctypes binding of libtcbnn_b200.so (the C ABI declared in include/tcbnn_b200.h).

The library is the product; this module only loads it and checks return codes.  There is
no fallback: if the shared object is missing, or a call fails, an exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtcbnn_b200.so")


class ConvDesc(C.Structure):
    """Mirror of tcbnn_conv_desc."""
    _fields_ = [(n, C.c_int) for n in
                ("B", "H", "W", "C", "O", "R", "S", "stride_h", "stride_w", "padding", "pool",
                 "pad_h", "pad_w", "OH", "OW")]


_P = C.c_void_p
_I = C.c_int
_LL = C.c_longlong
_SZ = C.c_size_t

# name -> (restype, argtypes); every symbol include/tcbnn_b200.h declares
SIGNATURES = {
    "tcbnn_version": (_I, []),
    "tcbnn_last_error": (C.c_char_p, []),
    "tcbnn_pack_rows": (_I, [_P, _I, _I, _I, _P, _P]),
    "tcbnn_unpack_rows": (_I, [_P, _I, _I, _I, _P, _P]),
    "tcbnn_pack_fc_weight": (_I, [_P, _I, _I, _I, _P, _P]),
    "tcbnn_pack_conv_filter": (_I, [_P, _I, _I, _I, _P, _P]),
    "tcbnn_pack_inconv_filter": (_I, [_P, _I, _I, _P, _P]),
    "tcbnn_gemm_workspace_bytes": (_SZ, [_I, _I, _I]),
    "tcbnn_gemm_launches": (_I, [_I, _I, _I, _SZ]),
    "tcbnn_set_gemm_path": (_I, [_I]),
    "tcbnn_gemm_status": (_I, [C.POINTER(C.c_int)]),
    "tcbnn_bgemm": (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _I, _P, _SZ, _P]),
    "tcbnn_fc_layer": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _P, _SZ, _P]),
    "tcbnn_out_layer": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _P, _SZ, _P]),
    "tcbnn_conv_shape": (_I, [C.POINTER(ConvDesc)]),
    "tcbnn_conv_prepared_bytes": (_SZ, [C.POINTER(ConvDesc)]),
    "tcbnn_conv_prepare": (_I, [C.POINTER(ConvDesc), _P, _P, _P]),
    "tcbnn_conv_layer": (_I, [C.POINTER(ConvDesc), _P, _P, _P, _P, _I, _I, _I, _I, _P, _LL, _P, _I, _P, _P]),
    "tcbnn_set_conv_path": (_I, [_I]),
    "tcbnn_conv_set_trace": (_I, [_P]),
    "tcbnn_set_gemm_plan": (_I, [_I, _I]),
    "tcbnn_mma_operand_probe": (_I, [_I, _I, _I, C.POINTER(C.c_double)]),
    "tcbnn_bulk_copy_rate": (_I, [_I, _I, _I, _I, _I, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "tcbnn_conv_status": (_I, [C.POINTER(ConvDesc), _P, C.POINTER(C.c_int)]),
    "tcbnn_inconv_layer": (_I, [C.POINTER(ConvDesc), _P, _P, _P, _P, _LL, _P, _I, _P, _P]),
    "tcbnn_noalloc_scratch_bytes": (_SZ, []),
    "tcbnn_fc_layer_noalloc": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _P]),
    "tcbnn_conv_workspace_bytes": (_SZ, [C.POINTER(ConvDesc)]),
    "tcbnn_conv_planes_bytes": (_SZ, [C.POINTER(ConvDesc)]),
    "tcbnn_conv_layer_w": (_I, [C.POINTER(ConvDesc), _P, _P, _P, _P, _I, _I, _I, _I, _P, _LL, _P, _I, _P, _P, _SZ, _P]),
    "tcbnn_conv_layer_x": (_I, [C.POINTER(ConvDesc), _P, _P, _P, _P, _I, _I, _I, _I, _P, _LL, _P, _I, _P, _P, _SZ, _I,
                                C.POINTER(ConvDesc), _P, _SZ, _P]),
    "tcbnn_inconv_specialized_layer_x": (_I, [_P, C.POINTER(ConvDesc), _P, _P, _P, _P, _LL, _P, _I, _P,
                                              C.POINTER(ConvDesc), _P, _SZ, _P]),
    "tcbnn_inconv_specialize": (_I, [C.POINTER(ConvDesc), _P, _P, _P, C.POINTER(C.c_void_p)]),
    "tcbnn_inconv_specialized_layer": (_I, [_P, C.POINTER(ConvDesc), _P, _P, _P, _P, _LL, _P, _I, _P, _P]),
    "tcbnn_inconv_release": (_I, [_P]),
    "tcbnn_inconv_specialize_selftest": (_I, [C.POINTER(ConvDesc), C.c_uint, C.POINTER(C.c_longlong)]),
    "tcbnn_inconv_layer_u8": (_I, [C.POINTER(ConvDesc), _P, _P, _P, _P, _P, _LL, _P, _I, _P, _P]),
    "tcbnn_mma_peak": (_I, [_I, _I, _I, C.POINTER(C.c_double)]),
    "tcbnn_wait_probe": (_I, [_I, C.POINTER(C.c_int)]),
    "tcbnn_conv_prefers_chunked_residual": (_I, [C.POINTER(ConvDesc)]),
}

RES_INT32, RES_INT16, RES_INT16_CHUNKED, RES_PROVEN = 4, 2, 18, 32      # TCBNN_RES_* of the header

_lib = None


class TcbnnError(RuntimeError):
    pass


def load():
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TcbnnError(
            "libtcbnn_b200.so is not built: run `python -m tcbnn_b200.build` "
            "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if a declared symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc):
    if rc != 0:
        raise TcbnnError(load().tcbnn_last_error().decode())


def call(name, *args):
    """Call an int-returning entry point and raise on a non-zero status."""
    check(getattr(load(), name)(*args))
