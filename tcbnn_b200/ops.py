"""Torch-tensor front end of the C ABI: device memory and streams come from torch, every
computation is a call into libtcbnn_b200.so.  Bit tensors are torch.int32 (same bytes as the
library's uint32 words)."""
import ctypes as C

import torch

from . import lib as _l
from .lib import ConvDesc


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _l.TcbnnError("tcbnn_b200 ops need CUDA tensors (no CPU path exists)")
        if t is not None and not t.is_contiguous():
            raise _l.TcbnnError("tcbnn_b200 ops need contiguous tensors")


def step128_words(k):
    """Words per bit row padded to 128 bits (STEP128(k)*4, utility.h:38)."""
    return ((k + 127) // 128) * 4


def pack_rows(x, ld_words=None):
    _need_cuda(x)
    rows, cols = x.shape
    ld = ld_words or step128_words(cols)
    out = torch.empty((rows, ld), dtype=torch.int32, device=x.device)
    _l.call("tcbnn_pack_rows", _ptr(x), rows, cols, ld, _ptr(out), _stream())
    return out


def unpack_rows(bits, cols):
    _need_cuda(bits)
    rows, ld = bits.shape
    out = torch.empty((rows, cols), dtype=torch.float32, device=bits.device)
    _l.call("tcbnn_unpack_rows", _ptr(bits), rows, cols, ld, _ptr(out), _stream())
    return out


def pack_fc_weight(W, ld_words=None):
    _need_cuda(W)
    K, N = W.shape
    ld = ld_words or step128_words(K)
    out = torch.empty((N, ld), dtype=torch.int32, device=W.device)
    _l.call("tcbnn_pack_fc_weight", _ptr(W), K, N, ld, _ptr(out), _stream())
    return out


def pack_conv_filter(F):
    """F: fp32 [R*S][C][O] -> bits [O][R*S][Cw]."""
    _need_cuda(F)
    RS, Cc, O = F.shape
    out = torch.empty((O, RS, (Cc + 31) // 32), dtype=torch.int32, device=F.device)
    _l.call("tcbnn_pack_conv_filter", _ptr(F), RS, Cc, O, _ptr(out), _stream())
    return out


def pack_inconv_filter(F):
    """F: fp32 [R*S][3][O] -> [R*S][3][Ow] words."""
    _need_cuda(F)
    RS, Cc, O = F.shape
    assert Cc == 3
    out = torch.empty((RS, 3, (O + 31) // 32), dtype=torch.int32, device=F.device)
    _l.call("tcbnn_pack_inconv_filter", _ptr(F), RS, O, _ptr(out), _stream())
    return out


def gemm_workspace(M, N, K, device):
    n = _l.load().tcbnn_gemm_workspace_bytes(M, N, K)
    return torch.empty((max(n, 4) // 4,), dtype=torch.int32, device=device) if n else None


def gemm_launches(M, N, K, workspace):
    """Kernels a GEMM-family call of this shape launches with this workspace tensor."""
    nbytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    return _l.load().tcbnn_gemm_launches(M, N, K, C.c_size_t(nbytes))


def _ws(ws):
    return (_ptr(ws), C.c_size_t(ws.numel() * 4 if ws is not None else 0))


def bgemm(A, B, K, out=None, workspace=None):
    _need_cuda(A, B)
    M, lda = A.shape
    N, ldb = B.shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.int32, device=A.device)
    _l.call("tcbnn_bgemm", _ptr(A), _ptr(B), M, N, K, lda, ldb, _ptr(out), out.shape[1],
            *_ws(workspace), _stream())
    return out


def fc_layer(A, W, thr, K, out=None, workspace=None):
    _need_cuda(A, W, thr)
    M, lda = A.shape
    N, ldw = W.shape
    if out is None:
        out = torch.zeros((M, step128_words(N)), dtype=torch.int32, device=A.device)
    _l.call("tcbnn_fc_layer", _ptr(A), _ptr(W), _ptr(thr), M, K, N, lda, ldw, _ptr(out),
            out.shape[1], *_ws(workspace), _stream())
    return out


def out_layer(A, W, scale, bias, K, out=None, workspace=None):
    _need_cuda(A, W, scale, bias)
    M, lda = A.shape
    N, ldw = W.shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=A.device)
    _l.call("tcbnn_out_layer", _ptr(A), _ptr(W), _ptr(scale), _ptr(bias), M, K, N, lda, ldw,
            _ptr(out), out.shape[1], *_ws(workspace), _stream())
    return out


def conv_desc(B, H, W, Cc, O, R, S, stride_h=1, stride_w=1, padding=True, pool=1):
    d = ConvDesc(B=B, H=H, W=W, C=Cc, O=O, R=R, S=S, stride_h=stride_h, stride_w=stride_w,
                 padding=int(bool(padding)), pool=pool)
    _l.call("tcbnn_conv_shape", C.byref(d))
    return d


def conv_prepare(d, filter_bits):
    _need_cuda(filter_bits)
    n = _l.load().tcbnn_conv_prepared_bytes(C.byref(d))
    if n == 0:
        raise _l.TcbnnError(_l.load().tcbnn_last_error().decode())
    blob = torch.empty((n,), dtype=torch.uint8, device=filter_bits.device)
    _l.call("tcbnn_conv_prepare", C.byref(d), _ptr(filter_bits), _ptr(blob), _stream())
    return blob


_scratch = {}


def conv_workspace(d, device):
    """A scratch tensor large enough for tcbnn_conv_layer_w on this descriptor, or None when the
    layer has no use for one.  One tensor per device, grown on demand and shared by every call
    that does not bring its own: callers running layers on several streams at once must pass
    separate workspaces."""
    n = _l.load().tcbnn_conv_workspace_bytes(C.byref(d))
    if n == 0:
        return None
    key = (device.type, device.index)
    t = _scratch.get(key)
    if t is None or t.numel() < n:
        _scratch[key] = None
        t = torch.empty((n,), dtype=torch.uint8, device=device)
        _scratch[key] = t
    return t


def conv_layer(d, x, prepared, thr, res_in=None, residual_channels=0, residual_pool=False,
               out=None, out_image_stride=None, save_residual=False, want_acc=False,
               res_out_buf=None, residual_dtype=torch.int32, workspace=None, workspace_ready=False,
               next_layer=None, res_in_chunked=False, res_out_chunked=False, res_out_proven=False):
    """x: [B][H][W][Cw] int32 words.  Returns (out_bits, res_out, acc_out).
    Residual tensors may be torch.int32 or torch.int16; res_in_chunked / res_out_chunked: the
    int16 tensor is laid out by 8-channel chunk (TCBNN_RES_INT16_CHUNKED, see chunked_to_nhwc).
    res_out_proven: the caller has proven that every saved int16 value fits (TCBNN_RES_PROVEN).
    workspace: uint8 scratch tensor for tcbnn_conv_layer_w; None = the shared one of
    conv_workspace(); False = none (tcbnn_conv_layer).
    next_layer: (descriptor, planes tensor) of the layer consuming this output: the layer also
    writes its output into that layer's input planes (new_planes()); the consumer is then called
    with workspace=planes, workspace_ready=True (tcbnn_conv_layer_x)."""
    _need_cuda(x, prepared, thr, res_in)
    if workspace is None:
        workspace = conv_workspace(d, x.device)
    elif workspace is False:
        workspace = None
    Ow = (d.O + 31) // 32
    stride = out_image_stride or d.OH * d.OW * Ow
    if out is None:
        out = torch.zeros((d.B, stride), dtype=torch.int32, device=x.device)
    P, Q = d.pool * d.OH, d.pool * d.OW
    res_out = res_out_buf
    if res_out is None and save_residual:
        res_out = torch.empty((d.B, P, Q, d.O), dtype=residual_dtype, device=x.device)
    acc_out = torch.empty((d.B, P, Q, d.O), dtype=torch.int32, device=x.device) if want_acc else None
    res_in_ch = res_in.shape[-1] if res_in is not None else 0
    args = (C.byref(d), _ptr(x), _ptr(prepared), _ptr(thr), _ptr(res_in),
            _residual_code(res_in, res_in_chunked),
            res_in_ch, residual_channels, int(bool(residual_pool)), _ptr(out),
            C.c_longlong(stride), _ptr(res_out),
            _residual_code(res_out, res_out_chunked, res_out_proven), _ptr(acc_out))
    if next_layer is not None or workspace_ready:
        nd, npl = next_layer if next_layer is not None else (None, None)
        _l.call("tcbnn_conv_layer_x", *args, _ptr(workspace),
                C.c_size_t(workspace.numel() if workspace is not None else 0), int(bool(workspace_ready)),
                C.byref(nd) if nd is not None else None, _ptr(npl),
                C.c_size_t(npl.numel() if npl is not None else 0), _stream())
    elif workspace is not None:
        _l.call("tcbnn_conv_layer_w", *args, _ptr(workspace), C.c_size_t(workspace.numel()), _stream())
    else:
        _l.call("tcbnn_conv_layer", *args, _stream())
    return out, res_out, acc_out


def _residual_code(t, chunked, proven=False):
    """The *_bytes argument of the conv entry points for a residual tensor."""
    if t is None:
        return 4
    flag = _l.RES_PROVEN if (proven and t.dtype == torch.int16) else 0
    if chunked:
        if t.dtype != torch.int16:
            raise _l.TcbnnError("chunked residuals are int16")
        return _l.RES_INT16_CHUNKED | flag
    return t.element_size() | flag


def conv_prefers_chunked_residual(d):
    """True for layers whose epilogue is fastest on residual tensors laid out by 8-channel chunk."""
    return bool(_l.load().tcbnn_conv_prefers_chunked_residual(C.byref(d)))


def chunked_to_nhwc(t):
    """A [B][P][Q][ch] int16 tensor whose memory holds the chunk-major layout [ch/8][B*P*Q][8]
    (TCBNN_RES_INT16_CHUNKED) -> the same values as a proper NHWC tensor."""
    B, P, Q, ch = t.shape
    return t.reshape(ch // 8, B * P * Q, 8).permute(1, 0, 2).reshape(B, P, Q, ch).contiguous()


def nhwc_to_chunked(t):
    """The inverse: NHWC values -> a tensor of the same shape whose memory is chunk-major."""
    B, P, Q, ch = t.shape
    return t.reshape(B * P * Q, ch // 8, 8).permute(1, 0, 2).contiguous().reshape(B, P, Q, ch)


def new_planes_bytes(d):
    return _l.load().tcbnn_conv_planes_bytes(C.byref(d))


def new_planes(d, device):
    """Zeroed input planes for the layer `d` when its producer writes them (next_layer=...), or
    None when the layer takes no pre-expanded input."""
    n = _l.load().tcbnn_conv_planes_bytes(C.byref(d))
    if not n:
        return None
    # the planes come first in the layer's workspace; a pooled layer keeps its pre-pool bits behind them
    return torch.zeros((max(n, _l.load().tcbnn_conv_workspace_bytes(C.byref(d))),), dtype=torch.uint8, device=device)


class InconvSpecialized:
    """A first-layer kernel compiled for one filter and one set of thresholds
    (tcbnn_inconv_specialize); pass it to inconv_layer(specialized=...)."""

    def __init__(self, d, filter_bits, thr):
        _need_cuda(filter_bits, thr)
        h = C.c_void_p(None)
        _l.call("tcbnn_inconv_specialize", C.byref(d), _ptr(filter_bits), _ptr(thr), _stream(), C.byref(h))
        self.handle = h

    def release(self):
        if self.handle is not None and self.handle.value:
            _l.call("tcbnn_inconv_release", self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def inconv_specialize(d, filter_bits, thr):
    return InconvSpecialized(d, filter_bits, thr)


def inconv_layer(d, x, filter_bits, thr, out=None, out_image_stride=None, save_residual=False,
                 want_acc=False, res_out_buf=None, residual_dtype=torch.int32, lut=None,
                 specialized=None, next_layer=None, res_out_chunked=False):
    """x: fp32 [B][3][H][W], or uint8 [B][3][H][W] together with lut (fp32 [3][256], the value
    of every byte per channel).  specialized: an InconvSpecialized built from the same filter
    and thresholds (filter_bits and thr are then not read).  Returns (out_bits, res_out, acc_out)."""
    _need_cuda(x, filter_bits, thr, lut)
    if (x.dtype == torch.uint8) != (lut is not None):
        raise _l.TcbnnError("inconv_layer: uint8 images need a lut, fp32 images must not have one")
    Ow = (d.O + 31) // 32
    stride = out_image_stride or d.OH * d.OW * Ow
    if out is None:
        out = torch.zeros((d.B, stride), dtype=torch.int32, device=x.device)
    P, Q = d.pool * d.OH, d.pool * d.OW
    res_out = res_out_buf
    if res_out is None and save_residual:
        res_out = torch.empty((d.B, P, Q, d.O), dtype=residual_dtype, device=x.device)
    acc_out = torch.empty((d.B, P, Q, d.O), dtype=torch.float32, device=x.device) if want_acc else None
    if next_layer is not None and specialized is None:
        raise _l.TcbnnError("inconv_layer: next_layer needs the specialised kernel")
    if specialized is not None:
        u8 = lut is not None
        nd, npl = next_layer if next_layer is not None else (None, None)
        _l.call("tcbnn_inconv_specialized_layer_x", specialized.handle, C.byref(d),
                None if u8 else _ptr(x), _ptr(x) if u8 else None, _ptr(lut), _ptr(out),
                C.c_longlong(stride), _ptr(res_out),
                _residual_code(res_out, res_out_chunked), _ptr(acc_out),
                C.byref(nd) if nd is not None else None, _ptr(npl),
                C.c_size_t(npl.numel() if npl is not None else 0), _stream())
    elif lut is not None:
        _l.call("tcbnn_inconv_layer_u8", C.byref(d), _ptr(x), _ptr(lut), _ptr(filter_bits), _ptr(thr),
                _ptr(out), C.c_longlong(stride), _ptr(res_out),
                res_out.element_size() if res_out is not None else 4, _ptr(acc_out), _stream())
    else:
        _l.call("tcbnn_inconv_layer", C.byref(d), _ptr(x), _ptr(filter_bits), _ptr(thr), _ptr(out),
                C.c_longlong(stride), _ptr(res_out),
                res_out.element_size() if res_out is not None else 4, _ptr(acc_out), _stream())
    return out, res_out, acc_out


def mma_peak(kind, warps_per_sm=32, iters=4000):
    t = C.c_double(0)
    _l.call("tcbnn_mma_peak", kind, warps_per_sm, iters, C.byref(t))
    return t.value


def set_gemm_path(path):
    """0 = automatic, 1 = warp-level b1 MMA kernel only."""
    _l.call("tcbnn_set_gemm_path", int(path))


def set_gemm_plan(pair=-1, splits=-1):
    """Force the tcgen05 GEMM's tile shape (1: 256 x 128, 0: 128 x 128) and split count; -1 = automatic."""
    _l.call("tcbnn_set_gemm_plan", int(pair), int(splits))


def gemm_status():
    s = C.c_int(0)
    _l.call("tcbnn_gemm_status", C.byref(s))
    return s.value


def set_conv_path(path):
    """0 = automatic, 1 = warp-level b1 MMA, 2 = tcgen05 (error when a layer is not eligible),
    3 = tcgen05 without the activation-stationary kernel, 4 / 5 = residual rows never / always
    staged in shared memory, 6 = one CTA per SM only, 7 = without the tile-per-group epilogues,
    8 = two CTAs per SM wherever they fit, 9 = one 64-channel block per stage, 10 = every n-tile the same number of CTAs
    (tcbnn_set_conv_path)."""
    _l.call("tcbnn_set_conv_path", int(path))


def conv_status(d, prepared):
    s = C.c_int(0)
    _l.call("tcbnn_conv_status", C.byref(d), _ptr(prepared), C.byref(s))
    return s.value
