"""Host-side layer objects with the names, constructor arguments and method names of the
reference's param.h classes (In128/Fc128/Out128/InConv128/Conv128 LayerParam), built on the
C ABI.  Differences that follow from the B200 design, not from the interface:

  * activations stay NHWC bit-packed (no HWNC 8x128 tiling) and residuals are unpadded NHWC
    int32, so get_output_gpu() hands the next layer an opaque device tensor exactly as the
    reference hands over an opaque uin32* (param.h:986);
  * every layer is a separate launch on the current stream (forward()), outputs are written
    with stores, so a layer object can be run any number of times;
  * weights come from a `config` object with read(n) -> n floats in the order launch_array
    consumes them (utility.h:188-196): filter/weight first, then thresholds;
  * the batch given to the constructor is the LARGEST batch the object will see: set_batch(n)
    (n <= that) makes the following forward() calls process the first n images in the same
    buffers, so a serving loop with a ragged last batch keeps its layer objects (the reference
    fixes the batch at construction, param.h:875-881).
"""
import numpy as np
import torch

from . import ops


class ArrayConfig:
    """In-memory stand-in for the reference's text weight file: read(n) returns the next n
    float32 values."""

    def __init__(self, arrays):
        if isinstance(arrays, np.ndarray):
            arrays = [arrays]
        self._arrays = [np.ascontiguousarray(a, dtype=np.float32).ravel() for a in arrays]
        self._i = 0
        self._off = 0

    def read(self, n):
        out = np.empty(n, dtype=np.float32)
        got = 0
        while got < n:
            if self._i >= len(self._arrays):
                raise ValueError("weight stream exhausted (launch_array would read past EOF)")
            a = self._arrays[self._i]
            take = min(n - got, a.size - self._off)
            out[got:got + take] = a[self._off:self._off + take]
            got += take
            self._off += take
            if self._off == a.size:
                self._i += 1
                self._off = 0
        return out


class TextConfig(ArrayConfig):
    """Whitespace-separated floats, the reference's file format (fscanf "%f")."""

    def __init__(self, path):
        super().__init__(np.loadtxt(path, dtype=np.float32).ravel())


def _residual_dtype(bound):
    """int16 when the running shortcut sum provably fits, else int32."""
    return torch.int16 if (bound is not None and bound <= 32767) else torch.int32


def _live_chunked(t, live):
    """A residual buffer sized for the constructor's batch that holds the chunk-major layout of the
    first `live` images: the view whose memory is exactly that layout."""
    B, P, Q, ch = t.shape
    return t.reshape(-1)[:live * P * Q * ch].reshape(live, P, Q, ch)


def _dev():
    if not torch.cuda.is_available():
        raise RuntimeError("tcbnn_b200 needs a CUDA device; there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


class In128LayerParam:
    """param.h:115-222.  fp32 [input_height][input_width] -> bit rows."""

    def __init__(self, name, input_height, input_width):
        self.name = name
        self.input_height = self.output_height = input_height
        self.input_width = self.output_width = input_width
        self.input_gpu = self.output_gpu = None
        self.live = input_height

    def set_batch(self, n):
        """Process the first n rows from now on (n <= the constructor's input_height)."""
        if not 0 < n <= self.input_height:
            raise ValueError("%s: batch %d outside 1..%d" % (self.name, n, self.input_height))
        self.live = n

    def initialize(self, input):
        dev = _dev()
        self.input_gpu = torch.empty((self.input_height, self.input_width), dtype=torch.float32, device=dev)
        self.set_input(input)
        self.output_gpu = torch.zeros((self.input_height, ops.step128_words(self.input_width)),
                                      dtype=torch.int32, device=dev)
        return self

    def set_input(self, input):
        src = input if torch.is_tensor(input) else torch.from_numpy(np.ascontiguousarray(input, dtype=np.float32))
        src = src.reshape(-1, self.input_width)
        self.input_gpu[:src.shape[0]].copy_(src, non_blocking=True)

    def forward(self):
        ops._l.call("tcbnn_pack_rows", ops._ptr(self.input_gpu), self.live, self.input_width,
                    self.output_gpu.shape[1], ops._ptr(self.output_gpu), ops._stream())

    def get_output_gpu(self):
        return self.output_gpu

    def download_output(self):
        return self.output_gpu.cpu().numpy().view(np.uint32)

    def download_full_output(self):
        return ops.unpack_rows(self.output_gpu, self.output_width).cpu().numpy()


class Fc128LayerParam:
    """param.h:224-385.  Hidden FC layer: bit GEMM + threshold + repack."""

    def __init__(self, name, input_height, input_width, weight_width):
        self.name = name
        self.input_height = self.output_height = input_height
        self.input_width = self.weight_height = input_width
        self.weight_width = self.output_width = self.bn_width = weight_width
        self.weight_gpu = self.bn_gpu = self.input_gpu = self.output_gpu = None
        self.live = input_height

    def set_batch(self, n):
        if not 0 < n <= self.input_height:
            raise ValueError("%s: batch %d outside 1..%d" % (self.name, n, self.input_height))
        self.live = n

    def initialize(self, config, prev_layer_gpu):
        dev = _dev()
        K, N = self.weight_height, self.weight_width
        w = torch.from_numpy(config.read(K * N).reshape(K, N)).to(dev)
        self.weight_gpu = ops.pack_fc_weight(w)
        self.bn = config.read(N)
        self.bn_gpu = torch.from_numpy(self.bn).to(dev)
        self.output_gpu = torch.zeros((self.input_height, ops.step128_words(N)), dtype=torch.int32, device=dev)
        self.workspace = ops.gemm_workspace(self.input_height, N, K, dev)
        self.launches = ops.gemm_launches(self.input_height, N, K, self.workspace)
        self.set_input_gpu(prev_layer_gpu)
        return self

    def set_input_gpu(self, t):
        M, K = self.input_height, self.input_width
        t = t.reshape(M, -1)
        if t.shape[1] * 32 < K or t.shape[1] % 2:
            raise ValueError("%s: input rows of %d words do not cover K=%d" % (self.name, t.shape[1], K))
        self.input_gpu = t

    def kernel_launches(self):
        return self.launches

    def forward(self):
        ops.fc_layer(self.input_gpu[:self.live], self.weight_gpu, self.bn_gpu, self.input_width,
                     out=self.output_gpu[:self.live], workspace=self.workspace)

    def get_output_gpu(self):
        return self.output_gpu

    def download_output(self):
        return self.output_gpu.cpu().numpy().view(np.uint32)

    def download_full_output(self):
        return ops.unpack_rows(self.output_gpu, self.output_width).cpu().numpy()


class Out128LayerParam:
    """param.h:388-531.  Output layer: bit GEMM + per-class scale and bias -> fp32 logits."""

    def __init__(self, name, input_height, input_width, weight_width):
        self.name = name
        self.input_height = self.output_height = input_height
        self.input_width = self.weight_height = input_width
        self.weight_width = self.output_width = weight_width
        self.weight_gpu = self.input_gpu = self.output_gpu = None
        self.live = input_height

    def set_batch(self, n):
        if not 0 < n <= self.input_height:
            raise ValueError("%s: batch %d outside 1..%d" % (self.name, n, self.input_height))
        self.live = n

    def initialize(self, config, prev_layer_gpu):
        dev = _dev()
        K, N = self.weight_height, self.weight_width
        w = torch.from_numpy(config.read(K * N).reshape(K, N)).to(dev)
        self.weight_gpu = ops.pack_fc_weight(w)
        self.bn_scale = config.read(N)
        self.bn_bias = config.read(N)
        self.bn_scale_gpu = torch.from_numpy(self.bn_scale).to(dev)
        self.bn_bias_gpu = torch.from_numpy(self.bn_bias).to(dev)
        self.output_gpu = torch.zeros((self.input_height, N), dtype=torch.float32, device=dev)
        self.workspace = ops.gemm_workspace(self.input_height, N, K, dev)
        self.launches = ops.gemm_launches(self.input_height, N, K, self.workspace)
        self.input_gpu = prev_layer_gpu.reshape(self.input_height, -1)
        return self

    def kernel_launches(self):
        return self.launches

    def forward(self):
        ops.out_layer(self.input_gpu[:self.live], self.weight_gpu, self.bn_scale_gpu, self.bn_bias_gpu,
                      self.input_width, out=self.output_gpu[:self.live], workspace=self.workspace)

    def get_output_gpu(self):
        return self.output_gpu

    def download_output(self):
        return self.output_gpu[:self.live].cpu().numpy()


class InConv128LayerParam:
    """param.h:701-870.  First conv layer on fp32 NCHW images."""

    def __init__(self, name, input_height, input_width, filter_height, filter_width,
                 input_channels, output_channels, batch, stride_height=1, stride_width=1,
                 padding=True, pool_height=1, pool_width=1, save_residual=False,
                 input_abs_bound=None):
        if pool_height != pool_width:
            raise ValueError("only square pooling windows are supported")
        self.name = name
        self.input_height, self.input_width = input_height, input_width
        self.filter_height, self.filter_width = filter_height, filter_width
        self.input_channels, self.output_channels, self.batch = input_channels, output_channels, batch
        self.stride_height, self.stride_width, self.padding = stride_height, stride_width, padding
        self.pool_height, self.pool_width, self.save_residual = pool_height, pool_width, save_residual
        # Bound of |saved residual| when the caller states max|input| (extension: lets the
        # residual be stored as int16).  Unknown -> int32 like the reference (param.h:758).
        self.residual_bound = None
        if input_abs_bound is not None:
            self.residual_bound = int(filter_height * filter_width * input_channels
                                      * float(input_abs_bound) * 1.001) + 2
        self.desc = ops.conv_desc(batch, input_height, input_width, input_channels, output_channels,
                                  filter_height, filter_width, stride_height, stride_width, padding,
                                  pool_height)
        self.pad_h, self.pad_w = self.desc.pad_h, self.desc.pad_w
        self.output_height, self.output_width = self.desc.OH, self.desc.OW
        self.output_residual_gpu = None

    def initialize(self, input, config, input_lut=None, specialize=True):
        """input: fp32 NCHW images as in the reference (param.h:760), or -- extension -- uint8 NCHW
        images with input_lut, fp32 [3][256]: the value of every byte per channel, i.e. the
        reader's normalisation tabulated (data.cpp:534-542).  Same results, a quarter of the
        host->device traffic.
        specialize: compile a kernel for this layer's filter and thresholds (layers of at most 128
        output channels; same results, several times faster than the kernel that reads the
        filter at run time, which is used otherwise)."""
        dev = _dev()
        d = self.desc
        u8 = input_lut is not None
        self.input_lut_gpu = None
        if u8:
            self.input_lut_gpu = torch.from_numpy(np.ascontiguousarray(input_lut, dtype=np.float32).reshape(3, 256)).to(dev)
        self.input_gpu = torch.empty((d.B, 3, d.H, d.W), dtype=torch.uint8 if u8 else torch.float32, device=dev)
        self.set_input(input)
        f = torch.from_numpy(config.read(d.R * d.S * 3 * d.O).reshape(d.R * d.S, 3, d.O)).to(dev)
        self.filter_gpu = ops.pack_inconv_filter(f)
        self.bn = config.read(d.O)
        self.bn_gpu = torch.from_numpy(self.bn).to(dev)
        self.specialized = None
        if specialize and d.O <= 128:
            try:
                self.specialized = ops.inconv_specialize(d, self.filter_gpu, self.bn_gpu)
            except Exception as e:      # no NVRTC on this machine: the general CUDA kernel runs
                import warnings
                warnings.warn("%s: first-layer kernel not specialised (%s)" % (self.name, e))
        Ow = (d.O + 31) // 32
        self.output_gpu = torch.zeros((d.B, d.OH, d.OW, Ow), dtype=torch.int32, device=dev)
        if self.save_residual:
            self.output_residual_gpu = torch.zeros((d.B, d.pool * d.OH, d.pool * d.OW, d.O),
                                                   dtype=_residual_dtype(self.residual_bound), device=dev)
        return self

    next_layer = None      # (consumer's descriptor, its planes): see Conv128LayerParam
    # The saved int16 residual is laid out by 8-channel chunk (TCBNN_RES_INT16_CHUNKED) instead of
    # NHWC: set by models.Network when this layer and the residual's consumers all handle it.
    residual_chunked = False

    def can_write_chunked_residual(self):
        d = self.desc
        return (self.specialized is not None and self.output_residual_gpu is not None and
                self.output_residual_gpu.dtype == torch.int16 and d.O % 8 == 0 and d.pool == 1)

    def download_output_residual(self):
        """The saved residual as int32 NHWC [B][P][Q][O] on the host, whatever its device layout."""
        d = self.desc
        t = self.output_residual_gpu
        if self.residual_chunked:
            t = ops.chunked_to_nhwc(_live_chunked(t, d.B))
        return t[:d.B].cpu().numpy().astype(np.int32)

    def set_batch(self, n):
        """Process the first n images from now on (n <= the constructor's batch); the compiled
        kernel does not depend on the batch."""
        if not 0 < n <= self.batch:
            raise ValueError("%s: batch %d outside 1..%d" % (self.name, n, self.batch))
        self.desc.B = n

    def set_input(self, input):
        src = input if torch.is_tensor(input) else torch.from_numpy(np.ascontiguousarray(input))
        if src.dtype != self.input_gpu.dtype:
            raise ValueError("%s: input dtype %s, layer was initialised for %s" % (self.name, src.dtype, self.input_gpu.dtype))
        src = src.reshape((-1,) + tuple(self.input_gpu.shape[1:]))
        self.input_gpu[:src.shape[0]].copy_(src, non_blocking=True)

    def forward(self):
        ops.inconv_layer(self.desc, self.input_gpu, self.filter_gpu, self.bn_gpu, out=self.output_gpu,
                         res_out_buf=self.output_residual_gpu, lut=self.input_lut_gpu,
                         specialized=self.specialized,
                         next_layer=self.next_layer if self.specialized is not None else None,
                         res_out_chunked=self.residual_chunked)

    def get_output_gpu(self):
        return self.output_gpu

    def get_output_residual_gpu(self):
        return self.output_residual_gpu

    def download_output(self):
        return self.output_gpu.cpu().numpy().view(np.uint32)

    def download_full_output(self):
        d = self.desc
        rows = d.B * d.OH * d.OW
        return ops.unpack_rows(self.output_gpu[:d.B].reshape(rows, -1), d.O).reshape(d.B, d.OH, d.OW, d.O).cpu().numpy()


class Conv128LayerParam:
    """param.h:872-1065.  Binary conv layer with threshold / OR-pool / residual fused."""

    def __init__(self, name, input_height, input_width, filter_height, filter_width,
                 input_channels, output_channels, batch, stride_height=1, stride_width=1,
                 padding=True, pool_height=1, pool_width=1, ahead_fc=False, save_residual=False,
                 inject_residual=False, residual_channels=0, residual_pool=False):
        if pool_height != pool_width:
            raise ValueError("only square pooling windows are supported")
        self.name = name
        self.input_height, self.input_width = input_height, input_width
        self.filter_height, self.filter_width = filter_height, filter_width
        self.input_channels, self.output_channels, self.batch = input_channels, output_channels, batch
        self.stride_height, self.stride_width, self.padding = stride_height, stride_width, padding
        self.pool_height, self.pool_width = pool_height, pool_width
        self.ahead_fc, self.save_residual = ahead_fc, save_residual
        self.inject_residual, self.residual_channels = inject_residual, residual_channels
        self.residual_pool = residual_pool
        self.desc = ops.conv_desc(batch, input_height, input_width, input_channels, output_channels,
                                  filter_height, filter_width, stride_height, stride_width, padding,
                                  pool_height)
        self.pad_h, self.pad_w = self.desc.pad_h, self.desc.pad_w
        self.output_height, self.output_width = self.desc.OH, self.desc.OW
        self.output_residual_gpu = self.input_residual_gpu = None
        self.residual_bound = None

    def initialize(self, config, prev_layer_gpu, input_residual_gpu=None, input_residual_bound=None):
        """input_residual_bound (extension): bound of |injected residual| if known; it decides
        whether this layer's saved residual can be int16."""
        dev = _dev()
        d = self.desc
        fan = d.C * d.R * d.S
        if not self.inject_residual:
            self.residual_bound = fan
        elif input_residual_bound is not None:
            self.residual_bound = fan + int(input_residual_bound)
        f = torch.from_numpy(config.read(d.R * d.S * d.C * d.O).reshape(d.R * d.S, d.C, d.O)).to(dev)
        self.filter_gpu = ops.pack_conv_filter(f)
        self.prepared = ops.conv_prepare(d, self.filter_gpu)
        self.bn = config.read(d.O)
        self.bn_gpu = torch.from_numpy(self.bn).to(dev)
        Ow = (d.O + 31) // 32
        words = d.OH * d.OW * Ow
        # a layer feeding an FC layer pads each image to a whole number of 128-bit rows
        self.out_image_stride = ops.step128_words(words * 32) if self.ahead_fc else words
        self.output_gpu = torch.zeros((d.B, self.out_image_stride), dtype=torch.int32, device=dev)
        if self.save_residual:
            self.output_residual_gpu = torch.zeros((d.B, d.pool * d.OH, d.pool * d.OW, d.O),
                                                   dtype=_residual_dtype(self.residual_bound), device=dev)
        self.set_input_gpu(prev_layer_gpu)
        if self.inject_residual:
            self.set_input_residual_gpu(input_residual_gpu)
        return self

    def set_batch(self, n):
        """Process the first n images from now on (n <= the constructor's batch).  The layout of the
        pre-expanded input planes depends on the batch, so planes a producer fills are cleared
        (their padding positions must read as zero)."""
        if not 0 < n <= self.batch:
            raise ValueError("%s: batch %d outside 1..%d" % (self.name, n, self.batch))
        if n != self.desc.B and self.input_planes is not None:
            self.input_planes.zero_()
        self.desc.B = n

    def set_input_gpu(self, t):
        d = self.desc
        self.input_gpu = t.reshape(self.batch, d.H, d.W, (d.C + 31) // 32)

    def set_input_residual_gpu(self, t):
        if t is None:
            raise ValueError("%s: inject_residual needs a residual tensor" % self.name)
        self.input_residual_gpu = t

    # Hand-over of the pre-expanded input between consecutive layers (tcbnn_conv_layer_x), wired
    # by models.Network: next_layer = (consumer's descriptor, its planes); input_planes = this
    # layer's planes when its producer fills them.
    next_layer = None
    input_planes = None
    # chunk-major int16 residual tensors (TCBNN_RES_INT16_CHUNKED), wired by models.Network
    residual_chunked = False            # this layer's saved residual
    input_residual_chunked = False      # the injected one

    def can_write_chunked_residual(self):
        return (self.output_residual_gpu is not None and self.output_residual_gpu.dtype == torch.int16 and
                ops.conv_prefers_chunked_residual(self.desc) and self.has_workspace())

    def can_read_chunked_residual(self):
        if self.desc.pool != 1 or not self.has_workspace() or ops.new_planes_bytes(self.desc) == 0:
            return False
        return bool(self.residual_pool) or ops.conv_prefers_chunked_residual(self.desc)

    def has_workspace(self):
        return ops.conv_workspace(self.desc, self.input_gpu.device) is not None

    def download_output_residual(self):
        """The saved residual as int32 NHWC [B][P][Q][O] on the host, whatever its device layout."""
        d = self.desc
        t = self.output_residual_gpu
        if self.residual_chunked:
            t = ops.chunked_to_nhwc(_live_chunked(t, d.B))
        return t[:d.B].cpu().numpy().astype(np.int32)

    def kernel_launches(self):
        """Kernels one forward() launches: a layer that runs on a pre-expanded input launches the
        expansion pass too unless its producer filled the planes."""
        has_ws = ops.conv_workspace(self.desc, self.input_gpu.device) is not None
        own_expand = self.input_planes is None and ops.new_planes_bytes(self.desc) > 0
        # a pooled NHWC int16 residual is reduced by a pass of its own; the chunk-major layout is
        # read in place by the kernel's tile-per-group epilogue (which also needs the saved
        # residual, if any, chunk-major)
        in_place = self.input_residual_chunked and (self.output_residual_gpu is None or self.residual_chunked)
        pools_residual = (self.inject_residual and self.residual_pool and has_ws and self.desc.pool == 1 and
                          self.input_residual_gpu is not None and self.input_residual_gpu.dtype == torch.int16 and
                          not in_place)
        pools_output = self.desc.pool != 1 and has_ws          # tcgen05 on the pre-pool grid + OR-pooling pass
        return 1 + int(own_expand) + int(pools_residual) + int(pools_output)

    def forward(self):
        ops.conv_layer(self.desc, self.input_gpu, self.prepared, self.bn_gpu,
                       res_in=self.input_residual_gpu if self.inject_residual else None,
                       residual_channels=self.residual_channels, residual_pool=self.residual_pool,
                       out=self.output_gpu, out_image_stride=self.out_image_stride,
                       res_out_buf=self.output_residual_gpu,
                       workspace=self.input_planes, workspace_ready=self.input_planes is not None,
                       next_layer=self.next_layer,
                       res_in_chunked=self.input_residual_chunked and self.inject_residual,
                       res_out_chunked=self.residual_chunked,
                       # int16 was chosen from the bound fan-in + bound of the injected residual
                       res_out_proven=self.residual_bound is not None and self.residual_bound <= 32767)

    def get_output_gpu(self):
        return self.output_gpu

    def get_output_residual_gpu(self):
        return self.output_residual_gpu

    def download_output(self):
        return self.output_gpu.cpu().numpy().view(np.uint32)

    def download_full_output(self):
        d = self.desc
        Ow = (d.O + 31) // 32
        bits = self.output_gpu[:d.B, :d.OH * d.OW * Ow].reshape(d.B * d.OH * d.OW, Ow).contiguous()
        return ops.unpack_rows(bits, d.O).reshape(d.B, d.OH, d.OW, d.O).cpu().numpy()
