"""Network topologies of the reference drivers as data, seeded synthetic weights and inputs,
and the GPU runner that chains the layer objects.

A topology is a list of layer specs (dicts).  The same list drives the GPU runner here and the
CPU oracle runner used by the tests, so both sides execute the identical network.

Topologies follow the reference drivers, not the textbook networks:
  * resnet18   : imagenet_resnet.cu:223-325 -- 7x7 stride-4 first layer (56x56x64, residual
                 saved), 16 binary 3x3 convs in 8 basic blocks (64/128/256/512; stride 2 at the
                 start of stages 2-4), every second conv adds the previous block's integer
                 residual (2x2 max-pooled when the stage changes), FC 25088->512, out 512->1000.
  * resnet_cifar: cifar10_resnet.cu:189-259 -- three-stage variant on 32x32 images.
  * vgg_cifar  : cifar10_vgg.cu:162-199 -- conv 3->128, 128->128+pool, ->256, 256+pool, ->512,
                 512+pool (feeds FC), FC 8192->1024->1024, out ->10.
  * mlp        : mnist_mlp.cu:112-126 -- 784 -> 1024 -> 1024 -> 1024 -> 10.
  * alexnet, vgg16_imagenet : alexnet.cu:141-178, imagenet_vgg.cu:217-280 (11x11 / 5x5 filters,
                 192 / 384 channels, pooled layers at 224 x 224).
"""
import numpy as np

from . import ops, param


def resnet18_spec(batch, image=224, classes=1000):
    L = [dict(type="inconv", name="Conv1", H=image, W=image, R=7, S=7, C=3, O=64,
              stride=4, pool=1, save_residual=True)]

    def conv(name, C, O, stride=1, **kw):
        L.append(dict(type="conv", name=name, C=C, O=O, R=3, S=3, stride=stride, pool=1, **kw))

    # stage 1
    conv("L1B1C1", 64, 64)
    conv("L1B1C2", 64, 64, save_residual=True, inject=0, residual_channels=64)
    conv("L1B2C1", 64, 64)
    conv("L1B2C2", 64, 64, save_residual=True, inject=2, residual_channels=128)
    # stage 2
    conv("L2B1C1", 64, 128, stride=2)
    conv("L2B1C2", 128, 128, save_residual=True, inject=4, residual_channels=128, residual_pool=True)
    conv("L2B2C1", 128, 128)
    conv("L2B2C2", 128, 128, save_residual=True, inject=6, residual_channels=128)
    # stage 3
    conv("L3B1C1", 128, 256, stride=2)
    conv("L3B1C2", 256, 256, save_residual=True, inject=8, residual_channels=128, residual_pool=True)
    conv("L3B2C1", 256, 256)
    conv("L3B2C2", 256, 256, save_residual=True, inject=10, residual_channels=256)
    # stage 4
    conv("L4B1C1", 256, 512, stride=2)
    conv("L4B1C2", 512, 512, save_residual=True, inject=12, residual_channels=256, residual_pool=True)
    conv("L4B2C1", 512, 512)
    conv("L4B2C2", 512, 512, ahead_fc=True, inject=14, residual_channels=512)
    L.append(dict(type="fc", name="Fc1", N=512))
    L.append(dict(type="out", name="Fout", N=classes))
    return dict(name="resnet18", batch=batch, layers=L)


def resnet_cifar_spec(batch, image=32, classes=10):
    """cifar10_resnet.cu:189-259 -- 3x3 first layer to 128 channels (residual saved), three stages
    of two basic blocks (128/256/512, stride 2 at the start of stages 2 and 3), FC -> 512 -> out."""
    L = [dict(type="inconv", name="Conv1", H=image, W=image, R=3, S=3, C=3, O=128, stride=1, pool=1,
              save_residual=True)]

    def conv(name, C, O, stride=1, **kw):
        L.append(dict(type="conv", name=name, C=C, O=O, R=3, S=3, stride=stride, pool=1, **kw))

    conv("L1B1C1", 128, 128)
    conv("L1B1C2", 128, 128, save_residual=True, inject=0, residual_channels=128)
    conv("L1B2C1", 128, 128)
    conv("L1B2C2", 128, 128, save_residual=True, inject=2, residual_channels=128)
    conv("L2B1C1", 128, 256, stride=2)
    conv("L2B1C2", 256, 256, save_residual=True, inject=4, residual_channels=128, residual_pool=True)
    conv("L2B2C1", 256, 256)
    conv("L2B2C2", 256, 256, save_residual=True, inject=6, residual_channels=256)
    conv("L3B1C1", 256, 512, stride=2)
    conv("L3B1C2", 512, 512, save_residual=True, inject=8, residual_channels=256, residual_pool=True)
    conv("L3B2C1", 512, 512)
    conv("L3B2C2", 512, 512, ahead_fc=True, inject=10, residual_channels=512)
    L.append(dict(type="fc", name="Fc1", N=512))
    L.append(dict(type="out", name="Fout", N=classes))
    return dict(name="resnet_cifar", batch=batch, layers=L)


def vgg_cifar_spec(batch, image=32, classes=10):
    L = [dict(type="inconv", name="Conv1", H=image, W=image, R=3, S=3, C=3, O=128, stride=1, pool=1)]
    for name, C, O, pool, afc in [("Conv2", 128, 128, 2, False), ("Conv3", 128, 256, 1, False),
                                  ("Conv4", 256, 256, 2, False), ("Conv5", 256, 512, 1, False),
                                  ("Conv6", 512, 512, 2, True)]:
        L.append(dict(type="conv", name=name, C=C, O=O, R=3, S=3, stride=1, pool=pool, ahead_fc=afc))
    L += [dict(type="fc", name="Fc1", N=1024), dict(type="fc", name="Fc2", N=1024),
          dict(type="out", name="Fout", N=classes)]
    return dict(name="vgg_cifar", batch=batch, layers=L)


def alexnet_spec(batch, image=224, hidden=4096, classes=1000):
    """alexnet.cu:141-178 -- 11x11/4 first layer with 2x2 pool (64 channels), 5x5 64->192 with
    pool, 3x3 192->384, 384->256, 256->256 with pool (feeds FC), FC -> hidden -> hidden -> out."""
    L = [dict(type="inconv", name="Conv1", H=image, W=image, R=11, S=11, C=3, O=64, stride=4, pool=2),
         dict(type="conv", name="Conv2", C=64, O=192, R=5, S=5, stride=1, pool=2),
         dict(type="conv", name="Conv3", C=192, O=384, R=3, S=3, stride=1, pool=1),
         dict(type="conv", name="Conv4", C=384, O=256, R=3, S=3, stride=1, pool=1),
         dict(type="conv", name="Conv5", C=256, O=256, R=3, S=3, stride=1, pool=2, ahead_fc=True),
         dict(type="fc", name="Fc1", N=hidden), dict(type="fc", name="Fc2", N=hidden),
         dict(type="out", name="Fout", N=classes)]
    return dict(name="alexnet", batch=batch, layers=L)


def vgg16_imagenet_spec(batch, image=224, hidden=4096, classes=1000):
    """imagenet_vgg.cu:217-280 -- thirteen 3x3 layers (64, 64+pool, 128, 128+pool, 256, 256,
    256+pool, 512, 512, 512+pool, 512, 512, 512+pool feeding FC), FC -> hidden -> hidden -> out."""
    L = [dict(type="inconv", name="Conv1", H=image, W=image, R=3, S=3, C=3, O=64, stride=1, pool=1)]
    cfg = [(64, 64, 2), (64, 128, 1), (128, 128, 2), (128, 256, 1), (256, 256, 1), (256, 256, 2),
           (256, 512, 1), (512, 512, 1), (512, 512, 2), (512, 512, 1), (512, 512, 1), (512, 512, 2)]
    for i, (C, O, pool) in enumerate(cfg):
        L.append(dict(type="conv", name="Conv%d" % (i + 2), C=C, O=O, R=3, S=3, stride=1, pool=pool,
                      ahead_fc=(i == len(cfg) - 1)))
    L += [dict(type="fc", name="Fc1", N=hidden), dict(type="fc", name="Fc2", N=hidden),
          dict(type="out", name="Fout", N=classes)]
    return dict(name="vgg16_imagenet", batch=batch, layers=L)


def mlp_spec(batch, features=784, hidden=1024, classes=10):
    L = [dict(type="in", name="Fin", K=features),
         dict(type="fc", name="Fc1", N=hidden), dict(type="fc", name="Fc2", N=hidden),
         dict(type="fc", name="Fc3", N=hidden), dict(type="out", name="Fout", N=classes)]
    return dict(name="mlp", batch=batch, layers=L)


def layer_shapes(spec):
    """Resolve H/W/K of every layer by walking the chain; returns a list of dicts with the
    resolved fields added (H, W, OH, OW, K)."""
    out = []
    H = W = Cprev = K = None
    for l in spec["layers"]:
        l = dict(l)
        t = l["type"]
        if t == "in":
            K = l["K"]
        elif t in ("inconv", "conv"):
            if t == "inconv":
                H, W = l["H"], l["W"]
            else:
                l["H"], l["W"] = H, W
            s, p, R = l["stride"], l["pool"], l["R"]
            bh = (H + s - 1) // s
            bw = (W + s - 1) // s
            l["OH"], l["OW"] = (bh + p - 1) // p, (bw + p - 1) // p
            H, W, Cprev = l["OH"], l["OW"], l["O"]
            K = H * W * Cprev
        elif t in ("fc", "out"):
            l["K"] = K
            K = l["N"]
        out.append(l)
    return out


def synthetic_weights(spec, seed):
    """Arrays in launch_array order (utility.h:188-196): per conv layer filter[R*S][C][O] then
    thresholds[O]; per FC weight[K][N] then thresholds[N]; output layer weight, scale, bias.
    Weights are +-1 (Bernoulli 0.5), thresholds N(0, sqrt(fan_in)); the first layer's
    thresholds are scaled to its fp32 input range."""
    g = np.random.Generator(np.random.PCG64(seed))
    arrays = []

    def pm1(shape):
        return (g.integers(0, 2, size=shape, dtype=np.int8).astype(np.float32) * 2 - 1)

    for l in layer_shapes(spec):
        t = l["type"]
        if t == "inconv":
            arrays.append(pm1((l["R"] * l["S"], 3, l["O"])))
            arrays.append((g.standard_normal(l["O"]) * np.sqrt(3 * l["R"] * l["S"])).astype(np.float32))
        elif t == "conv":
            fan = l["C"] * l["R"] * l["S"]
            arrays.append(pm1((l["R"] * l["S"], l["C"], l["O"])))
            arrays.append((g.standard_normal(l["O"]) * np.sqrt(fan)).astype(np.float32))
        elif t == "fc":
            arrays.append(pm1((l["K"], l["N"])))
            arrays.append((g.standard_normal(l["N"]) * np.sqrt(l["K"])).astype(np.float32))
        elif t == "out":
            arrays.append(pm1((l["K"], l["N"])))
            arrays.append((g.standard_normal(l["N"]) * 0.1 + 1.0).astype(np.float32))
            arrays.append(g.standard_normal(l["N"]).astype(np.float32))
    return arrays


def synthetic_input(spec, seed, batch=None):
    """Seeded stand-in for the datasets, with the value ranges the reference readers produce:
    images are uint8 uniform, scaled to [0,1] and normalised per channel (data.cpp:295-315,
    534-542); MLP features are uniform[0,1) minus 0.5 because In128 binarises at 0."""
    g = np.random.Generator(np.random.PCG64(seed))
    B = batch or spec["batch"]
    first = spec["layers"][0]
    if first["type"] == "in":
        return (g.random((B, first["K"]), dtype=np.float32) - np.float32(0.5))
    u8 = g.integers(0, 256, size=(B, 3, first["H"], first["W"]), dtype=np.uint8)
    mean = np.array([0.485, 0.456, 0.406], dtype=np.float32).reshape(1, 3, 1, 1)
    std = np.array([0.229, 0.224, 0.225], dtype=np.float32).reshape(1, 3, 1, 1)
    return ((u8.astype(np.float32) / np.float32(255.0)) - mean) / std


# max |value| synthetic_input() can produce for images: (1 - 0.406) / 0.225
SYNTHETIC_IMAGE_ABS_BOUND = 2.65


def synthetic_input_u8(spec, seed, batch=None):
    """The same synthetic images as synthetic_input(), as bytes plus the per-channel table of
    their fp32 values: lut[c][v] is computed with the arithmetic synthetic_input() applies, so
    lut[c][u8] reproduces its output bit for bit.  Returns (uint8 [B][3][H][W], fp32 [3][256])."""
    g = np.random.Generator(np.random.PCG64(seed))
    B = batch or spec["batch"]
    first = spec["layers"][0]
    if first["type"] == "in":
        raise ValueError("byte input is for image networks")
    u8 = g.integers(0, 256, size=(B, 3, first["H"], first["W"]), dtype=np.uint8)
    mean = np.array([0.485, 0.456, 0.406], dtype=np.float32).reshape(3, 1)
    std = np.array([0.229, 0.224, 0.225], dtype=np.float32).reshape(3, 1)
    v = np.arange(256, dtype=np.float32).reshape(1, 256)
    lut = ((v / np.float32(255.0)) - mean) / std
    return u8, lut.astype(np.float32)


class Network:
    """Chain of layer objects built from a spec, the way the reference drivers build theirs
    (new XLayerParam(...) ; initialize(config, prev->get_output_gpu(), residual))."""

    def __init__(self, spec, weights, input_host, input_abs_bound=None, input_lut=None, handover=True):
        """input_abs_bound: max |pixel value| the caller guarantees; with it the residual chain
        is provably small and is stored as int16 instead of int32.
        input_lut: images arrive as uint8 with this [3][256] table of their fp32 values.
        handover: producers write the pre-expanded input of the conv layers that follow them."""
        self.spec = spec
        B = spec["batch"]
        cfg = weights if hasattr(weights, "read") else param.ArrayConfig(weights)
        self.layers = []
        prev = None
        for l in layer_shapes(spec):
            t = l["type"]
            if t == "in":
                obj = param.In128LayerParam(l["name"], B, l["K"]).initialize(input_host)
            elif t == "inconv":
                obj = param.InConv128LayerParam(l["name"], l["H"], l["W"], l["R"], l["S"], 3, l["O"], B,
                                                l["stride"], l["stride"], True, l["pool"], l["pool"],
                                                l.get("save_residual", False),
                                                input_abs_bound=input_abs_bound).initialize(
                                                    input_host, cfg, input_lut=input_lut)
            elif t == "conv":
                inj = l.get("inject")
                obj = param.Conv128LayerParam(l["name"], l["H"], l["W"], l["R"], l["S"], l["C"], l["O"], B,
                                              l["stride"], l["stride"], True, l["pool"], l["pool"],
                                              l.get("ahead_fc", False), l.get("save_residual", False),
                                              inj is not None, l.get("residual_channels", 0),
                                              l.get("residual_pool", False))
                res = self.layers[inj].get_output_residual_gpu() if inj is not None else None
                rb = self.layers[inj].residual_bound if inj is not None else None
                obj.initialize(cfg, prev.get_output_gpu(), res, rb)
            elif t == "fc":
                obj = param.Fc128LayerParam(l["name"], B, l["K"], l["N"]).initialize(cfg, prev.get_output_gpu())
            elif t == "out":
                obj = param.Out128LayerParam(l["name"], B, l["K"], l["N"]).initialize(cfg, prev.get_output_gpu())
            else:
                raise ValueError(t)
            self.layers.append(obj)
            prev = obj
        if handover:
            self._wire_handover()
            self._wire_residual_layouts()

    def _wire_handover(self):
        """Consecutive conv layers: where the consumer runs on a pre-expanded input, its producer
        writes that input itself (tcbnn_conv_layer_x) and the consumer skips its expansion pass."""
        for prod, cons in zip(self.layers, self.layers[1:]):
            if type(cons).__name__ != "Conv128LayerParam":
                continue
            kind = type(prod).__name__
            if kind == "Conv128LayerParam":
                dense = prod.out_image_stride == prod.desc.OH * prod.desc.OW * ((prod.desc.O + 31) // 32)
                if prod.desc.pool != 1 or not dense:
                    continue
            elif kind == "InConv128LayerParam":
                if getattr(prod, "specialized", None) is None:
                    continue
            else:
                continue
            planes = ops.new_planes(cons.desc, cons.input_gpu.device)
            if planes is None:
                continue
            prod.next_layer = (cons.desc, planes)
            cons.input_planes = planes

    def _wire_residual_layouts(self):
        """An int16 residual tensor is kept in the chunk-major layout (TCBNN_RES_INT16_CHUNKED)
        when the layer that saves it and every layer that injects it move residual rows directly
        between registers and memory: one thread per pixel then touches whole lines per warp."""
        consumers = {}
        for l in self.layers:
            if type(l).__name__ == "Conv128LayerParam" and l.inject_residual:
                for p in self.layers:
                    if getattr(p, "output_residual_gpu", None) is l.input_residual_gpu and p.output_residual_gpu is not None:
                        consumers.setdefault(id(p), (p, []))[1].append(l)
        for p, cons in consumers.values():
            if p.can_write_chunked_residual() and all(c.can_read_chunked_residual() for c in cons):
                p.residual_chunked = True
                for c in cons:
                    c.input_residual_chunked = True

    def set_input(self, x):
        self.layers[0].set_input(x)

    def set_batch(self, n):
        """Run the following passes on the first n images (n <= the batch the network was built
        for) without rebuilding anything: buffers keep their size, kernels take the live batch.
        The logits of the live images are the first n rows of the output."""
        for l in self.layers:
            l.set_batch(n)
        self.live_batch = n

    def forward(self):
        for l in self.layers:
            l.forward()
        return self.layers[-1].get_output_gpu()

    def forward_graph(self):
        """forward() replayed from a CUDA graph: the layer launches (every entry point takes the
        stream and none allocates or synchronises) are captured once per input buffer, after one
        eager pass that lets the first layer compile its kernel variants, and replayed as one
        submission on the current stream.  Same launches, same results; the host's per-launch
        work and the gaps between the launches go away."""
        import torch
        first = self.layers[0]
        key = (first.input_gpu.data_ptr(), getattr(self, "live_batch", None))
        graphs = self.__dict__.setdefault("_graphs", {})
        g = graphs.get(key)
        if g is None:
            self.forward()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            # thread_local: only this thread's calls are checked during the capture; another
            # thread (e.g. a communicator's watchdog polling its events) is left alone
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self.forward()
            graphs[key] = g
        g.replay()
        return self.layers[-1].get_output_gpu()


class HostFeeder:
    """Feeds a Network from pinned host batches with the host->device copy of batch i+1 running
    on its own stream while batch i is being computed (two device input buffers).  Every batch
    still pays its own copy; only the waiting is overlapped."""

    def __init__(self, net, graph=True):
        """graph: run each forward pass as a CUDA-graph replay (Network.forward_graph)."""
        self.graph = graph
        import torch
        self.net = net
        self.first = net.layers[0]
        self.bufs = [self.first.input_gpu, torch.empty_like(self.first.input_gpu)]
        self.copy_stream = torch.cuda.Stream()
        self.copied = [torch.cuda.Event(), torch.cuda.Event()]
        self.free = [torch.cuda.Event(), torch.cuda.Event()]
        self.read_stream = torch.cuda.Stream()
        self.computed = torch.cuda.Event()
        self.read_done = torch.cuda.Event()
        self.n = 0
        self.pending = None

    def _enqueue_copy(self, slot, x_host):
        import torch
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.free[slot])
            self.bufs[slot].copy_(x_host.reshape(self.bufs[slot].shape), non_blocking=True)
            self.copied[slot].record(self.copy_stream)

    def run(self, batches, on_result=None, result_host=None):
        """batches: iterable of pinned host tensors; on_result(logits_device) is called after
        each forward pass has been queued.  result_host: pinned host tensor that receives every
        batch's logits; that device->host read runs on a third stream, beside the next batch's
        compute and input copy, and the next pass's output layer waits for it."""
        import torch
        main = torch.cuda.current_stream()
        for ev in self.free:
            ev.record(main)
        self.read_done.record(main)
        it = iter(batches)
        nxt = next(it, None)
        slot = 0
        if nxt is not None:
            self._enqueue_copy(slot, nxt)
        while nxt is not None:
            cur_slot = slot
            nxt = next(it, None)
            if nxt is not None:
                slot ^= 1
                self._enqueue_copy(slot, nxt)
            main.wait_event(self.copied[cur_slot])
            self.first.input_gpu = self.bufs[cur_slot]
            main.wait_event(self.read_done)          # the logits buffer is about to be rewritten
            out = self.net.forward_graph() if self.graph else self.net.forward()
            self.free[cur_slot].record(main)
            if on_result is not None:
                on_result(out)
            if result_host is not None:
                self.computed.record(main)
                with torch.cuda.stream(self.read_stream):
                    self.read_stream.wait_event(self.computed)
                    result_host.copy_(out, non_blocking=True)
                    self.read_done.record(self.read_stream)
        main.wait_event(self.read_done)
