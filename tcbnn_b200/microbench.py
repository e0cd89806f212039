"""Kernel microbenchmarks on the standalone configurations of the reference's side benchmarks.

    python -m tcbnn_b200.microbench --case c1 [--iters 50]
    python -m tcbnn_b200.microbench --case c2 [--batch 256] [--iters 20]

c1: bit GEMM 1024 x 1024 x 4096 (bmm/benchmark-bmm.cu shape), int32 output.
c2: one binary conv layer, NHWC batch x 56 x 56 x 128 -> 128 channels, 3x3, stride 1, pad 1,
    threshold + repack (bconv/benchmark-bconv.cu shape), optionally saving an int32 residual.
conv: one binary 3x3 conv layer of any ResNet-18 shape: --hw, --cin, --cout, --stride,
    --residual (int16 residual injected and saved, as in every second conv of a basic block).
stem: the fp32 first layer, batch x 3 x 224 x 224 -> 56 x 56 x 64, 7x7 stride 4, int16 residual.
Prints one JSON line: tera bit-ops/s (2*M*N*K, all taps counted, the reference's formula at
bmm/bmma_op_test/main_test.cu:368) and the fraction of the b1 MMA issue rate measured in the
same process.  Seeded synthetic operands (Bernoulli 0.5 bits)."""
import argparse
import json

import torch

from . import ops


def _words(shape, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=dev, generator=g)


_GRAPH = False


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if _GRAPH:
        # the calls recorded once and replayed: device time without the host's launch cost
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(iters):
                    fn()
            graph.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            side.synchronize()
        return e0.elapsed_time(e1) / iters
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _l_pack(x, out):
    from . import lib as _lib
    import ctypes as C
    _lib.call("tcbnn_pack_rows", C.c_void_p(x.data_ptr()), x.shape[0], x.shape[1], out.shape[1],
              C.c_void_p(out.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="c2", choices=["c1", "c2", "conv", "stem", "net", "pack"])
    ap.add_argument("--net", default="vgg_cifar",
                    choices=["mlp", "vgg_cifar", "resnet_cifar", "alexnet", "vgg16_imagenet", "resnet18"],
                    help="net: which reference driver's topology (C3 = mlp at batch 8192, C4 = vgg_cifar at 1024)")
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--cin", type=int, default=64)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--residual", action="store_true", help="c2: also save the int32 residual")
    ap.add_argument("--chunked", action="store_true",
                    help="conv --residual: int16 residuals in the chunk-major layout (TCBNN_RES_INT16_CHUNKED)")
    ap.add_argument("--mnk", default="1024,1024,4096", help="c1: M,N,K of the bit GEMM")
    ap.add_argument("--gemm-path", type=int, default=0, help="c1: 0 automatic, 1 warp-level b1 MMA only")
    ap.add_argument("--gemm-plan", default="-1,-1", help="c1: pair,splits forced on the tcgen05 GEMM (-1 automatic)")
    ap.add_argument("--trace", action="store_true", help="c1: print the kernel's cycle counters")
    ap.add_argument("--gemm-mode", default="int32", choices=["int32", "fc", "out"],
                    help="c1: int32 sums, threshold bits (Fc layer) or scale + bias (Out layer)")
    ap.add_argument("--graph", action="store_true",
                    help="time the calls as one replayed CUDA graph (small kernels: the host cannot launch fast enough)")
    ap.add_argument("--no-peak", action="store_true")
    ap.add_argument("--specialized", action="store_true", help="stem: the kernel compiled for the filter")
    a = ap.parse_args()
    global _GRAPH
    _GRAPH = a.graph
    dev = torch.device("cuda", 0)
    if a.case == "net":
        import numpy as np
        from . import models
        spec = getattr(models, a.net + "_spec")(a.batch)
        net = models.Network(spec, models.synthetic_weights(spec, 1),
                             torch.from_numpy(np.ascontiguousarray(models.synthetic_input(spec, 2))),
                             input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND if "resnet" in a.net else None)
        for _ in range(3):
            net.forward()
        torch.cuda.synchronize()
        ev = []
        for _ in range(a.iters):
            for l in net.layers:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                l.forward()
                e1.record()
                ev.append((l.name, e0, e1))
        torch.cuda.synchronize()
        per = {}
        for n, e0, e1 in ev:
            per[n] = per.get(n, 0.0) + e0.elapsed_time(e1) / a.iters
        ms = sum(per.values())
        print(json.dumps({"case": "net", "net": a.net, "batch": a.batch, "ms": ms,
                          "images_per_s": a.batch / (ms * 1e-3), "layer_ms": {k: round(v, 4) for k, v in per.items()}}))
        return
    if a.case == "pack":
        # the input layer (In128LayerFMT): fp32 rows -> bit rows.  Memory-bound: 4 bytes read and
        # 1/8 byte written per value.  Rows x 784 features; the default 262144 rows (822 MB) do
        # not fit in L2.
        rows = a.batch if a.batch != 256 else 262144
        x = torch.rand((rows, 784), device=dev) - 0.5
        out = ops.pack_rows(x)
        ms = _time(lambda: _l_pack(x, out), a.iters)
        nbytes = x.numel() * 4 + out.numel() * 4
        print(json.dumps({"case": "pack", "workload": "fp32 [%d][784] -> bit rows (tcbnn_pack_rows)" % rows, "ms": ms,
                          "bytes": nbytes, "gb_per_s": nbytes / (ms * 1e-3) / 1e9}))
        return
    if a.case == "c1":
        M, N, K = (int(v) for v in a.mnk.split(","))
        ld = ops.step128_words(K)
        A, B = _words((M, ld), 1, dev), _words((N, ld), 2, dev)
        ops.set_gemm_plan(*(int(v) for v in a.gemm_plan.split(",")))
        ws = ops.gemm_workspace(M, N, K, dev)
        ops.set_gemm_path(a.gemm_path)
        if a.gemm_mode == "int32":
            out = torch.empty((M, N), dtype=torch.int32, device=dev)
            fn = lambda: ops.bgemm(A, B, K, out=out, workspace=ws)
        elif a.gemm_mode == "fc":
            thr = torch.randn(N, device=dev) * K ** 0.5
            out = torch.zeros((M, ops.step128_words(N)), dtype=torch.int32, device=dev)
            fn = lambda: ops.fc_layer(A, B, thr, K, out=out, workspace=ws)
        else:
            sc, bi = torch.randn(N, device=dev), torch.randn(N, device=dev)
            out = torch.empty((M, N), dtype=torch.float32, device=dev)
            fn = lambda: ops.out_layer(A, B, sc, bi, K, out=out, workspace=ws)
        ms = _time(fn, a.iters)
        if a.trace:
            from . import lib as _lib
            import ctypes as C
            tb = torch.zeros(16, dtype=torch.int64, device=dev)
            _lib.call("tcbnn_conv_set_trace", C.c_void_p(tb.data_ptr()))
            fn()
            torch.cuda.synchronize()
            _lib.call("tcbnn_conv_set_trace", C.c_void_p(0))
            t = tb.tolist()
            print(json.dumps({"trace": {"loader_wait_free": t[10], "mma_total": t[11], "mma_wait_full": t[12],
                                        "epilogue_wait": t[13], "kblocks": t[14], "epilogue": t[15], "cta_total": t[9]}}))
        ops.set_gemm_path(0)
        work = 2.0 * M * N * K
        desc = "bit GEMM %dx%dx%d (%s, %d launches)" % (M, N, K, a.gemm_mode,
                                                       1 if a.gemm_path else ops.gemm_launches(M, N, K, ws))
    elif a.case == "stem":
        Bn = a.batch
        d = ops.conv_desc(Bn, 224, 224, 3, 64, 7, 7, 4, 4)
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        x = torch.randn((Bn, 3, 224, 224), device=dev, generator=g)
        f = ops.pack_inconv_filter(torch.randn((49, 3, 64), device=dev, generator=g))
        thr = torch.randn((64,), device=dev, generator=g) * 12.0
        out = torch.zeros((Bn, d.OH * d.OW * 2), dtype=torch.int32, device=dev)
        res = torch.empty((Bn, d.OH, d.OW, 64), dtype=torch.int16, device=dev)
        spec = ops.inconv_specialize(d, f, thr) if a.specialized else None
        ms = _time(lambda: ops.inconv_layer(d, x, f, thr, out=out, res_out_buf=res, specialized=spec), a.iters)
        work = 2.0 * Bn * d.OH * d.OW * 64 * 49 * 3
        desc = "fp32 first layer %dx3x224x224 -> 56x56x64 (7x7/4), int16 residual; ops = fp32 add/sub" % Bn
    elif a.case == "conv":
        Bn, H, C, O, st = a.batch, a.hw, a.cin, a.cout, a.stride
        d = ops.conv_desc(Bn, H, H, C, O, 3, 3, st, st)
        x, f = _words((Bn, H, H, C // 32), 2, dev), _words((O, 9, C // 32), 3, dev)
        g = torch.Generator(device=dev)
        g.manual_seed(4)
        thr = torch.randn((O,), device=dev, generator=g) * (9 * C) ** 0.5
        prep = ops.conv_prepare(d, f)
        out = torch.zeros((Bn, d.OH * d.OW * (O // 32)), dtype=torch.int32, device=dev)
        rin = rout = None
        if a.residual:
            rin = torch.randint(-500, 500, (Bn, d.OH, d.OW, O), dtype=torch.int16, device=dev, generator=g)
            rout = torch.empty((Bn, d.OH, d.OW, O), dtype=torch.int16, device=dev)
        ch = bool(a.chunked and a.residual)
        ms = _time(lambda: ops.conv_layer(d, x, prep, thr, res_in=rin, residual_channels=O if rin is not None else 0,
                                          out=out, res_out_buf=rout, res_in_chunked=ch, res_out_chunked=ch,
                                          res_out_proven=ch), a.iters)
        work = 2.0 * Bn * d.OH * d.OW * O * 9 * C
        desc = "bit conv %dx%dx%dx%d -> %d, 3x3 stride %d%s%s" % (Bn, H, H, C, O, st, " + int16 residual in/out" if a.residual else "",
                                                                " (chunk-major)" if ch else "")
    else:
        Bn, H, C, O = a.batch, 56, 128, 128
        d = ops.conv_desc(Bn, H, H, C, O, 3, 3)
        x, f = _words((Bn, H, H, C // 32), 2, dev), _words((O, 9, C // 32), 3, dev)
        g = torch.Generator(device=dev)
        g.manual_seed(4)
        thr = torch.randn((O,), device=dev, generator=g) * 8.0
        prep = ops.conv_prepare(d, f)
        out = torch.zeros((Bn, H * H * (O // 32)), dtype=torch.int32, device=dev)
        res = torch.empty((Bn, H, H, O), dtype=torch.int32, device=dev) if a.residual else None
        ms = _time(lambda: ops.conv_layer(d, x, prep, thr, out=out, res_out_buf=res), a.iters)
        work = 2.0 * Bn * H * H * O * 9 * C
        desc = "bit conv %dx56x56x128 -> 128, 3x3%s" % (Bn, " + int32 residual" if a.residual else "")
    tops = work / (ms * 1e-3) / 1e12
    peak = None if a.no_peak else ops.mma_peak(0, 32, 4000)
    print(json.dumps({"case": a.case, "workload": desc, "ms": ms, "tops": tops,
                      "b1_mma_peak_tops": peak, "frac_of_b1_peak": tops / peak if peak else None}))


if __name__ == "__main__":
    main()
