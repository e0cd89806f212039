#!/usr/bin/env python
"""Benchmark of the binarised ResNet-18 forward pass (the reference driver's topology,
imagenet_resnet.cu:223-325) at batch 1024 per GPU on synthetic 224x224 images.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

One JSON line on stdout (rank 0).  `value` is images/s with the inputs already in HBM;
`e2e` is the same pass driven from pinned host buffers (H2D of the fp32 images and D2H of the
logits inside the timed region).  `--impl reference` times the CPU oracle (the reference has
no CPU path of its own; the oracle is its restatement) on a bounded sample of the same
workload with all host threads.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "resnet18_bnn_inference_throughput"
UNIT = "images/s"
PUBLISHED_IMAGES_PER_S = 5600.0      # reference README.md:15, Turing GPU


def conv_ops(spec_layers):
    """Algorithmic bit-ops of the binary conv layers per image: 2*M*N*K, all taps counted."""
    total = 0
    for l in spec_layers:
        if l["type"] == "conv":
            total += 2 * (l["OH"] * l["pool"]) * (l["OW"] * l["pool"]) * l["O"] * l["R"] * l["S"] * l["C"]
    return total


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Number of samples read so far (to delimit a window of the run)."""
        return len(self.lines)

    def stop(self, first=0, last=None):
        """Summary of the samples [first, last) (marks); the whole record if that window holds
        fewer than three samples (a timed region of a few tens of milliseconds)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = self.lines[first:last]
        whole = len(window) < 3
        if whole:
            window = self.lines
        for ln in window:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "window": "warm-up, timed region and per-layer pass" if whole else "timed region and per-layer pass"}


def run_reference(args, rank, world):
    """CPU arm: the oracle on the host cores, bounded sample, all threads."""
    if rank != 0:
        return
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import networks as onet
    import oracle as orc
    from tcbnn_b200 import models
    L = orc.lib(native=True)
    orc.use_all_cores(L)
    threads = orc.num_threads(L)
    sample = max(1, min(args.batch, args.cpu_images))
    spec = models.resnet18_spec(sample)
    w = models.synthetic_weights(spec, 1234)
    x = models.synthetic_input(spec, 4321)
    for _ in range(min(args.warmup, 1)):
        onet.run(spec, w, x, L=L)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        onet.run(spec, w, x, L=L)
    dt = (time.perf_counter() - t0) / args.steps
    v = sample / dt
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "b1/int32",
        "data": "synthetic",
        "config": {"workload": "C5 ResNet-18 BNN 224x224 (reference driver topology), batch 1024 per GPU",
                   "note": "CPU oracle (reference has no CPU path); each step = %d images" % sample},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d images per step, full network incl. weight packing" % sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1024, help="images per GPU")
    ap.add_argument("--impl", default="tcbnn_b200", choices=["tcbnn_b200", "reference"])
    ap.add_argument("--cpu-images", type=int, default=64, help="images in the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    from tcbnn_b200 import dist as tdist
    from tcbnn_b200 import models, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # stdout carries the one JSON line and nothing else: from here on file descriptor 1 points at
    # stderr (libraries such as NCCL print their version banner to it) and the line goes to the
    # saved descriptor at the end
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    tdist.init("nccl", dev)

    B = args.batch
    spec = models.resnet18_spec(B)
    shapes = models.layer_shapes(spec)
    weights = models.synthetic_weights(spec, 1234)               # same weights on every rank
    x_host = torch.from_numpy(models.synthetic_input(spec, tdist.shard_seed(4321, rank))).pin_memory()
    net = models.Network(spec, weights, x_host, input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND)
    del weights
    logits_host = torch.empty((B, 1000), dtype=torch.float32).pin_memory()
    gathered = torch.empty((world * B, 1000), dtype=torch.float32, device=dev) if world > 1 else None

    def step(events=None):
        if events is None:
            out = net.forward_graph()
        else:
            for l in net.layers:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                l.forward()
                e1.record()
                events.append((l, e0, e1))
            out = net.layers[-1].get_output_gpu()
        if world > 1:
            tdist.gather_logits(out, gathered)
        return out

    def sync():
        tdist.barrier()
        torch.cuda.synchronize()

    # clocks and throttle reasons are sampled every 20 ms from before the warm-up on (nvidia-smi
    # needs a moment to start), and the samples of the timed window are picked out by marks
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    sync()

    # ---- device-resident throughput ------------------------------------------------------
    mark0 = sampler.mark()
    # The timed region replays the forward pass from a CUDA graph (the same launches as one
    # submission).  A second pass of the same K steps, layer by layer with a CUDA event pair
    # around each, gives the per-layer times the roofline figures use.
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    sync()
    ms = t0.elapsed_time(t1)
    events = []
    for _ in range(args.steps):
        step(events)
    sync()
    clocks = sampler.stop(mark0, sampler.mark()) if rank == 0 else None

    # ---- end to end from host buffers ----------------------------------------------------
    # Every step copies its images from pinned host memory and reads its logits back; the copy
    # of step i+1 runs on a second stream while step i computes (models.HostFeeder).
    # `e2e` feeds the images as bytes (uint8 + per-channel value table, tcbnn_inconv_layer_u8:
    # the reader's normalisation happens in the first layer, results identical);
    # `e2e_fp32_images` feeds the reference's fp32 images.
    def timed_feed(network, batch_host):
        feeder = models.HostFeeder(network)

        def on_result(out):
            if world > 1:
                tdist.gather_logits(out, gathered)

        feeder.run([batch_host] * 2, on_result, logits_host)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        feeder.run([batch_host] * args.steps, on_result, logits_host)   # ends by waiting for the last read
        e1.record()
        sync()
        return e0.elapsed_time(e1)

    ms_e2e_f32 = timed_feed(net, x_host)
    u8_np, lut = models.synthetic_input_u8(spec, tdist.shard_seed(4321, rank))
    x8_host = torch.from_numpy(u8_np).pin_memory()
    net8 = models.Network(spec, models.synthetic_weights(spec, 1234), x8_host,
                          input_abs_bound=models.SYNTHETIC_IMAGE_ABS_BOUND, input_lut=lut)
    ms_e2e = timed_feed(net8, x8_host)

    ms, ms_e2e, ms_e2e_f32 = tdist.max_over_ranks([ms, ms_e2e, ms_e2e_f32], dev)

    if rank == 0:
        conv_ms, launches = 0.0, 0
        per_layer = {}
        for l, a, b in events:
            d = a.elapsed_time(b)
            per_layer[l.name] = per_layer.get(l.name, 0.0) + d / args.steps
            if type(l).__name__ == "Conv128LayerParam":
                conv_ms += d
            if hasattr(l, "kernel_launches"):
                launches += l.kernel_launches()
            else:
                launches += 2 if getattr(l, "workspace", None) is not None else 1
        n_conv = sum(1 for l in shapes if l["type"] == "conv")
        ops_per_step = conv_ops(shapes) * B
        achieved = ops_per_step * args.steps / (conv_ms * 1e-3) / 1e12
        peak_b1 = ops.mma_peak(0, 32, 4000)
        peak = ops.mma_peak(3, 1, 20000)
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "conv_traffic.json")
        if os.path.exists(tpath):
            traffic = json.load(open(tpath)).get("dram_bytes_per_launch_avg")
        out = {
            "metric": METRIC, "value": world * B * args.steps / (ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": world * B * args.steps / (ms * 1e-3) / PUBLISHED_IMAGES_PER_S,
            "dtype": "b1/int32", "data": "synthetic",
            "config": {"workload": "C5 ResNet-18 BNN 224x224 (reference driver topology), batch %d per GPU" % B,
                       "l2": "inputs (%.0f MB fp32 images per step) larger than L2" % (x_host.numel() * 4 / 1e6),
                       "parallelism": "batch-sharded x%d, NCCL all-gather of logits" % world,
                       "baseline_note": "vs_baseline divides by the 5.6 K images/s the reference README quotes for a Turing GPU"},
            "e2e": {"value": world * B * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": x8_host.numel(), "d2h_bytes_per_step": logits_host.numel() * 4,
                    "input": "uint8 NCHW images + [3][256] fp32 value table (normalisation fused into the first layer)"},
            "e2e_fp32_images": {"value": world * B * args.steps / (ms_e2e_f32 * 1e-3), "unit": UNIT,
                                "h2d_bytes_per_step": x_host.numel() * 4,
                                "d2h_bytes_per_step": logits_host.numel() * 4,
                                "input": "fp32 NCHW images, the reference's interface"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "kernel": "tcgen05 int8 implicit-GEMM conv kernels k_conv_umma_ws / _pre / _as (%d layers per step)" % n_conv,
                         "timing": "CUDA event pairs around each layer, a second pass of the same %d steps right after the timed (graph-replayed) one" % args.steps,
                         "peak_source": "tcgen05.mma kind::i8 128x256x32 issue rate measured in this run by tcbnn_mma_peak(3) (of measured)",
                         "b1_mma_peak": peak_b1, "frac_of_b1_mma_peak": achieved / peak_b1},
            "layer_ms": {k: round(v, 4) for k, v in per_layer.items()},
        }
        if not args.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline(args.cpu_images)
        os.write(json_fd, (json.dumps(out) + "\n").encode())
    tdist.finish()


def cpu_baseline(images):
    """The CPU oracle timed on this box's host cores on a bounded sample of the workload."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import networks as onet
    import oracle as orc
    from tcbnn_b200 import models
    L = orc.lib(native=True)
    orc.use_all_cores(L)
    spec = models.resnet18_spec(images)
    w = models.synthetic_weights(spec, 1234)
    x = models.synthetic_input(spec, 4321)
    t0 = time.perf_counter()
    onet.run(spec, w, x, L=L)
    dt = time.perf_counter() - t0
    return {"value": images / dt, "unit": UNIT, "cores": orc.num_threads(L), "kind": "port",
            "sample": "%d images, one pass of the full network (OpenMP oracle)" % images}


if __name__ == "__main__":
    main()
