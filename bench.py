#!/usr/bin/env python
"""Benchmark of the B200 LUT6 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

Headline workload (BASELINE config 1): BinaryLut6 bit-packed inference forward, 16384 -> 16384 nodes,
2^20 frames per GPU, Bernoulli(0.5) inputs, random 6-input wiring, random 64-bit tables.  One step is
one forward over the whole batch.  `value` = node-frames/s with inputs resident in HBM; `e2e` = the same
through the public operator with HOST buffers (pinned H2D of x, D2H of y inside the timed region).
Frames shard across ranks with no collective (weak scaling: every rank holds 2^20 frames).

The `fp32` object reports the other half of the metric -- StochasticLut6 / DifferentiableLut6 forward and
backward on one 8192 -> 8192 layer slice of config 4 -- with the roofline that bounds each (FP32 pipe or HBM) and, at one
GPU, the reference's CPU code on the same operators.  Further objects: `train` / `train_binary` (the frame-sharded config-4
training step, in probability mode and in the reference's default binary mode), `cnn` (the config-3 LUT-CNN step) and
`operators` (every other operator of the path: bit-input variants, binary mode, StochasticBatchNormalization, Adam, the
convolution lowering), each with its time and roofline fraction.

`--impl reference` times the reference's own CPU implementation (oracle/_ref, the unmodified BinaryBrain
headers, AVX2 + OpenMP on all host cores) on a bounded frame sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_IN = N_OUT = 16384
FRAMES = 1 << 20
TRAIN_NODES = 65536                  # config 4 layer width
TRAIN_FRAMES = 4096                  # frames per GPU and step in the training section (6 saved activations of 1 GiB each)
CPU_SAMPLE_FRAMES = 1 << 18          # bounded sample for the CPU legs (the full batch needs 8 GiB of host copies)
FALLBACK_HBM_GBS = 6650.0            # the pool's earlier measurement, used only when MEASURED_PEAKS.json is absent
# dram__bytes_read.sum + dram__bytes_write.sum of one k_binary_lut6_pipe launch: ncu on a 131072-frame launch gave
# 449.7 MB + 244.6 MB (profiles/binary_lut6_16384x16384_131072frames.md); traffic grows with frames, so x8 for 2^20 frames.
NCU_TRAFFIC_BYTES_PER_FRAME = (449.7e6 + 244.6e6) / 131072


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured", d
    return FALLBACK_HBM_GBS, "fallback", {}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 8 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 8 for i in range(4) if r[4 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def make_inputs(torch, device, frames, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    words = frames // 32
    x = torch.randint(-2**31, 2**31 - 1, (N_IN, words), dtype=torch.int32, device=device, generator=g)       # Bernoulli(0.5) bits
    key = torch.rand((N_OUT, N_IN), device=device, generator=g) if N_IN <= 4096 else None
    if key is not None:
        idx = key.topk(6, dim=1).indices.to(torch.int32).contiguous()
    else:   # 6 distinct inputs per node: draw, then re-draw the few rows with a repeat
        idx = torch.randint(0, N_IN, (N_OUT, 6), device=device, generator=g)
        for _ in range(8):
            s = idx.sort(dim=1).values
            bad = (s[:, 1:] == s[:, :-1]).any(dim=1)
            if not bool(bad.any()):
                break
            idx[bad] = torch.randint(0, N_IN, (int(bad.sum()), 6), device=device, generator=g)
        idx = idx.to(torch.int32).contiguous()
    table = torch.randint(-2**31, 2**31 - 1, (N_OUT, 2), dtype=torch.int32, device=device, generator=g)
    return x, idx, table


def cpu_reference_leg(steps, warmup, frames=CPU_SAMPLE_FRAMES):
    """BinaryLutN<6,Bit>::Forward of the unmodified reference headers (AVX2 + OpenMP), or the C port when _ref is absent."""
    import numpy as np
    from oracle import port, ref
    rng = np.random.default_rng(1)
    words = frames // 32
    x = rng.integers(0, 2**32, (N_IN, words), dtype=np.uint64).astype(np.uint32)
    idx = rng.integers(0, N_IN, (N_OUT, 6)).astype(np.int32)
    table = rng.integers(-2**31, 2**31, (N_OUT, 2)).astype(np.int32)
    use_ref = ref.available()
    times = []
    for i in range(warmup + steps):
        if use_ref:
            t = ref.binary_lut6(x, idx, table, frames)["t_fwd"]
        else:
            t0 = time.perf_counter()
            port.binary_lut6_forward(x, idx, table, frames)
            t = time.perf_counter() - t0
        if i >= warmup:
            times.append(t)
    cores = ref.num_threads() if use_ref else (os.cpu_count() or 1)
    per_step = sum(times) / len(times)
    return {"value": N_OUT * frames / per_step, "unit": "node-frames/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"BinaryLut6 {N_IN}->{N_OUT} nodes, {frames} of {FRAMES} frames per step, mean of {len(times)} steps, "
                      f"{'bb::BinaryLutN<6,Bit>::Forward AVX2+OpenMP' if use_ref else 'C port, OpenMP'}"}, per_step


def fp32_cpu_reference(nodes=8192):
    """The reference's own CPU code (oracle/_ref: AVX2 + OpenMP StochasticLutN, scalar DifferentiableLutN whose backward is serial) on
    the fp32 operators, same node count, at a reduced frame count (stated in the result; never extrapolated)."""
    import numpy as np
    import oracle
    ref = oracle.ref
    if not ref.available():
        return None
    rng = np.random.default_rng(7)
    idx = np.stack([rng.permutation(nodes)[:6] for _ in range(nodes)]).astype(np.int32)
    W = np.clip(rng.normal(0.5, 0.01, (nodes, 64)), 0, 1).astype(np.float32)
    out = {"cores": ref.num_threads(), "kind": "reference", "unit": "node-frames/s"}
    F = 1024
    x, dy = rng.random((nodes, F), dtype=np.float32), rng.random((nodes, F), dtype=np.float32)
    r = ref.stochastic_lut6(x, idx, W, dy=dy)                        # warm-up (first-touch of the buffers, OpenMP team start)
    r = ref.stochastic_lut6(x, idx, W, dy=dy)
    out["sl6_forward"] = {"value": nodes * F / r["t_fwd"], "frames": F}
    out["sl6_backward"] = {"value": nodes * F / r["t_bwd"], "frames": F}
    F = 256                                                           # DifferentiableLutN's CPU backward is a serial loop over nodes
    x, dy = rng.random((nodes, F), dtype=np.float32), rng.random((nodes, F), dtype=np.float32)
    r = ref.differentiable_lut6(x, idx, W, binary=False, dy=dy)
    out["dl6_forward_training"] = {"value": nodes * F / r["t_fwd"], "frames": F}
    out["dl6_backward"] = {"value": nodes * F / r["t_bwd"], "frames": F}
    return out


def fp32_section(torch, ops, steps):
    """SL6 / DL6 forward and backward on one 8192 -> 8192 node layer, 16384 frames (x, y, dy, dx: 512 MiB each, > L2)."""
    I = O = 8192
    F = 16384
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(2)
    x = torch.rand((I, F), device=dev, generator=g)
    dy = torch.rand((O, F), device=dev, generator=g)
    idx = torch.randint(0, I, (O, 6), device=dev, generator=g).to(torch.int32)
    W = (torch.randn((O, 64), device=dev, generator=g) * 0.01 + 0.5).clamp_(0, 1)
    dW = torch.zeros((O, 64), device=dev)
    rm, rv = torch.zeros(O, device=dev), torch.ones(O, device=dev)
    y = torch.empty((O, F), device=dev)
    dx = torch.empty((I, F), device=dev)
    state = {}

    def dl_fwd():
        state["y"], state["mean"], state["rstd"] = ops.differentiable_lut6_forward_training(x, idx, W, rm, rv, F, y=y, binary=False)

    cases = {
        "sl6_forward":  (lambda: ops.stochastic_lut6_forward(x, idx, W, F, y=y), 126.0, 8.0),
        "sl6_backward": (lambda: ops.stochastic_lut6_backward(x, dy, idx, W, dW, I, F, dx=dx), 505.0, 12.0),
        "dl6_forward_training": (dl_fwd, 136.0, 16.0),
        "dl6_backward": (lambda: ops.differentiable_lut6_backward(x, dy, idx, W, dW, state["mean"], state["rstd"], I, F, dx=dx, binary=False),
                         525.0 + 126.0, 24.0),
    }
    props = torch.cuda.get_device_properties(0)
    hbm, which, _ = measured_peaks()
    out = {"layer": f"{I}->{O} nodes, {F} frames", "fp32_peak_note": "SMs*128 lanes*2*sm_clock at the max SM clock"}
    fp32_peak = props.multi_processor_count * 128 * 2 * 1.965e9
    for name, (fn, flops, bytes_) in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / 1e3 / steps
        nf = O * F / sec
        t_fp, t_hbm = flops / fp32_peak, bytes_ / (hbm * 1e9)
        out[name] = {"node_frames_per_s": nf, "ms": sec * 1e3, "bound": "fp32" if t_fp > t_hbm else "hbm",
                     "frac_of_roofline": nf * max(t_fp, t_hbm), "fp32_frac": nf * t_fp, "hbm_frac": nf * t_hbm,
                     "algorithmic_flops_per_nf": flops, "algorithmic_bytes_per_nf": bytes_}
    out["hbm_peak"] = f"{hbm} GB/s of {which}"
    return out


def train_section(torch, ops, dist, world, rank, steps, binary=False):
    """Config-4 style training step, frame-sharded: 6 stacked DifferentiableLut6 layers of TRAIN_NODES nodes (fp32, batch norm on),
    TRAIN_FRAMES frames per GPU (global batch = that x world), MSE loss on the last layer, backward with the per-layer dW all-reduce
    overlapped with the next layer's backward, Adam.  Reports forward+backward node-frames/s over all ranks."""
    from binarybrain_b200.dist import ShardedDifferentiableLut6
    nodes, frames, layers_n = TRAIN_NODES, TRAIN_FRAMES, 6
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(3)          # same seed on every rank: replicated wiring and tables
    layers = []
    for _ in range(layers_n):
        idx = torch.randint(0, nodes, (nodes, 6), device=dev, generator=g).to(torch.int32)
        W = (torch.randn((nodes, 64), device=dev, generator=g) * 0.01 + 0.5).clamp_(0, 1)
        layers.append(ShardedDifferentiableLut6(idx, W, nodes, binary=binary))
    opt = ops.Adam([l.W for l in layers], [l.dW for l in layers])
    gd = torch.Generator(device=dev).manual_seed(100 + rank)  # each rank draws its own frame shard
    x0 = torch.rand((nodes, frames), device=dev, generator=gd)
    target = torch.rand((nodes, frames), device=dev, generator=gd)
    total = frames * world
    acts = [torch.empty((nodes, frames), device=dev) for _ in range(layers_n)]
    grads = [torch.empty((nodes, frames), device=dev) for _ in range(2)]
    loss_buf = torch.zeros(1024, dtype=torch.float64, device=dev)

    def step():
        h = x0
        for l, a in zip(layers, acts):
            ops.clamp_(l.W)
            h = l.forward(h, frames, total, y=a)
        dy, _ = ops.mean_squared_error(h, target, frames, batch_size=total, loss_buf=loss_buf, dy=grads[0])   # mean over the GLOBAL batch
        for k, l in enumerate(reversed(layers)):
            dy = l.backward(dy, dx=grads[(k + 1) % 2])
        for l in layers:
            l.wait_grad()
        opt.update()

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    sec = ms / 1e3 / steps
    return {"workload": f"config 4 (frame-sharded training): {layers_n} x DifferentiableLut6 {nodes}->{nodes}, {frames} frames per GPU "
                        f"(global batch {total}), fp32{', binary mode' if binary else ''}, batch norm, MSE, Adam; dW all-reduce overlapped with backward",
            "node_frames_per_s": layers_n * nodes * total / sec, "ms_per_step": sec * 1e3, "steps": steps, "n_gpus": world,
            "allreduce_bytes_per_step": layers_n * (nodes * 64 * 4 + 2 * nodes * 2 * 8) if world > 1 else 0}


def build_config3_network(dev, seed=5, ops=None):
    """BASELINE config 3, the LUT-CNN, from the host-side classes: two conv blocks (each two bb::Convolution2d of per-pixel
    DifferentiableLut6 layers with 3x3 'same' lowering, then 2x2 MaxPooling) and a dense head 4096 -> 1024 -> 420 -> 70 -> 10.
    Random 6-distinct wiring, tables N(0.5, 0.01), fp32, batch norm on."""
    import torch
    from binarybrain_b200.conv import Convolution2d, MaxPooling, Sequential
    from binarybrain_b200.dist import ShardedDifferentiableLut6
    g = torch.Generator(device=dev).manual_seed(seed)

    def lut(n_in, n_out):
        idx = torch.rand((n_out, n_in), device=dev, generator=g).argsort(dim=1)[:, :6].to(torch.int32).contiguous()
        W = (torch.randn((n_out, 64), device=dev, generator=g) * 0.01 + 0.5).clamp_(0, 1)
        return ShardedDifferentiableLut6(idx, W, n_in, ops=ops, binary=False, sharded=False)       # runs on one rank only: no collectives

    def conv(c, hw, widths):
        return Convolution2d([lut(a, b) for a, b in zip(widths[:-1], widths[1:])], c, hw, hw, 3, 3, padding="same", ops=ops)

    return Sequential([
        conv(3, 32, [27, 216, 36, 32]), conv(32, 32, [288, 216, 36, 32]), MaxPooling(32, 32, 32, 2, 2, ops=ops),
        conv(32, 16, [288, 384, 64]), conv(64, 16, [576, 384, 64]), MaxPooling(64, 16, 16, 2, 2, ops=ops),
        lut(4096, 1024), lut(1024, 420), lut(420, 70), lut(70, 10)])


def cnn_section(torch, ops, steps):
    """Config 3: LUT-CNN forward + backward on 256 synthetic 3x32x32 images (one GPU).  Node-frames count the LUT evaluations of
    one forward pass (per-pixel layers run on 256 * oh * ow frames)."""
    B = 256
    net = build_config3_network(torch.device("cuda"))
    x = torch.rand((3 * 32 * 32, B), device="cuda")
    dy = torch.rand((10, ops.fp32_stride(B)), device="cuda")

    def step():
        for l in net.lut_layers():
            ops.clamp_(l.W)
        net.forward(x, B)
        net.backward(dy)

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / steps
    nf = B * (1024 * (216 + 36 + 32) * 2 + 256 * (384 + 64) * 2 + (1024 + 420 + 70 + 10))
    return {"workload": "config 3 (LUT-CNN): 3x32x32 images, batch 256, 2 conv blocks of per-pixel DifferentiableLut6 trees with 3x3 Im2Col / "
                        "Col2Im and 2x2 MaxPooling, dense head 4096->1024->420->70->10, fp32, batch norm; forward + backward",
            "node_frames_per_s": nf / sec, "ms_per_step": sec * 1e3, "steps": steps, "n_gpus": 1}


def operators_section(torch, ops, steps):
    """Every other operator of the path on the same 8192 -> 8192 x 16384-frame layer (bit inputs: same node counts, 16384 frames), each with
    its algorithmic bytes / flops per node-frame and the fraction of max(HBM, FP32) roofline time, plus the lowering operators at a config-3
    block shape and Adam.  One launch sequence per operator call, timed with CUDA events over `steps` calls after 3 warm-ups."""
    I = O = 8192
    F = 16384
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(4)
    idx = torch.rand((O, I), device=dev, generator=g).argsort(dim=1)[:, :6].to(torch.int32).contiguous()
    W = (torch.randn((O, 64), device=dev, generator=g) * 0.01 + 0.5).clamp_(0, 1)
    dW = torch.zeros((O, 64), device=dev)
    xb = torch.randint(-2**31, 2**31 - 1, (I, ops.bit_stride(F)), device=dev, generator=g, dtype=torch.int32)
    xf = torch.rand((I, F), device=dev, generator=g)
    dy = torch.rand((O, F), device=dev, generator=g)
    rm, rv = torch.zeros(O, device=dev), torch.ones(O, device=dev)
    yf = torch.empty((O, F), device=dev)
    ybit = torch.zeros((O, ops.bit_stride(F)), dtype=torch.int32, device=dev)
    dx = torch.empty((I, F), device=dev)
    st = {}

    def dl_bit_fwd():
        _, st["mean"], st["rstd"] = ops.differentiable_lut6_forward_training(xb, idx, W, rm, rv, F, y=ybit)

    def dl_binary_fwd():
        _, st["bmean"], st["brstd"] = ops.differentiable_lut6_forward_training(xf, idx, W, rm, rv, F, y=yf, binary=True)

    def sbn_fwd():
        st["sy"], st["smean"], st["srstd"] = ops.stochastic_bn_forward_training(xf, rm, rv, F)

    adam = ops.Adam([W], [dW])
    # lowering at the first conv block of config 3: 32 channels, 32x32, batch 256
    c, hw, B = 32, 32, 256
    img = torch.rand((c * hw * hw, B), device=dev, generator=g)
    cols = ops.im2col_forward(img, B, c, hw, hw, 3, 3, padding="same")
    colsb_in = torch.randint(-2**31, 2**31 - 1, (c * hw * hw, ops.bit_stride(B)), device=dev, generator=g, dtype=torch.int32)
    z = torch.rand((c, B * hw * hw), device=dev, generator=g)
    pooled, am = ops.maxpool_forward(img, B, c, hw, hw, 2, 2)
    gp = torch.rand_like(pooled)
    nf = float(O) * F
    px = float(c) * hw * hw * B                       # image elements
    cases = {   # name: (callable, units per call, algorithmic bytes per unit, algorithmic flops per unit)
        "sl6_forward_bit_fp32": (lambda: ops.stochastic_lut6_forward(xb, idx, W, F, y=yf), nf, 4.125, 0.0),       # per-pattern value lookup
        # bit in, bit out: evaluated as a BinaryLut6 forward with a per-node truth table (no per-frame fp32 tree), so the bound is HBM
        "sl6_forward_bit_bit": (lambda: ops.stochastic_lut6_forward(xb, idx, W, F, y=ybit, bit_output=True), nf, 0.25, 0.0),
        "sl6_backward_bit": (lambda: ops.stochastic_lut6_backward(xb, dy, idx, W, dW, I, F, dx=dx), nf, 8.125, 505.0),
        "dl6_forward_training_bit": (dl_bit_fwd, nf, 0.375, 0.0),       # x read twice (pattern histogram, then the table forward)
        "dl6_forward_inference_bit": (lambda: ops.differentiable_lut6_forward_inference(xb, idx, W, rm, rv, F, y=ybit), nf, 0.25, 0.0),
        "dl6_forward_inference_fp32": (lambda: ops.differentiable_lut6_forward_inference(xf, idx, W, rm, rv, F, y=yf, binary=False), nf, 8.0, 136.0),
        "dl6_backward_bit": (lambda: ops.differentiable_lut6_backward(xb, dy, idx, W, dW, st["mean"], st["rstd"], I, F, dx=dx), nf, 12.125, 651.0),
        # binary mode on fp32 frames (the reference's default mode): forward by the fp32 tree, backward through the per-pattern tables
        "dl6_forward_training_fp32_binary": (dl_binary_fwd, nf, 13.0, 0.0),     # x read, pattern byte written and read, y written
        "sl6_forward_fp32_binary": (lambda: ops.stochastic_lut6_forward(xf, idx, W, F, y=yf, binary=True), nf, 8.0, 0.0),
        "dl6_backward_fp32_binary": (lambda: ops.differentiable_lut6_backward(xf, dy, idx, W, dW, st["bmean"], st["brstd"], I, F, dx=dx, binary=True),
                                     nf, 24.0, 651.0),
        "sl6_backward_fp32_binary": (lambda: ops.stochastic_lut6_backward(xf, dy, idx, W, dW, I, F, dx=dx, binary=True), nf, 12.0, 505.0),
        "sbn_forward_training": (sbn_fwd, nf, 12.0, 8.0),
        "sbn_backward": (lambda: ops.stochastic_bn_backward(xf, dy, st["smean"], st["srstd"], F), nf, 20.0, 12.0),
        "adam_update": (lambda: adam.update(), float(W.numel()), 28.0, 12.0),
        "im2col_forward_fp32": (lambda: ops.im2col_forward(img, B, c, hw, hw, 3, 3, padding="same"), px * 9, 4.0 + 4.0 / 9, 0.0),
        "im2col_forward_bit": (lambda: ops.im2col_forward(colsb_in, B, c, hw, hw, 3, 3, padding="same"), px * 9, (1 + 1.0 / 9) / 8, 0.0),
        "im2col_backward_fp32": (lambda: ops.im2col_backward(cols, B, c, hw, hw, 3, 3, padding="same"), px * 9, 4.0 + 4.0 / 9, 1.0),
        "col2im_forward_fp32": (lambda: ops.col2im_forward(z, c, hw, hw, B), px, 8.0, 0.0),
        "col2im_backward_fp32": (lambda: ops.col2im_backward(img, c, hw, hw, B), px, 8.0, 0.0),
        "maxpool_forward_fp32": (lambda: ops.maxpool_forward(img, B, c, hw, hw, 2, 2), px, 4.0 + 2.0, 1.0),
        "maxpool_backward_fp32": (lambda: ops.maxpool_backward(am, gp, B, c, hw, hw, 2, 2), px, 4.0 + 2.0, 0.0),
    }
    props = torch.cuda.get_device_properties(0)
    hbm, which, _ = measured_peaks()
    fp32_peak = props.multi_processor_count * 128 * 2 * 1.965e9
    out = {"layer": f"{I}->{O} nodes, {F} frames (bit inputs: same frames, 32 per word); lowering: {c} channels {hw}x{hw}, batch {B}, 3x3 same / 2x2 pool",
           "unit": "node-frames (LUT, SBN), table entries (Adam), output elements (lowering: Im2Col counts the 9x expanded buffer)",
           "hbm_peak": f"{hbm} GB/s of {which}"}
    for name, (fn, units, bytes_, flops) in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / 1e3 / steps
        t_fp, t_hbm = flops / fp32_peak, bytes_ / (hbm * 1e9)
        out[name] = {"units_per_s": units / sec, "ms": sec * 1e3, "bound": "fp32" if t_fp > t_hbm else "hbm",
                     "frac_of_roofline": units / sec * max(t_fp, t_hbm), "algorithmic_bytes_per_unit": round(bytes_, 4),
                     "algorithmic_flops_per_unit": flops}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--frames", type=int, default=FRAMES, help="frames per GPU (default: the full 2^20 of config 1)")
    ap.add_argument("--no-extras", action="store_true", help="skip the fp32 section, the e2e leg and the CPU baseline")
    ap.add_argument("--fp32-only", action="store_true", help="run and print only the fp32 section (profiling aid)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": f"config 1: BinaryLut6 forward {N_IN}->{N_OUT} nodes, 2^20 frames per GPU bit-packed (x, y 2 GiB each)",
              "frames_per_gpu": args.frames, "sharding": "frames, no collective", "l2": "inputs (2 GiB) exceed L2 (126 MB); no flush"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        base, per_step = cpu_reference_leg(args.steps, args.warmup)
        line = {"impl": "reference", "metric": "BinaryLut6 forward node-frames/s", "value": base["value"], "unit": "node-frames/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "u32 bit-packed", "data": "synthetic", "config": config,
                "cpu_baseline": base, "e2e": {"value": base["value"], "unit": "node-frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    import torch
    from binarybrain_b200 import abi, ops          # raises if the CUDA library is missing: there is no CPU fallback
    abi.lib()
    assert torch.cuda.is_available(), "bench.py --impl ours needs a CUDA device"
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"          # keep NCCL's version banner off stdout: stdout carries exactly one JSON line
        import torch.distributed as dist
        import datetime
        # a collective that is not matched on every rank fails after three minutes instead of holding the GPUs for NCCL's default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=180))
    if args.fp32_only:
        print(json.dumps({"fp32": fp32_section(torch, ops, max(1, args.steps))}))
        return 0
    W = max(args.warmup, 3)
    frames = args.frames
    x, idx, table = make_inputs(torch, "cuda", frames, seed=1 + rank)
    y = torch.empty_like(x)

    def step():
        ops.binary_lut6_forward(x, idx, table, frames, y=y)

    for _ in range(W):
        step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    # keep the sampler alive long enough to have seen the loaded clocks at least a few times
    t_keep = time.time()
    while len(sampler.rows) < 3 and time.time() - t_keep < 1.0:
        step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    if dist:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    sec_per_step = ms / 1e3 / args.steps
    value = world * N_OUT * frames / sec_per_step

    hbm, which, _ = measured_peaks()
    algo_bytes = frames * (N_IN + N_OUT) / 8 + 32 * N_OUT            # x + y bit rows, wiring + table per node
    achieved = algo_bytes / sec_per_step / 1e9
    line = {"metric": "BinaryLut6 forward node-frames/s", "value": value, "unit": "node-frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": W, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32 bit-packed", "data": "synthetic", "config": config, "clocks": clocks, "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                         "traffic": NCU_TRAFFIC_BYTES_PER_FRAME * frames, "peak_source": f"of {which}", "kernel": "k_binary_lut6",
                         "algorithmic_bytes_per_launch": algo_bytes}}

    if not args.no_extras:
        # end to end through the operator with host buffers: H2D of x, kernel, D2H of y, every step
        hx = torch.empty(x.shape, dtype=torch.int32).pin_memory()
        hy = torch.empty(y.shape, dtype=torch.int32).pin_memory()
        hx.copy_(x)
        torch.cuda.synchronize()
        k = max(2, min(args.steps, 5))
        hidx, htab = idx.cpu(), table.cpu()
        for i in range(1 + k):
            if i == 1:
                torch.cuda.synchronize()
                if dist:
                    dist.barrier()
                t0 = time.perf_counter()
            # one call through the C ABI with HOST buffers: upload of x, kernel and download of y happen inside (chunk-pipelined)
            ops.binary_lut6_forward_host(hx, hidx, htab, frames, y=hy)
        if dist:
            dist.barrier()
        dt = time.perf_counter() - t0
        if dist:
            t = torch.tensor([dt], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        line["e2e"] = {"value": world * N_OUT * frames / (dt / k), "unit": "node-frames/s", "h2d_bytes_per_step": hx.numel() * 4,
                       "d2h_bytes_per_step": hy.numel() * 4, "steps": k}
        del hx, hy, x, y
        torch.cuda.empty_cache()
        line["train"] = train_section(torch, ops, dist, world, rank, max(2, min(args.steps, 5)))
        torch.cuda.empty_cache()
        # the same step in the reference's default binary mode (inputs 0.5 +- bias by x > 0.5, outputs binarised)
        line["train_binary"] = train_section(torch, ops, dist, world, rank, max(2, min(args.steps, 5)), binary=True)
        if rank == 0:
            torch.cuda.empty_cache()
            line["fp32"] = fp32_section(torch, ops, max(3, min(args.steps, 10)))
            torch.cuda.empty_cache()
            line["cnn"] = cnn_section(torch, ops, max(2, min(args.steps, 5)))
            torch.cuda.empty_cache()
            line["operators"] = operators_section(torch, ops, max(3, min(args.steps, 10)))
            if world == 1:
                line["cpu_baseline"], _ = cpu_reference_leg(3, 1)
                line["fp32"]["cpu_baseline"] = fp32_cpu_reference()
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
