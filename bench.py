#!/usr/bin/env python
"""Benchmark of the B200 LUT6 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras] [--only SECTION]

Headline workload: the frame-sharded training step on six stacked DifferentiableLut6 layers of 65536 nodes (fp32, batch norm
fused, MSE loss on the last layer, Adam), at a FIXED global batch of 32768 frames per step whatever the number of GPUs
(strong scaling; one GPU holds ten 8 GiB frame buffers).  Rank r owns the frames [r G/N, (r+1) G/N).  Per layer and step the ranks
exchange the batch-norm sums of the forward and of the backward pass (two blocking all-reduces of [65536, 2] fp64) and the
table gradients ([65536, 64] fp32, all-reduced asynchronously under the next layer's backward).  One step is forward +
backward + Adam over the whole global batch; `value` = layers x nodes x G / step time (node-frames/s, each counted once for
its forward and backward together) with the inputs resident in HBM; `e2e` = the same step with this rank's input and target
shards uploaded from pinned host memory every step (double-buffered on a copy stream) and the loss read back.
`roofline` is that of the kernel that dominates the step, the fused batch-norm + LUT backward (k_lut6_backward_pipe), timed
with CUDA events around every one of its launches inside the timed steps.

Sub-objects: `binary_lut6` (BinaryLut6 bit-packed inference forward, 16384 -> 16384 nodes, 2^20 frames per GPU, with its own
roofline, host-buffer e2e and CPU baseline), `fp32` (StochasticLut6 / DifferentiableLut6 forward and backward on one 65536 -> 65536
x 4096-frame layer, each against the roofline that bounds it), `train_binary` (the same six layers in the reference's binary
mode, 4096 frames per GPU), `train_cpp` (one GPU: the headline's six layers, forward + backward + Adam, through the C++ host
classes), `cnn` (the LUT-CNN step through the C++ host classes) and `operators` (every other operator of the path).

`--impl reference` times the reference's own CPU implementation (oracle/_ref, the unmodified BinaryBrain headers, OpenMP on all
host cores) on a bounded sample of the headline workload.
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

TRAIN_NODES = 65536                  # layer width of the training workload
TRAIN_LAYERS = 6
TRAIN_GLOBAL_BATCH = 32768           # frames per step over all GPUs (8 GiB per fp32 frame buffer on one GPU)
CPU_TRAIN_SAMPLE_FRAMES = 8          # the reference's DifferentiableLutN backward is a serial loop over nodes (~2e5 node-frames/s)
BL6_NODES = 16384
BL6_FRAMES = 1 << 20
FALLBACK_HBM_GBS = 6650.0            # the pool's earlier measurement, used only when MEASURED_PEAKS.json is absent
SM_CLOCK_HZ = 1.965e9                # clocks.max.sm of the B200s of this pool
# Algorithmic work per node-frame (one LUT evaluation) of the kernels the rooflines are quoted on, counted for the 63-interpolation
# tree: forward 126 flops; backward 126 (recomputed forward) + 63 x 5 (reverse pass) + 64 (table-gradient sums) = 505.
FLOPS_FWD, FLOPS_BWD = 126.0, 505.0
# what the centred-polynomial kernels issue instead: 63 FMA forward; backward 31 + 1 FMA forward halves, 41 packed FMA + 40 packed
# mul/add + 7 scalar operations in the reverse pass, 12 for input conditioning
FLOPS_FWD_EXECUTED, FLOPS_BWD_EXECUTED = 126.0 + 12.0, 379.0
# dram__bytes_read.sum + dram__bytes_write.sum of one k_binary_lut6_pipe launch: ncu on a 131072-frame launch; traffic grows with frames
NCU_BL6_TRAFFIC_BYTES_PER_FRAME = (449.7e6 + 244.6e6) / 131072
# the same for one k_lut6_backward_pipe<BN> launch on a 65536 -> 65536 x 4096-frame layer: 11.379 GB read + 5.201 GB written for 2.68e8
# node-frames; the tile width does not depend on the frame count, so the traffic grows in proportion to the frames of a launch
NCU_BWD_TRAFFIC_BYTES_PER_NF = (11.379342e9 + 5.201327e9) / (65536 * 4096)


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


def fp32_peak_flops(torch):
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count * 128 * 2 * SM_CLOCK_HZ


class TimedOps:
    """The operator module with CUDA events around every call of one operator (on the current stream, where it launches)."""

    def __init__(self, ops, torch, name):
        self._ops, self._torch, self._name, self.pairs, self.enabled = ops, torch, name, [], False

    def __getattr__(self, attr):
        fn = getattr(self._ops, attr)
        if attr != self._name:
            return fn

        def timed(*a, **k):
            if not self.enabled:
                return fn(*a, **k)
            e0, e1 = self._torch.cuda.Event(enable_timing=True), self._torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **k)
            e1.record()
            self.pairs.append((e0, e1))
            return r
        return timed

    def mean_ms(self):
        return sum(a.elapsed_time(b) for a, b in self.pairs) / max(1, len(self.pairs))


# ------------------------------------------------------------------------------------------------ the training step
class TrainingWorkload:
    """Six stacked DifferentiableLut6 layers, frame-sharded; replicated wiring / tables / Adam state, one frame shard per rank."""

    def __init__(self, torch, ops, world, rank, frames_per_gpu, total_frames, binary=False, timed=None):
        from binarybrain_b200.dist import ShardedDifferentiableLut6
        self.torch, self.ops, self.world, self.frames, self.total = torch, ops, world, frames_per_gpu, total_frames
        nodes, dev = TRAIN_NODES, "cuda"
        g = torch.Generator(device=dev).manual_seed(3)          # same seed on every rank: replicated wiring and tables
        self.layers = []
        for _ in range(TRAIN_LAYERS):
            idx = torch.randint(0, nodes, (nodes, 6), device=dev, generator=g).to(torch.int32)
            W = (torch.randn((nodes, 64), device=dev, generator=g) * 0.01 + 0.5).clamp_(0, 1)
            self.layers.append(ShardedDifferentiableLut6(idx, W, nodes, ops=timed if timed is not None else ops, binary=binary))
        self.opt = ops.Adam([l.W for l in self.layers], [l.dW for l in self.layers])
        gd = torch.Generator(device=dev).manual_seed(100 + rank)  # each rank draws its own frame shard
        self.x0 = torch.rand((nodes, frames_per_gpu), device=dev, generator=gd)
        self.target = torch.rand((nodes, frames_per_gpu), device=dev, generator=gd)
        self.acts = [torch.empty((nodes, frames_per_gpu), device=dev) for _ in range(TRAIN_LAYERS)]
        self.grads = [torch.empty((nodes, frames_per_gpu), device=dev) for _ in range(2)]
        self.loss_buf = torch.zeros(1024, dtype=torch.float64, device=dev)

    def step(self, x=None, target=None):
        ops = self.ops
        h = self.x0 if x is None else x
        for l, a in zip(self.layers, self.acts):
            ops.clamp_(l.W)
            h = l.forward(h, self.frames, self.total, y=a)
        dy, _ = ops.mean_squared_error(h, self.target if target is None else target, self.frames, batch_size=self.total,
                                       loss_buf=self.loss_buf, dy=self.grads[0])         # mean over the GLOBAL batch
        for k, l in enumerate(reversed(self.layers)):
            dy = l.backward(dy, dx=self.grads[(k + 1) % 2])
        for l in self.layers:
            l.wait_grad()
        self.opt.update()

    # our kernels per step: per layer clamp, table conversion, statistics forward, finalize, normalise; the loss; per layer the
    # backward statistics, finalize, the clear of dx, table conversion, the backward kernel, the table-gradient kernel; Adam
    LAUNCHES_PER_STEP = TRAIN_LAYERS * 5 + 1 + TRAIN_LAYERS * 6 + 1

    def allreduce_bytes(self):
        return TRAIN_LAYERS * (TRAIN_NODES * 64 * 4 + 2 * TRAIN_NODES * 2 * 8) if self.world > 1 else 0


def timed_steps(torch, dist, fn, steps, warmup, sampler=None):
    """`warmup` untimed calls, then exactly `steps` calls between barrier + synchronize, timed with CUDA events; max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    if sampler:
        sampler.start()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / 1e3 / steps


def bind_to_gpu_numa_node(torch, local_rank):
    """Keeps this rank's threads (and with them the first touch of its page-locked buffers) on the NUMA node its GPU hangs off, so that
    eight ranks' host-to-device copies do not all cross the socket interconnect.  Returns the node, or None when the platform does not
    say (no sysfs entry, node -1, or none of the node's cores in this process's affinity mask)."""
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read())
        if node < 0:
            return None
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (AttributeError, OSError, ValueError):
        return None


def train_e2e(torch, dist, wl, steps):
    """The training step fed from pinned host memory: every step uploads this rank's input and target shards (on a copy stream,
    into the spare one of two device buffers, while the previous step computes) and reads the loss back."""
    nbytes = wl.x0.numel() * 4
    hx = ht = None
    why = None
    try:
        with open("/proc/meminfo") as f:
            avail = next(int(l.split()[1]) * 1024 for l in f if l.startswith("MemAvailable"))
        if avail < 3 * 2 * nbytes:          # this rank's two buffers, with room to spare (the other ranks pin theirs at the same time)
            why = f"host memory: {avail >> 30} GiB available, {2 * nbytes >> 30} GiB of pinned buffers needed per rank"
        else:
            hx = torch.empty(wl.x0.shape, dtype=torch.float32, pin_memory=True)
            ht = torch.empty(wl.target.shape, dtype=torch.float32, pin_memory=True)
    except (RuntimeError, OSError, StopIteration) as e:
        why = f"pinned host buffers: {e}"
    # every rank takes the same branch: the timed loop below holds collectives, so one rank without its buffers means no rank runs it
    ok = torch.tensor([0 if why else 1], device="cuda", dtype=torch.int32)
    if dist:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        del hx, ht
        return {"value": None, "unavailable": why or "another rank could not pin its host buffers"}
    hx.copy_(wl.x0)
    ht.copy_(wl.target)
    bufs = [(wl.x0, wl.target), (torch.empty_like(wl.x0), torch.empty_like(wl.target))]
    copy_stream = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    ready = [torch.cuda.Event(), torch.cuda.Event()]          # upload into buffer b complete
    freed = [torch.cuda.Event(), torch.cuda.Event()]          # the step that read buffer b has finished
    for e in freed:
        e.record(main)

    def upload(b):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[b])
            bufs[b][0].copy_(hx, non_blocking=True)
            bufs[b][1].copy_(ht, non_blocking=True)
            ready[b].record(copy_stream)

    losses = []
    torch.cuda.synchronize()
    upload(0)
    t0 = None
    for i in range(1 + steps):                                 # the first step is the warm-up of the pipeline
        if i == 1:
            torch.cuda.synchronize()
            if dist:
                dist.barrier()
            t0 = time.perf_counter()
        b = i & 1
        if i < steps:
            upload(b ^ 1)                                      # next step's inputs travel while this step computes
        main.wait_event(ready[b])
        wl.step(bufs[b][0], bufs[b][1])
        freed[b].record(main)
        losses.append(float(wl.loss_buf.sum().item()) / wl.total)          # device -> host read of the step's result
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    dt = time.perf_counter() - t0
    if dist:
        t = torch.tensor([dt], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    del hx, ht, bufs
    return {"value": TRAIN_LAYERS * TRAIN_NODES * wl.total / (dt / steps), "unit": "node-frames/s", "h2d_bytes_per_step": 2 * nbytes,
            "d2h_bytes_per_step": wl.loss_buf.numel() * 8, "steps": steps, "ms_per_step": dt / steps * 1e3,
            "note": "per rank: input + target shard from pinned host memory each step, double-buffered on a copy stream; loss read back",
            "last_loss": losses[-1]}


def cpu_train_reference(steps, warmup):
    """The reference's own DifferentiableLutN<6> (oracle/_ref: unmodified headers) forward + backward on one 65536-node layer of the
    training workload at a reduced frame count; the C restatement when _ref is absent.  Returns (cpu_baseline object, seconds per step)."""
    import numpy as np
    import oracle
    ref, port = oracle.ref, oracle.port
    nodes, F = TRAIN_NODES, CPU_TRAIN_SAMPLE_FRAMES
    rng = np.random.default_rng(7)
    idx = rng.integers(0, nodes, (nodes, 6)).astype(np.int32)
    W = np.clip(rng.normal(0.5, 0.01, (nodes, 64)), 0, 1).astype(np.float32)
    x, dy = rng.random((nodes, F), dtype=np.float32), rng.random((nodes, F), dtype=np.float32)
    use_ref = ref.available()
    cores = ref.use_all_cores() if use_ref else (os.cpu_count() or 1)
    times = []
    for i in range(warmup + steps):
        if use_ref:
            r = ref.differentiable_lut6(x, idx, W, binary=False, dy=dy)
            t = r["t_fwd"] + r["t_bwd"]
        else:
            t0 = time.perf_counter()
            p = port.dl6_forward_train(x, idx, W, np.zeros(nodes, np.float32), np.ones(nodes, np.float32), binary=False)
            port.dl6_backward(x, dy, idx, W, p["mean"], p["rstd"], nodes, binary=False)
            t = time.perf_counter() - t0
        if i >= warmup:
            times.append(t)
    per_step = sum(times) / len(times)
    return {"value": nodes * F / per_step, "unit": "node-frames/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"one DifferentiableLut6 layer {nodes}->{nodes} of the six, {F} of {TRAIN_GLOBAL_BATCH} frames, forward + backward, mean of "
                      f"{len(times)} steps; {'bb::DifferentiableLutN<6,float> (forward OpenMP over nodes, backward a serial loop)' if use_ref else 'C port, OpenMP'}"}, per_step


# ------------------------------------------------------------------------------------------------ BinaryLut6
def bl6_inputs(torch, device, frames, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    words = frames // 32
    x = torch.randint(-2**31, 2**31 - 1, (BL6_NODES, words), dtype=torch.int32, device=device, generator=g)       # Bernoulli(0.5) bits
    idx = torch.randint(0, BL6_NODES, (BL6_NODES, 6), device=device, generator=g)
    for _ in range(8):   # 6 distinct inputs per node: re-draw the few rows with a repeat
        s = idx.sort(dim=1).values
        bad = (s[:, 1:] == s[:, :-1]).any(dim=1)
        if not bool(bad.any()):
            break
        idx[bad] = torch.randint(0, BL6_NODES, (int(bad.sum()), 6), device=device, generator=g)
    idx = idx.to(torch.int32).contiguous()
    table = torch.randint(-2**31, 2**31 - 1, (BL6_NODES, 2), dtype=torch.int32, device=device, generator=g)
    return x, idx, table


def bl6_cpu_reference(steps, warmup, frames):
    """BinaryLutN<6,Bit>::Forward of the unmodified reference headers (AVX2 + OpenMP), or the C port when _ref is absent."""
    import numpy as np
    from oracle import port, ref
    rng = np.random.default_rng(1)
    words = frames // 32
    x = rng.integers(0, 2**32, (BL6_NODES, words), dtype=np.uint64).astype(np.uint32)
    idx = rng.integers(0, BL6_NODES, (BL6_NODES, 6)).astype(np.int32)
    table = rng.integers(-2**31, 2**31, (BL6_NODES, 2)).astype(np.int32)
    use_ref = ref.available()
    cores = ref.use_all_cores() if use_ref else (os.cpu_count() or 1)
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
    per_step = sum(times) / len(times)
    return {"value": BL6_NODES * frames / per_step, "unit": "node-frames/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"BinaryLut6 {BL6_NODES}->{BL6_NODES} nodes, {frames} of {BL6_FRAMES} frames per step, mean of {len(times)} steps, "
                      f"{'bb::BinaryLutN<6,Bit>::Forward AVX2+OpenMP' if use_ref else 'C port, OpenMP'}"}


def binary_lut6_section(torch, ops, dist, world, rank, steps, warmup, frames, extras):
    """BinaryLut6 bit-packed inference forward, 16384 -> 16384 nodes, `frames` frames per GPU (frames shard with no collective)."""
    x, idx, table = bl6_inputs(torch, "cuda", frames, seed=1 + rank)
    y = torch.empty_like(x)
    sec = timed_steps(torch, dist, lambda: ops.binary_lut6_forward(x, idx, table, frames, y=y), steps, warmup)
    hbm, which, _ = measured_peaks()
    algo_bytes = frames * (BL6_NODES + BL6_NODES) / 8 + 32 * BL6_NODES            # x + y bit rows, wiring + table per node
    achieved = algo_bytes / sec / 1e9
    out = {"workload": f"BinaryLut6 forward {BL6_NODES}->{BL6_NODES} nodes, {frames} frames per GPU bit-packed (x, y {frames * BL6_NODES // 8 >> 20} MiB each; "
                       "inputs exceed L2, no flush)", "metric": "BinaryLut6 forward node-frames/s", "value": world * BL6_NODES * frames / sec,
           "unit": "node-frames/s", "ms_per_step": sec * 1e3, "steps": steps, "scaling": "weak", "dtype": "u32 bit-packed", "gpu_launches": steps,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                        "traffic": NCU_BL6_TRAFFIC_BYTES_PER_FRAME * frames, "peak_source": f"of {which}", "kernel": "k_binary_lut6_pipe",
                        "algorithmic_bytes_per_launch": algo_bytes}}
    if extras and rank == 0:
        # the same launch through the truth-table-immediate kernel (15 logic operations per word instead of 63, one indexed branch per
        # table byte): kept measurable because it is the formulation with the fewest operations and still the slower one
        sec_imm = time_op(torch, lambda: ops.binary_lut6_forward(x, idx, table, frames, y=y, lop3_immediate=True), max(2, min(steps, 5)))
        out["lop3_immediate_variant"] = {"ms_per_step": sec_imm * 1e3, "frac": algo_bytes / sec_imm / 1e9 / hbm, "kernel": "k_binary_lut6_imm"}
    if extras and world == 1:
        # end to end through the operator with host buffers: H2D of x, kernel, D2H of y, every step (chunk-pipelined inside the call)
        hx = torch.empty(x.shape, dtype=torch.int32).pin_memory()
        hy = torch.empty(y.shape, dtype=torch.int32).pin_memory()
        hx.copy_(x)
        torch.cuda.synchronize()
        k = max(2, min(steps, 5))
        hidx, htab = idx.cpu(), table.cpu()
        for i in range(1 + k):
            if i == 1:
                torch.cuda.synchronize()
                t0 = time.perf_counter()
            ops.binary_lut6_forward_host(hx, hidx, htab, frames, y=hy)
        dt = time.perf_counter() - t0
        out["e2e"] = {"value": BL6_NODES * frames / (dt / k), "unit": "node-frames/s", "h2d_bytes_per_step": hx.numel() * 4,
                      "d2h_bytes_per_step": hy.numel() * 4, "steps": k}
        del hx, hy
        out["cpu_baseline"] = bl6_cpu_reference(3, 1, frames)
    return out


# ------------------------------------------------------------------------------------------------ single operators
def time_op(torch, fn, steps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / steps


def fp32_cpu_reference(nodes=8192):
    """The reference's own CPU code (oracle/_ref: AVX2 + OpenMP StochasticLutN, scalar DifferentiableLutN whose backward is serial) on
    the fp32 operators at a reduced size (stated in the result; never extrapolated)."""
    import numpy as np
    import oracle
    ref = oracle.ref
    if not ref.available():
        return None
    rng = np.random.default_rng(7)
    idx = np.stack([rng.permutation(nodes)[:6] for _ in range(nodes)]).astype(np.int32)
    W = np.clip(rng.normal(0.5, 0.01, (nodes, 64)), 0, 1).astype(np.float32)
    out = {"cores": ref.use_all_cores(), "kind": "reference", "unit": "node-frames/s", "nodes": nodes}
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


def fp32_section(torch, ops, steps, nodes=TRAIN_NODES, frames=4096):
    """SL6 / DL6 forward and backward on the layer the training step runs per GPU at eight GPUs: 65536 -> 65536 nodes, 4096 frames
    (x, y, dy, dx: 1 GiB each, larger than L2).  Fractions: `frac_of_roofline` on the algorithmic flops / bytes of the 63-interpolation
    formulation, `executed_fp32_frac` on the flops the centred-polynomial kernels really issue."""
    I = O = nodes
    F = frames
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

    cases = {   # name: (callable, algorithmic flops, algorithmic bytes, executed flops) per node-frame
        "sl6_forward":  (lambda: ops.stochastic_lut6_forward(x, idx, W, F, y=y), FLOPS_FWD, 8.0, FLOPS_FWD_EXECUTED),
        "sl6_backward": (lambda: ops.stochastic_lut6_backward(x, dy, idx, W, dW, I, F, dx=dx), FLOPS_BWD, 12.0, FLOPS_BWD_EXECUTED),
        "dl6_forward_training": (dl_fwd, FLOPS_FWD + 10.0, 16.0, FLOPS_FWD_EXECUTED + 10.0),
        # statistics pass (a second evaluation of the tree) + apply pass
        "dl6_backward": (lambda: ops.differentiable_lut6_backward(x, dy, idx, W, dW, state["mean"], state["rstd"], I, F, dx=dx, binary=False),
                         525.0 + FLOPS_FWD, 24.0, FLOPS_BWD_EXECUTED + 10.0 + FLOPS_FWD_EXECUTED + 10.0),
    }
    hbm, which, _ = measured_peaks()
    fp32_peak = fp32_peak_flops(torch)
    out = {"layer": f"{I}->{O} nodes, {F} frames", "fp32_peak_tflops": fp32_peak / 1e12,
           "fp32_peak_note": "SMs * 128 lanes * 2 * 1.965 GHz (clocks.max.sm)", "hbm_peak": f"{hbm} GB/s of {which}"}
    for name, (fn, flops, bytes_, flops_exec) in cases.items():
        sec = time_op(torch, fn, steps)
        nf = O * F / sec
        t_fp, t_hbm = flops / fp32_peak, bytes_ / (hbm * 1e9)
        out[name] = {"node_frames_per_s": nf, "ms": sec * 1e3, "bound": "fp32" if t_fp > t_hbm else "hbm",
                     "frac_of_roofline": nf * max(t_fp, t_hbm), "fp32_frac": nf * t_fp, "hbm_frac": nf * t_hbm,
                     "executed_fp32_frac": nf * flops_exec / fp32_peak,
                     "algorithmic_flops_per_nf": flops, "algorithmic_bytes_per_nf": bytes_, "executed_flops_per_nf": flops_exec}
    return out


def build_lut_cnn(core):
    """The LUT-CNN from the C++ host classes (binarybrain_b200.core): two conv blocks (each two bb::Convolution2d of per-pixel
    DifferentiableLut6 layers with 3x3 'same' lowering, then 2x2 bb::MaxPooling) and a dense head 4096 -> 1024 -> 420 -> 70 -> 10.  Seeded
    random 6-distinct wiring and N(0.5, 0.01) tables as the classes draw them, fp32, batch norm on, probability mode."""
    luts = []

    def lut(n):
        layer = core.DifferentiableLut6_fp32_fp32.create([n], seed=1 + len(luts))
        layer.send_command("binary false")
        luts.append(layer)
        return layer

    def conv(widths):
        seq = core.Sequential.create()
        for n in widths:
            seq.add(lut(n))
        return core.Convolution2d_fp32_fp32.create(seq, 3, 3, padding="same")

    net = core.Sequential.create()
    net.add(conv([216, 36, 32]))
    net.add(conv([216, 36, 32]))
    net.add(core.MaxPooling_fp32_fp32.create(2, 2))
    net.add(conv([384, 64]))
    net.add(conv([384, 64]))
    net.add(core.MaxPooling_fp32_fp32.create(2, 2))
    for n in (1024, 420, 70, 10):
        net.add(lut(n))
    net.set_input_shape([3, 32, 32])
    return net, luts


def cnn_section(torch, steps):
    """LUT-CNN forward + backward on 256 synthetic 3x32x32 images (one GPU), driven through the C++ host classes (bb::Sequential,
    bb::Convolution2d, bb::MaxPooling, bb::DifferentiableLutN over the C ABI).  Node-frames count the LUT evaluations of one forward
    pass (per-pixel layers run on 256 * oh * ow frames)."""
    import numpy as np
    import binarybrain_b200.core as core
    B = 256
    net, _ = build_lut_cnn(core)
    rng = np.random.default_rng(5)
    x = core.FrameBuffer.from_numpy_fp32(rng.random((B, 3, 32, 32), dtype=np.float32))
    dy = core.FrameBuffer.from_numpy_fp32(rng.random((B, 10), dtype=np.float32))
    x.lock_device()
    dy.lock_device()                                 # both stay current on the device: the steps below move nothing over PCIe

    def step():
        net.forward(x, True)
        net.backward(dy)

    sec = time_op(torch, step, steps)
    nf = B * (1024 * (216 + 36 + 32) * 2 + 256 * (384 + 64) * 2 + (1024 + 420 + 70 + 10))
    return {"workload": "LUT-CNN: 3x32x32 images, batch 256, 2 conv blocks of per-pixel DifferentiableLut6 trees with 3x3 Im2Col / "
                        "Col2Im and 2x2 MaxPooling, dense head 4096->1024->420->70->10, fp32, batch norm; forward + backward through the C++ host classes",
            "node_frames_per_s": nf / sec, "ms_per_step": sec * 1e3, "steps": steps, "n_gpus": 1}


def train_cpp_section(torch, steps):
    """The headline's six layers at the headline's shape (one GPU, all of the global batch) through the C++ host classes: bb::Sequential
    of bb::DifferentiableLutN forward (training) + backward, bb::OptimizerAdam update.  Frame buffers come from the library's device
    heap; input and output gradient are filled on the device once."""
    import binarybrain_b200.core as core
    from binarybrain_b200 import abi
    F, nodes = TRAIN_GLOBAL_BATCH, TRAIN_NODES
    net, layers = core.Sequential.create(), []
    for k in range(TRAIN_LAYERS):
        layer = core.DifferentiableLut6_fp32_fp32.create([nodes], seed=1 + k)
        layer.send_command("binary false")
        net.add(layer)
        layers.append(layer)
    net.set_input_shape([nodes])
    opt = core.OptimizerAdam_fp32.create()
    for layer in layers:
        opt.set_variables(layer.W(), layer.dW())

    def device_frames(seed):
        fb = core.FrameBuffer(F, [nodes])
        src = torch.rand((nodes, F), device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed))
        abi.call("bbcu_int32_FrameBufferCopy", fb.lock_device(), src.data_ptr(), nodes, 0, 0, F, 0, 0, fb.get_frame_stride() // 4, F, None)
        torch.cuda.synchronize()
        return fb

    x, dy = device_frames(11), device_frames(12)
    torch.cuda.empty_cache()

    def step():
        net.forward(x, True)
        net.backward(dy)
        opt.update()

    sec = time_op(torch, step, steps)
    del net, layers, opt, x, dy
    torch.cuda.synchronize()
    abi.lib().bbcu_LocalHeap_GarbageCollect()         # the section's frame buffers go back to the driver before the next one allocates
    return {"workload": f"{TRAIN_LAYERS} x DifferentiableLut6 {TRAIN_NODES}->{TRAIN_NODES}, fp32, batch norm, {F} frames, forward + backward + Adam "
                        "through the C++ host classes (bb::Sequential, bb::DifferentiableLutN, bb::OptimizerAdam), one GPU",
            "node_frames_per_s": TRAIN_LAYERS * nodes * F / sec, "ms_per_step": sec * 1e3, "steps": steps}


def operators_section(torch, ops, steps):
    """Every other operator of the path on an 8192 -> 8192 x 16384-frame layer, each with its algorithmic bytes / flops per node-frame
    and the fraction of max(HBM, FP32) roofline time, plus the lowering operators on 32-channel 32x32 images and Adam.  One launch
    sequence per operator call, timed with CUDA events over `steps` back-to-back calls; operators whose device time at the layer's
    shape would be below the ~20 us a call costs on the host run on a larger case (bit -> bit forwards: 262144 frames; Col2Im and
    MaxPooling: batch 2048; Adam: eight 65536 x 64 tables), named in `layer`."""
    I = O = 8192
    F = 16384
    FB = 262144                                       # frames of the bit -> bit forwards
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
    xbb = torch.randint(-2**31, 2**31 - 1, (I, ops.bit_stride(FB)), device=dev, generator=g, dtype=torch.int32)
    ybb = torch.zeros((O, ops.bit_stride(FB)), dtype=torch.int32, device=dev)
    dx = torch.empty((I, F), device=dev)
    st = {}
    _, st["mean"], st["rstd"] = ops.differentiable_lut6_forward_training(xb, idx, W, rm, rv, F, y=ybit)      # statistics of the bit backward case

    def dl_bit_fwd():
        ops.differentiable_lut6_forward_training(xbb, idx, W, rm, rv, FB, y=ybb)

    def dl_binary_fwd():
        _, st["bmean"], st["brstd"] = ops.differentiable_lut6_forward_training(xf, idx, W, rm, rv, F, y=yf, binary=True)

    def sbn_fwd():
        st["sy"], st["smean"], st["srstd"] = ops.stochastic_bn_forward_training(xf, rm, rv, F)

    tables = [(torch.randn((65536, 64), device=dev, generator=g) * 0.01 + 0.5) for _ in range(8)]
    adam = ops.Adam(tables, [torch.rand((65536, 64), device=dev, generator=g) for _ in range(8)])
    # lowering at the LUT-CNN's 32-channel conv: 32x32 images, batch 256 for Im2Col (its output is 9x the image), 2048 for the rest
    c, hw, B, B2 = 32, 32, 256, 2048
    img = torch.rand((c * hw * hw, B), device=dev, generator=g)
    cols = ops.im2col_forward(img, B, c, hw, hw, 3, 3, padding="same")
    colsb_in = torch.randint(-2**31, 2**31 - 1, (c * hw * hw, ops.bit_stride(B2)), device=dev, generator=g, dtype=torch.int32)
    colsb_out = torch.empty((c * 9, ops.bit_stride(B2 * hw * hw)), device=dev, dtype=torch.int32)
    img2 = torch.rand((c * hw * hw, B2), device=dev, generator=g)
    z = torch.rand((c, B2 * hw * hw), device=dev, generator=g)
    pooled, am = ops.maxpool_forward(img2, B2, c, hw, hw, 2, 2)
    gp = torch.rand_like(pooled)
    nf = float(O) * F
    nfb = float(O) * FB
    px = float(c) * hw * hw * B                       # image elements
    px2 = float(c) * hw * hw * B2
    cases = {   # name: (callable, units per call, algorithmic bytes per unit, algorithmic flops per unit)
        "sl6_forward_bit_fp32": (lambda: ops.stochastic_lut6_forward(xb, idx, W, F, y=yf), nf, 4.125, 0.0),       # per-pattern value lookup
        # bit in, bit out: evaluated as a BinaryLut6 forward with a per-node truth table (no per-frame fp32 tree), so the bound is HBM
        "sl6_forward_bit_bit": (lambda: ops.stochastic_lut6_forward(xbb, idx, W, FB, y=ybb, bit_output=True), nfb, 0.25, 0.0),
        "sl6_backward_bit": (lambda: ops.stochastic_lut6_backward(xb, dy, idx, W, dW, I, F, dx=dx), nf, 8.125, 505.0),
        "dl6_forward_training_bit": (dl_bit_fwd, nfb, 0.375, 0.0),      # x read twice (pattern histogram, then the table forward)
        "dl6_forward_inference_bit": (lambda: ops.differentiable_lut6_forward_inference(xbb, idx, W, rm, rv, FB, y=ybb), nfb, 0.25, 0.0),
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
        "adam_update": (lambda: adam.update(), 8.0 * 65536 * 64, 32.0, 12.0),      # W, m, v read and written, dW read, then cleared (Update = Step + ZeroGrad)
        "im2col_forward_fp32": (lambda: ops.im2col_forward(img, B, c, hw, hw, 3, 3, padding="same"), px * 9, 4.0 + 4.0 / 9, 0.0),
        "im2col_forward_bit": (lambda: ops.im2col_forward(colsb_in, B2, c, hw, hw, 3, 3, padding="same", y=colsb_out), px2 * 9, (1 + 1.0 / 9) / 8, 0.0),
        "im2col_backward_fp32": (lambda: ops.im2col_backward(cols, B, c, hw, hw, 3, 3, padding="same"), px * 9, 4.0 + 4.0 / 9, 1.0),
        "col2im_forward_fp32": (lambda: ops.col2im_forward(z, c, hw, hw, B2), px2, 8.0, 0.0),
        "col2im_backward_fp32": (lambda: ops.col2im_backward(img2, c, hw, hw, B2), px2, 8.0, 0.0),
        "maxpool_forward_fp32": (lambda: ops.maxpool_forward(img2, B2, c, hw, hw, 2, 2), px2, 4.0 + 2.0, 1.0),
        "maxpool_backward_fp32": (lambda: ops.maxpool_backward(am, gp, B2, c, hw, hw, 2, 2), px2, 4.0 + 2.0, 0.0),
    }
    hbm, which, _ = measured_peaks()
    fp32_peak = fp32_peak_flops(torch)
    out = {"layer": f"{I}->{O} nodes, {F} frames (bit -> bit forwards: {FB} frames); lowering: {c} channels {hw}x{hw}, 3x3 same / 2x2 pool, batch {B} "
                    f"(Im2Col fp32) and {B2} (Im2Col bit, Col2Im, MaxPooling); Adam: 8 tables of 65536 x 64",
           "unit": "node-frames (LUT, SBN), table entries (Adam), output elements (lowering: Im2Col counts the 9x expanded buffer)",
           "hbm_peak": f"{hbm} GB/s of {which}"}
    for name, (fn, units, bytes_, flops) in cases.items():
        sec = time_op(torch, fn, steps)
        t_fp, t_hbm = flops / fp32_peak, bytes_ / (hbm * 1e9)
        out[name] = {"units_per_s": units / sec, "ms": sec * 1e3, "bound": "fp32" if t_fp > t_hbm else "hbm",
                     "frac_of_roofline": units / sec * max(t_fp, t_hbm), "algorithmic_bytes_per_unit": round(bytes_, 4),
                     "algorithmic_flops_per_unit": flops}
    return out


METRIC = "LUT6 node-frames/s, training step forward+backward fp32 (DifferentiableLut6 x6, 65536 nodes)"


def train_config(world, frames):
    return {"workload": f"frame-sharded training step: {TRAIN_LAYERS} x DifferentiableLut6 {TRAIN_NODES}->{TRAIN_NODES}, fp32, batch norm, MSE, Adam; "
                        f"global batch G = {frames * world} frames per step at every GPU count (strong scaling), {frames} frames per GPU",
            "global_batch": frames * world, "frames_per_gpu": frames, "sharding": "frames; all-reduce of batch-norm sums (2 per layer, blocking) and of "
            "the table gradients (1 per layer, overlapped with the next layer's backward)",
            "l2": f"every frame buffer ({TRAIN_NODES * frames * 4 >> 20} MiB) exceeds L2 (126 MB); no flush"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--global-batch", type=int, default=TRAIN_GLOBAL_BATCH, help="frames per step over all GPUs (default: 32768)")
    ap.add_argument("--bl6-frames", type=int, default=BL6_FRAMES, help="frames per GPU of the BinaryLut6 section (default: 2^20)")
    ap.add_argument("--no-extras", action="store_true", help="headline only: no e2e leg, no sub-sections, no CPU baseline")
    ap.add_argument("--only", default=None, choices=["train", "binary_lut6", "fp32", "operators", "train_cpp"], help="run and print one section (profiling aid)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.global_batch % (32 * world) != 0:
        raise SystemExit("--global-batch must be a multiple of 32 frames per GPU")
    frames = args.global_batch // world
    config = train_config(world, frames)

    if args.impl == "reference":
        if rank != 0:
            return 0
        # a launcher may have exported OMP_NUM_THREADS=1 (torch.distributed.run does): the CPU arm uses every core it may run on
        ncores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        os.environ["OMP_NUM_THREADS"] = str(ncores)
        base, per_step = cpu_train_reference(args.steps, args.warmup)
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "node-frames/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
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
    numa_node = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else None       # (one rank alone keeps every core for the CPU baseline)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ.pop("NCCL_DEBUG", None)         # NCCL prints its version banner on stdout at VERSION and above: stdout carries one JSON line
        import torch.distributed as dist
        import datetime
        # a collective that is not matched on every rank fails after three minutes instead of holding the GPUs for NCCL's default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=180))
    W = max(args.warmup, 3)
    if args.only == "fp32":
        print(json.dumps({"fp32": fp32_section(torch, ops, max(1, args.steps))}))
        return 0
    if args.only == "train_cpp":
        print(json.dumps({"train_cpp": train_cpp_section(torch, max(1, args.steps))}))
        return 0
    if args.only == "operators":
        print(json.dumps({"operators": operators_section(torch, ops, max(1, args.steps))}))
        return 0
    if args.only == "binary_lut6":
        print(json.dumps({"binary_lut6": binary_lut6_section(torch, ops, dist, world, rank, args.steps, W, args.bl6_frames, False)}))
        return 0

    # ---- headline: the training step
    timed = TimedOps(ops, torch, "dl6_backward_apply")
    wl = TrainingWorkload(torch, ops, world, rank, frames, frames * world, timed=timed)
    for _ in range(W):
        wl.step()
    timed.enabled = True
    sampler = ClockSampler(local_rank)
    sec = timed_steps(torch, dist, wl.step, args.steps, 0, sampler)
    timed.enabled = False
    # let the sampler see the loaded clocks at least a few times.  The step holds collectives, so every rank runs the same number of
    # extra steps: whether to run them is agreed on (MAX over ranks), and their count follows from `sec`, which is the same everywhere
    short = torch.tensor([1 if len(sampler.rows) < 3 else 0], device="cuda", dtype=torch.int32)
    if dist:
        dist.all_reduce(short, op=dist.ReduceOp.MAX)
    if int(short.item()):
        for _ in range(int(min(64, max(1, round(0.8 / sec))))):
            wl.step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    value = TRAIN_LAYERS * TRAIN_NODES * frames * world / sec
    hbm, which, _ = measured_peaks()
    fp32_peak = fp32_peak_flops(torch)
    k_ms = timed.mean_ms()                                           # one backward operator call: dx clear, finalize, table conversion, the kernel, dW
    k_nf = TRAIN_NODES * frames
    achieved_tf = FLOPS_BWD * k_nf / (k_ms / 1e3) / 1e12
    line = {"metric": METRIC, "value": value, "unit": "node-frames/s", "n_gpus": world, "steps": args.steps, "warmup": W,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "clocks": clocks, "gpu_launches": args.steps * TrainingWorkload.LAUNCHES_PER_STEP,
            "allreduce_bytes_per_step": wl.allreduce_bytes(),
            "roofline": {"bound": "fp32", "kernel": "k_lut6_backward_pipe<BN> (one bbcu_fp32_DifferentiableLut6_BackwardApply call: dx clear, table conversion, the kernel, dW)",
                         "achieved": achieved_tf, "peak": fp32_peak / 1e12, "unit": "TFLOP/s", "frac": achieved_tf * 1e12 / fp32_peak,
                         "executed_frac": (FLOPS_BWD_EXECUTED + 10.0) * k_nf / (k_ms / 1e3) / fp32_peak,
                         # the same fraction against the peak at the SM clock sampled during the step (a long step runs under the power cap)
                         "frac_at_sampled_clock": (achieved_tf * 1e12 / (fp32_peak * clocks["sm_mhz"] * 1e6 / SM_CLOCK_HZ)) if clocks.get("sm_mhz") else None,
                         "peak_source": "FP32 CUDA-core peak = SMs * 128 lanes * 2 * 1.965 GHz; the path has no tensor-core work",
                         "ms_per_launch": k_ms, "launches_timed": len(timed.pairs), "node_frames_per_launch": k_nf,
                         "algorithmic_flops_per_nf": FLOPS_BWD, "algorithmic_bytes_per_nf": 12.0,
                         "hbm_achieved_gbs": 12.0 * k_nf / (k_ms / 1e3) / 1e9, "hbm_peak_gbs": hbm, "hbm_frac": 12.0 * k_nf / (k_ms / 1e3) / 1e9 / hbm,
                         "hbm_peak_source": f"of {which}",
                         "traffic": None if NCU_BWD_TRAFFIC_BYTES_PER_NF is None else NCU_BWD_TRAFFIC_BYTES_PER_NF * k_nf}}

    dbg = (lambda m: print(f"[bench rank {rank}] {m}", file=sys.stderr, flush=True)) if os.environ.get("BENCH_DEBUG") else (lambda m: None)
    dbg("headline done")
    if not args.no_extras:
        line["e2e"] = train_e2e(torch, dist, wl, max(2, min(args.steps, 5)))
        line["e2e"]["host_numa_node"] = numa_node
    dbg("e2e done")
    del wl
    torch.cuda.empty_cache()
    if args.only == "train" or args.no_extras:
        if dist:
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps(line))
        return 0

    k = max(2, min(args.steps, 5))
    line["binary_lut6"] = binary_lut6_section(torch, ops, dist, world, rank, max(3, min(args.steps, 10)), 3, args.bl6_frames, True)
    torch.cuda.empty_cache()
    dbg("binary_lut6 done")
    # the same six layers in the reference's binary mode (inputs 0.5 +- bias by x > 0.5, outputs binarised), 4096 frames per GPU
    wb = TrainingWorkload(torch, ops, world, rank, 4096, 4096 * world, binary=True)
    sec_b = timed_steps(torch, dist, wb.step, k, 2)
    line["train_binary"] = {"workload": f"{TRAIN_LAYERS} x DifferentiableLut6 {TRAIN_NODES}->{TRAIN_NODES}, binary mode, 4096 frames per GPU (weak scaling)",
                            "node_frames_per_s": TRAIN_LAYERS * TRAIN_NODES * 4096 * world / sec_b, "ms_per_step": sec_b * 1e3, "steps": k, "n_gpus": world}
    del wb
    torch.cuda.empty_cache()
    dbg("train_binary done")
    if rank == 0:
        if world == 1:
            line["train_cpp"] = train_cpp_section(torch, k)
            torch.cuda.empty_cache()
        line["fp32"] = fp32_section(torch, ops, max(3, min(args.steps, 10)))
        torch.cuda.empty_cache()
        line["cnn"] = cnn_section(torch, k)
        torch.cuda.empty_cache()
        line["operators"] = operators_section(torch, ops, max(3, min(args.steps, 10)))
        if world == 1:
            line["cpu_baseline"], _ = cpu_train_reference(2, 1)
            line["fp32"]["cpu_baseline"] = fp32_cpu_reference()
    dbg("sections done")
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
