#!/usr/bin/env python
"""Benchmark of the inference hot path on B200.

    python bench.py --gpus N --steps K --warmup W                 # this back end, headline workload
    python bench.py --workload <name> [--batch B] [--scaling strong]
    python bench.py --impl reference --gpus N ...                 # the reference's CPU path (oracle port)

Headline workload (default): the reference's example CNN in QLinear int8 form (QuantizeLinear ->
2x[QLinearConv, ReLU, MaxPool] -> 2x QLinearMatMul -> DequantizeLinear) on seeded synthetic 1x28x28 inputs,
batch 65536 per GPU (weak scaling) or 65536 in total split across the ranks (`--scaling strong`); a step is
one pass of the plan over the batch.  Other workloads: small_cnn_fp32 (the same network in FP32), qconv3a..3d
(the standalone QLinearConv sweep), qconv4a..4e (single MobileNetV2-style layers), mobilenetv2_int8, tinyyolo_int8,
tinyyolo_fp32.

Every workload prints ONE JSON line on rank 0 with
  value     device-resident throughput (inputs already in HBM, CUDA events on the context's stream),
  e2e       the same call on pinned HOST buffers (H2D of the inputs and D2H of the result inside the timed region),
  roofline  the dominant step: algorithmic bytes or MACs (zant_b200_plan_step_cost) / its mean launch time against
            the measured peaks, plus `whole_step` for the pass as a whole,
  cpu_baseline  the CPU oracle (the reference's algorithm restated) on a bounded sample with every host core; the
            sample's outputs are also compared with what the GPU produced for the same images.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

BATCH_PER_GPU = 65536
METRIC = "int8 images/sec (small CNN, QLinear int8, batch 65536 per GPU)"
MACS_PER_IMAGE = 194688 + 2230272 + 819200 + 5120
L2_BYTES = 126 << 20

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of ONE GPU, named by its UUID, while a timed region runs
    (a CUDA ordinal is not a physical index when CUDA_VISIBLE_DEVICES is set)."""

    def __init__(self, gpu_uuid, period_ms=200):
        self.gpu = gpu_uuid
        self.period_ms = period_ms
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"], gpu=self.gpu)
        time.sleep(self.period_ms / 1e3 + 0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for line in self.lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    power_w_max=max(power) if power else None, reasons=sorted(reasons), samples=len(sm), gpu=self.gpu)


def gpu_uuid(torch, local):
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:       # noqa: BLE001  (older builds have no uuid attribute)
        return str(local)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the four fused steps of the int8 CNN at batch 65536,
# from the ncu captures summarised under profiles/ (index = fused step).
NCU_DRAM_TRAFFIC_B65536 = [205.9e6 + 253.1e6, 302.1e6 + 80.6e6, 105.7e6 + 9.6e6, 33.6e6 + 0.0]


# ------------------------------------------------------------------------------------------------
# Workloads.  Each one knows how to build its graph for a batch, how to make seeded synthetic inputs, and
# what the CPU oracle should run for the same samples.
# ------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    metric = ""
    dtype = "int8"
    default_batch = 1
    flush_l2 = False          # True: inputs fit in L2, so L2 is flushed between timed passes
    l2_note = ""
    cpu_probe = 2             # images of the first oracle run that sizes the CPU sample
    cpu_max_images = 2048     # per thread: the oracle materialises the reference's im2col matrix for its whole batch

    def __init__(self, zb, models, ctx):
        self.zb, self.models, self.ctx = zb, models, ctx

    def graph(self, batch):
        raise NotImplementedError

    def inputs(self, batch, seed):
        raise NotImplementedError

    # what the oracle runs for `x` (a slice of the GPU's own input) -> array comparable with the GPU's output rows
    def oracle_run(self, zo, graph_oracle, x):
        g = self.graph(x.shape[0])
        return graph_oracle.run(zo, g, x)[g.output]

    def config(self, batch):
        return {}


class SmallCnnInt8(Workload):
    name = "small_cnn_int8"
    metric = METRIC
    default_batch = BATCH_PER_GPU
    l2_note = "inputs larger than L2 (205 MB of float input per step at batch 65536)"
    cpu_probe = 4

    def __init__(self, zb, models, ctx):
        super().__init__(zb, models, ctx)
        # calibration through the FP32 network (configuration 1 at batch 256): on the GPU through the FP32 plan, or, in the
        # CPU-only reference arm, through the oracle (the two agree bit for bit; a test checks it)
        fp32, cx = models.small_cnn_fp32(256), models.small_cnn_input(256, models.DEFAULT_SEED + 1)
        if ctx is not None:
            self.scales = models.calibrate_on_gpu(ctx, fp32, cx)
        else:
            zo = ge.load_oracle()
            import graph_oracle
            self.scales = graph_oracle.calibrate(zo, fp32, cx)

    def graph(self, batch):
        return self.models.small_cnn_int8(batch, act_scales=self.scales)

    def inputs(self, batch, seed):
        return np.random.default_rng(seed).random((batch, 1, 28, 28), dtype=np.float32)

    def config(self, batch):
        return dict(workload="small CNN int8 (QLinear form of the reference's example net)", calibration="256 seeded samples, FP32 plan on the GPU",
                    macs_per_image=MACS_PER_IMAGE)


class SmallCnnFp32(Workload):
    name = "small_cnn_fp32"
    metric = "FP32 images/sec (small CNN, the reference's example net)"
    dtype = "f32"
    default_batch = 4096
    l2_note = "activations larger than L2 (354 MB after the first convolution at batch 4096)"
    cpu_probe = 4

    def graph(self, batch):
        return self.models.small_cnn_fp32(batch)

    def inputs(self, batch, seed):
        return np.random.default_rng(seed).random((batch, 1, 28, 28), dtype=np.float32)

    def config(self, batch):
        return dict(workload="small CNN FP32 (configuration 1)", macs_per_image=MACS_PER_IMAGE)


class QConvSweep(Workload):
    default_batch = 256
    flush_l2 = True
    l2_note = "256 MiB written, then 256 MiB read, between passes (inputs not in L2, no dirty lines of the flush left to write back)"
    cpu_probe = 1
    cpu_max_images = 8

    def __init__(self, zb, models, ctx, case):
        super().__init__(zb, models, ctx)
        self.case = case[:2]
        self.default_batch = models.QCONV_SWEEP[self.case]["N"]
        self.channels_last = case.endswith("_nhwc")
        self.name = "qconv" + case
        self.metric = f"int8 images/sec (standalone QLinearConv, sweep case {case})"

    def graph(self, batch):
        return self.models.qconv_graph(self.case, batch=batch, channels_last=self.channels_last)[0]

    def inputs(self, batch, seed):
        # the sweep's own seeded tensor (the seed argument only matters for the CPU threads' extra samples)
        c = self.models.qconv_graph(self.case, batch=batch, seed=self.models.DEFAULT_SEED + (seed % 1000), channels_last=self.channels_last)[1]
        return c["x"]

    def oracle_run(self, zo, graph_oracle, x):
        xn = np.ascontiguousarray(x.transpose(0, 3, 1, 2)) if self.channels_last else x
        g = self.models.qconv_graph(self.case, batch=x.shape[0])[0]
        y = graph_oracle.run(zo, g, xn)[g.output]
        return np.ascontiguousarray(y.transpose(0, 2, 3, 1)) if self.channels_last else y

    def config(self, batch):
        c = self.models.QCONV_SWEEP[self.case]
        return dict(workload=f"QLinearConv sweep case {self.name[5:]}", layout="NHWC int8 in and out (channels-last entry point)" if self.channels_last else "NCHW int8 in and out",
                    **{k: c[k] for k in ("C", "H", "W", "K", "k", "s", "p", "group")})


class MobileNetV2Int8(Workload):
    name = "mobilenetv2_int8"
    metric = "int8 images/sec (MobileNetV2-style classifier, 224x224)"
    default_batch = 1024
    l2_note = "inputs and activations larger than L2 (154 MB of uint8 input at batch 1024)"
    cpu_probe = 1
    cpu_max_images = 8

    def graph(self, batch):
        return self.models.mobilenetv2_int8(batch)

    def inputs(self, batch, seed):
        return np.random.default_rng(seed).integers(0, 256, (batch, 3, 224, 224), dtype=np.uint8)

    def config(self, batch):
        return dict(workload="MobileNetV2-style int8 classifier (width 1.0), 224x224")


class TinyYolo(Workload):
    default_batch = 32
    l2_note = "activations larger than L2 (the first layer's output alone is 354 MB in FP32, 88 MB in int8, at batch 32)"
    cpu_probe = 1
    cpu_max_images = 2

    def __init__(self, zb, models, ctx, int8):
        super().__init__(zb, models, ctx)
        self.int8 = int8
        self.name = "tinyyolo_int8" if int8 else "tinyyolo_fp32"
        self.dtype = "int8" if int8 else "f32"
        self.metric = "images/sec (Tiny-YOLOv3-style detector, 416x416, " + ("int8" if int8 else "FP32") + ")"
        if int8:
            small, cx = models.tiny_yolo_fp32(2), models.tiny_yolo_input(2)
            if ctx is not None:
                self.scales = models.activation_scales_on_gpu(ctx, small, cx)
            else:
                zo = ge.load_oracle()
                import graph_oracle
                vals = graph_oracle.run(zo, small, cx)
                self.scales = models.act_scales_from({t["name"]: vals[i] for i, t in enumerate(small.tensors) if t["data"] is None and i != small.input})

    def graph(self, batch):
        f = self.models.tiny_yolo_fp32(batch)
        return self.models.tiny_yolo_int8(f, self.scales) if self.int8 else f

    def inputs(self, batch, seed):
        return np.random.default_rng(seed).random((batch, 3, 416, 416), dtype=np.float32)

    def config(self, batch):
        return dict(workload="Tiny-YOLOv3-style detector, 416x416, " + ("int8 QDQ" if self.int8 else "FP32"))


WORKLOADS = ["small_cnn_int8", "small_cnn_fp32", "qconv3a", "qconv3b", "qconv3c", "qconv3d", "qconv3a_nhwc", "qconv3c_nhwc",
             "qconv4a", "qconv4b", "qconv4c", "qconv4d", "qconv4e",      # single MobileNetV2-style layers (profiler captures)
             "mobilenetv2_int8", "tinyyolo_int8", "tinyyolo_fp32"]


def make_workload(name, zb, models, ctx):
    if name == "small_cnn_int8":
        return SmallCnnInt8(zb, models, ctx)
    if name == "small_cnn_fp32":
        return SmallCnnFp32(zb, models, ctx)
    if name.startswith("qconv"):
        return QConvSweep(zb, models, ctx, name[len("qconv"):])
    if name == "mobilenetv2_int8":
        return MobileNetV2Int8(zb, models, ctx)
    return TinyYolo(zb, models, ctx, name == "tinyyolo_int8")


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle (the reference's algorithm restated in C++) on a bounded sample, one thread per
# host core on independent sample shards.  Thread 0 runs the first images of the GPU's own input so
# that its outputs can be compared with what the GPU produced.
# ------------------------------------------------------------------------------------------------
def cpu_reference_rate(wl, budget_s=12.0, x_gpu=None, y_gpu=None, tf32_mode=0):
    zo = ge.load_oracle()
    import graph_oracle
    cores = os.cpu_count() or 1
    t0 = time.perf_counter()
    wl.oracle_run(zo, graph_oracle, wl.inputs(wl.cpu_probe, 1))
    per_image = max((time.perf_counter() - t0) / wl.cpu_probe, 1e-6)
    n = int(min(max(budget_s / per_image, 1), wl.cpu_max_images))
    if x_gpu is not None:
        n = min(n, x_gpu.shape[0])
    outs = [None] * cores

    def run_shard(i):
        x = x_gpu[:n] if (i == 0 and x_gpu is not None) else wl.inputs(n, 10 + i)
        outs[i] = wl.oracle_run(zo, graph_oracle, np.ascontiguousarray(x))

    threads = [threading.Thread(target=run_shard, args=(i,)) for i in range(cores)]
    t0 = time.perf_counter()
    for t in threads: t.start()
    for t in threads: t.join()
    wall = time.perf_counter() - t0
    res = dict(value=n * cores / wall, unit="images/s", cores=cores, kind="port",
               sample=f"{n} images per thread x {cores} threads of the same workload ({wl.name}), oracle port of the reference's CPU algorithm "
                      f"({wall:.1f} s wall); the reference (Zig) cannot be built here")
    if y_gpu is not None and outs[0] is not None:
        a, b = np.ascontiguousarray(outs[0]), np.ascontiguousarray(y_gpu[:n])
        how = "the first images of the GPU's own batch through the oracle against the GPU's output rows"
        if tf32_mode:
            # tensor-core float path: the stated tolerance instead of bit identity
            floor = 1.0 if tf32_mode == 1 else 1e-1
            bound = 2e-3 * np.maximum(np.abs(a), floor * np.abs(a).max())
            worst = float((np.abs(a - b) / bound).max())
            same = a.shape == b.shape and worst <= 1.0
            res["parity"] = dict(images=n, bit_exact=False, within_tolerance=bool(same), worst_over_bound=worst,
                                 tolerance=f"|y - ref| <= 2e-3 * max(|ref|, {floor:g} * max|ref|)", how=how)
        else:
            same = a.shape == b.shape and (np.array_equal(a.view(np.uint32), b.view(np.uint32)) if a.dtype == np.float32 else np.array_equal(a, b))
            res["parity"] = dict(images=n, bit_exact=bool(same), how=how)
        if not same:
            raise SystemExit(f"bench: the GPU's output differs from the CPU oracle on the first {n} images of the batch")
    return res


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU path (its algorithm as restated by the oracle: the Zig toolchain is
    not available) on the host cores, on the same workload, metric and unit; each step a bounded sample."""
    if rank != 0:
        return
    zb = ge.load_package()
    from zant_b200 import models
    wl = make_workload(args.workload, zb, models, None)
    batch = args.batch or wl.default_batch
    for _ in range(max(args.warmup, 0)):
        cpu_reference_rate(wl, budget_s=1.0)
    vals, res = [], None
    for _ in range(max(args.steps, 1)):
        res = cpu_reference_rate(wl, budget_s=4.0)
        vals.append(res["value"])
    v = float(np.mean(vals))
    res["value"] = v
    cfg = dict(wl.config(batch), batch_per_gpu=batch, note="the CPU arm times a bounded sample of the workload per step")
    line = dict(impl="reference", metric=wl.metric, value=v, unit="images/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=None, higher_is_better=True, scaling=args.scaling, vs_baseline=None, dtype=wl.dtype, data="synthetic",
                config=cfg, cpu_baseline=res,
                e2e=dict(value=v, unit="images/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def roofline_of(costs, per_step_ms, names, peaks, tensor_peak_tops, tensor_peak_label):
    """Roofline of the dominant step (largest share of the pass) and the per-step table."""
    rows = []
    for i, ((macs, nbytes), ms) in enumerate(zip(costs, per_step_ms)):
        secs = max(ms, 1e-9) / 1e3
        tops, gbs = 2.0 * macs / secs / 1e12, nbytes / secs / 1e9
        rows.append(dict(step=i, kernel=names[i], ms=round(ms, 5), tops=round(tops, 1), tops_frac=round(tops / tensor_peak_tops, 4),
                         gbs=round(gbs, 1), hbm_frac=round(gbs / peaks["hbm_gbs"], 4), macs=macs, bytes=nbytes))
    top = int(np.argmax(per_step_ms)) if per_step_ms else 0
    macs, nbytes = costs[top]
    secs = per_step_ms[top] / 1e3
    ridge = tensor_peak_tops * 1e12 / (peaks["hbm_gbs"] * 1e9)
    if macs and 2.0 * macs / max(nbytes, 1) > ridge:
        ach = 2.0 * macs / secs / 1e12
        roof = dict(bound="tensor", achieved=ach, peak=tensor_peak_tops, unit="TFLOP/s", frac=ach / tensor_peak_tops,
                    peak_source=tensor_peak_label)
    else:
        ach = nbytes / secs / 1e9
        roof = dict(bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"],
                    peak_source=peaks["source"] + " (MEASURED_PEAKS.json hbm_gbs)" if peaks["source"] == "measured" else "fallback")
    roof.update(traffic=None, kernel=f"{top}:{names[top]}", launch_ms=per_step_ms[top], algorithmic_bytes=nbytes, macs=macs,
                share_of_pass=per_step_ms[top] / max(sum(per_step_ms), 1e-9))
    return roof, rows


def whole_step_roofline(graph, costs, ms, peaks, tensor_peak_tops, itemsize):
    """The pass as one unit: all MACs against the tensor peak, and the bytes a fully fused pass could not avoid
    (graph input, graph output and every initializer once) against HBM; `frac` = the larger floor / the time."""
    macs = sum(c[0] for c in costs)
    t = graph.tensors
    nbytes = sum(int(np.prod(x["shape"])) * itemsize[x["dtype"]] for i, x in enumerate(t) if x["data"] is not None or i in (graph.input, graph.output))
    secs = ms / 1e3
    tensor_floor_ms = 2.0 * macs / (tensor_peak_tops * 1e12) * 1e3
    hbm_floor_ms = nbytes / (peaks["hbm_gbs"] * 1e9) * 1e3
    unfused_bytes = sum(c[1] for c in costs)
    return dict(macs=macs, min_bytes=nbytes, tops=2.0 * macs / secs / 1e12, tops_frac=2.0 * macs / secs / 1e12 / tensor_peak_tops,
                gbs_min_bytes=nbytes / secs / 1e9, tensor_floor_ms=tensor_floor_ms, hbm_floor_ms=hbm_floor_ms,
                frac=max(tensor_floor_ms, hbm_floor_ms) / ms, bound="tensor" if tensor_floor_ms > hbm_floor_ms else "hbm",
                per_step_bytes_total=unfused_bytes, hbm_floor_of_the_steps_ms=unfused_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3)


def run_gpu_arm(args, rank, world, local):
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    zb = ge.load_package()
    zb.lib()
    from zant_b200 import models
    ctx = zb.Context(local)
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local))
    fuse = not args.no_fuse
    if args.dtype in ("tf32", "tf32x3"):
        ctx.set_tf32(1 if args.dtype == "tf32" else 2)

    int8_peak = ctx.measure_int8_peak(20000)          # resident-tile tcgen05 probe, ~15 ms per launch, best of four
    peaks = measured_peaks()
    wl = make_workload(args.workload, zb, models, ctx)
    tensor_peak, tensor_label = int8_peak, "int8 tensor peak measured in this run by zant_b200_measure_int8_peak (burst)"
    if wl.dtype == "f32":
        tensor_peak = peaks["bf16_tflops"] / 2.0
        tensor_label = "TF32 dense peak taken as half the measured bf16 rate (MEASURED_PEAKS.json bf16_tflops / 2)"

    # this rank's samples: a fixed batch per GPU (weak), or its shard of one global batch (strong)
    if args.scaling == "strong":
        total = args.batch or wl.default_batch
        _begin, batch = zb.shard_range(total, world, rank)
    else:
        batch = args.batch or wl.default_batch
        total = batch * world
    graph = wl.graph(batch)
    plan = zb.Plan(ctx, graph, fuse=fuse)
    out_np_dtype = zb.NP_DTYPE[graph.tensors[graph.output]["dtype"]]
    out_shape = tuple(graph.tensors[graph.output]["shape"])
    x_host = torch.from_numpy(np.ascontiguousarray(wl.inputs(batch, models.DEFAULT_SEED + 100 + rank))).pin_memory()
    y_host = torch.from_numpy(np.zeros(out_shape, out_np_dtype)).pin_memory()
    x_dev = x_host.cuda(non_blocking=False)
    y_dev = torch.empty_like(y_host, device="cuda")
    in_bytes, out_bytes = x_host.numel() * x_host.element_size(), y_host.numel() * y_host.element_size()
    if wl.flush_l2:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")      # larger than L2
        clean = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")      # read after the write: L2 then holds clean lines

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def timed(fn, steps):
        """Milliseconds for `steps` calls of fn: barrier + synchronize on both sides, CUDA events on the context's
        stream, maximum over ranks.  With L2 flushing every call is bracketed on its own and the times are summed."""
        with torch.cuda.stream(stream):
            barrier()
            ctx.reset_launch_count()
            if wl.flush_l2:
                ms = 0.0
                for _ in range(steps):
                    flush.fill_(1)
                    clean.max()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream); fn(); e1.record(stream)
                    torch.cuda.synchronize()
                    ms += e0.elapsed_time(e1)
                launches = ctx.launch_count()
                barrier()
            else:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(steps):
                    fn()
                e1.record(stream)
                barrier()
                ms = e0.elapsed_time(e1)
                launches = ctx.launch_count()
        return max_over_ranks(ms), launches

    resident = lambda: plan.run(x_dev, out=y_dev)        # noqa: E731

    # End to end: the same batch from pinned host memory.  The headline workload cuts it into chunks that alternate
    # between two contexts (streams) so that the H2D copy of one chunk overlaps the kernels of the previous one.
    n_chunks = args.e2e_chunks if (args.e2e_chunks > 1 and batch % args.e2e_chunks == 0 and batch // args.e2e_chunks >= 256) else 1
    cb = batch // n_chunks
    extra_plans, ctx2 = [], None
    if n_chunks > 1:
        ctx2 = zb.Context(local)
        if args.dtype in ("tf32", "tf32x3"):
            ctx2.set_tf32(1 if args.dtype == "tf32" else 2)
        chunk_graph = wl.graph(cb)
        extra_plans = [zb.Plan(ctx, chunk_graph, fuse=fuse), zb.Plan(ctx2, chunk_graph, fuse=fuse)]
        stream2 = torch.cuda.ExternalStream(ctx2.stream, device=torch.device("cuda", local))

        def end_to_end():
            # order the two streams behind the timing event's stream, run, and join them again
            ev = torch.cuda.Event(); ev.record(stream); stream2.wait_event(ev)
            for c in range(n_chunks):
                extra_plans[c % 2].run(x_host[c * cb:(c + 1) * cb], out=y_host[c * cb:(c + 1) * cb])
            ev2 = torch.cuda.Event(); ev2.record(stream2); stream.wait_event(ev2)
    else:
        end_to_end = lambda: plan.run(x_host, out=y_host)    # noqa: E731

    # graph replay runs on the arena's own input buffer (one more device copy of the input): worth it where the launch
    # cost dominates, i.e. for the small per-rank batches of a strong-scaling split
    use_graph = args.graph or (args.scaling == "strong" and not wl.flush_l2 and in_bytes <= (32 << 20))
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            resident()
    sampler = ClockSampler(gpu_uuid(torch, local)).start() if rank == 0 else None
    if use_graph:
        plan.use_graph(True)
        with torch.cuda.stream(stream):
            for _ in range(3):
                resident()
    ms, launches = timed(resident, args.steps)
    if use_graph:
        plan.use_graph(False)

    # per-step times: a second, untimed series with one CUDA event in front of every step
    with torch.cuda.stream(stream):
        plan.profile(True)
        if wl.flush_l2:
            for _ in range(args.steps):
                flush.fill_(1); clean.max(); resident()
        else:
            for _ in range(args.steps):
                resident()
        torch.cuda.synchronize()
        step_ms, runs = plan.profile_read()
        plan.profile(False)

    with torch.cuda.stream(stream):
        for _ in range(2):
            end_to_end()
    ms_e2e, _ = timed(end_to_end, args.steps)
    torch.cuda.synchronize()
    # the host-buffer path must produce what the resident path produced
    with torch.cuda.stream(stream):
        resident()
    torch.cuda.synchronize()
    if not torch.equal(y_dev.cpu(), y_host):
        raise SystemExit("bench: end-to-end result differs from the device-resident result")

    # a bare pinned->device copy of the same input on every rank at once: the ceiling the host side puts on e2e
    with torch.cuda.stream(stream):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        e0.record(stream)
        for _ in range(reps):
            x_dev.copy_(x_host, non_blocking=True)
        e1.record(stream)
        barrier()
        copy_ms = max_over_ranks(e0.elapsed_time(e1)) / reps
    h2d_plain = dict(bytes=in_bytes, ms=copy_ms, gbs_per_rank=in_bytes / (copy_ms / 1e3) / 1e9, gbs_all_ranks=in_bytes * world / (copy_ms / 1e3) / 1e9,
                     images_per_s_ceiling=total / (copy_ms / 1e3),
                     how="cudaMemcpyAsync pinned host -> device of one step's input on every rank at the same time, max over ranks")

    sustained = None
    if args.sustain_seconds > 0 and not wl.flush_l2:
        # the resident step looped for seconds with the clock sampler running: the rate under the power cap, and the
        # tensor-core probe looped the same way as its denominator
        s2 = ClockSampler(gpu_uuid(torch, local)).start() if rank == 0 else None
        per_step = ms / args.steps
        n_iter = int(max(args.sustain_seconds * 1e3 / max(per_step, 1e-3), 10))
        ms_s, _ = timed(resident, n_iter)
        c2 = s2.stop() if s2 else None
        sustained = dict(seconds=ms_s / 1e3, steps=n_iter, ms_per_step=ms_s / n_iter, value=total * n_iter / (ms_s / 1e3), unit="images/s", clocks=c2)
        if rank == 0 and wl.dtype == "int8":
            s3 = ClockSampler(gpu_uuid(torch, local)).start()
            sustained["int8_peak_tops_sustained"] = ctx.measure_int8_peak_sustained(args.sustain_seconds)
            sustained["int8_peak_clocks"] = s3.stop()
    clocks = sampler.stop() if sampler else None

    latency = None
    if rank == 0 and args.workload in ("small_cnn_int8", "small_cnn_fp32"):
        # batch-1 latency of one predict() call on pinned host buffers (host clock around run + synchronize),
        # with separate launches and with the plan's captured CUDA graph
        p1 = zb.Plan(ctx, wl.graph(1), fuse=fuse)
        x1, y1 = x_host[:1], torch.empty((1,) + out_shape[1:], dtype=y_host.dtype).pin_memory()
        latency = {}
        for mode in ("launches", "graph"):
            p1.use_graph(mode == "graph")
            for _ in range(50):
                p1.run(x1, out=y1)
            ctx.synchronize()
            samples = []
            for _ in range(300):
                t0 = time.perf_counter()
                p1.run(x1, out=y1)
                ctx.synchronize()
                samples.append((time.perf_counter() - t0) * 1e6)
            latency[mode + "_us_median"] = round(float(np.median(samples)), 2)
        latency["kernels_per_call"] = p1.launches_per_run
        p1.close()

    if rank == 0:
        names = plan.step_names()
        costs = plan.step_costs()
        per_step = [m / max(runs, 1) for m in step_ms]
        roof, rows = roofline_of(costs, per_step, names, peaks, tensor_peak, tensor_label)
        fused_cnn = args.workload == "small_cnn_int8" and len(names) == 4 and fuse
        if fused_cnn:
            top = int(np.argmax(per_step))
            roof["traffic"] = NCU_DRAM_TRAFFIC_B65536[top] * batch / 65536
            roof["traffic_source"] = "ncu capture at batch 65536 (profiles/), scaled by batch"
        itemsize = {0: 4, 1: 1, 2: 1, 3: 4}
        whole = whole_step_roofline(graph, costs, ms / args.steps, peaks, tensor_peak, itemsize)
        roof["whole_step"] = whole
        by_kind = {}
        for r in rows:
            by_kind[r["kernel"]] = by_kind.get(r["kernel"], 0.0) + r["ms"]
        top_rows = rows if (len(rows) <= 8 or args.all_steps) else sorted(rows, key=lambda r: -r["ms"])[:8]
        cpu = None
        if not args.skip_cpu and world == 1:
            cpu = cpu_reference_rate(wl, x_gpu=x_host.numpy(), y_gpu=y_host.numpy(), tf32_mode={"tf32": 1, "tf32x3": 2}.get(args.dtype, 0))
        value = total * args.steps / (ms / 1e3)
        cfg = dict(wl.config(batch), batch_per_gpu=batch, global_batch=total, fused=fuse, l2=wl.l2_note, cuda_graph=bool(use_graph),
                   parallelism=f"sample-sharded x{world}, no collective")
        line = dict(metric=wl.metric, value=value, unit="images/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms / args.steps, higher_is_better=True, scaling=args.scaling, vs_baseline=None,
                    dtype=(args.dtype if args.dtype != "native" else wl.dtype), data="synthetic", config=cfg,
                    roofline=roof, int8_peak_tops=int8_peak, bf16_tflops_measured=peaks["bf16_tflops"],
                    per_kernel=top_rows, ms_by_step_kind={k: round(v, 4) for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1])},
                    cpu_baseline=cpu,
                    e2e=dict(value=total * args.steps / (ms_e2e / 1e3), unit="images/s", h2d_bytes_per_step=in_bytes, d2h_bytes_per_step=out_bytes,
                             ms_per_step=ms_e2e / args.steps, chunks=n_chunks,
                             how="plan.run on pinned host buffers" + (", chunks alternate between two contexts (copy/compute overlap)" if n_chunks > 1 else "")),
                    h2d_plain_copy=h2d_plain, sustained=sustained, gpu_launches=int(launches) * world, clocks=clocks,
                    arena_bytes=plan.arena_bytes, batch1_latency=latency)
        print(json.dumps(line), flush=True)
    for p in extra_plans:
        p.close()
    plan.close()
    # The contexts (and their streams) stay alive until the process exits: torch's allocators record events on every
    # stream a buffer was used on when that buffer is freed, which for the pinned host buffers happens at interpreter exit.
    torch.cuda.synchronize()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="zant_b200", choices=["zant_b200", "reference"])
    ap.add_argument("--workload", default="small_cnn_int8", choices=WORKLOADS,
                    help="small_cnn_int8 is the headline workload; the qconv cases time one standalone operator")
    ap.add_argument("--batch", type=int, default=0, help="images per GPU per step (weak) or in total (strong); 0 = the workload's own")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--dtype", default="native", choices=["native", "tf32", "tf32x3"],
                    help="tf32: float contractions on the tensor cores, one pass; tf32x3: the same with split operands (three MMAs per K step)")
    ap.add_argument("--graph", action="store_true", help="replay the plan as one CUDA graph in the timed region")
    ap.add_argument("--no-fuse", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--all-steps", action="store_true", help="per_kernel lists every step of the plan in order (default: the eight longest)")
    ap.add_argument("--sustain-seconds", type=float, default=2.0, help="length of the sustained-rate loop (0 = skip)")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="chunks of the batch that the end-to-end path pipelines")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    run_gpu_arm(args, rank, world, local)


if __name__ == "__main__":
    main()
