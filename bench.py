#!/usr/bin/env python
"""Benchmark of the int8 inference hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this back end
    python bench.py --impl reference --gpus N ...            # the reference's CPU path (oracle port)

Workload: the reference's example CNN in QLinear int8 form (QuantizeLinear -> 2x[QLinearConv, ReLU,
MaxPool] -> 2x QLinearMatMul -> DequantizeLinear) on seeded synthetic 1x28x28 inputs, batch 65536
per GPU; a step is one pass of the plan over the batch.  `value` times the step with the batch
already resident in HBM; `e2e` times the same call with pinned HOST buffers (H2D of the float
inputs and D2H of the logits inside the timed region).  Prints one JSON line on rank 0.
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

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    reasons=sorted(reasons), samples=len(sm))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def step_costs(graph):
    """Algorithmic work of every graph node: MACs and bytes (each operand and result once)."""
    itemsize = {0: 4, 1: 1, 2: 1, 3: 4}
    out = {}
    for i, n in enumerate(graph.nodes):
        ts = [graph.tensors[t] for t in n["inputs"] if t >= 0] + [graph.tensors[t] for t in n["outputs"]]
        nbytes = sum(int(np.prod(t["shape"])) * itemsize[t["dtype"]] for t in ts)
        macs = 0
        if n["op"] in ("QLinearConv", "Conv"):
            w = graph.tensors[n["inputs"][1]]["shape"]; y = graph.tensors[n["outputs"][0]]["shape"]
            macs = int(np.prod(y)) * w[1] * w[2] * w[3]
        elif n["op"] in ("QLinearMatMul", "MatMul"):
            a = graph.tensors[n["inputs"][0]]["shape"]; b = graph.tensors[n["inputs"][1]]["shape"]
            macs = a[0] * a[1] * b[1]
        out[i] = dict(op=n["op"], macs=macs, bytes=nbytes, out=graph.tensors[n["outputs"][0]]["name"])
    return out


def fused_step_costs(batch, n_classes=10):
    """Algorithmic work of the four fused steps of the int8 CNN (per launch): every tensor that
    crosses a kernel boundary counted once at its storage type, weights included.  Of the 13 x 13 pooled
    pixels of stage 1 the next stage's pool reads 12 x 12: only those are stored and counted (MACs stay the
    layer's nominal ones)."""
    return [
        dict(op="conv1 fused", out="pool1", macs=batch * 194688, bytes=batch * (784 * 4 + 12 * 12 * 32) + 32 * 9),
        dict(op="conv2 fused tcgen05", out="pool2", macs=batch * 2230272, bytes=batch * (12 * 12 * 32 + 1600) + 64 * 288),
        dict(op="fc1 tcgen05", out="relu3", macs=batch * 819200, bytes=batch * (1600 + 512) + 1600 * 512),
        dict(op="fc2+dequant", out="logits", macs=batch * 512 * n_classes, bytes=batch * (512 + 4 * n_classes) + 512 * n_classes),
    ]


# dram__bytes_read.sum + dram__bytes_write.sum per launch at batch 65536, from the ncu captures
# summarised under profiles/ (index = fused step).
NCU_DRAM_TRAFFIC_B65536 = [205.9e6 + 253.1e6, 302.1e6 + 80.6e6, 105.7e6 + 9.6e6, 33.6e6 + 0.0]


def cpu_reference_rate(batch_hint, scales, budget_s=12.0):
    """Times the CPU oracle (the reference's algorithm restated) on a bounded sample of the
    workload with every host core (independent sample shards, one thread each)."""
    zo = ge.load_oracle()
    import graph_oracle
    zb = ge.load_package()
    from zant_b200 import models
    cores = os.cpu_count() or 1

    def run_shard(n, seed, box):
        g = models.small_cnn_int8(n, act_scales=scales)
        x = models.small_cnn_input(n, seed)
        t0 = time.perf_counter()
        graph_oracle.run(zo, g, x)
        box.append(time.perf_counter() - t0)

    probe = []
    run_shard(4, 1, probe)
    per_image = max(probe[0] / 4, 1e-6)
    n = int(min(max(budget_s / per_image, 4), 2048))
    boxes = [[] for _ in range(cores)]
    threads = [threading.Thread(target=run_shard, args=(n, 10 + i, boxes[i])) for i in range(cores)]
    t0 = time.perf_counter()
    for t in threads: t.start()
    for t in threads: t.join()
    wall = time.perf_counter() - t0
    return dict(value=n * cores / wall, unit="images/s", cores=cores, kind="port",
                sample=f"{n} images per thread x {cores} threads of the same int8 CNN, oracle port of the reference's CPU algorithm "
                       f"({wall:.1f} s wall); the reference (Zig) cannot be built here")


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    scales = dict(relu1=0.02, relu2=0.05, relu3=0.05, logits=0.1)
    vals = []
    for _ in range(max(args.warmup, 0)):
        cpu_reference_rate(BATCH_PER_GPU, scales, budget_s=1.0)
    res = None
    for _ in range(max(args.steps, 1)):
        res = cpu_reference_rate(BATCH_PER_GPU, scales, budget_s=4.0)
        vals.append(res["value"])
    v = float(np.mean(vals))
    res["value"] = v
    line = dict(impl="reference", metric=METRIC, value=v, unit="images/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=None, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="int8", data="synthetic",
                config=dict(workload="small CNN int8 (QLinear), batch 65536 per GPU; CPU arm times a bounded sample per step",
                            batch_per_gpu=BATCH_PER_GPU), cpu_baseline=res,
                e2e=dict(value=v, unit="images/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line), flush=True)


def run_qconv_workload(args, zb, ctx, models, torch, stream, rank, world, local, int8_peak_tops):
    """One case of the standalone QLinearConv sweep (--workload qconv3a..3d): the batch of 256
    NCHW int8 images resident in HBM, one plan step per pass; images/s plus the op's roofline."""
    name = args.workload[len("qconv"):]
    channels_last = name.endswith("_nhwc")
    graph, c = models.qconv_graph(name[:2], channels_last=channels_last)
    plan = zb.Plan(ctx, graph, fuse=not args.no_fuse)
    x_dev = torch.from_numpy(c["x"]).cuda()
    y_dev = torch.empty(tuple(graph.tensors[graph.output]["shape"]), dtype=torch.int8, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")      # larger than L2
    clean = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")      # read after the write: see the timing loop
    run = lambda: plan.run(x_dev, out=y_dev)    # noqa: E731
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            run()
        torch.cuda.synchronize()
        sampler = ClockSampler(local) if rank == 0 else None
        if sampler:
            sampler.start()
        ctx.reset_launch_count()
        times = []
        for _ in range(args.steps):
            flush.fill_(1)                                                # evict x, w and y from L2 between passes
            clean.max()                                                   # ... and read another buffer, so that L2 holds clean lines: the
            #                                                               timed kernel does not pay for writing the flush buffer back
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream); run(); e1.record(stream)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        launches = ctx.launch_count()
        clocks = sampler.stop() if sampler else None
    ms = float(np.mean(times))
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        peaks = measured_peaks()
        ridge = int8_peak_tops * 1e12 / (peaks["hbm_gbs"] * 1e9)
        tops, gbs = 2.0 * c["macs"] / (ms / 1e3) / 1e12, c["bytes"] / (ms / 1e3) / 1e9
        if 2.0 * c["macs"] / c["bytes"] > ridge:
            roof = dict(bound="tensor", achieved=tops, peak=int8_peak_tops, unit="TFLOP/s", frac=tops / int8_peak_tops)
        else:
            roof = dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"])
        roof.update(traffic=None, kernel=" + ".join(plan.step_names()), launch_ms=ms, algorithmic_bytes=c["bytes"], macs=c["macs"],
                    peak_source=peaks["source"], tops=tops, gbs=gbs)
        shape = {k: c[k] for k in ("N", "C", "H", "W", "K", "k", "s", "p", "group")}
        line = dict(metric=f"int8 images/sec (standalone QLinearConv, sweep case {name})", value=c["N"] * world / (ms / 1e3), unit="images/s",
                    n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="weak",
                    vs_baseline=None, dtype="int8", data="synthetic",
                    config=dict(workload=f"QLinearConv sweep case {name}", layout="NHWC int8 in and out (channels-last entry point)" if channels_last else "NCHW int8 in and out", l2="256 MiB written, then 256 MiB read, between passes (inputs not in L2, no dirty lines of the flush left to write back)",
                                parallelism=f"replicas x{world}, no collective", **shape),
                    roofline=roof, int8_peak_tops=int8_peak_tops, cpu_baseline=None, e2e=None, gpu_launches=int(launches) * world, clocks=clocks)
        print(json.dumps(line), flush=True)
    plan.close()


def run_graph_workload(args, zb, ctx, models, torch, stream, rank, world, local, int8_peak_tops):
    """Whole-network workloads beside the headline one (--workload mobilenetv2_int8 | tinyyolo_int8 |
    tinyyolo_fp32): device-resident images/s of one plan pass per step, with the per-step time table."""
    if args.workload == "mobilenetv2_int8":
        batch = args.batch if args.batch != BATCH_PER_GPU else 1024
        graph = models.mobilenetv2_int8(batch)
        x = models.mobilenetv2_input(batch)
        name = "MobileNetV2-style int8 classifier, 224x224"
    else:
        batch = args.batch if args.batch != BATCH_PER_GPU else 32
        fp32 = models.tiny_yolo_fp32(batch)
        x = models.tiny_yolo_input(batch)
        if args.workload == "tinyyolo_int8":
            small = models.tiny_yolo_fp32(2)
            scales = models.activation_scales_on_gpu(ctx, small, models.tiny_yolo_input(2))
            graph = models.tiny_yolo_int8(fp32, scales)
        else:
            graph = fp32
        name = "Tiny-YOLOv3-style detector, 416x416, " + ("int8" if args.workload == "tinyyolo_int8" else "FP32")
    plan = zb.Plan(ctx, graph, fuse=not args.no_fuse)
    x_dev = torch.from_numpy(x).cuda()
    out_shape = tuple(graph.tensors[graph.output]["shape"])
    y_dev = torch.empty(out_shape, dtype=torch.float32, device="cuda")
    run = lambda: plan.run(x_dev, out=y_dev)    # noqa: E731
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            run()
        torch.cuda.synchronize()
        sampler = ClockSampler(local) if rank == 0 else None
        if sampler:
            sampler.start()
        plan.profile(True)
        ctx.reset_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        launches = ctx.launch_count()
        step_ms, runs = plan.profile_read()
        plan.profile(False)
        clocks = sampler.stop() if sampler else None
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        names = plan.step_names()
        per = [m / max(runs, 1) for m in step_ms]
        by_kind = {}
        for n, m in zip(names, per):
            by_kind[n] = by_kind.get(n, 0.0) + m
        top = sorted(range(len(per)), key=lambda i: -per[i])[:8]
        macs = graph.meta.get("macs_per_image") if hasattr(graph, "meta") else None
        line = dict(metric=f"images/sec ({name})", value=batch * world / (ms / 1e3), unit="images/s", n_gpus=world, steps=args.steps,
                    warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="f32" if args.workload == "tinyyolo_fp32" else "int8", data="synthetic",
                    config=dict(workload=name, batch_per_gpu=batch, l2="activations larger than L2", parallelism=f"sample-sharded x{world}, no collective"),
                    roofline=None, int8_peak_tops=int8_peak_tops, macs_per_image=macs,
                    tops=(2.0 * macs * batch / (ms / 1e3) / 1e12) if macs else None,
                    ms_by_step_kind={k: round(v, 4) for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1])},
                    top_steps=[dict(step=i, kind=names[i], ms=round(per[i], 4)) for i in top],
                    cpu_baseline=None, e2e=None, gpu_launches=int(launches) * world, clocks=clocks, arena_bytes=plan.arena_bytes)
        print(json.dumps(line), flush=True)
    plan.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="zant_b200", choices=["zant_b200", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="images per GPU per step")
    ap.add_argument("--no-fuse", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--workload", default="small_cnn_int8", choices=["small_cnn_int8", "qconv3a", "qconv3b", "qconv3c", "qconv3d", "qconv3a_nhwc", "qconv3c_nhwc", "mobilenetv2_int8", "tinyyolo_int8", "tinyyolo_fp32"],
                    help="small_cnn_int8 is the headline workload; the qconv cases time one standalone operator")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="chunks of the batch that the end-to-end path pipelines")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

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
    batch = args.batch

    int8_peak_tops = ctx.measure_int8_peak(20000) if rank == 0 else None   # resident-tile tcgen05 probe, ~15 ms

    if args.workload != "small_cnn_int8":
        fn = run_qconv_workload if args.workload.startswith("qconv") else run_graph_workload
        fn(args, zb, ctx, models, torch, stream, rank, world, local, ctx.measure_int8_peak(20000))
        ctx.close()
        if world > 1:
            dist.destroy_process_group()
        return

    # calibration on the GPU through the FP32 plan (configuration 1 at batch 256), then the int8 graph
    scales = models.calibrate_on_gpu(ctx, models.small_cnn_fp32(256), models.small_cnn_input(256, models.DEFAULT_SEED + 1))
    graph = models.small_cnn_int8(batch, act_scales=scales)
    plan = zb.Plan(ctx, graph, fuse=not args.no_fuse)

    begin, count = zb.shard_range(batch * world, world, rank)   # this rank's samples of the global batch
    gen = torch.Generator(device="cpu").manual_seed(models.DEFAULT_SEED + 100 + rank)
    x_host = torch.rand((batch, 1, 28, 28), generator=gen, dtype=torch.float32).pin_memory()
    y_host = torch.empty((batch, 10), dtype=torch.float32).pin_memory()
    x_dev = x_host.cuda(non_blocking=False)
    y_dev = torch.empty((batch, 10), dtype=torch.float32, device="cuda")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, profile=False):
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            if profile:
                plan.profile(True)
            ctx.reset_launch_count()
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
        launches = ctx.launch_count()
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches

    resident = lambda: plan.run(x_dev, out=y_dev)        # noqa: E731

    # End to end: the same batch from pinned host memory, cut into chunks that alternate between two
    # contexts (streams) so that the H2D copy of one chunk overlaps the kernels of the previous one.
    n_chunks = args.e2e_chunks if batch % args.e2e_chunks == 0 else 1
    cb = batch // n_chunks
    if n_chunks > 1:
        ctx2 = zb.Context(local)
        chunk_graph = models.small_cnn_int8(cb, act_scales=scales)
        chunk_plans = [zb.Plan(ctx, chunk_graph, fuse=not args.no_fuse), zb.Plan(ctx2, chunk_graph, fuse=not args.no_fuse)]
        stream2 = torch.cuda.ExternalStream(ctx2.stream, device=torch.device("cuda", local))

        def end_to_end():
            # order the two streams behind the timing event's stream, run, and join them again
            ev = torch.cuda.Event(); ev.record(stream); stream2.wait_event(ev)
            for c in range(n_chunks):
                chunk_plans[c % 2].run(x_host[c * cb:(c + 1) * cb], out=y_host[c * cb:(c + 1) * cb])
            ev2 = torch.cuda.Event(); ev2.record(stream2); stream.wait_event(ev2)
    else:
        end_to_end = lambda: plan.run(x_host, out=y_host)    # noqa: E731

    for _ in range(args.warmup):
        resident()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms, launches = timed(resident, args.steps, profile=True)
    step_ms, runs = plan.profile_read()
    plan.profile(False)
    clocks = sampler.stop() if sampler else None

    for _ in range(2):
        end_to_end()
    ms_e2e, _ = timed(end_to_end, args.steps)
    torch.cuda.synchronize()
    # the pipelined path must produce what the resident path produced
    resident()
    torch.cuda.synchronize()
    if not torch.equal(y_dev.cpu(), y_host):
        raise SystemExit("bench: end-to-end result differs from the device-resident result")

    latency = None
    if rank == 0:
        # batch-1 latency of one predict() call on pinned host buffers (host clock around run + synchronize),
        # with separate launches and with the plan's captured CUDA graph
        g1 = models.small_cnn_int8(1, act_scales=scales)
        p1 = zb.Plan(ctx, g1, fuse=not args.no_fuse)
        x1, y1 = x_host[:1], torch.empty((1, 10), dtype=torch.float32).pin_memory()
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
        peaks = measured_peaks()
        total_images = batch * world * args.steps
        value = total_images / (ms / 1e3)
        names = plan.step_names()
        costs = step_costs(graph)
        per_step = [m / max(runs, 1) for m in step_ms]
        # dominant kernel = the step with the largest share of the timed region
        top = int(np.argmax(per_step)) if per_step else 0
        # map the step back to its node: unfused plans have one step per non-Reshape node
        node_ids = [i for i, n in enumerate(graph.nodes) if n["op"] != "Reshape"]
        shares = {f"{i}:{names[i]}": round(per_step[i] / max(sum(per_step), 1e-9), 4) for i in range(len(names))}
        roof = None
        fused_costs = fused_step_costs(batch) if (len(names) == 4 and not args.no_fuse) else None
        if len(names) == len(node_ids) or fused_costs:
            c = fused_costs[top] if fused_costs else costs[node_ids[top]]
            int8_peak = int8_peak_tops      # measured on this GPU by the resident-tile tcgen05 kind::i8 probe
            intensity = 2.0 * c["macs"] / max(c["bytes"], 1)
            ridge = int8_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)
            secs = per_step[top] / 1e3
            if c["macs"] and intensity > ridge:
                ach = 2.0 * c["macs"] / secs / 1e12
                roof = dict(bound="tensor", achieved=ach, peak=int8_peak, unit="TFLOP/s", frac=ach / int8_peak)
            else:
                ach = c["bytes"] / secs / 1e9
                roof = dict(bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"])
            traffic = NCU_DRAM_TRAFFIC_B65536[top] * batch / 65536 if fused_costs else None
            roof.update(traffic=traffic, traffic_source="ncu capture at batch 65536 (profiles/), scaled by batch" if traffic else None, kernel=f"{names[top]} -> {c['out']}", launch_ms=per_step[top], peak_source=peaks["source"] +
                        (" (int8 tensor peak measured in this run by zant_b200_measure_int8_peak)" if roof["bound"] == "tensor" else ""),
                        algorithmic_bytes=c["bytes"], macs=c["macs"])
        else:
            roof = dict(bound="hbm", achieved=None, peak=peaks["hbm_gbs"], unit="GB/s", frac=None, traffic=None,
                        kernel="fused plan: see step_share", peak_source=peaks["source"])
        per_kernel = None
        if fused_costs:
            per_kernel = []
            for i, c in enumerate(fused_costs):
                secs = per_step[i] / 1e3
                tens = 2.0 * c["macs"] / secs / 1e12
                gbs = c["bytes"] / secs / 1e9
                per_kernel.append(dict(kernel=names[i], ms=round(per_step[i], 5), tops=round(tens, 1), tops_frac=round(tens / int8_peak_tops, 4),
                                       gbs=round(gbs, 1), hbm_frac=round(gbs / peaks["hbm_gbs"], 4)))
        cpu = None if args.skip_cpu else cpu_reference_rate(batch, scales)
        line = dict(metric=METRIC, value=value, unit="images/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="int8",
                    data="synthetic",
                    config=dict(workload="small CNN int8 (QLinear form of the reference's example net), batch 65536 per GPU",
                                batch_per_gpu=batch, global_batch=batch * world, fused=not args.no_fuse,
                                l2="inputs larger than L2 (205 MB of float input per step)", calibration="256 seeded samples, FP32 plan on the GPU",
                                macs_per_image=MACS_PER_IMAGE, parallelism=f"sample-sharded x{world}, no collective"),
                    roofline=roof, int8_peak_tops=int8_peak_tops, bf16_tflops_measured=peaks["bf16_tflops"], per_kernel=per_kernel, step_share=shares, step_ms={f"{i}:{names[i]}": round(per_step[i], 5) for i in range(len(names))},
                    cpu_baseline=cpu,
                    e2e=dict(value=total_images / (ms_e2e / 1e3), unit="images/s", h2d_bytes_per_step=batch * 784 * 4,
                             d2h_bytes_per_step=batch * 10 * 4, ms_per_step=ms_e2e / args.steps, chunks=n_chunks,
                             how="plan.run on pinned host buffers, chunks alternate between two contexts (copy/compute overlap)"),
                    gpu_launches=int(launches) * world, clocks=clocks, arena_bytes=plan.arena_bytes, batch1_latency=latency)
        print(json.dumps(line), flush=True)
    plan.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
