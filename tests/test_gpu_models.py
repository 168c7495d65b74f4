"""Whole-graph parity: the plan (the run-time form of a generated predict()) against the oracle
executing the same graph node by node; then size-independent properties at the full batch."""
import numpy as np
import pytest

import graph_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(zb):
    from zant_b200 import models
    return models


@pytest.fixture(scope="module")
def scales(zb, ctx, models):
    fp32 = models.small_cnn_fp32(256)
    return models.calibrate_on_gpu(ctx, fp32, models.small_cnn_input(256, models.DEFAULT_SEED + 1))


@pytest.mark.parametrize("batch", [1, 5])
@pytest.mark.parametrize("fuse", [False, True])
def test_small_cnn_fp32_matches_oracle(zb, ctx, oracle, models, batch, fuse):
    g = models.small_cnn_fp32(batch)
    x = models.small_cnn_input(batch, 77)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g, fuse=fuse)
    got = plan.run(x)
    ref = want[g.output]
    # FP32 contract: |gpu - ref| <= 1e-4 * max(|ref|, 1e-2 * max|ref|); the exact kernels are in fact bit-identical.
    tol = 1e-4 * np.maximum(np.abs(ref), 1e-2 * np.abs(ref).max())
    assert np.all(np.abs(got - ref) <= tol)
    if not fuse:
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
        for name in ("conv1", "pool1", "conv2", "pool2", "fc1", "relu3"):
            tid = g.id_of(name)
            assert np.array_equal(plan.read_tensor(tid).view(np.uint32), want[tid].view(np.uint32)), name
    plan.close()


def test_calibration_agrees_with_oracle(zb, ctx, oracle, models, scales):
    fp32 = models.small_cnn_fp32(16)
    x = models.small_cnn_input(16, models.DEFAULT_SEED + 1)
    cpu = graph_oracle.calibrate(oracle, fp32, x)
    gpu = models.calibrate_on_gpu(ctx, fp32, x)
    assert cpu == gpu
    assert all(0 < v < 10 for v in scales.values())


@pytest.mark.parametrize("batch", [1, 9])
@pytest.mark.parametrize("fuse", [False, True])
def test_small_cnn_int8_bit_exact(zb, ctx, oracle, models, scales, batch, fuse):
    g = models.small_cnn_int8(batch, act_scales=scales)
    x = models.small_cnn_input(batch, 99)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g, fuse=fuse)
    got = plan.run(x)
    assert np.array_equal(got.view(np.uint32), want[g.output].view(np.uint32))
    if not fuse:
        for name in ("xq", "conv1", "pool1", "conv2", "pool2", "fc1", "fc2"):
            tid = g.id_of(name)
            assert np.array_equal(plan.read_tensor(tid), want[tid]), name
    # the quantized network is not degenerate: logits differ between samples and use many codes
    assert len(np.unique(want[g.id_of("fc2")])) > 4
    plan.close()


@pytest.mark.parametrize("amplitude", [(300, 3000, 20000, 500), (2000, 400000, 100000, 3000), (2000, 600000, 100000, 3000)])
def test_small_cnn_int8_with_biases_bit_exact(zb, ctx, oracle, models, scales, amplitude):
    """Non-zero int32 biases through the fused chain (conv1 adds them as the MMA's C operand, conv2 after the
    window max, the two matrix products in their epilogues): small ones and ones that saturate most outputs."""
    batch = 7
    g = models.small_cnn_int8(batch, act_scales=scales, bias_amplitude=amplitude)
    x = models.small_cnn_input(batch, 123)
    want = graph_oracle.run(oracle, g, x)
    for fuse in (True, False):
        plan = zb.Plan(ctx, g, fuse=fuse)
        got = plan.run(x)
        assert np.array_equal(got.view(np.uint32), want[g.output].view(np.uint32)), fuse
        if fuse:
            assert any("Fused" in n for n in plan.step_names())
        plan.close()
    if amplitude[1] <= 3000:      # the moderate biases leave the activations spread over many codes
        assert len(np.unique(want[g.id_of("pool2")])) > 16


@pytest.mark.parametrize("zp", [7, 128])
def test_small_cnn_int8_with_an_input_zero_point(zb, ctx, oracle, models, scales, zp):
    """uint8 input codes with a non-zero zero point through the fused chain: stage 1 quantises with explicit clamps (zero
    point 0 takes the conversion + saturating pack alone) and folds -zp * sum(w) into its bias."""
    batch = 9
    g = models.small_cnn_int8(batch, act_scales=scales, bias_amplitude=(100, 1000, 5000, 300))
    assert g.nodes[0]["op"] == "QuantizeLinear" and g.nodes[1]["op"] == "QLinearConv"
    g.nodes[0]["attrs"]["y_zp"] = zp
    g.nodes[1]["attrs"]["x_zp"] = zp
    x = models.small_cnn_input(batch, 321) - (0.25 if zp else 0.0)      # some inputs below zero: the lower clamp matters
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g, fuse=True)
    got = plan.run(x)
    assert any("Fused" in n for n in plan.step_names())
    assert np.array_equal(got.view(np.uint32), want[g.output].view(np.uint32))
    plan.close()
    assert len(np.unique(want[g.id_of("pool1")])) > 16


@pytest.mark.parametrize("n_classes,batch", [(1, 3), (3, 33), (8, 17), (9, 40)])
def test_small_cnn_int8_class_counts_and_ragged_batches(zb, ctx, oracle, models, scales, n_classes, batch):
    """The last fused kernel has one instantiation per block of eight classes, and the batch sizes here end in
    partly filled tiles of every stage (groups of 4 images, 128 pool windows, 128 and 16 rows)."""
    g = models.small_cnn_int8(batch, act_scales=scales, n_classes=n_classes, bias_amplitude=(100, 1000, 5000, 300))
    x = models.small_cnn_input(batch, 321)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g, fuse=True)
    assert any("Fused" in n for n in plan.step_names())
    got = plan.run(x)
    assert got.shape == (batch, n_classes)
    assert np.array_equal(got.view(np.uint32), want[g.output].view(np.uint32))
    plan.close()


def test_int8_close_to_fp32(zb, ctx, models, scales):
    """Sanity of the quantisation itself: int8 logits track the FP32 logits."""
    batch = 64
    x = models.small_cnn_input(batch, 5)
    pf = zb.Plan(ctx, models.small_cnn_fp32(batch), fuse=False)
    pq = zb.Plan(ctx, models.small_cnn_int8(batch, act_scales=scales), fuse=True)
    yf, yq = pf.run(x), pq.run(x)
    pf.close(); pq.close()
    assert np.abs(yf - yq).max() <= 0.15 * np.abs(yf).max()
    assert (yf.argmax(1) == yq.argmax(1)).mean() > 0.8


def test_full_batch_properties(zb, ctx, oracle, models, scales):
    """Batch 4096: (1) fused and unfused plans agree bit for bit, (2) samples are independent —
    any slice of the big batch equals a small-batch run of the same samples, which the oracle
    checks on 4 of them, (3) sharding the batch over ranks reproduces the unsharded result."""
    batch = 4096
    x = models.small_cnn_input(batch, 1234)
    g = models.small_cnn_int8(batch, act_scales=scales)
    p0, p1 = zb.Plan(ctx, g, fuse=False), zb.Plan(ctx, g, fuse=True)
    y0, y1 = p0.run(x), p1.run(x)
    p0.close(); p1.close()
    assert np.array_equal(y0, y1)
    idx = [0, 1777, 4094, 4095]
    gs = models.small_cnn_int8(len(idx), act_scales=scales)
    want = graph_oracle.run(oracle, gs, x[idx])[gs.output]
    assert np.array_equal(y1[idx], want)
    world = 3
    parts = []
    for r in range(world):
        b, c = zb.shard_range(batch, world, r)
        ps = zb.Plan(ctx, models.small_cnn_int8(c, act_scales=scales), fuse=True)
        parts.append(ps.run(x[b:b + c]))
        ps.close()
    assert np.array_equal(np.concatenate(parts), y1)


def test_plan_accepts_device_buffers(zb, ctx, models, scales):
    torch = pytest.importorskip("torch")
    batch = 32
    g = models.small_cnn_int8(batch, act_scales=scales)
    x = models.small_cnn_input(batch, 8)
    plan = zb.Plan(ctx, g, fuse=True)
    want = plan.run(x)
    xd = torch.from_numpy(x).cuda()
    yd = torch.empty((batch, 10), dtype=torch.float32, device="cuda")
    plan.run(xd, out=yd)
    ctx.synchronize()
    assert np.array_equal(yd.cpu().numpy(), want)
    assert plan.launches_per_run > 0
    plan.close()


def test_plan_rejects_bad_graphs(zb, ctx, models):
    g = models.small_cnn_fp32(2)
    g.tensors[g.id_of("conv1")]["shape"] = [2, 32, 25, 26]
    with pytest.raises(zb.ZantError) as e:
        zb.Plan(ctx, g)
    assert e.value.name == "InvalidDimensions"


@pytest.mark.parametrize("name,batch", [("3a", 2), ("3b", 4), ("3c", 2), ("3d", 2)])
def test_qconv_sweep_reduced_batch(zb, ctx, oracle, models, name, batch):
    """Configuration 3 shapes at a batch the oracle finishes in seconds: bit-exact."""
    c = models.qconv_case(name, batch=batch)
    kw = dict(stride=c["stride"], pads=c["pads"], dilations=c["dilations"], group=c["group"])
    got = ctx.qlinearconv(c["x"], c["x_scale"], 0, c["w"], c["w_scale"], None, c["y_scale"], 0, **kw)
    want = oracle.qlinearconv(c["x"], c["x_scale"], 0, c["w"], c["w_scale"], None, c["y_scale"], 0, **kw)
    assert np.array_equal(got, want)


# ------------------------------------------------------------------------------------------------
# Configuration 4 (MobileNetV2-style int8) and configuration 5 (Tiny-YOLOv3-style FP32 + int8) at a
# resolution the oracle finishes in seconds; the layer tables, channel counts and operator mix are
# those of the full-size networks.
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("batch,res", [(1, 96), (2, 64)])
def test_mobilenetv2_int8_bit_exact(zb, ctx, oracle, models, batch, res):
    g = models.mobilenetv2_int8(batch, res=res, classes=1000)
    x = models.mobilenetv2_input(batch, res)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g, fuse=True)
    got = plan.run(x)
    assert np.array_equal(got.view(np.uint32), want[g.output].view(np.uint32))
    names = plan.step_names()
    # pointwise convs: the filters-on-lanes kernel; the smallest planes: im2col + GEMM; depthwise: its own kernel
    assert "QLinearConv(tc-pointwise)" in names and "QLinearConv(tc)" in names and "QLinearConv(depthwise)" in names
    # spot-check intermediates of each operator kind: depthwise conv, residual add, global pool
    kinds = {}
    for n in g.nodes:
        key = n["op"] + ("dw" if n["attrs"].get("group", 1) > 1 else "")
        kinds.setdefault(key, n["outputs"][0])
    for key, tid in kinds.items():
        if g.tensors[tid]["data"] is None and tid != g.output:
            assert np.array_equal(plan.read_tensor(tid), want[tid]), key
    assert len(np.unique(want[g.output])) > 20
    plan.close()


def test_tiny_yolo_fp32_matches_oracle(zb, ctx, oracle, models):
    g = models.tiny_yolo_fp32(1, res=96)
    x = models.tiny_yolo_input(1, 96)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g, fuse=True)
    got = plan.run(x)
    for name, ref, out in (("head26", want[g.output], got), ("head13", want[g.meta["head13"]], plan.read_tensor(g.meta["head13"]))):
        tol = 1e-4 * np.maximum(np.abs(ref), 1e-2 * np.abs(ref).max())     # the FP32 contract of the float path
        assert np.all(np.abs(out - ref) <= tol), name
        assert np.array_equal(out.view(np.uint32), ref.view(np.uint32)), name  # exact kernels: in fact bit-identical
    plan.close()


def test_tiny_yolo_int8_bit_exact(zb, ctx, oracle, models):
    f = models.tiny_yolo_fp32(2, res=64)
    x = models.tiny_yolo_input(2, 64)
    scales = models.activation_scales_on_gpu(ctx, f, x)
    q = models.tiny_yolo_int8(f, scales)
    want = graph_oracle.run(oracle, q, x)
    plan = zb.Plan(ctx, q, fuse=True)
    got = plan.run(x)
    assert np.array_equal(got.view(np.uint32), want[q.output].view(np.uint32))
    assert np.array_equal(plan.read_tensor(q.meta["head13"]), want[q.meta["head13"]])
    assert any(n.startswith("QLinearConv(tc-implicit)") for n in plan.step_names())
    # the quantized detector tracks the FP32 one
    ref = graph_oracle.run(oracle, f, x)[f.output]
    assert np.abs(got - ref).max() <= 0.2 * np.abs(ref).max()
    plan.close()


def test_full_size_graphs_plan_and_run(zb, ctx, models):
    """Full-size configurations 4 and 5 (224x224 and 416x416): the plans build, run and are
    deterministic; sample 0 of a batch of 2 equals a batch-1 run (samples are independent)."""
    g2, g1 = models.mobilenetv2_int8(2), models.mobilenetv2_int8(1)
    x = models.mobilenetv2_input(2)
    p2, p1 = zb.Plan(ctx, g2), zb.Plan(ctx, g1)
    y2, y2b, y1 = p2.run(x), p2.run(x), p1.run(x[:1])
    p2.close(); p1.close()
    assert y2.shape == (2, 1000) and np.array_equal(y2, y2b) and np.array_equal(y2[:1], y1)
    f = models.tiny_yolo_fp32(1)
    pf = zb.Plan(ctx, f)
    yf = pf.run(models.tiny_yolo_input(1))
    assert yf.shape == (1, 255, 26, 26) and np.isfinite(yf).all()
    assert pf.read_tensor(f.meta["head13"]).shape == (1, 255, 13, 13)
    pf.close()


def test_plan_graph_replay_matches_separate_launches(zb, ctx, models, scales):
    """One captured CUDA graph per run: same bytes as the step-by-step run, host and device buffers."""
    import torch
    for g, x in ((models.small_cnn_int8(4, act_scales=scales), models.small_cnn_input(4)),
                 (models.mobilenetv2_int8(1, res=96, classes=1000), models.mobilenetv2_input(1, 96))):
        plan = zb.Plan(ctx, g, fuse=True)
        want = plan.run(x).copy()
        plan.use_graph(True)
        before = ctx.launch_count()
        got = plan.run(x)
        assert ctx.launch_count() - before == plan.launches_per_run
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        xd = torch.from_numpy(x).cuda()
        yd = torch.empty(tuple(want.shape), dtype=torch.float32, device="cuda")
        plan.run(xd, out=yd)
        ctx.synchronize()
        assert np.array_equal(yd.cpu().numpy().view(np.uint32), want.view(np.uint32))
        # a second input through the same graph
        x2 = np.ascontiguousarray(x[::-1]) if x.shape[0] > 1 else (255 - x if x.dtype == np.uint8 else 1.0 - x)
        plan.use_graph(False)
        want2 = plan.run(x2).copy()
        plan.use_graph(True)
        assert np.array_equal(plan.run(x2).view(np.uint32), want2.view(np.uint32))
        plan.close()
