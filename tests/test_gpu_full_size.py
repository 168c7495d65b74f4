"""Oracle parity at the sizes the benchmark configurations state.

Samples of a batch are independent, so the GPU runs the full-size workload and the oracle runs a few
of its samples (first, last, and the ones either side of a tile edge of every stage); every tensor of
the graph that the plan materialises is compared, not just the output, so that each kernel variant
the full size selects (row blocks on 416- and 208-wide planes, the 3->16 stem at 416, 112x112 1x1
tiles, width segments, the 65536-image fused chain) is checked where it is used."""
import numpy as np
import pytest

import graph_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(zb):
    from zant_b200 import models
    return models


def _materialised(zb, plan, graph):
    """(tensor id, array) for every activation tensor the plan keeps in its arena."""
    for tid, t in enumerate(graph.tensors):
        if t["data"] is not None:
            continue
        try:
            yield tid, plan.read_tensor(tid)
        except zb.ZantError as e:
            assert e.name == "Unsupported"          # interior of a fused chain: not materialised


def _same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    if a.dtype == np.float32:
        return np.array_equal(a.view(np.uint32), b.view(np.uint32))
    return np.array_equal(a, b)


def _fp32_rule(got, ref):
    """|gpu - ref| <= 1e-4 * max(|ref|, 1e-2 * max|ref|): the float-path tolerance."""
    return np.all(np.abs(got - ref) <= 1e-4 * np.maximum(np.abs(ref), 1e-2 * np.abs(ref).max()))


def test_cfg1_small_cnn_fp32_batch_4096(zb, ctx, oracle, models):
    batch = 4096
    g = models.small_cnn_fp32(batch)
    x = models.small_cnn_input(batch, 4096)
    plan = zb.Plan(ctx, g, fuse=False)
    got = plan.run(x)
    idx = [0, 2047, 4095]
    gs = models.small_cnn_fp32(len(idx))
    want = graph_oracle.run(oracle, gs, x[idx])
    assert _fp32_rule(got[idx], want[gs.output])
    checked = 0
    for tid, arr in _materialised(zb, plan, g):
        assert _same_bits(arr[idx], want[tid]), g.tensors[tid]["name"]
        checked += 1
    assert checked >= 12
    plan.close()


def test_cfg2_small_cnn_int8_batch_65536_fused(zb, ctx, oracle, models):
    batch = 65536
    scales = models.calibrate_on_gpu(ctx, models.small_cnn_fp32(256), models.small_cnn_input(256, models.DEFAULT_SEED + 1))
    g = models.small_cnn_int8(batch, act_scales=scales)
    x = models.small_cnn_input(batch, 65536)
    plan = zb.Plan(ctx, g, fuse=True)
    assert sum("Fused" in n for n in plan.step_names()) == 4
    got = plan.run(x)
    plan.close()
    # groups of 3 images (stage 1), 128 pool windows = 3.56 images (stage 2), 128-row tiles (fc1), 16-row tiles (fc2)
    idx = [0, 1, 2, 3, 4, 15, 16, 127, 128, 129, 32767, 32768, 65407, 65408, 65533, 65534, 65535]
    gs = models.small_cnn_int8(len(idx), act_scales=scales)
    want = graph_oracle.run(oracle, gs, x[idx])[gs.output]
    assert _same_bits(got[idx], want)
    assert len(np.unique(got)) > 50


@pytest.mark.parametrize("name,channels_last", [("3a", False), ("3a", True), ("3b", False), ("3c", False), ("3c", True), ("3d", False)])
def test_cfg3_qconv_sweep_batch_256(zb, ctx, oracle, models, name, channels_last):
    g, c = models.qconv_graph(name, channels_last=channels_last)
    assert c["N"] == 256
    plan = zb.Plan(ctx, g)
    got = plan.run(c["x"])
    plan.close()
    for i in (0, 1, 255):
        xi = c["x"][i:i + 1]
        if channels_last:
            xi = np.ascontiguousarray(xi.transpose(0, 3, 1, 2))
        want = oracle.qlinearconv(xi, c["x_scale"], 0, c["w"], c["w_scale"], None, c["y_scale"], 0, stride=c["stride"], pads=c["pads"],
                                  dilations=c["dilations"], group=c["group"])
        gi = got[i:i + 1].transpose(0, 3, 1, 2) if channels_last else got[i:i + 1]
        assert np.array_equal(gi, want), (name, i)


def test_cfg4_mobilenetv2_int8_224(zb, ctx, oracle, models):
    batch = 2
    g = models.mobilenetv2_int8(batch)
    x = models.mobilenetv2_input(batch)
    want = graph_oracle.run(oracle, g, x)
    for fuse in (True, False):
        plan = zb.Plan(ctx, g, fuse=fuse)
        got = plan.run(x)
        assert _same_bits(got, want[g.output]), fuse
        checked = 0
        for tid, arr in _materialised(zb, plan, g):
            assert _same_bits(arr, want[tid]), (fuse, g.tensors[tid]["name"], g.tensors[tid]["shape"])
            checked += 1
        assert checked >= 20
        plan.close()
    assert len(np.unique(want[g.output])) > 20


def test_cfg5_tiny_yolo_fp32_416(zb, ctx, oracle, models):
    g = models.tiny_yolo_fp32(1)
    x = models.tiny_yolo_input(1)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g)
    got = plan.run(x)
    assert _fp32_rule(got, want[g.output])
    assert _fp32_rule(plan.read_tensor(g.meta["head13"]), want[g.meta["head13"]])
    for tid, arr in _materialised(zb, plan, g):
        assert _same_bits(arr, want[tid]), (g.tensors[tid]["name"], g.tensors[tid]["shape"])
    plan.close()


def test_cfg5_tiny_yolo_int8_416(zb, ctx, oracle, models):
    f = models.tiny_yolo_fp32(1)
    x = models.tiny_yolo_input(1)
    scales = models.activation_scales_on_gpu(ctx, f, x)
    q = models.tiny_yolo_int8(f, scales)
    want = graph_oracle.run(oracle, q, x)
    for fuse in (True, False):
        plan = zb.Plan(ctx, q, fuse=fuse)
        got = plan.run(x)
        assert _same_bits(got, want[q.output]), fuse
        checked = 0
        for tid, arr in _materialised(zb, plan, q):
            assert _same_bits(arr, want[tid]), (fuse, q.tensors[tid]["name"], q.tensors[tid]["shape"])
            checked += 1
        assert checked >= 10
        plan.close()
    assert len(np.unique(want[q.meta["head13"]])) > 20
