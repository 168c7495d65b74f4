"""Generic epilogue fusion in the plan: QLinearConv -> [Relu | LeakyRelu | Clip] -> [MaxPool 2x2 / 2] as one step.

The generator emits one call per node (src/codeGen/predict.zig:73-92); the plan folds the activation into the producer's
epilogue (a flag, or a 256-entry table on the finished codes) and, where the implicit-GEMM kernel's tiling allows, the
pool too.  Every case is compared bit for bit with the oracle running the graph node by node, and with the unfused plan."""
import numpy as np
import pytest

import graph_oracle

pytestmark = pytest.mark.gpu
F32, I8, U8, I32 = 0, 1, 2, 3


def chain_graph(zb, N, C, H, W, M, k, pad, act, pool, ydt=I8, xdt=I8, seed=0, y_zp=0, extra_consumer=False):
    """x -> QLinearConv -> act -> MaxPool (each optional after the convolution)."""
    rng = np.random.default_rng(seed + C + M + H)
    g = zb.Graph("chain")
    x = g.tensor("x", xdt, (N, C, H, W))
    w = g.tensor("w", I8, (M, C, k, k), rng.integers(-127, 128, (M, C, k, k), dtype=np.int8))
    ws = g.tensor("ws", F32, (M,), (rng.random(M, dtype=np.float32) * 0.01 + 0.002).astype(np.float32))
    b = g.tensor("b", I32, (M,), rng.integers(-500, 500, M).astype(np.int32))
    OH, OW = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    s_conv = float(np.float32(0.02 * np.sqrt(C * k * k) * 0.35))
    c = g.tensor("conv", ydt, (N, M, OH, OW))
    g.node("QLinearConv", [x, w, ws, -1, b], [c], x_scale=0.02, x_zp=0 if xdt == I8 else 128, y_scale=s_conv, y_zp=y_zp,
           strides=(1, 1), pads=(pad,) * 4, dilations=(1, 1), group=1, auto_pad="NOTSET")
    cur = c
    if act is not None:
        a = g.tensor("act", ydt, (N, M, OH, OW))
        if act == "relu":
            g.node("Relu", [cur], [a], x_scale=s_conv, x_zp=y_zp, y_scale=s_conv, y_zp=y_zp)
        elif act == "relu_rescale":
            g.node("Relu", [cur], [a], x_scale=s_conv, x_zp=y_zp, y_scale=s_conv * 0.7, y_zp=y_zp)
        elif act == "leaky":
            g.node("LeakyRelu", [cur], [a], alpha=0.1, x_scale=s_conv, x_zp=y_zp, y_scale=s_conv * 0.8, y_zp=y_zp)
        else:
            g.node("Clip", [cur], [a], alpha=0.0, beta=6.0, x_scale=s_conv, x_zp=y_zp, y_scale=s_conv, y_zp=y_zp)
        cur = a
    if pool:
        p = g.tensor("pool", ydt, (N, M, OH // 2, OW // 2))
        g.node("MaxPool", [cur], [p], kernel_shape=(2, 2), strides=(2, 2), dilations=(1, 1), pads=(0, 0, 0, 0), auto_pad="NOTSET")
        cur = p
    if extra_consumer:
        # a second reader of the convolution's own output: it must stay materialised, nothing may be fused behind it
        e = g.tensor("extra", ydt, (N, M, OH, OW))
        g.node("Relu", [c], [e], x_scale=s_conv, x_zp=y_zp, y_scale=s_conv, y_zp=y_zp)
    g.input, g.output = x, cur
    xin = rng.integers(0, 256, (N, C, H, W), dtype=np.uint8) if xdt == U8 else rng.integers(-128, 128, (N, C, H, W), dtype=np.int8)
    return g, xin


CASES = [
    # N  C   H    W   M  k pad act            pool  ydt  expect (substring of the fused step's name)
    (2, 16, 28, 28, 32, 3, 1, "leaky", True, I8, "tc-implicit)+ActivationLut+MaxPool"),      # BH = 4
    (2, 16, 40, 40, 16, 3, 1, "leaky", True, I8, "tc-implicit)+ActivationLut+MaxPool"),      # BH = 3 -> 2
    (1, 32, 52, 52, 64, 3, 1, "relu", True, I8, "tc-implicit)+Relu+MaxPool"),                # BH = 2
    (1, 16, 104, 104, 32, 3, 1, "leaky", True, I8, "tc-implicit)+ActivationLut+MaxPool"),    # single-row blocks in pairs
    (1, 16, 208, 208, 16, 3, 1, "leaky", True, I8, "tc-implicit)+ActivationLut+MaxPool"),    # two column segments
    (1, 16, 29, 32, 16, 3, 0, "leaky", True, I8, "+MaxPool"),                                # 27 x 30 output: the last row is dropped
    (2, 16, 32, 28, 16, 3, 0, "clip", True, I8, "+ActivationLut+MaxPool"),                   # no padding: 30 x 26 output, pooled 15 x 13
    (1, 16, 56, 56, 32, 3, 1, "leaky", True, U8, "+ActivationLut+MaxPool"),                  # unsigned codes: unsigned maximum
    (1, 16, 104, 104, 128, 3, 1, None, True, I8, "tc-implicit)+MaxPool"),                    # pool alone, two filter tiles
    (2, 16, 28, 28, 32, 3, 1, "relu_rescale", False, I8, "+ActivationLut"),                  # activation alone (table)
    (2, 64, 28, 28, 32, 1, 0, "leaky", True, I8, "tc-pointwise)+ActivationLut"),             # 1x1, 32 filters (four pixel groups on the lanes): table fused, pool stays a step
    (2, 64, 28, 28, 96, 1, 0, "leaky", True, I8, "tc-pointwise)+ActivationLut"),             # 1x1, 96 filters: the filters-on-lanes kernel with the table
    (2, 3, 64, 64, 16, 3, 1, "leaky", True, I8, "tc-stem)+ActivationLut"),                   # stem (patches in shared memory): table fused, pool separate
    (2, 4, 64, 64, 16, 3, 1, "leaky", True, I8, "small-c)+ActivationLut"),                   # four channels: warp-level stem kernel
    (2, 16, 13, 13, 32, 3, 1, "leaky", False, I8, "+ActivationLut"),                         # im2col path (odd width)
    (1, 8, 9, 9, 8, 3, 1, "leaky", True, I8, "QLinearConv+ActivationLut"),                   # generic kernel
]


@pytest.mark.parametrize("case", CASES, ids=[f"chain{i}" for i in range(len(CASES))])
def test_conv_activation_pool_groups_are_bit_exact(zb, ctx, oracle, case):
    N, C, H, W, M, k, pad, act, pool, ydt, expect = case
    g, x = chain_graph(zb, N, C, H, W, M, k, pad, act, pool, ydt=ydt, y_zp=0 if ydt == I8 else 30)
    want = graph_oracle.run(oracle, g, x)[g.output]
    fused = zb.Plan(ctx, g, fuse=True)
    names = fused.step_names()
    got = fused.run(x)
    fused.close()
    plain = zb.Plan(ctx, g, fuse=False)
    n_plain = len(plain.step_names())
    got_plain = plain.run(x)
    plain.close()
    assert np.array_equal(got_plain, want)
    assert np.array_equal(got, want), names
    assert any(expect in n for n in names), names
    assert len(names) < n_plain
    if "+MaxPool" in expect:
        assert len(names) == 1
    assert len(np.unique(want)) > 8


def test_depthwise_and_uint8_input_groups(zb, ctx, oracle):
    """Depthwise kernel with a table behind it, and a uint8 input with a non-zero zero point in front of a fused group."""
    rng = np.random.default_rng(3)
    g = zb.Graph("dw")
    C = 32
    x = g.tensor("x", I8, (2, C, 28, 28))
    w = g.tensor("w", I8, (C, 1, 3, 3), rng.integers(-127, 128, (C, 1, 3, 3), dtype=np.int8))
    ws = g.tensor("ws", F32, (C,), (rng.random(C, dtype=np.float32) * 0.01 + 0.002).astype(np.float32))
    c = g.tensor("conv", I8, (2, C, 28, 28)); a = g.tensor("act", I8, (2, C, 28, 28))
    g.node("QLinearConv", [x, w, ws, -1, -1], [c], x_scale=0.02, x_zp=0, y_scale=0.05, y_zp=0, strides=(1, 1), pads=(1, 1, 1, 1), dilations=(1, 1),
           group=C, auto_pad="NOTSET")
    g.node("LeakyRelu", [c], [a], alpha=0.1, x_scale=0.05, x_zp=0, y_scale=0.04, y_zp=0)
    g.input, g.output = x, a
    xin = rng.integers(-128, 128, (2, C, 28, 28), dtype=np.int8)
    want = graph_oracle.run(oracle, g, xin)[g.output]
    plan = zb.Plan(ctx, g)
    assert plan.step_names() == ["QLinearConv(depthwise)+ActivationLut"]
    assert np.array_equal(plan.run(xin), want)
    plan.close()
    g2, x2 = chain_graph(zb, 2, 16, 52, 52, 32, 3, 1, "leaky", True, xdt=U8)
    want2 = graph_oracle.run(oracle, g2, x2)[g2.output]
    p2 = zb.Plan(ctx, g2)
    assert len(p2.step_names()) == 1 and np.array_equal(p2.run(x2), want2)
    p2.close()


def test_tensors_with_other_readers_are_not_fused_away(zb, ctx, oracle):
    """The convolution's output has a second consumer: it stays materialised and the group is left alone."""
    g, x = chain_graph(zb, 1, 16, 28, 28, 16, 3, 1, "leaky", True, extra_consumer=True)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(ctx, g)
    assert np.array_equal(plan.run(x), want[g.output])
    assert np.array_equal(plan.read_tensor("conv"), want[g.id_of("conv")])
    assert np.array_equal(plan.read_tensor("extra"), want[g.id_of("extra")])
    plan.close()


def test_fused_networks_have_no_standalone_activation_or_pool_behind_implicit_convs(zb, ctx):
    """Tiny-YOLOv3-style int8 at full size: no LeakyRelu table runs as its own step any more, and the pools behind
    the implicit-GEMM layers are gone; MobileNetV2-style: ReLU6 stays inside the producers."""
    from zant_b200 import models
    f = models.tiny_yolo_fp32(1)
    scales = models.activation_scales_on_gpu(ctx, models.tiny_yolo_fp32(1, res=96), models.tiny_yolo_input(1, 96))
    plan = zb.Plan(ctx, models.tiny_yolo_int8(f, scales))
    names = plan.step_names()
    plan.close()
    assert "ActivationLut" not in names
    assert sum(n == "MaxPool" for n in names) <= 3          # behind the stem kernel, the 26-wide layer (im2col path) and the stride-1 pool
    assert sum("+MaxPool" in n for n in names) >= 3
    pm = zb.Plan(ctx, models.mobilenetv2_int8(1))
    assert not any(n in ("Relu", "Clip", "ActivationLut") for n in pm.step_names())
    pm.close()
