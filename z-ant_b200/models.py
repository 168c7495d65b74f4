"""Seeded synthetic graphs for the benchmark configurations.

Everything here is workload synthesis: random He-normal weights and uniform inputs from a seeded
numpy generator (there are no datasets or checkpoints), frozen into `Graph` objects that a `Plan`
executes.  Shapes follow the reference's example network (src/main.zig:41-305 in the Z-Ant tree:
Conv 1->32 3x3, ReLU, MaxPool 2, Conv 32->64 3x3, ReLU, MaxPool 2, Flatten 1600, Dense 512, ReLU,
Dense 10) on MNIST-shaped 1x28x28 inputs.
"""
import numpy as np

from . import F32, I8, I32, U8, Graph, Plan, conv_output_shape, get_pooling_output_shape

DEFAULT_SEED = 0x5A4E54


def he_normal(rng, shape, fan_in):
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def small_cnn_input(batch, seed=DEFAULT_SEED + 1):
    """[batch,1,28,28] float32, uniform in [0,1)."""
    return np.random.default_rng(seed).random((batch, 1, 28, 28), dtype=np.float32)


def small_cnn_weights(seed=DEFAULT_SEED):
    rng = np.random.default_rng(seed)
    return dict(
        w1=he_normal(rng, (32, 1, 3, 3), 9), b1=np.zeros(32, np.float32),
        w2=he_normal(rng, (64, 32, 3, 3), 288), b2=np.zeros(64, np.float32),
        w3=he_normal(rng, (1600, 512), 1600), b3=np.zeros(512, np.float32),
        w4=he_normal(rng, (512, 10), 512), b4=np.zeros(10, np.float32),
    )


POOL = dict(kernel_shape=(2, 2), strides=(2, 2), dilations=(1, 1), pads=(0, 0, 0, 0), auto_pad="NOTSET")
CONV = dict(strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1, auto_pad="NOTSET")


def small_cnn_fp32(batch, seed=DEFAULT_SEED):
    """Configuration 1: the FP32 example CNN, node for node as the generator would emit it
    (Conv with bias, Relu, MaxPool, Reshape, MatMul + Add for the dense layers)."""
    w = small_cnn_weights(seed)
    g = Graph("small_cnn_fp32")
    x = g.tensor("x", F32, (batch, 1, 28, 28))
    c1s = conv_output_shape((batch, 1, 28, 28), (32, 1, 3, 3), (1, 1), (0, 0, 0, 0), (1, 1), "NOTSET")
    c1 = g.tensor("conv1", F32, c1s); r1 = g.tensor("relu1", F32, c1s)
    p1s = get_pooling_output_shape(c1s, (2, 2), (2, 2)); p1 = g.tensor("pool1", F32, p1s)
    c2s = conv_output_shape(p1s, (64, 32, 3, 3), (1, 1), (0, 0, 0, 0), (1, 1), "NOTSET")
    c2 = g.tensor("conv2", F32, c2s); r2 = g.tensor("relu2", F32, c2s)
    p2s = get_pooling_output_shape(c2s, (2, 2), (2, 2)); p2 = g.tensor("pool2", F32, p2s)
    fl = g.tensor("flat", F32, (batch, 1600))
    m3 = g.tensor("fc1_mm", F32, (batch, 512)); a3 = g.tensor("fc1", F32, (batch, 512)); r3 = g.tensor("relu3", F32, (batch, 512))
    m4 = g.tensor("fc2_mm", F32, (batch, 10)); a4 = g.tensor("logits", F32, (batch, 10))
    W1 = g.tensor("W1", F32, (32, 1, 3, 3), w["w1"]); B1 = g.tensor("B1", F32, (32,), w["b1"])
    W2 = g.tensor("W2", F32, (64, 32, 3, 3), w["w2"]); B2 = g.tensor("B2", F32, (64,), w["b2"])
    W3 = g.tensor("W3", F32, (1600, 512), w["w3"]); B3 = g.tensor("B3", F32, (512,), w["b3"])
    W4 = g.tensor("W4", F32, (512, 10), w["w4"]); B4 = g.tensor("B4", F32, (10,), w["b4"])
    g.node("Conv", [x, W1, B1], [c1], **CONV)
    g.node("Relu", [c1], [r1])
    g.node("MaxPool", [r1], [p1], **POOL)
    g.node("Conv", [p1, W2, B2], [c2], **CONV)
    g.node("Relu", [c2], [r2])
    g.node("MaxPool", [r2], [p2], **POOL)
    g.node("Reshape", [p2], [fl])
    g.node("MatMul", [fl, W3], [m3])
    g.node("Add", [m3, B3], [a3])
    g.node("Relu", [a3], [r3])
    g.node("MatMul", [r3, W4], [m4])
    g.node("Add", [m4, B4], [a4])
    g.input, g.output = x, a4
    g.meta = dict(macs_per_image=194688 + 2230272 + 819200 + 5120, calib_tensors=["relu1", "relu2", "relu3", "logits"])
    return g


def act_scales_from(acts):
    """Per-tensor symmetric activation scales max|a| / 127 (zero point 0)."""
    out = {}
    for name, a in acts.items():
        m = np.float32(np.abs(a).max())
        out[name] = float(np.float32(m / np.float32(127.0))) if m > 0 else 1.0
    return out


def calibrate_on_gpu(ctx, fp32_graph, calib_x):
    """Runs the FP32 graph on the calibration batch through a Plan and reads the activation ranges."""
    plan = Plan(ctx, fp32_graph, fuse=False)
    try:
        plan.run(calib_x)
        acts = {n: plan.read_tensor(n) for n in fp32_graph.meta["calib_tensors"]}
    finally:
        plan.close()
    return act_scales_from(acts)


def quantize_weights(w, axis):
    """Symmetric int8 per-output-channel: s[k] = max|w[k]| / 127, w_q = rne(w / s[k])."""
    red = tuple(i for i in range(w.ndim) if i != axis)
    m = np.abs(w).max(axis=red).astype(np.float32)
    s = (m / np.float32(127.0)).astype(np.float32)
    s[s == 0] = np.float32(1.0)
    shape = [1] * w.ndim
    shape[axis] = -1
    q = np.rint(w / s.reshape(shape)).clip(-127, 127).astype(np.int8)
    return q, s


def small_cnn_int8(batch, seed=DEFAULT_SEED, act_scales=None):
    """Configuration 2: the same CNN in QLinear form.  QuantizeLinear(1/255, uint8) on the input,
    QLinearConv / QLinearMatMul with int8 per-output-channel weights and int32 zero biases, int8
    activations with zero point 0 (scales from `act_scales`), ReLU and MaxPool on the int8 codes,
    DequantizeLinear at the end."""
    if act_scales is None:
        act_scales = dict(relu1=0.02, relu2=0.05, relu3=0.05, logits=0.1)
    w = small_cnn_weights(seed)
    q1, s1 = quantize_weights(w["w1"], 0)
    q2, s2 = quantize_weights(w["w2"], 0)
    q3, s3 = quantize_weights(w["w3"], 1)
    q4, s4 = quantize_weights(w["w4"], 1)
    sx = float(np.float32(1.0) / np.float32(255.0))
    a1, a2, a3, a4 = (act_scales[k] for k in ("relu1", "relu2", "relu3", "logits"))
    g = Graph("small_cnn_int8")
    x = g.tensor("x", F32, (batch, 1, 28, 28))
    xq = g.tensor("xq", U8, (batch, 1, 28, 28))
    c1 = g.tensor("conv1", I8, (batch, 32, 26, 26)); r1 = g.tensor("relu1", I8, (batch, 32, 26, 26)); p1 = g.tensor("pool1", I8, (batch, 32, 13, 13))
    c2 = g.tensor("conv2", I8, (batch, 64, 11, 11)); r2 = g.tensor("relu2", I8, (batch, 64, 11, 11)); p2 = g.tensor("pool2", I8, (batch, 64, 5, 5))
    fl = g.tensor("flat", I8, (batch, 1600))
    f1 = g.tensor("fc1", I8, (batch, 512)); r3 = g.tensor("relu3", I8, (batch, 512))
    f2 = g.tensor("fc2", I8, (batch, 10)); y = g.tensor("logits", F32, (batch, 10))
    W1 = g.tensor("W1", I8, (32, 1, 3, 3), q1); S1 = g.tensor("S1", F32, (32,), s1); B1 = g.tensor("B1", I32, (32,), np.zeros(32, np.int32))
    W2 = g.tensor("W2", I8, (64, 32, 3, 3), q2); S2 = g.tensor("S2", F32, (64,), s2); B2 = g.tensor("B2", I32, (64,), np.zeros(64, np.int32))
    W3 = g.tensor("W3", I8, (1600, 512), q3); S3 = g.tensor("S3", F32, (512,), s3); B3 = g.tensor("B3", I32, (512,), np.zeros(512, np.int32))
    W4 = g.tensor("W4", I8, (512, 10), q4); S4 = g.tensor("S4", F32, (10,), s4); B4 = g.tensor("B4", I32, (10,), np.zeros(10, np.int32))
    qconv = dict(strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1, auto_pad="NOTSET")
    g.node("QuantizeLinear", [x], [xq], y_scale=sx, y_zp=0)
    g.node("QLinearConv", [xq, W1, S1, -1, B1], [c1], x_scale=sx, x_zp=0, y_scale=a1, y_zp=0, **qconv)
    g.node("Relu", [c1], [r1], x_scale=a1, x_zp=0, y_scale=a1, y_zp=0)
    g.node("MaxPool", [r1], [p1], **POOL)
    g.node("QLinearConv", [p1, W2, S2, -1, B2], [c2], x_scale=a1, x_zp=0, y_scale=a2, y_zp=0, **qconv)
    g.node("Relu", [c2], [r2], x_scale=a2, x_zp=0, y_scale=a2, y_zp=0)
    g.node("MaxPool", [r2], [p2], **POOL)
    g.node("Reshape", [p2], [fl])
    g.node("QLinearMatMul", [fl, W3, S3, -1, B3], [f1], x_scale=a2, x_zp=0, y_scale=a3, y_zp=0)
    g.node("Relu", [f1], [r3], x_scale=a3, x_zp=0, y_scale=a3, y_zp=0)
    g.node("QLinearMatMul", [r3, W4, S4, -1, B4], [f2], x_scale=a3, x_zp=0, y_scale=a4, y_zp=0)
    g.node("DequantizeLinear", [f2], [y], x_scale=a4, x_zp=0)
    g.input, g.output = x, y
    g.meta = dict(macs_per_image=194688 + 2230272 + 819200 + 5120, act_scales=dict(act_scales))
    return g


# ------------------------------------------------------------------------------------------------
# Configuration 3: stand-alone int8 QLinearConv sweep (NCHW at the boundary), every scale 0.02,
# every zero point 0, activations uniform in [-128,127], weights uniform in [-127,127].
# ------------------------------------------------------------------------------------------------
QCONV_SWEEP = {
    "3a": dict(N=256, C=64, H=56, W=56, K=64, k=3, s=1, p=1, group=1),
    "3b": dict(N=256, C=256, H=14, W=14, K=512, k=3, s=2, p=1, group=1),
    "3c": dict(N=256, C=256, H=56, W=56, K=64, k=1, s=1, p=0, group=1),
    "3d": dict(N=256, C=128, H=56, W=56, K=128, k=3, s=1, p=1, group=128),
}


def qconv_case(name, batch=None, seed=DEFAULT_SEED):
    c = dict(QCONV_SWEEP[name])
    if batch is not None:
        c["N"] = batch
    rng = np.random.default_rng(seed + sum(ord(ch) for ch in name))
    x = rng.integers(-128, 128, (c["N"], c["C"], c["H"], c["W"]), dtype=np.int8)
    w = rng.integers(-127, 128, (c["K"], c["C"] // c["group"], c["k"], c["k"]), dtype=np.int8)
    c.update(x=x, w=w, x_scale=0.02, w_scale=np.array([0.02], np.float32), y_scale=0.02,
             stride=(c["s"], c["s"]), pads=(c["p"],) * 4, dilations=(1, 1))
    oh = (c["H"] + 2 * c["p"] - c["k"]) // c["s"] + 1
    c["macs"] = c["N"] * c["K"] * oh * oh * (c["C"] // c["group"]) * c["k"] * c["k"]
    c["bytes"] = x.size + w.size + c["N"] * c["K"] * oh * oh
    return c
