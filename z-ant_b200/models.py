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


def small_cnn_int8(batch, seed=DEFAULT_SEED, act_scales=None, bias_amplitude=None, n_classes=10):
    """Configuration 2: the same CNN in QLinear form.  QuantizeLinear(1/255, uint8) on the input,
    QLinearConv / QLinearMatMul with int8 per-output-channel weights and int32 zero biases, int8
    activations with zero point 0 (scales from `act_scales`), ReLU and MaxPool on the int8 codes,
    DequantizeLinear at the end.  `bias_amplitude` (four integers, one per layer) replaces the zero
    biases of the configuration with seeded uniform int32 values in [-amplitude, amplitude] (tests);
    `n_classes` below 10 keeps the first columns of the last layer (tests)."""
    if act_scales is None:
        act_scales = dict(relu1=0.02, relu2=0.05, relu3=0.05, logits=0.1)
    w = small_cnn_weights(seed)
    q1, s1 = quantize_weights(w["w1"], 0)
    q2, s2 = quantize_weights(w["w2"], 0)
    q3, s3 = quantize_weights(w["w3"], 1)
    q4, s4 = quantize_weights(w["w4"][:, :n_classes], 1)
    sx = float(np.float32(1.0) / np.float32(255.0))
    a1, a2, a3, a4 = (act_scales[k] for k in ("relu1", "relu2", "relu3", "logits"))
    brng = np.random.default_rng(seed + 17)
    b1, b2, b3, b4 = (np.zeros(n, np.int32) if bias_amplitude is None else brng.integers(-amp, amp + 1, n).astype(np.int32)
                      for n, amp in zip((32, 64, 512, n_classes), bias_amplitude or (0, 0, 0, 0)))
    g = Graph("small_cnn_int8")
    x = g.tensor("x", F32, (batch, 1, 28, 28))
    xq = g.tensor("xq", U8, (batch, 1, 28, 28))
    c1 = g.tensor("conv1", I8, (batch, 32, 26, 26)); r1 = g.tensor("relu1", I8, (batch, 32, 26, 26)); p1 = g.tensor("pool1", I8, (batch, 32, 13, 13))
    c2 = g.tensor("conv2", I8, (batch, 64, 11, 11)); r2 = g.tensor("relu2", I8, (batch, 64, 11, 11)); p2 = g.tensor("pool2", I8, (batch, 64, 5, 5))
    fl = g.tensor("flat", I8, (batch, 1600))
    f1 = g.tensor("fc1", I8, (batch, 512)); r3 = g.tensor("relu3", I8, (batch, 512))
    f2 = g.tensor("fc2", I8, (batch, n_classes)); y = g.tensor("logits", F32, (batch, n_classes))
    W1 = g.tensor("W1", I8, (32, 1, 3, 3), q1); S1 = g.tensor("S1", F32, (32,), s1); B1 = g.tensor("B1", I32, (32,), b1)
    W2 = g.tensor("W2", I8, (64, 32, 3, 3), q2); S2 = g.tensor("S2", F32, (64,), s2); B2 = g.tensor("B2", I32, (64,), b2)
    W3 = g.tensor("W3", I8, (1600, 512), q3); S3 = g.tensor("S3", F32, (512,), s3); B3 = g.tensor("B3", I32, (512,), b3)
    W4 = g.tensor("W4", I8, (512, n_classes), q4); S4 = g.tensor("S4", F32, (n_classes,), s4); B4 = g.tensor("B4", I32, (n_classes,), b4)
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
    g.meta = dict(macs_per_image=194688 + 2230272 + 819200 + 512 * n_classes, act_scales=dict(act_scales))
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
    # single layers of the MobileNetV2-style network (ReLU6 fused), sized for profiler captures
    "4a": dict(N=64, C=16, H=112, W=112, K=96, k=1, s=1, p=0, group=1, act="relu6", y_scale=0.1),     # expansion 1x1, output-heavy
    "4b": dict(N=256, C=64, H=14, W=14, K=384, k=1, s=1, p=0, group=1, act="relu6", y_scale=0.1),     # 1x1 on 196-byte planes
    "4c": dict(N=128, C=384, H=14, W=14, K=384, k=3, s=1, p=1, group=384, act="relu6", y_scale=0.1),  # depthwise on 14 x 14
    "4d": dict(N=256, C=160, H=7, W=7, K=960, k=1, s=1, p=0, group=1, act="relu6", y_scale=0.1),      # 1x1 on 49-byte planes
    "4e": dict(N=64, C=3, H=224, W=224, K=32, k=3, s=2, p=1, group=1, act="relu6", y_scale=0.1),      # the stem: 3x3, stride 2, three channels
}


def qconv_case(name, batch=None, seed=DEFAULT_SEED):
    c = dict(QCONV_SWEEP[name])
    if batch is not None:
        c["N"] = batch
    rng = np.random.default_rng(seed + sum(ord(ch) for ch in name))
    x = rng.integers(-128, 128, (c["N"], c["C"], c["H"], c["W"]), dtype=np.int8)
    # the weights come from a generator of their own, so that they do not depend on the batch size
    wrng = np.random.default_rng(DEFAULT_SEED + 7919 + sum(ord(ch) for ch in name))
    w = wrng.integers(-127, 128, (c["K"], c["C"] // c["group"], c["k"], c["k"]), dtype=np.int8)
    c.update(x=x, w=w, x_scale=0.02, w_scale=np.array([0.02], np.float32), y_scale=c.get("y_scale", 0.02), act=c.get("act"),
             stride=(c["s"], c["s"]), pads=(c["p"],) * 4, dilations=(1, 1))
    oh = (c["H"] + 2 * c["p"] - c["k"]) // c["s"] + 1
    c["macs"] = c["N"] * c["K"] * oh * oh * (c["C"] // c["group"]) * c["k"] * c["k"]
    c["bytes"] = x.size + w.size + c["N"] * c["K"] * oh * oh
    return c


# ------------------------------------------------------------------------------------------------
# Small graph-building helpers for the larger synthetic networks below.
# ------------------------------------------------------------------------------------------------
def qconv_graph(name, batch=None, seed=DEFAULT_SEED, channels_last=False):
    """One sweep case as a one-node graph (int8 in and out); returns (graph, case).  NCHW tensors as the
    reference has them, or, with `channels_last`, the same values as [N,H,W,C] -> [N,OH,OW,K]
    (case["x"] is then the transposed input)."""
    c = qconv_case(name, batch, seed)
    g = Graph("qconv_" + name + ("_nhwc" if channels_last else ""))
    oh = (c["H"] + 2 * c["p"] - c["k"]) // c["s"] + 1
    if channels_last:
        c["x"] = np.ascontiguousarray(c["x"].transpose(0, 2, 3, 1))
    x = g.tensor("x", I8, c["x"].shape)
    w = g.tensor("w", I8, c["w"].shape, c["w"])
    ws = g.tensor("w_scale", F32, (1,), c["w_scale"])
    y = g.tensor("y", I8, (c["N"], oh, oh, c["K"]) if channels_last else (c["N"], c["K"], oh, oh))
    g.node("QLinearConv", [x, w, ws, -1, -1], [y], x_scale=c["x_scale"], x_zp=0, y_scale=c["y_scale"], y_zp=0,
           strides=c["stride"], pads=c["pads"], dilations=c["dilations"], group=c["group"], auto_pad="NOTSET", activation=c["act"],
           channels_last=1 if channels_last else 0)
    g.input, g.output = x, y
    return g, c


class _Builder:
    def __init__(self, name, seed):
        self.g = Graph(name)
        self.rng = np.random.default_rng(seed)
        self.n = 0

    def act(self, dtype, shape, name=None):
        self.n += 1
        return self.g.tensor(name or f"t{self.n}", dtype, shape)

    def const(self, dtype, arr, name=None):
        self.n += 1
        arr = np.asarray(arr)
        return self.g.tensor(name or f"c{self.n}", dtype, arr.shape, arr)

    def shape(self, tid):
        return list(self.g.tensors[tid]["shape"])


def _conv_out(h, k, s, p):
    return (h + 2 * p - k) // s + 1


# ------------------------------------------------------------------------------------------------
# Configuration 4: MobileNetV2-style int8 classifier (width 1.0).  Stem 3->32 3x3 s2, 17 inverted
# residual blocks (1x1 expand x6, 3x3 depthwise, 1x1 project, residual Add where shapes match) with
# ReLU6, channels 16/24/32/64/96/160/320 with repeats (1,2,3,4,3,3,1) and strides (1,2,2,2,1,2,1),
# Conv 320->1280 1x1, GlobalAveragePool, 1280->classes, DequantizeLinear.  Weights: He-normal,
# symmetric int8 per output channel.  Activation scales are fixed by construction instead of
# calibrated: 6/127 after every ReLU6 (its exact range), 0.1 for the linear projection / residual
# tensors, 0.05 for the pooled features and 0.1 for the logits; all zero points 0, int8 throughout.
# ------------------------------------------------------------------------------------------------
MBV2_STAGES = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]


def mobilenetv2_int8(batch, res=224, classes=1000, seed=DEFAULT_SEED):
    b = _Builder("mobilenetv2_int8", seed + 4)
    g = b.g
    S6, SL = float(np.float32(6.0) / np.float32(127.0)), 0.1
    sx = float(np.float32(1.0) / np.float32(255.0))
    x = b.act(U8, (batch, 3, res, res), "x")
    macs = 0

    def qconv(src, s_in, cin, cout, k, stride, group, s_out, act, x_dtype_scale=None):
        nonlocal macs
        n, _, h, w_ = b.shape(src)
        p = k // 2
        oh, ow = _conv_out(h, k, stride, p), _conv_out(w_, k, stride, p)
        wf = he_normal(b.rng, (cout, cin // group, k, k), (cin // group) * k * k)
        wq, ws = quantize_weights(wf, 0)
        out = b.act(I8, (n, cout, oh, ow))
        g.node("QLinearConv", [src, b.const(I8, wq), b.const(F32, ws), -1, b.const(I32, np.zeros(cout, np.int32))], [out],
               x_scale=s_in, x_zp=0, y_scale=s_out, y_zp=0, strides=(stride, stride), pads=(p, p, p, p), dilations=(1, 1),
               group=group, auto_pad="NOTSET", activation=act)
        macs += oh * ow * cout * (cin // group) * k * k
        return out

    cur = qconv(x, sx, 3, 32, 3, 2, 1, S6, "relu6")
    s_cur, cin = S6, 32
    for t, c, reps, stride in MBV2_STAGES:
        for i in range(reps):
            st = stride if i == 0 else 1
            src, s_src = cur, s_cur
            h = cur
            if t != 1:
                h = qconv(h, s_cur, cin, cin * t, 1, 1, 1, S6, "relu6")
            h = qconv(h, S6, cin * t, cin * t, 3, st, cin * t, S6, "relu6")
            h = qconv(h, S6, cin * t, c, 1, 1, 1, SL, None)
            if st == 1 and cin == c:
                o = b.act(I8, b.shape(h))
                g.node("QLinearAdd", [src, h], [o], x_scale=s_src, x_zp=0, b_scale=SL, b_zp=0, y_scale=SL, y_zp=0)
                h = o
            cur, s_cur, cin = h, SL, c
    cur = qconv(cur, s_cur, 320, 1280, 1, 1, 1, S6, "relu6")
    n = b.shape(cur)[0]
    gap = b.act(I8, (n, 1280, 1, 1))
    g.node("QLinearGlobalAveragePool", [cur], [gap], x_scale=S6, x_zp=0, y_scale=0.05, y_zp=0)
    flat = b.act(I8, (n, 1280))
    g.node("Reshape", [gap], [flat])
    wf = he_normal(b.rng, (1280, classes), 1280)
    wq, ws = quantize_weights(wf, 1)
    fc = b.act(I8, (n, classes))
    g.node("QLinearMatMul", [flat, b.const(I8, wq), b.const(F32, ws), -1, b.const(I32, np.zeros(classes, np.int32))], [fc],
           x_scale=0.05, x_zp=0, y_scale=0.1, y_zp=0)
    y = b.act(F32, (n, classes), "logits")
    g.node("DequantizeLinear", [fc], [y], x_scale=0.1, x_zp=0)
    g.input, g.output = x, y
    g.meta = dict(macs_per_image=macs + 1280 * classes)
    return g


def mobilenetv2_input(batch, res=224, seed=DEFAULT_SEED + 5):
    return np.random.default_rng(seed).integers(0, 256, (batch, 3, res, res), dtype=np.uint8)


# ------------------------------------------------------------------------------------------------
# Configuration 5: Tiny-YOLOv3-style detector.  Backbone: [Conv 3x3 + LeakyReLU(0.1) + MaxPool 2/2]
# with channels 16/32/64/128/256, then 512 with a stride-1 2x2 MaxPool (SAME_UPPER), then Conv 1024.
# Heads: Conv 1x1 1024->256; head 1 = Conv 3x3 256->512, Conv 1x1 ->255 on the 13x13 grid; head 2 =
# Conv 1x1 256->128, Resize x2 nearest, Concat with the 26x26x256 feature, Conv 3x3 ->256, 1x1 ->255.
# (The 1x1 1024->256 in front of both heads is the choice made where the description is ambiguous.)
# The graph has two outputs; the plan returns head 2 (26x26) and head 1 is read as an intermediate.
# ------------------------------------------------------------------------------------------------
def tiny_yolo_fp32(batch, res=416, seed=DEFAULT_SEED, out_ch=255):
    b = _Builder("tiny_yolo_fp32", seed + 6)
    g = b.g
    x = b.act(F32, (batch, 3, res, res), "x")
    macs = 0

    def conv(src, cout, k, act=True, name=None):
        nonlocal macs
        n, cin, h, w_ = b.shape(src)
        p = k // 2
        wf = he_normal(b.rng, (cout, cin, k, k), cin * k * k)
        c = b.act(F32, (n, cout, h, w_))
        g.node("Conv", [src, b.const(F32, wf), b.const(F32, np.zeros(cout, np.float32))], [c], strides=(1, 1), pads=(p, p, p, p),
               dilations=(1, 1), group=1, auto_pad="NOTSET")
        macs += h * w_ * cout * cin * k * k
        if not act:
            g.tensors[c]["name"] = name or g.tensors[c]["name"]
            return c
        a = b.act(F32, (n, cout, h, w_), name)
        g.node("LeakyRelu", [c], [a], alpha=0.1)
        return a

    def pool(src, stride):
        n, c, h, w_ = b.shape(src)
        if stride == 2:
            o = b.act(F32, (n, c, h // 2, w_ // 2))
            g.node("MaxPool", [src], [o], kernel_shape=(2, 2), strides=(2, 2), dilations=(1, 1), pads=(0, 0, 0, 0), auto_pad="NOTSET")
        else:
            o = b.act(F32, (n, c, h, w_))
            g.node("MaxPool", [src], [o], kernel_shape=(2, 2), strides=(1, 1), dilations=(1, 1), pads=(0, 0, 0, 0), auto_pad="SAME_UPPER")
        return o

    cur = x
    feat26 = None
    for i, ch in enumerate((16, 32, 64, 128, 256)):
        cur = conv(cur, ch, 3)
        if ch == 256:
            feat26 = cur
        cur = pool(cur, 2)
    cur = pool(conv(cur, 512, 3), 1)
    cur = conv(cur, 1024, 3)
    neck = conv(cur, 256, 1)
    head1 = conv(conv(neck, 512, 3), out_ch, 1, act=False, name="head13")
    up_in = conv(neck, 128, 1)
    n, c, h, w_ = b.shape(up_in)
    up = b.act(F32, (n, c, 2 * h, 2 * w_))
    g.node("Resize", [up_in], [up], scales=(1.0, 1.0, 2.0, 2.0), coord_mode="half_pixel")
    cat = b.act(F32, (n, c + 256, 2 * h, 2 * w_))
    g.node("Concat", [up, feat26], [cat], axis=1)
    head2 = conv(conv(cat, 256, 3), out_ch, 1, act=False, name="head26")
    g.input, g.output = x, head2
    g.meta = dict(macs_per_image=macs, head13=head1, head26=head2)
    return g


def tiny_yolo_input(batch, res=416, seed=DEFAULT_SEED + 7):
    return np.random.default_rng(seed).random((batch, 3, res, res), dtype=np.float32)


def tiny_yolo_int8(fp32_graph, act_scales):
    """QDQ/QLinear form of a tiny_yolo_fp32 graph: QuantizeLinear(uint8, 1/255) on the input, every
    Conv -> QLinearConv (int8 per-channel weights from the FP32 graph's own weights), LeakyReLU as a
    requantising 256-entry table, MaxPool / Resize / Concat on int8 codes (Concat inputs are brought
    to one scale by the producer's y_scale), DequantizeLinear on the 26x26 head.
    `act_scales`: tensor name -> scale for every FP32 activation tensor (zero point 0)."""
    f = fp32_graph
    b = _Builder("tiny_yolo_int8", 0)
    g = b.g
    sx = float(np.float32(1.0) / np.float32(255.0))
    m = {}            # fp32 tensor id -> (int8 tensor id, scale)
    xin = b.act(F32, f.tensors[f.input]["shape"], "x")
    xq = b.act(U8, f.tensors[f.input]["shape"], "xq")
    g.node("QuantizeLinear", [xin], [xq], y_scale=sx, y_zp=0)
    m[f.input] = (xq, sx)
    # Concat needs equal scales on its inputs: give both producers the larger of the two scales.
    forced = {}
    for n in f.nodes:
        if n["op"] == "Concat":
            s = max(act_scales[f.tensors[i]["name"]] for i in n["inputs"])
            for i in n["inputs"]:
                forced[i] = s
            forced[n["outputs"][0]] = s
    # Resize / MaxPool keep the scale of their input; propagate forced scales backwards through them.
    changed = True
    while changed:
        changed = False
        for n in f.nodes:
            if n["op"] in ("Resize", "MaxPool") and n["outputs"][0] in forced and n["inputs"][0] not in forced:
                forced[n["inputs"][0]] = forced[n["outputs"][0]]
                changed = True

    def scale_of(tid):
        return forced.get(tid, act_scales[f.tensors[tid]["name"]])

    for n in f.nodes:
        op, a = n["op"], n["attrs"]
        out_t = f.tensors[n["outputs"][0]]
        o = n["outputs"][0]
        if op == "Conv":
            src, s_in = m[n["inputs"][0]]
            wf = f.tensors[n["inputs"][1]]["data"]
            wq, ws = quantize_weights(wf, 0)
            s_out = scale_of(o)
            q = b.act(I8, out_t["shape"], out_t["name"])
            g.node("QLinearConv", [src, b.const(I8, wq), b.const(F32, ws), -1, b.const(I32, np.zeros(wq.shape[0], np.int32))], [q],
                   x_scale=s_in, x_zp=0, y_scale=s_out, y_zp=0, strides=a["strides"], pads=a["pads"], dilations=a["dilations"],
                   group=1, auto_pad="NOTSET")
            m[o] = (q, s_out)
        elif op == "LeakyRelu":
            src, s_in = m[n["inputs"][0]]
            s_out = scale_of(o)
            q = b.act(I8, out_t["shape"], out_t["name"])
            g.node("LeakyRelu", [src], [q], alpha=a["alpha"], x_scale=s_in, x_zp=0, y_scale=s_out, y_zp=0)
            m[o] = (q, s_out)
        elif op in ("MaxPool", "Resize"):
            src, s_in = m[n["inputs"][0]]
            q = b.act(I8, out_t["shape"], out_t["name"])
            g.node(op, [src], [q], **a)
            m[o] = (q, s_in)
        elif op == "Concat":
            srcs = [m[i] for i in n["inputs"]]
            assert len({s for _, s in srcs}) == 1
            q = b.act(I8, out_t["shape"], out_t["name"])
            g.node("Concat", [s for s, _ in srcs], [q], **a)
            m[o] = (q, srcs[0][1])
        else:
            raise NotImplementedError(op)
    last, s_last = m[f.output]
    y = b.act(F32, f.tensors[f.output]["shape"], "head26_f32")
    g.node("DequantizeLinear", [last], [y], x_scale=s_last, x_zp=0)
    g.input, g.output = xin, y
    g.meta = dict(macs_per_image=f.meta["macs_per_image"], head13=m[f.meta["head13"]][0], head13_scale=m[f.meta["head13"]][1])
    return g


def activation_scales_on_gpu(ctx, fp32_graph, calib_x):
    """max|a|/127 of every non-constant tensor of an FP32 graph, from one run of its plan."""
    plan = Plan(ctx, fp32_graph, fuse=False)
    try:
        plan.run(calib_x)
        acts = {t["name"]: plan.read_tensor(i) for i, t in enumerate(fp32_graph.tensors) if t["data"] is None and i != fp32_graph.input}
    finally:
        plan.close()
    return act_scales_from(acts)
