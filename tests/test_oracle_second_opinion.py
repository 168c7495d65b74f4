"""An independent second opinion on the quantized part of the oracle.

The reference has no quantized operators, so the C++ oracle's QLinearConv / QLinearMatMul / QLinearAdd /
global average pool restate the ONNX definitions and nothing in the reference can pin them.  This file
checks them against a differently built computation: the integer accumulation comes from PyTorch's CPU
convolution / matmul on float64 tensors (exact for these magnitudes: every partial sum is far below 2^53),
and the requantisation is written here in numpy from the pinned formula
    M = (x_scale * w_scale) / y_scale;  y = sat(rne(float32(acc) * M) + y_zp);  activation on the codes.
PyTorch is test infrastructure only; nothing in the product imports it."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

I8, U8, I32 = 1, 2, 3
NPDT = {I8: np.int8, U8: np.uint8}


def q(rng, shape, dt):
    return rng.integers(0, 256, shape, dtype=np.uint8) if dt == U8 else rng.integers(-128, 128, shape, dtype=np.int8)


def requant(acc, mult, y_zp, ydt, act, y_scale):
    """acc int64 [..], mult float32 broadcastable to acc."""
    v = acc.astype(np.float32) * mult.astype(np.float32)
    v = np.clip(v, np.float32(-512.0), np.float32(511.0))
    t = np.rint(v).astype(np.int64) + y_zp
    lo, hi = (0, 255) if ydt == U8 else (-128, 127)
    t = np.clip(t, lo, hi)
    if act in ("relu", "relu6"):
        t = np.maximum(t, y_zp)
    if act == "relu6":
        six = np.clip(np.rint(np.clip(np.float32(6.0) / np.float32(y_scale), -512, 511)).astype(np.int64) + y_zp, lo, hi)
        t = np.minimum(t, six)
    return t.astype(NPDT[ydt])


def multipliers(x_scale, w_scale, y_scale):
    xw = np.float32(x_scale) * w_scale.astype(np.float32)
    return (xw / np.float32(y_scale)).astype(np.float32)


def torch_qconv(x, x_zp, w, w_zp, bias, stride, pads, dil, group):
    """Exact integer accumulator of QLinearConv, via float64 conv2d; pads = (top, left, bottom, right)."""
    xf = torch.from_numpy(x.astype(np.float64) - x_zp)
    wzp = np.zeros(w.shape[0], np.int64) if w_zp is None else np.broadcast_to(np.asarray(w_zp, np.int64), (w.shape[0],))
    wf = torch.from_numpy(w.astype(np.float64) - wzp.reshape(-1, 1, 1, 1))
    t, l, b, r = pads
    xf = torch.nn.functional.pad(xf, (l, r, t, b))          # zero = (x_zp - x_zp): padding contributes nothing
    acc = torch.nn.functional.conv2d(xf, wf, None, stride=stride, padding=0, dilation=dil, groups=group).numpy()
    acc = np.rint(acc).astype(np.int64)
    if bias is not None:
        acc = acc + bias.astype(np.int64).reshape(1, -1, 1, 1)
    return acc


CASES = [
    # N C H W M k stride pads dil group xdt ydt xzp yzp per_channel bias act
    (2, 1, 28, 28, 32, 3, (1, 1), (0, 0, 0, 0), (1, 1), 1, U8, I8, 0, 0, True, True, "relu"),
    (2, 32, 13, 13, 64, 3, (1, 1), (0, 0, 0, 0), (1, 1), 1, I8, I8, 0, 0, True, True, "relu"),
    (1, 16, 9, 9, 24, 3, (1, 1), (1, 1, 1, 1), (1, 1), 1, I8, I8, 0, 0, False, False, None),
    (2, 8, 10, 7, 12, 3, (2, 2), (1, 1, 1, 1), (1, 1), 1, U8, U8, 128, 3, True, True, "relu6"),
    (1, 6, 8, 8, 9, 1, (1, 1), (0, 0, 0, 0), (1, 1), 3, I8, I8, -3, 5, True, True, None),
    (2, 16, 11, 11, 16, 3, (1, 1), (1, 1, 1, 1), (1, 1), 16, I8, I8, 0, 0, True, True, "relu6"),
    (1, 16, 12, 12, 16, 3, (2, 2), (0, 1, 1, 0), (1, 1), 16, I8, U8, 2, 10, False, False, "relu"),
    (1, 4, 9, 9, 5, 2, (1, 1), (0, 0, 0, 0), (2, 2), 1, I8, I8, 0, 0, True, False, None),
    # shapes of the tensor-core paths: 64 -> 64 3x3 on 56x56, 256 -> 64 1x1, stride-2 256 -> 512, depthwise 128
    (1, 64, 56, 56, 64, 3, (1, 1), (1, 1, 1, 1), (1, 1), 1, I8, I8, 0, 0, False, False, None),
    (1, 256, 28, 28, 64, 1, (1, 1), (0, 0, 0, 0), (1, 1), 1, I8, I8, 0, 0, True, True, "relu"),
    (1, 256, 14, 14, 512, 3, (2, 2), (1, 1, 1, 1), (1, 1), 1, I8, I8, 0, 0, False, False, None),
    (1, 128, 56, 56, 128, 3, (1, 1), (1, 1, 1, 1), (1, 1), 128, I8, I8, 0, 0, False, True, "relu6"),
    (1, 3, 64, 64, 32, 3, (2, 2), (1, 1, 1, 1), (1, 1), 1, U8, I8, 0, 0, True, True, "relu6"),
]


@pytest.mark.parametrize("case", CASES, ids=[f"case{i}" for i in range(len(CASES))])
def test_qlinearconv_oracle_agrees_with_torch(oracle, case):
    N, C, H, W, M, k, stride, pads, dil, group, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(1000 + N + C * 3 + M)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C // group, k, k), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    wz = rng.integers(-3, 4, M if per_ch else 1).astype(np.int32) if xzp else None
    bias = rng.integers(-2000, 2000, M).astype(np.int32) if has_bias else None
    y_scale = float(np.float32(0.02 * np.sqrt(C // group * k * k)))
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, wz, y_scale, yzp, bias=bias, y_dtype=ydt, stride=stride, pads=pads,
                              dilations=dil, group=group, activation=act)
    acc = torch_qconv(x, xzp, w, wz, bias, stride, pads, dil, group)
    mult = multipliers(0.02, np.broadcast_to(ws, (M,)), y_scale).reshape(1, M, 1, 1)
    second = requant(acc, mult, yzp, ydt, act, y_scale)
    assert want.shape == second.shape
    assert np.array_equal(want, second)
    assert len(np.unique(want)) > 8


@pytest.mark.parametrize("M,K,N", [(5, 1600, 512), (130, 512, 10), (33, 70, 9), (256, 1280, 1000)])
@pytest.mark.parametrize("adt,ydt,azp,yzp,act", [(I8, I8, 0, 0, "relu"), (U8, U8, 128, 7, None), (I8, I8, 9, -4, "relu6")])
def test_qlinearmatmul_oracle_agrees_with_torch(oracle, M, K, N, adt, ydt, azp, yzp, act):
    rng = np.random.default_rng(M + K + N)
    a = q(rng, (M, K), adt)
    b = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bs = (rng.random(N, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bz = rng.integers(-2, 3, N).astype(np.int32) if azp else None
    bias = rng.integers(-3000, 3000, N).astype(np.int32)
    ys = float(np.float32(0.02 * np.sqrt(K)))
    want = oracle.qlinearmatmul(a, 0.02, azp, b, bs, bz, ys, yzp, bias, ydt, act)
    af = torch.from_numpy(a.astype(np.float64) - azp)
    bf = torch.from_numpy(b.astype(np.float64) - (0 if bz is None else bz.astype(np.float64).reshape(1, N)))
    acc = np.rint((af @ bf).numpy()).astype(np.int64) + bias.astype(np.int64).reshape(1, N)
    second = requant(acc, multipliers(0.02, bs, ys).reshape(1, N), yzp, ydt, act, ys)
    assert np.array_equal(want, second)


def test_quantize_add_gap_oracle_agree_with_numpy(oracle):
    rng = np.random.default_rng(11)
    x = ((rng.random(5000, dtype=np.float32) - 0.5) * 8).astype(np.float32)
    for dt, scale, zp in ((U8, 1 / 255, 0), (I8, 0.02, 0), (I8, 0.013, -7), (U8, 0.031, 128)):
        lo, hi = (0, 255) if dt == U8 else (-128, 127)
        v = np.clip(x / np.float32(scale), np.float32(-512), np.float32(511))
        second = np.clip(np.rint(v).astype(np.int64) + zp, lo, hi).astype(NPDT[dt])
        assert np.array_equal(oracle.quantize_linear(x, scale, zp, dt), second)
        back = (second.astype(np.int32) - zp).astype(np.float32) * np.float32(scale)
        assert np.array_equal(oracle.dequantize_linear(second, scale, zp).view(np.uint32), back.view(np.uint32))
    a, b = q(rng, (3, 8, 5, 5), I8), q(rng, (3, 8, 5, 5), I8)
    fa = (a.astype(np.int32) - 3).astype(np.float32) * np.float32(0.031)
    fb = (b.astype(np.int32) + 4).astype(np.float32) * np.float32(0.017)
    v = np.clip((fa + fb) / np.float32(0.045), np.float32(-512), np.float32(511))
    second = np.clip(np.rint(v).astype(np.int64) + 1, -128, 127).astype(np.int8)
    assert np.array_equal(oracle.qlinearadd(a, 0.031, 3, b, 0.017, -4, 0.045, 1, None), second)
    x4 = q(rng, (2, 16, 7, 7), I8)
    s = (x4.astype(np.int64) - 2).sum(axis=(2, 3))
    v = (s.astype(np.float32) * np.float32(0.047)) / np.float32(49.0) / np.float32(0.05)
    second = np.clip(np.rint(np.clip(v, -512, 511)).astype(np.int64) + 0, -128, 127).astype(np.int8).reshape(2, 16, 1, 1)
    assert np.array_equal(oracle.qlinear_global_avgpool(x4, 0.047, 2, 0.05, 0).reshape(2, 16, 1, 1), second)
