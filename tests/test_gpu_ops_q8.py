"""Quantized operators: CUDA against the pinned int8 definitions of the oracle, bit for bit.

The reference tree has no quantized operators, so these definitions are the contract; the
oracle itself is pinned by hand-computed vectors in tests/test_oracle_quant.py.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
I8, U8, I32 = 1, 2, 3
NP = {I8: np.int8, U8: np.uint8}


def q(rng, shape, dt):
    return rng.integers(0, 256, shape, dtype=np.uint8) if dt == U8 else rng.integers(-128, 128, shape, dtype=np.int8)


@pytest.mark.parametrize("n", [0, 1, 5, 784, 4099])
@pytest.mark.parametrize("dt,scale,zp", [(U8, 1 / 255, 0), (I8, 0.02, 0), (I8, 0.013, -7), (U8, 0.031, 128)])
def test_quantize_dequantize(ctx, oracle, n, dt, scale, zp):
    rng = np.random.default_rng(n)
    x = (rng.random(n, dtype=np.float32) * 12 - 4).astype(np.float32)
    if n > 4:
        x[:5] = [0.5 * scale, 1.5 * scale, 2.5 * scale, -0.5 * scale, 1e30]   # ties and saturation
    got, want = ctx.quantize_linear(x, scale, zp, dt), oracle.quantize_linear(x, scale, zp, dt)
    assert np.array_equal(got, want)
    back_g, back_o = ctx.dequantize_linear(want, scale, zp), oracle.dequantize_linear(want, scale, zp)
    assert np.array_equal(back_g.view(np.uint32), back_o.view(np.uint32))


def test_dequantize_int32(ctx, oracle):
    acc = np.random.default_rng(1).integers(-2**31, 2**31 - 1, 1000, dtype=np.int64).astype(np.int32)
    a, b = ctx.dequantize_linear(acc, 0.0004, 0), oracle.dequantize_linear(acc, 0.0004, 0)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


QCONV = [
    # N C H W M k stride pads dil group xdt ydt xzp yzp per_channel bias act
    (2, 1, 28, 28, 32, 3, (1, 1), (0, 0, 0, 0), (1, 1), 1, U8, I8, 0, 0, True, True, "relu"),
    (2, 32, 13, 13, 64, 3, (1, 1), (0, 0, 0, 0), (1, 1), 1, I8, I8, 0, 0, True, True, "relu"),
    (1, 16, 9, 9, 24, 3, (1, 1), (1, 1, 1, 1), (1, 1), 1, I8, I8, 0, 0, False, False, None),
    (2, 8, 10, 7, 12, 3, (2, 2), (1, 1, 1, 1), (1, 1), 1, U8, U8, 128, 3, True, True, "relu6"),
    (1, 6, 8, 8, 9, 1, (1, 1), (0, 0, 0, 0), (1, 1), 3, I8, I8, -3, 5, True, True, None),
    (2, 16, 11, 11, 16, 3, (1, 1), (1, 1, 1, 1), (1, 1), 16, I8, I8, 0, 0, True, True, "relu6"),   # depthwise
    (1, 16, 12, 12, 16, 3, (2, 2), (0, 1, 1, 0), (1, 1), 16, I8, U8, 2, 10, False, False, "relu"),  # depthwise s2
    (1, 4, 9, 9, 5, 2, (1, 1), (0, 0, 0, 0), (2, 2), 1, I8, I8, 0, 0, True, False, None),
]


@pytest.mark.parametrize("case", QCONV, ids=[f"qconv{i}" for i in range(len(QCONV))])
def test_qlinearconv(ctx, oracle, case):
    N, C, H, W, M, k, stride, pads, dil, group, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N + C * 3 + M)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C // group, k, k), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    wz = rng.integers(-3, 4, M if per_ch else 1).astype(np.int32) if xzp else None
    bias = rng.integers(-2000, 2000, M).astype(np.int32) if has_bias else None
    y_scale = 0.02 * np.sqrt(C // group * k * k)
    kw = dict(bias=bias, y_dtype=ydt, stride=stride, pads=pads, dilations=dil, group=group, activation=act)
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, wz, y_scale, yzp, **kw)
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, wz, y_scale, yzp, **kw)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert len(np.unique(want)) > 8   # the case is not saturated into triviality


@pytest.mark.parametrize("auto_pad", ["SAME_UPPER", "SAME_LOWER", "VALID"])
def test_qlinearconv_auto_pad(ctx, oracle, auto_pad):
    rng = np.random.default_rng(3)
    x = q(rng, (1, 4, 9, 10), I8)
    w = rng.integers(-127, 128, (6, 4, 3, 3), dtype=np.int8)
    kw = dict(stride=(2, 2), pads=(0, 0, 0, 0), auto_pad=auto_pad)
    got = ctx.qlinearconv(x, 0.02, 0, w, [0.02], None, 0.3, 0, **kw)
    want = oracle.qlinearconv(x, 0.02, 0, w, [0.02], None, 0.3, 0, **kw)
    assert got.shape == want.shape and np.array_equal(got, want)


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (3, 1600, 512), (5, 512, 10), (33, 70, 129), (128, 128, 128), (2, 17, 3)])
@pytest.mark.parametrize("adt,ydt,azp,yzp,act", [(I8, I8, 0, 0, "relu"), (U8, U8, 128, 7, None), (I8, I32, 0, 0, None)])
def test_qlinearmatmul(ctx, oracle, M, K, N, adt, ydt, azp, yzp, act):
    rng = np.random.default_rng(M + K + N)
    a = q(rng, (M, K), adt)
    b = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bs = (rng.random(N, dtype=np.float32) * 0.01 + 0.001).astype(np.float32)
    bz = rng.integers(-2, 3, N).astype(np.int32) if azp else None
    bias = rng.integers(-500, 500, N).astype(np.int32)
    ys = 0.02 * np.sqrt(K)
    got = ctx.qlinearmatmul(a, 0.02, azp, b, bs, bz, ys, yzp, bias, ydt, act)
    want = oracle.qlinearmatmul(a, 0.02, azp, b, bs, bz, ys, yzp, bias, ydt, act)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt,act", [(I8, None), (U8, "relu"), (I8, "relu6")])
def test_qlinearadd(ctx, oracle, dt, act):
    rng = np.random.default_rng(17)
    a, b = q(rng, (3, 24, 7, 7), dt), q(rng, (3, 24, 7, 7), dt)
    zp = 0 if dt == I8 else 120
    got = ctx.qlinearadd(a, 0.031, zp, b, 0.017, zp - 3 if dt == U8 else -4, 0.045, zp, act)
    want = oracle.qlinearadd(a, 0.031, zp, b, 0.017, zp - 3 if dt == U8 else -4, 0.045, zp, act)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", [I8, U8])
@pytest.mark.parametrize("hw", [(7, 7), (1, 1), (5, 13)])
def test_qlinear_global_avgpool(ctx, oracle, dt, hw):
    x = q(np.random.default_rng(5), (3, 40) + hw, dt)
    got = ctx.qlinear_global_avgpool(x, 0.05, 3, 0.02, -1 if dt == I8 else 9)
    want = oracle.qlinear_global_avgpool(x, 0.05, 3, 0.02, -1 if dt == I8 else 9)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", [I8, U8])
@pytest.mark.parametrize("shape", [(8, 640, 7, 7), (5, 1001, 5, 13), (4099, 1, 1, 3), (17, 300, 16, 16)])
def test_qlinear_global_avgpool_many_small_planes(ctx, oracle, dt, shape):
    """At least 4096 planes of at most 256 bytes: the thread-per-plane kernel (word loads, masked first and last word)."""
    x = q(np.random.default_rng(shape[1]), shape, dt)
    zp = 3 if dt == I8 else 131
    got = ctx.qlinear_global_avgpool(x, 0.05, zp, 0.02, -1 if dt == I8 else 9)
    want = oracle.qlinear_global_avgpool(x, 0.05, zp, 0.02, -1 if dt == I8 else 9)
    assert np.array_equal(got, want)
    assert len(np.unique(want)) > 16


@pytest.mark.parametrize("dt", [I8, U8])
def test_maxpool_q8(ctx, oracle, dt):
    x = q(np.random.default_rng(6), (2, 16, 13, 13), dt)
    for args in (((2, 2), (2, 2), (1, 1), (0, 0, 0, 0), "NOTSET"), ((2, 2), (1, 1), (1, 1), (0, 0, 0, 0), "SAME_UPPER"),
                 ((3, 3), (2, 2), (1, 1), (1, 1, 1, 1), "NOTSET")):
        assert np.array_equal(ctx.onnx_maxpool(x, *args), oracle.onnx_maxpool(x, *args))


@pytest.mark.parametrize("dt", [I8, U8])
@pytest.mark.parametrize("shape", [(2, 5, 16, 24), (1, 3, 2, 8), (3, 16, 52, 104)])
def test_maxpool_q8_2x2_stride2_rows_of_whole_words(ctx, oracle, dt, shape):
    """The packed-byte kernel (even H, W % 8 == 0) against the oracle."""
    x = q(np.random.default_rng(shape[3]), shape, dt)
    args = ((2, 2), (2, 2), (1, 1), (0, 0, 0, 0), "NOTSET")
    assert np.array_equal(ctx.onnx_maxpool(x, *args), oracle.onnx_maxpool(x, *args))


@pytest.mark.parametrize("dt", [I8, U8])
@pytest.mark.parametrize("n", [1, 15, 16, 4097])
def test_leaky_relu_lut(ctx, oracle, dt, n):
    lut = oracle.build_leaky_lut(dt, 0.05, 3 if dt == U8 else 0, 0.1, 0.04, 5 if dt == U8 else 0)
    x = q(np.random.default_rng(n), (n,), dt)
    got, want = ctx.lut_q8(x, lut), oracle.lut_q8(x, lut)
    assert np.array_equal(got, want)
    # the table equals dequantise -> LeakyReLU -> quantise computed element by element
    zi, zo = (3, 5) if dt == U8 else (0, 0)
    ref = oracle.quantize_linear(oracle.leakyReLU(oracle.dequantize_linear(x, 0.05, zi), 0.1), 0.04, zo, dt)
    assert np.array_equal(want, ref)


# ---- tensor-core path (im2col into the GEMM-blocked layout + tcgen05 GEMM): taken for group 1,
# ---- zero weight zero points and at least 256 output positions
TC_QCONV = [
    # N C H W M k stride pads dil xdt ydt xzp yzp per_channel bias act
    (2, 64, 20, 20, 64, 3, (1, 1), (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, False, False, None),
    (4, 24, 17, 19, 40, 3, (2, 2), (1, 0, 2, 1), (1, 1), U8, U8, 128, 7, True, True, "relu6"),
    (2, 7, 23, 23, 130, 5, (1, 2), (2, 2, 2, 2), (2, 1), I8, I8, -5, 3, True, True, "relu"),
    (2, 256, 16, 16, 300, 1, (1, 1), (0, 0, 0, 0), (1, 1), I8, U8, 0, 100, True, True, None),
    (4, 3, 32, 32, 32, 3, (2, 2), (1, 1, 1, 1), (1, 1), U8, I8, 0, 0, True, False, "relu6"),
    (4, 40, 14, 14, 72, 1, (1, 1), (0, 0, 0, 0), (1, 1), I8, I8, 3, 0, True, True, "relu6"),     # 1x1 on 14x14 (196-byte planes): implicit GEMM, rows copied by warps
    (8, 200, 6, 6, 130, 1, (1, 1), (0, 0, 0, 0), (1, 1), U8, U8, 128, 4, True, True, None),      # 1x1, 200 channels (4 K groups, last partial)
    (8, 64, 14, 14, 96, 3, (2, 2), (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, True, True, "relu"),      # sweep case 3b in small: tap-major im2col
    (6, 80, 13, 11, 40, 3, (1, 2), (2, 0, 1, 1), (2, 1), U8, I8, 77, -5, True, False, None),     # tap-major, 80 channels, odd geometry
    (3, 16, 30, 30, 24, 5, (3, 3), (2, 2, 2, 2), (1, 1), I8, U8, -9, 30, False, True, "relu6"),  # tap-major, 25 taps of 16 channels
]


DW_QCONV = [
    # N C H W stride xdt ydt xzp yzp per_channel bias act
    (2, 128, 56, 56, 1, I8, I8, 0, 0, False, False, None),        # sweep case 3d
    (3, 24, 28, 28, 1, U8, U8, 128, 9, True, True, "relu6"),      # four planes per warp, zero points
    (2, 40, 8, 8, 1, I8, I8, -4, 0, True, True, "relu"),          # 16 planes per warp
    (1, 7, 20, 112, 1, I8, U8, 3, 120, True, False, None),        # 28 of 32 lanes
    (2, 96, 112, 112, 2, I8, I8, 0, 0, True, True, "relu6"),      # stride 2
    (3, 18, 16, 24, 2, U8, I8, 7, -3, True, True, None),          # stride 2, uint8 input
    (1, 5, 4, 8, 2, I8, I8, 0, 0, False, False, "relu"),          # smallest stride-2 plane
    (3, 48, 14, 14, 1, I8, I8, 0, 0, True, True, "relu6"),        # rows that are not whole words
    (5, 21, 7, 7, 1, U8, U8, 100, 3, True, True, None),           # 49-byte planes, tensor size not a multiple of 4
    (2, 36, 14, 14, 2, I8, I8, -2, 0, True, True, "relu6"),       # stride 2 onto 7x7
    (1, 3, 5, 9, 1, I8, U8, 0, 17, False, False, None),           # odd sizes
    (2, 8, 6, 10, 2, U8, I8, 9, 0, True, False, "relu"),          # stride 2, 10 -> 5 columns
    (3, 5, 1, 8, 1, I8, I8, 4, 0, True, True, None),              # 8 columns per lane: one row
    (2, 6, 2, 16, 1, U8, U8, 11, 2, True, True, "relu"),          # two rows
    (2, 7, 3, 24, 1, I8, I8, 0, 0, False, True, None),            # three rows
    (1, 9, 4, 40, 1, I8, I8, -1, 0, True, False, "relu6"),        # four rows, 5 lanes of 8 per plane
    (2, 3, 5, 64, 1, I8, U8, 0, 9, True, True, None),             # five rows
    (1, 2, 9, 128, 1, U8, I8, 200, 0, True, True, None),          # widest plane the kernel takes
    (3, 40, 28, 28, 2, I8, I8, 0, 0, True, True, "relu6"),        # stride 2 from whole-word rows onto 14 x 14: only the output is staged
    (2, 12, 12, 20, 2, U8, U8, 5, 3, True, True, None),           # the same onto 6 x 10
    (4, 7, 9, 9, 1, I8, I8, 2, 0, True, True, "relu"),            # 81-byte planes: a word spans two planes (flat form)
    (3, 10, 6, 7, 1, U8, I8, 130, 0, True, False, None),          # 42-byte planes, uint8 input
    (5, 52, 14, 14, 1, U8, U8, 128, 9, True, True, "relu6"),      # rows form: 16 batches of 16 planes and a tail of 4, general requantisation
    (9, 30, 7, 7, 1, I8, I8, 3, 0, True, True, "relu"),           # rows form on 7 x 7: batches of 32 planes, a tail of 14
    (4, 64, 7, 7, 1, U8, I8, 0, 0, False, True, "relu6"),         # rows form, whole batches only
    (2, 40, 20, 14, 1, I8, I8, -6, 0, True, False, None),         # rows form, 20 rows of 14: 12 planes per batch
    (32, 96, 14, 14, 1, I8, I8, 0, 0, True, True, "relu6"),       # rows form, more batches than CTAs: every CTA loops
    (6, 40, 14, 14, 2, I8, I8, 0, 0, True, True, "relu6"),        # rows form, stride 2 onto 7 x 7: batches of 32 planes and a tail of 16
    (4, 48, 28, 28, 2, U8, I8, 0, 0, True, True, "relu6"),        # rows form, stride 2 onto 14 x 14: whole batches of 16 planes
    (3, 30, 28, 28, 2, U8, U8, 131, 4, True, True, None),         # the same with zero points and a tail of 10 planes
    (5, 32, 13, 14, 2, I8, I8, -3, 0, False, True, "relu"),       # 13 rows: the last output row reads the padding row below
    (16, 144, 14, 14, 2, I8, I8, 0, 0, True, True, "relu6"),      # stride 2, every CTA loops
]


@pytest.mark.parametrize("case", DW_QCONV, ids=[f"dw{i}" for i in range(len(DW_QCONV))])
def test_qlinearconv_depthwise3x3(zb, ctx, oracle, case):
    N, C, H, W, stride, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 41 + C + H + W)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (C, 1, 3, 3), dtype=np.int8)
    ws = (rng.random(C if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, C).astype(np.int32) if has_bias else None
    kw = dict(bias=bias, y_dtype=ydt, stride=(stride, stride), pads=(1, 1, 1, 1), dilations=(1, 1), group=C, activation=act)
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, None, 0.045, yzp, **kw)
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, None, 0.045, yzp, **kw)
    assert np.array_equal(got, want)
    assert len(np.unique(want)) > 16


# stride-1 cases run the implicit-GEMM or the pointwise kernel (one launch), the others im2col + GEMM (two launches)
TC_QCONV_LAUNCHES = [1, 2, 2, 1, 2, 1, 1, 2, 2, 2]

IMPLICIT_QCONV = [
    # N C H W M k stride pads dil xdt ydt xzp yzp per_channel bias act
    (2, 64, 56, 56, 64, 3, (1, 1), (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, False, False, None),         # sweep case 3a, 8-byte rows
    (3, 3, 32, 32, 32, 3, (1, 1), (1, 1, 1, 1), (1, 1), U8, I8, 0, 0, True, True, "relu6"),          # 3 channels of a 32-channel stage
    (2, 40, 24, 28, 72, 3, (1, 1), (1, 0, 1, 2), (1, 1), U8, U8, 128, 7, True, True, "relu"),        # partial second block, odd pads, zero points
    (1, 16, 40, 144, 24, 3, (1, 1), (1, 1, 1, 1), (1, 1), I8, I8, -3, 5, True, True, None),          # two width segments
    (2, 32, 36, 36, 48, 5, (1, 1), (4, 4, 4, 4), (2, 2), I8, I8, 0, -4, True, False, "relu"),        # 5x5 dilated
    (2, 96, 20, 20, 300, 1, (1, 1), (0, 0, 0, 0), (1, 1), I8, U8, 0, 100, True, True, None),         # pointwise, 256-wide filter tiles
    (5, 256, 8, 8, 64, 1, (1, 1), (0, 0, 0, 0), (1, 1), I8, I8, 2, 0, False, True, "relu6"),          # pointwise, 64 pixels per image
    (2, 33, 12, 16, 130, 3, (1, 1), (0, 0, 0, 0), (1, 1), I8, I8, 0, 0, True, True, None),           # no padding, 2 filter tiles
    (3, 32, 30, 56, 64, 3, (1, 1), (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, True, True, "relu"),          # 4 row blocks per tile, 3 in the last tile
    (1, 16, 9, 144, 24, 3, (1, 1), (1, 1, 1, 1), (1, 1), U8, I8, 5, 0, True, True, None),            # width segments, 2 row blocks, 1 in the last tile
    (2, 128, 28, 28, 128, 3, (1, 1), (1, 1, 1, 1), (1, 1), I8, U8, 0, 3, True, False, None),         # 128-wide filter tile: 2 row blocks
    (3, 96, 14, 14, 160, 1, (1, 1), (0, 0, 0, 0), (1, 1), I8, I8, 0, 0, True, True, "relu6"),        # pointwise, 196-byte planes: rows copied by warps, channel padding
    (3, 40, 10, 10, 24, 1, (1, 1), (0, 0, 0, 0), (1, 1), U8, U8, 9, 5, True, True, None),            # pointwise, 100-byte planes, one tile per image
    (2, 192, 14, 14, 300, 1, (1, 1), (0, 0, 0, 0), (1, 1), I8, I8, -2, 0, False, True, "relu"),      # pointwise, 196-byte planes, streamed weights, 2 channel stages
]


@pytest.mark.parametrize("case", IMPLICIT_QCONV, ids=[f"implicit{i}" for i in range(len(IMPLICIT_QCONV))])
def test_qlinearconv_implicit_gemm(ctx, oracle, case):
    N, C, H, W, M, k, stride, pads, dil, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 37 + C + M + W)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C, k, k), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, M).astype(np.int32) if has_bias else None
    y_scale = 0.015 * np.sqrt(C * k * k)
    kw = dict(bias=bias, y_dtype=ydt, stride=stride, pads=pads, dilations=dil, group=1, activation=act)
    before = ctx.launch_count()
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    launches = ctx.launch_count() - before
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    assert np.array_equal(got, want)
    assert launches == 1
    assert len(np.unique(want)) > 16


# 1x1 / stride 1 / no padding.  Planes of whole words and more than 32 filters: filters on the accumulator lanes, activations
# straight from NCHW (tc_pw_nchw.cuh); the other cases take the implicit-GEMM kernel or im2col + GEMM.
POINTWISE_QCONV = [
    # N C H W M xdt ydt xzp yzp per_channel bias act
    (2, 32, 112, 112, 16, I8, I8, 0, 0, True, True, "relu6"),       # 12544-pixel planes (49 tiles), half a lane quarter of filters, 32-byte stores
    (2, 16, 112, 112, 96, I8, I8, 0, 0, True, True, None),          # 16 channels: half a K step of zero weights
    (3, 24, 56, 56, 144, U8, I8, 128, 0, True, True, "relu"),       # 13 tiles per image, the last of 64 pixels; two filter tiles, the second of 16
    (2, 144, 28, 28, 32, I8, I8, -3, 0, False, True, "relu6"),      # 784-byte planes: tiles of 208 pixels, 16-byte stores; five K steps in stages of two
    (3, 64, 14, 14, 384, U8, U8, 7, 9, True, True, None),           # 196-byte planes: word copies in, bulk copy out; three filter tiles; general requantisation
    (2, 960, 7, 7, 160, I8, I8, 0, 0, True, True, "relu"),          # 49-byte planes (im2col + GEMM)
    (3, 960, 14, 14, 160, I8, I8, 0, 0, True, True, "relu"),        # the deepest K the pointwise kernel takes
    (6, 320, 7, 7, 1280, I8, I8, 2, 0, True, False, None),          # ten filter tiles
    (5, 20, 9, 9, 10, I8, U8, -1, 30, True, True, "relu"),          # 81-byte planes
    (5, 20, 6, 6, 10, I8, U8, -1, 30, True, True, "relu"),          # 36-byte planes, 10 filters: the staged tile (360 bytes per image) is copied out by threads
    (6, 12, 6, 10, 20, U8, I8, 9, 0, False, True, None),            # 60-byte planes, word copies
    (2, 8, 4, 36, 6, I8, I8, 0, 0, True, True, "relu"),             # 144-pixel planes: a second pixel block of 16
    (1, 64, 16, 17, 130, I8, I8, 0, -4, True, True, None),          # 272 pixels: two tiles of 144; non-zero output zero point
    (2, 32, 28, 28, 96, I8, I8, 0, 0, True, True, "relu6"),         # ReLU6 with a six below 127: the clamp of the accumulator (per-filter bounds)
    (2, 48, 14, 14, 64, U8, I8, 128, 0, False, True, "relu6"),      # the same on 14 x 14 planes, one multiplier for all filters
    (3, 96, 56, 56, 24, I8, I8, 0, 0, True, True, None),            # 24 filters: four pixel groups of 32 lanes (block-diagonal weights), tiles of 4 x 208 pixels, the last one partly empty
    (2, 200, 24, 24, 40, U8, U8, 3, 7, True, True, "relu"),         # 40 filters: two groups of 64 lanes, 7 K steps per group, general requantisation
    (2, 64, 16, 16, 12, I8, I8, 0, 0, True, False, "relu6"),        # 12 filters but too few pixels for eight groups: the implicit-GEMM kernel
]


@pytest.mark.parametrize("case", POINTWISE_QCONV, ids=[f"pointwise{i}" for i in range(len(POINTWISE_QCONV))])
def test_qlinearconv_pointwise(ctx, oracle, case):
    N, C, H, W, M, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 43 + C + M + W)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C, 1, 1), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, M).astype(np.int32) if has_bias else None
    y_scale = 0.015 * np.sqrt(C)
    kw = dict(bias=bias, y_dtype=ydt, stride=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1, activation=act)
    before = ctx.launch_count()
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    launches = ctx.launch_count() - before
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    assert np.array_equal(got, want)
    assert launches == 1 if (H * W) % 4 == 0 else launches <= 2
    assert len(np.unique(want)) > 16


NHWC_QCONV = [
    # N C H W M k pads dil xdt ydt xzp yzp per_channel bias act        (channels-last in and out)
    (2, 64, 56, 56, 64, 3, (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, True, True, "relu"),        # sweep case 3a: 64-byte rows, 4 row blocks, resident weights
    (2, 128, 28, 28, 128, 3, (1, 1, 1, 1), (1, 1), I8, U8, 0, 3, True, False, None),       # 128-byte rows, 128-wide filter tile, general requantisation
    (1, 64, 40, 144, 32, 3, (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, False, True, "relu6"),     # two width segments
    (2, 256, 20, 20, 320, 1, (0, 0, 0, 0), (1, 1), U8, I8, 128, 0, True, True, None),      # 1x1, two channel stages, two filter tiles (streamed weights)
    (2, 64, 36, 36, 48, 5, (4, 4, 4, 4), (2, 2), I8, I8, 0, -4, True, False, "relu"),      # 5x5 dilated
    (3, 192, 14, 14, 64, 3, (0, 0, 0, 0), (1, 1), U8, U8, 7, 9, True, True, None),         # three 64-channel stages, no padding with an input zero point
    (1, 64, 30, 56, 64, 3, (1, 1, 1, 1), (1, 1), I8, I8, 0, 0, True, True, None),          # 3 row blocks in the last tile
]


@pytest.mark.parametrize("case", NHWC_QCONV, ids=[f"nhwc{i}" for i in range(len(NHWC_QCONV))])
def test_qlinearconv_channels_last(ctx, oracle, case):
    N, C, H, W, M, k, pads, dil, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 43 + C + M + W)
    x = q(rng, (N, H, W, C), xdt)
    w = rng.integers(-127, 128, (M, C, k, k), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, M).astype(np.int32) if has_bias else None
    y_scale = 0.015 * np.sqrt(C * k * k)
    kw = dict(bias=bias, y_dtype=ydt, stride=(1, 1), pads=pads, dilations=dil, group=1, activation=act)
    before = ctx.launch_count()
    got = ctx.qlinearconv_nhwc(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    assert ctx.launch_count() - before == 1
    want = oracle.qlinearconv(np.ascontiguousarray(x.transpose(0, 3, 1, 2)), 0.02, xzp, w, ws, None, y_scale, yzp, **kw).transpose(0, 2, 3, 1)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert len(np.unique(want)) > 16


def test_qlinearconv_channels_last_as_a_plan_node(ctx, zb, oracle):
    """The sweep case 3a, small batch, as a one-node plan with channels_last=1."""
    import torch
    from zant_b200 import models
    graph, c = models.qconv_graph("3a", batch=4, channels_last=True)
    plan = zb.Plan(ctx, graph)
    assert plan.step_names() == ["QLinearConv(tc-nhwc)"]
    x = torch.from_numpy(c["x"]).cuda()
    y = torch.empty(tuple(graph.tensors[graph.output]["shape"]), dtype=torch.int8, device="cuda")
    plan.run(x, out=y)
    want = oracle.qlinearconv(np.ascontiguousarray(c["x"].transpose(0, 3, 1, 2)), c["x_scale"], 0, c["w"], c["w_scale"], None, c["y_scale"], 0,
                              y_dtype=I8, stride=c["stride"], pads=c["pads"], dilations=c["dilations"], group=1, activation=None)
    assert np.array_equal(y.cpu().numpy(), want.transpose(0, 2, 3, 1))
    plan.close()


def test_qlinearconv_channels_last_refuses_other_shapes(ctx, zb):
    rng = np.random.default_rng(5)
    x = q(rng, (1, 8, 8, 32), I8)                              # 32 channels: not a whole 64-byte operand row
    w = rng.integers(-127, 128, (16, 32, 3, 3), dtype=np.int8)
    with pytest.raises(zb.ZantError) as e:
        ctx.qlinearconv_nhwc(x, 0.02, 0, w, np.float32(0.01), None, 0.5, 0)
    assert e.value.name == "Unsupported" or e.value.status == -103


SMALLC_QCONV = [
    # N C H W M stride pads xdt ydt xzp yzp per_channel bias act        (3x3 on at most four channels: network stems)
    (5, 3, 64, 64, 32, 2, (1, 1, 1, 1), U8, I8, 0, 0, True, True, "relu6"),       # MobileNet-style stem, 32-pixel units
    (1, 3, 48, 112, 16, 1, (1, 1, 1, 1), U8, I8, 3, 0, True, True, None),         # detector-style stem, 16-pixel units
    (2, 1, 40, 60, 48, 1, (0, 1, 1, 0), I8, U8, 0, 7, True, True, "relu"),        # one channel, odd output width: byte stores, partial units
    (4, 4, 66, 72, 64, 2, (0, 0, 0, 0), I8, I8, -5, -3, False, False, None),      # four channels, 64 filters, no padding, general requantisation
    (8, 3, 50, 52, 32, 2, (1, 0, 0, 1), U8, U8, 128, 100, True, True, "relu6"),   # asymmetric pads
    (1, 2, 20, 512, 16, 1, (1, 1, 1, 1), I8, I8, 0, 0, True, False, "relu"),      # wide rows, one band per few rows
]


@pytest.mark.parametrize("case", SMALLC_QCONV, ids=[f"smallc{i}" for i in range(len(SMALLC_QCONV))])
def test_qlinearconv_small_channel_count(ctx, oracle, case):
    N, C, H, W, M, s, pads, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 41 + C + M + W)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C, 3, 3), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, M).astype(np.int32) if has_bias else None
    y_scale = 0.03 * np.sqrt(C * 9)
    kw = dict(bias=bias, y_dtype=ydt, stride=(s, s), pads=pads, dilations=(1, 1), group=1, activation=act)
    before = ctx.launch_count()
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    launches = ctx.launch_count() - before
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert launches == 1
    assert len(np.unique(want)) > 16


STEM_QCONV = [
    # N C H W M stride pads xdt ydt xzp yzp per_channel bias act      (3x3 on at most three channels, rows of whole 16-byte units:
    #                                                                  patches written in shared memory for the filters-on-lanes kernel)
    (3, 3, 96, 96, 32, 2, (0, 0, 1, 1), U8, I8, 0, 0, True, True, "relu6"),        # pads below and right only; 48 x 48 output, one tile and a bit
    (4, 3, 64, 96, 24, 2, (1, 1, 1, 1), U8, I8, 128, 0, True, True, "relu"),       # 24 filters in 32-lane groups; zero point 128 in the padding
    (2, 3, 50, 64, 64, 1, (1, 1, 1, 1), I8, U8, -7, 9, True, True, None),          # 64 filters (two groups), signed input, general requantisation
    (1, 1, 72, 128, 16, 1, (0, 1, 1, 1), I8, I8, 5, -2, False, False, "relu"),     # one channel, eight groups, no padding above
    (8, 2, 52, 64, 8, 2, (1, 1, 0, 0), U8, U8, 17, 3, True, True, "relu6"),        # eight filters; 26 x 32 output: groups of 112 pixels, the last ragged
    (1, 3, 224, 224, 32, 2, (1, 1, 1, 1), U8, I8, 0, 0, True, True, "relu6"),      # the MobileNet stem itself: 13 tiles, the last partly empty
    (1, 3, 64, 416, 16, 1, (1, 1, 1, 1), U8, I8, 0, 0, True, True, None),          # detector rows: a tile spans five output rows
]


@pytest.mark.parametrize("case", STEM_QCONV, ids=[f"stem{i}" for i in range(len(STEM_QCONV))])
def test_qlinearconv_stem_patches(ctx, oracle, case):
    N, C, H, W, M, s, pads, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 43 + C + M + W)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C, 3, 3), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, M).astype(np.int32) if has_bias else None
    y_scale = 0.03 * np.sqrt(C * 9)
    kw = dict(bias=bias, y_dtype=ydt, stride=(s, s), pads=pads, dilations=(1, 1), group=1, activation=act)
    before = ctx.launch_count()
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    launches = ctx.launch_count() - before
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert launches == 1
    assert len(np.unique(want)) > 16


@pytest.mark.parametrize("case,launches", list(zip(TC_QCONV, TC_QCONV_LAUNCHES)), ids=[f"tcqconv{i}" for i in range(len(TC_QCONV))])
def test_qlinearconv_tensor_core_path(ctx, oracle, case, launches):
    N, C, H, W, M, k, stride, pads, dil, xdt, ydt, xzp, yzp, per_ch, has_bias, act = case
    rng = np.random.default_rng(N * 31 + C + M)
    x = q(rng, (N, C, H, W), xdt)
    w = rng.integers(-127, 128, (M, C, k, k), dtype=np.int8)
    ws = (rng.random(M if per_ch else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-3000, 3000, M).astype(np.int32) if has_bias else None
    y_scale = 0.015 * np.sqrt(C * k * k)
    kw = dict(bias=bias, y_dtype=ydt, stride=stride, pads=pads, dilations=dil, group=1, activation=act)
    before = ctx.launch_count()
    got = ctx.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    n_launches = ctx.launch_count() - before
    want = oracle.qlinearconv(x, 0.02, xzp, w, ws, None, y_scale, yzp, **kw)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert n_launches == launches    # a tensor-core path, not the generic kernel
    assert len(np.unique(want)) > 8


@pytest.mark.parametrize("M,K,N", [(256, 64, 64), (1000, 1600, 512), (300, 70, 10), (513, 1280, 1000)])
@pytest.mark.parametrize("adt,ydt,azp,yzp,act", [(I8, I8, 0, 0, "relu"), (U8, U8, 128, 7, None), (I8, I8, 9, -4, "relu6")])
def test_qlinearmatmul_tensor_core_path(ctx, oracle, M, K, N, adt, ydt, azp, yzp, act):
    rng = np.random.default_rng(M + K + N)
    a = q(rng, (M, K), adt)
    b = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bs = (rng.random(N, dtype=np.float32) * 0.01 + 0.001).astype(np.float32)
    bias = rng.integers(-500, 500, N).astype(np.int32)
    ys = 0.02 * np.sqrt(K)
    before = ctx.launch_count()
    got = ctx.qlinearmatmul(a, 0.02, azp, b, bs, None, ys, yzp, bias, ydt, act)
    assert ctx.launch_count() - before == 2
    want = oracle.qlinearmatmul(a, 0.02, azp, b, bs, None, ys, yzp, bias, ydt, act)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt,scale,zp", [(U8, 1 / 255, 0), (I8, 0.02, 0), (I8, 0.013, -7), (U8, 0.031, 128), (I8, 0.1, 127), (U8, 3.7e-3, 255)])
def test_quantize_rounding_boundaries(ctx, oracle, dt, scale, zp):
    """QuantizeLinear takes the division only where a multiply cannot prove the rounding.  The values that decide it: every
    k + 0.5 of the output range times the scale, the floats next to each of them, the clamp bounds, and non-finite inputs."""
    s = np.float32(scale)
    lo, hi = (0, 255) if dt == U8 else (-128, 127)
    ks = np.arange(lo - zp - 3, hi - zp + 4, dtype=np.float32)
    centre = ((ks + np.float32(0.5)) * s).astype(np.float32)
    xs = [centre, np.nextafter(centre, np.float32(np.inf)), np.nextafter(centre, np.float32(-np.inf)), (ks * s).astype(np.float32)]
    for _ in range(3):                                        # a few more steps away from the boundary, both ways
        xs.append(np.nextafter(xs[1] if len(xs) % 2 else xs[2], np.float32(np.inf if len(xs) % 2 else -np.inf)))
    special = np.array([np.inf, -np.inf, np.nan, 0.0, -0.0, 1e30, -1e30, 1e-40], np.float32)
    x = np.concatenate(xs + [special]).astype(np.float32)
    x = np.concatenate([x, np.zeros((-len(x)) % 4, np.float32)])          # the vector path takes whole float4s
    got, want = ctx.quantize_linear(x, scale, zp, dt), oracle.quantize_linear(x, scale, zp, dt)
    assert np.array_equal(got, want)


def test_fused_cnn_input_quantisation_on_rounding_boundaries(zb, ctx, oracle):
    """The fused first stage of the int8 CNN quantises its float input itself: images made of rounding-boundary values."""
    import graph_oracle
    from zant_b200 import models
    g = models.small_cnn_int8(6)
    s = np.float32(1.0) / np.float32(255.0)
    ks = np.arange(0, 28 * 28, dtype=np.float32) % 256
    centre = ((ks + np.float32(0.5)) * s).astype(np.float32).reshape(1, 1, 28, 28)
    x = np.concatenate([centre, np.nextafter(centre, np.float32(np.inf)), np.nextafter(centre, np.float32(-np.inf)),
                        centre[:, :, ::-1], np.full_like(centre, 2.0), np.full_like(centre, -1.0)]).astype(np.float32)
    want = graph_oracle.run(oracle, g, x)[g.output]
    plan = zb.Plan(ctx, g, fuse=True)
    assert any("Fused" in n for n in plan.step_names())
    assert np.array_equal(plan.run(x).view(np.uint32), want.view(np.uint32))
    plan.close()


@pytest.mark.parametrize("dt,a_s,a_zp,b_s,b_zp,y_s,y_zp,act", [
    (I8, 0.031, 0, 0.017, -4, 0.045, 0, None), (U8, 0.031, 120, 0.017, 117, 0.045, 120, "relu"), (I8, 0.1, 0, 0.1, 0, 0.1, 0, None),
    (I8, 0.05, 3, 0.025, -7, 0.0125, 5, "relu6"), (I8, 0.047244094, 0, 0.1, 0, 0.1, 0, None), (U8, 0.02, 0, 0.02, 255, 0.01, 7, None)])
def test_qlinearadd_every_code_pair(ctx, oracle, dt, a_s, a_zp, b_s, b_zp, y_s, y_zp, act):
    """All 65536 pairs of codes: the vector kernel takes the division only where a multiply cannot prove the rounding (exact
    halves are common here: equal scales, scale ratios of two)."""
    codes = np.arange(256, dtype=np.uint8).view(np.int8 if dt == I8 else np.uint8)
    a = np.repeat(codes, 256).reshape(1, 256, 16, 16)
    b = np.tile(codes, 256).reshape(1, 256, 16, 16)
    got = ctx.qlinearadd(a, a_s, a_zp, b, b_s, b_zp, y_s, y_zp, act)
    want = oracle.qlinearadd(a, a_s, a_zp, b, b_s, b_zp, y_s, y_zp, act)
    assert np.array_equal(got, want)
