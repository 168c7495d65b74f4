"""Hand-computed vectors for the quantized oracle functions.

The reference tree contains no quantized operators, so there is nothing of its own to pin these
against ("parity unpinned"); the vectors below pin the arithmetic order stated in
include/zant_b200.h with cases small enough to verify on paper (power-of-two scales make every
intermediate exact).
"""
import numpy as np

I8, U8, I32 = 1, 2, 3


def test_quantize_linear_ties_to_even_and_saturation(oracle):
    x = np.array([0.0, 0.25, 0.75, 1.25, -0.25, -0.75, 100.0, -100.0, 0.5, 1.0], np.float32)
    # scale 0.5: x/s = 0, .5, 1.5, 2.5, -.5, -1.5, 200, -200, 1, 2 -> rne 0,0,2,2,-0,-2,(clamped),..,1,2
    assert oracle.quantize_linear(x, 0.5, 0, I8).tolist() == [0, 0, 2, 2, 0, -2, 127, -128, 1, 2]
    assert oracle.quantize_linear(x, 0.5, 10, U8).tolist() == [10, 10, 12, 12, 10, 8, 210, 0, 11, 12]


def test_dequantize_linear(oracle):
    q = np.array([-128, -1, 0, 1, 127], np.int8)
    assert oracle.dequantize_linear(q, 0.5, 1).tolist() == [-64.5, -1.0, -0.5, 0.0, 63.0]


def test_qlinearconv_by_hand(oracle):
    # 1x1x3x3 input, 1x1x2x2 kernel of ones, scales 0.5*0.5/0.25 = 1 -> y = acc + bias
    x = np.arange(1, 10, dtype=np.int8).reshape(1, 1, 3, 3)
    w = np.ones((1, 1, 2, 2), np.int8)
    y = oracle.qlinearconv(x, 0.5, 0, w, [0.5], None, 0.25, 0, bias=np.array([3], np.int32))
    assert y.reshape(-1).tolist() == [12 + 3, 16 + 3, 24 + 3, 28 + 3]
    # zero points: (x - 1) and (w - (-1)) = 2 -> acc = 2 * sum(x - 1); multiplier 0.125 ; y_zp 5
    y = oracle.qlinearconv(x, 0.5, 1, w, [0.5], [-1], 2.0, 5, y_dtype=U8)
    assert y.reshape(-1).tolist() == [int(np.rint(2 * s * 0.125)) + 5 for s in (8, 12, 20, 24)]
    # padding contributes zero in the real domain even with a non-zero x zero point
    y = oracle.qlinearconv(np.full((1, 1, 1, 1), 5, np.int8), 1.0, 5, np.ones((1, 1, 3, 3), np.int8), [1.0], None, 1.0, 0, pads=(1, 1, 1, 1))
    assert y.reshape(-1).tolist() == [0]
    # fused activations
    xn = np.array([-4, 4, 40, 100], np.int8).reshape(1, 1, 2, 2)
    one = np.ones((1, 1, 1, 1), np.int8)
    assert oracle.qlinearconv(xn, 0.5, 0, one, [1.0], None, 0.5, 0).reshape(-1).tolist() == [-4, 4, 40, 100]
    assert oracle.qlinearconv(xn, 0.5, 0, one, [1.0], None, 0.5, 0, activation="relu").reshape(-1).tolist() == [0, 4, 40, 100]
    assert oracle.qlinearconv(xn, 0.5, 0, one, [1.0], None, 0.5, 0, activation="relu6").reshape(-1).tolist() == [0, 4, 12, 12]


def test_depthwise_by_hand(oracle):
    x = np.stack([np.full((2, 2), 1, np.int8), np.full((2, 2), 2, np.int8)])[None]
    w = np.array([3, -5], np.int8).reshape(2, 1, 1, 1)
    y = oracle.qlinearconv(x, 1.0, 0, w, [1.0, 0.5], None, 1.0, 0, group=2)
    assert y[0, 0].reshape(-1).tolist() == [3] * 4 and y[0, 1].reshape(-1).tolist() == [-5] * 4   # -10 * 0.5


def test_qlinearmatmul_by_hand(oracle):
    a = np.array([[1, 2], [3, 4]], np.int8)
    b = np.array([[1, -1], [2, 0]], np.int8)
    y = oracle.qlinearmatmul(a, 0.5, 0, b, [0.5, 1.0], None, 0.25, 0)
    assert y.tolist() == [[5, -2], [11, -6]]             # acc [[5,-1],[11,-3]] * multipliers [1, 2]
    y = oracle.qlinearmatmul(a, 0.5, 0, b, [0.5, 1.0], None, 0.25, 0, y_dtype=I32)
    assert y.tolist() == [[5, -1], [11, -3]]
    # rne at a tie: acc 1 * multiplier 0.5 -> 0.5 -> 0 ; acc 3 * 0.5 = 1.5 -> 2
    y = oracle.qlinearmatmul(np.array([[1], [3]], np.int8), 1.0, 0, np.array([[1]], np.int8), [1.0], None, 2.0, 0)
    assert y.reshape(-1).tolist() == [0, 2]


def test_qlinearadd_and_gap_by_hand(oracle):
    a = np.array([10, -20, 127], np.int8)
    b = np.array([4, 8, 127], np.int8)
    # (a*0.5 + b*0.25) / 0.5 = a + b/2
    assert oracle.qlinearadd(a, 0.5, 0, b, 0.25, 0, 0.5, 0).tolist() == [12, -16, 127]
    x = np.array([[1, 2, 3, 4], [10, 10, 10, 12]], np.int8).reshape(1, 2, 2, 2)
    # sums 10 and 42; * 0.5 / 4 / 0.25 = 5 and 21
    assert oracle.qlinear_global_avgpool(x, 0.5, 0, 0.25, 0).reshape(-1).tolist() == [5, 21]


def test_leaky_lut_by_hand(oracle):
    lut = oracle.build_leaky_lut(I8, 1.0, 0, 0.5, 1.0, 0)
    codes = np.array([-4, -3, -1, 0, 5], np.int8)
    # leaky(0.5): -2, -1.5 -> -2 (tie to even), -0.5 -> 0 (tie to even), 0, 5
    assert oracle.lut_q8(codes, lut).tolist() == [-2, -2, 0, 0, 5]


def test_oracle_conv_second_opinion_torch(oracle):
    """Independent check of the FP32 oracle against torch's CPU convolution (different algorithm,
    so only to tolerance)."""
    import torch
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 5, 12, 11)).astype(np.float32)
    w = rng.standard_normal((7, 5, 3, 3)).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    got = oracle.Conv(x, w, b, (2, 1), (1, 2, 1, 2), (1, 1), None, "NOTSET")
    ref = torch.nn.functional.conv2d(torch.nn.functional.pad(torch.from_numpy(x), (2, 2, 1, 1)), torch.from_numpy(w),
                                     torch.from_numpy(b), stride=(2, 1)).numpy()
    assert got.shape == ref.shape and np.allclose(got, ref, rtol=1e-4, atol=1e-4)


def test_oracle_qconv_second_opinion_numpy(oracle):
    rng = np.random.default_rng(1)
    x = rng.integers(-128, 128, (1, 3, 6, 6), dtype=np.int8)
    w = rng.integers(-127, 128, (4, 3, 3, 3), dtype=np.int8)
    got = oracle.qlinearconv(x, 0.02, 0, w, [0.02], None, 0.02 * 5, 0, pads=(1, 1, 1, 1))
    xp = np.pad(x.astype(np.int64), ((0, 0), (0, 0), (1, 1), (1, 1)))
    acc = np.zeros((1, 4, 6, 6), np.int64)
    for kh in range(3):
        for kw in range(3):
            acc += np.einsum("nchw,mc->nmhw", xp[:, :, kh:kh + 6, kw:kw + 6], w[:, :, kh, kw].astype(np.int64))
    m = np.float32(np.float32(0.02) * np.float32(0.02)) / np.float32(0.02 * 5)
    ref = np.clip(np.rint(acc.astype(np.float32) * m), -128, 127).astype(np.int8)
    assert np.array_equal(got, ref)
