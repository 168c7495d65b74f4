"""FP32 operators: CUDA (through the C ABI) against the CPU oracle on seeded random inputs.

The back end's FP32 kernels keep the reference's order of operations (sequential k, separate
multiply and add), so the comparison is bit-exact, which is stricter than the 1e-4 relative
tolerance the float path is allowed.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rnd(rng, shape):
    return rng.standard_normal(shape).astype(np.float32)


def same(a, b):
    assert a.shape == b.shape, (a.shape, b.shape)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), f"max |d| = {np.abs(a - b).max()}"


CONV_CASES = [
    # N, C, H, W, M, KH, KW, stride, pads, dilations, auto_pad, bias
    (1, 1, 28, 28, 32, 3, 3, (1, 1), (0, 0, 0, 0), (1, 1), "NOTSET", True),
    (3, 32, 13, 13, 64, 3, 3, (1, 1), (0, 0, 0, 0), (1, 1), "NOTSET", True),
    (2, 3, 17, 19, 5, 3, 3, (2, 2), (1, 1, 1, 1), (1, 1), "NOTSET", False),
    (2, 4, 9, 11, 7, 2, 3, (1, 2), (0, 1, 2, 0), (2, 1), "NOTSET", True),
    (1, 5, 10, 10, 70, 3, 3, (1,), None, None, "SAME_UPPER", True),
    (1, 5, 11, 9, 3, 3, 2, (2,), None, None, "SAME_LOWER", False),
    (2, 2, 8, 8, 4, 5, 5, (1, 1), None, (1,), "VALID", True),
    (1, 3, 8, 8, 4, 1, 1, (1, 1), (1, 1, 1, 1), None, None, True),      # pads ignored without auto_pad
    (2, 17, 6, 6, 130, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1), "NOTSET", True),  # K and M not multiples of the tile
    (1, 1, 5, 5, 1, 2, 2, (1,), None, (2,), None, True),
]


@pytest.mark.parametrize("case", CONV_CASES, ids=[f"conv{i}" for i in range(len(CONV_CASES))])
def test_conv_lean(ctx, oracle, case):
    N, C, H, W, M, KH, KW, stride, pads, dil, ap, has_bias = case
    rng = np.random.default_rng(100 + N * 7 + C)
    x, w = rnd(rng, (N, C, H, W)), rnd(rng, (M, C, KH, KW))
    b = rnd(rng, (M,)) if has_bias else None
    if ap is None and pads is not None and any(pads):
        # Quirk of the reference: the allocating wrapper sizes the output WITH the pads, the lean
        # function ignores pads when auto_pad is null, so the call ends in InvalidDimensions.
        with pytest.raises(oracle.OracleError) as eo:
            oracle.Conv(x, w, b, stride, pads, dil, None, ap)
        with pytest.raises(Exception) as ez:
            ctx.Conv(x, w, b, stride, pads, dil, None, ap)
        assert eo.value.name == ez.value.name == "InvalidDimensions"
        pads = None
    want = oracle.Conv(x, w, b, stride, pads, dil, None, ap)
    got = ctx.conv_lean(x, w, want.shape, b, stride, pads, dil, None, ap)
    same(got, want)


def test_conv_zero_pad_taps_are_multiplied_like_the_reference(ctx, oracle):
    # The reference multiplies the zero padding by the weight (0 * inf = NaN); skipping the tap would hide that.
    x = np.ones((1, 1, 3, 3), np.float32)
    w = np.full((1, 1, 3, 3), np.inf, np.float32)
    want = oracle.Conv(x, w, None, (1,), (1, 1, 1, 1), None, None, "NOTSET")
    got = ctx.conv_lean(x, w, want.shape, None, (1,), (1, 1, 1, 1), None, None, "NOTSET")
    assert np.array_equal(np.isnan(got), np.isnan(want))


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (2, 2, 2), (7, 1600, 512), (3, 512, 10), (65, 33, 129), (128, 64, 64), (1, 300, 70)])
def test_mat_mul(ctx, oracle, M, K, N):
    rng = np.random.default_rng(M * 1000 + K + N)
    a, b = rnd(rng, (M, K)), rnd(rng, (K, N))
    same(ctx.mat_mul(a, b), oracle.mat_mul(a, b))


def test_mat_mul_uses_last_two_dims_only(ctx, oracle):
    rng = np.random.default_rng(3)
    a, b = rnd(rng, (1, 1, 5, 6)), rnd(rng, (1, 1, 6, 4))
    same(ctx.mat_mul(a, b), oracle.mat_mul(a, b))


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("cmode", ["none", "full", "row", "col", "scalar"])
def test_gemm(ctx, oracle, ta, tb, cmode):
    rng = np.random.default_rng(11 + ta * 2 + tb)
    rows, K, cols = 37, 53, 29
    a = rnd(rng, (1, 1, K, rows) if ta else (1, 1, rows, K))
    b = rnd(rng, (1, 1, cols, K) if tb else (1, 1, K, cols))
    c = {"none": None, "full": (1, 1, rows, cols), "row": (1, 1, 1, cols), "col": (1, 1, rows, 1), "scalar": (1, 1, 1, 1)}[cmode]
    c = None if c is None else rnd(rng, c)
    same(ctx.gemm(a, b, c, 1.5, -0.75, ta, tb), oracle.gemm(a, b, c, 1.5, -0.75, ta, tb))


def test_gemm_classifier_shape(ctx, oracle):
    rng = np.random.default_rng(12)
    a, b, c = rnd(rng, (1, 1, 4, 1280)), rnd(rng, (1, 1, 1000, 1280)), rnd(rng, (1, 1, 1, 1000))
    same(ctx.gemm(a, b, c, 1.0, 1.0, False, True), oracle.gemm(a, b, c, 1.0, 1.0, False, True))


POOL_CASES = [
    ((2, 32, 26, 26), (2, 2), (2, 2), (1, 1), (0, 0, 0, 0), "NOTSET", False),
    ((1, 64, 11, 11), (2, 2), (2, 2), (1, 1), (0, 0, 0, 0), "NOTSET", False),
    ((1, 3, 13, 13), (2, 2), (1, 1), (1, 1), (0, 0, 0, 0), "SAME_UPPER", False),
    ((1, 3, 13, 13), (2, 2), (1, 1), (1, 1), (0, 0, 0, 0), "SAME_LOWER", False),
    ((2, 2, 9, 7), (3, 2), (2, 1), (2, 2), (1, 0, 1, 1), "NOTSET", False),
    ((1, 2, 7, 7), (3, 3), (2, 2), (1, 1), (0, 0, 0, 0), "NOTSET", True),
    ((1, 1, 6, 6), (2, 2), (2, 2), (1, 1), (0, 0, 0, 0), "VALID", False),
]


@pytest.mark.parametrize("case", POOL_CASES, ids=[f"pool{i}" for i in range(len(POOL_CASES))])
def test_onnx_maxpool(ctx, oracle, case):
    xs, k, s, d, p, ap, ceil = case
    x = rnd(np.random.default_rng(7), xs)
    same(ctx.onnx_maxpool(x, k, s, d, p, ap, ceil), oracle.onnx_maxpool(x, k, s, d, p, ap, ceil))


@pytest.mark.parametrize("n", [0, 1, 3, 4, 1023, 4096, 100003])
def test_activations(ctx, oracle, n):
    x = rnd(np.random.default_rng(n), (n,))
    if n:
        x[0] = 0.0
    if n > 2:
        x[1], x[2] = -0.0, np.float32(1e-38)
    same(ctx.ReLU(x), oracle.ReLU(x))
    same(ctx.leakyReLU(x, 0.1), oracle.leakyReLU(x, 0.1))
    same(ctx.leakyReLU(x, 0.01), oracle.leakyReLU(x, 0.01))
    same(ctx.clip(x, 0.0, 6.0), oracle.clip(x, 0.0, 6.0))


def test_relu_does_not_need_a_zeroed_output(ctx):
    # lean_ReLU writes only positive inputs (the generated code zeroes outputs first); this back end writes all.
    x = np.array([-1.0, 2.0, -3.0, 4.0, 0.0], np.float32)
    out = np.full(5, 7.0, np.float32)
    ctx.ReLU(x, out=out)
    assert out.tolist() == [0.0, 2.0, 0.0, 4.0, 0.0]


ADD_CASES = [((2, 3, 4, 5), (2, 3, 4, 5)), ((6, 512), (512,)), ((2, 3, 4, 5), (5,)), ((2, 3, 4, 5), (1, 1, 4, 5)),
             ((4, 5), (2, 3, 4, 5)), ((2, 8, 6, 6), (8, 1, 1)), ((2, 3, 1, 5), (1, 3, 4, 1)), ((24,), (2, 3, 4)), ((3, 1), (1, 4))]


@pytest.mark.parametrize("sa,sb", ADD_CASES, ids=[f"add{i}" for i in range(len(ADD_CASES))])
def test_sum_tensors(ctx, oracle, sa, sb):
    rng = np.random.default_rng(len(sa) * 10 + len(sb))
    a, b = rnd(rng, sa), rnd(rng, sb)
    want, flag = oracle.sum_tensors(a, b, return_flag=True)
    same(ctx.sum_tensors(a, b), want)
    # flag != 0 marks shapes where the reference itself indexes outside the operand (documented deviation)
    if (sa, sb) == ((2, 8, 6, 6), (8, 1, 1)):
        assert flag == 1


def test_sum_tensors_incompatible(zb, ctx):
    with pytest.raises(zb.ZantError) as e:
        ctx.sum_tensors(np.zeros((2, 3), np.float32), np.zeros((4,), np.float32))
    assert e.value.name == "IncompatibleBroadcastShapes"


@pytest.mark.parametrize("nt", [1, 2, 3, 8, 9, 17])
def test_sum_tensor_list(ctx, oracle, nt):
    rng = np.random.default_rng(nt)
    ts = [rnd(rng, (5, 7, 3)) for _ in range(nt)]
    same(ctx.sum_tensor_list(ts), oracle.sum_tensor_list(ts))


CONCAT_CASES = [([(2, 128, 6, 6), (2, 256, 6, 6)], 1), ([(3, 4), (5, 4), (1, 4)], 0), ([(2, 3, 5), (2, 3, 2), (2, 3, 1)], -1),
                ([(2, 3), (3,)], 0), ([(1, 7, 3, 3)], 1), ([(2, 3, 4, 5), (2, 3, 4, 5)], 2)]


@pytest.mark.parametrize("shapes,axis", CONCAT_CASES, ids=[f"cat{i}" for i in range(len(CONCAT_CASES))])
@pytest.mark.parametrize("dt", [np.float32, np.int8, np.uint8])
def test_concatenate(ctx, oracle, shapes, axis, dt):
    rng = np.random.default_rng(9)
    ts = [(rng.standard_normal(s) * 50).astype(dt) for s in shapes]
    got, want = ctx.concatenate(ts, axis), oracle.concatenate(ts, axis)
    assert got.shape == want.shape and np.array_equal(got, want)


RESIZE_CASES = [((2, 128, 13, 13), [1, 1, 2, 2], None, "half_pixel"), ((1, 3, 5, 7), [1, 1, 2, 2], None, "asymmetric"),
                ((1, 2, 4, 4), [1, 1, 1.5, 2.5], None, "half_pixel"), ((1, 2, 6, 6), None, [1, 2, 9, 4], "align_corners"),
                ((4,), [2.0], None, "half_pixel"), ((3, 5), None, [7, 2], "asymmetric")]


@pytest.mark.parametrize("xs,scales,sizes,cm", RESIZE_CASES, ids=[f"rs{i}" for i in range(len(RESIZE_CASES))])
@pytest.mark.parametrize("dt", [np.float32, np.uint8])
def test_resize_nearest(ctx, oracle, xs, scales, sizes, cm, dt):
    x = (np.random.default_rng(4).standard_normal(xs) * 40).astype(dt)
    got, want = ctx.resize(x, "nearest", scales, sizes, cm), oracle.resize(x, "nearest", scales, sizes, cm)
    assert got.shape == want.shape and np.array_equal(got, want)


REDUCE_CASES = [((2, 1280, 7, 7), [2, 3], True), ((2, 3, 4, 5), [1], False), ((2, 3, 4, 5), [0, 2], True), ((2, 3, 4, 5), [-1], False),
                ((2, 3, 4, 5), [3, 1], True), ((6, 5), None, True), ((2, 3, 4), [0, 1, 2], False)]


@pytest.mark.parametrize("xs,axes,keep", REDUCE_CASES, ids=[f"rm{i}" for i in range(len(REDUCE_CASES))])
def test_reduce_mean(ctx, oracle, xs, axes, keep):
    x = rnd(np.random.default_rng(8), xs)
    same(ctx.reduce_mean(x, axes, keep, False), oracle.reduce_mean(x, axes, keep, False))


def test_reduce_mean_noop(ctx, oracle):
    x = rnd(np.random.default_rng(8), (3, 4))
    same(ctx.reduce_mean(x, None, True, True), x)


def test_reshape(ctx, oracle):
    x = rnd(np.random.default_rng(2), (4, 64, 5, 5))
    got = ctx.reshape(x, [0, "SIZE_MAX"])
    assert got.shape == (4, 1600) and np.array_equal(got, x.reshape(4, 1600))


def test_device_pointers_are_used_in_place(ctx, oracle):
    torch = pytest.importorskip("torch")
    x = rnd(np.random.default_rng(21), (5, 1000))
    xd = torch.from_numpy(x).cuda()
    yd = torch.empty_like(xd)
    ctx.ReLU(xd, out=yd)
    ctx.synchronize()
    same(yd.cpu().numpy(), oracle.ReLU(x))


# ------------------------------------------------------------------------------------------------
# Sigmoid / Softmax / Tanh / Ceil / Mul / Div (the next operators the code generator can emit).
# Mul, Div and Ceil are single rounded operations: bit-identical.  The others go through exp / tanh
# of two different math libraries: the FP32 contract (1e-4 relative) with a much tighter bound in fact.
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [0, 1, 7, 1024, 100003])
def test_mul_div_ceil_bit_identical(ctx, oracle, n):
    rng = np.random.default_rng(n + 3)
    a = (rng.standard_normal(n) * 50).astype(np.float32)
    b = (rng.standard_normal(n) * 3 + 0.5).astype(np.float32)
    for name in ("mul", "div"):
        got, want = getattr(ctx, name)(a, b), getattr(oracle, name)(a, b)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
    x = np.concatenate([a, np.array([np.inf, -np.inf, np.nan, -0.0, 2.0], np.float32)])
    assert np.array_equal(ctx.ceil(x).view(np.uint32), oracle.ceil(x).view(np.uint32))


def test_mul_div_reject_different_sizes(zb, ctx):
    for fn in (ctx.mul, ctx.div):
        with pytest.raises(zb.ZantError) as e:
            fn(np.zeros((2, 3), np.float32), np.zeros((3, 3), np.float32))
        assert e.value.name == "MismatchedShape"


@pytest.mark.parametrize("n", [1, 33, 4096, 70001])
def test_sigmoid_tanh(ctx, oracle, n):
    x = (np.random.default_rng(n).standard_normal(n) * 6).astype(np.float32)
    for name in ("sigmoid", "tanh"):
        got, want = getattr(ctx, name)(x), getattr(oracle, name)(x)
        tol = 1e-4 * np.maximum(np.abs(want), 1e-2 * np.abs(want).max())
        assert np.all(np.abs(got - want) <= tol), name
        assert np.abs(got - want).max() <= 4e-7, name          # a few units in the last place of values below 1


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 10), (257, 1000), (4096, 7)])
def test_softmax_rows(ctx, oracle, rows, cols):
    x = (np.random.default_rng(rows * cols).standard_normal((rows, cols)) * 8).astype(np.float32)
    got, want = ctx.softmax(x), oracle.softmax(x)
    tol = 1e-4 * np.maximum(np.abs(want), 1e-2 * np.abs(want).max())
    assert np.all(np.abs(got - want) <= tol)
    assert np.all(np.abs(got.astype(np.float64).sum(axis=1) - 1.0) < 1e-5)


def test_next_operators_in_a_plan(zb, ctx, oracle):
    """MatMul -> Sigmoid -> Mul -> Div -> Tanh -> Ceil -> Softmax as plan nodes against the graph oracle."""
    import graph_oracle
    rng = np.random.default_rng(5)
    g = zb.Graph("next_ops")
    F32 = zb.F32
    x = g.tensor("x", F32, (6, 16))
    w = g.tensor("w", F32, (16, 12), rng.standard_normal((16, 12)).astype(np.float32))
    s = g.tensor("s", F32, (6, 12), (rng.standard_normal((6, 12)) * 4).astype(np.float32))
    d = g.tensor("d", F32, (6, 12), (rng.random((6, 12)) + 0.5).astype(np.float32))
    ids = [g.tensor(n, F32, (6, 12)) for n in ("mm", "sig", "mul", "div", "tanh", "ceil", "soft")]
    g.node("MatMul", [x, w], [ids[0]])
    g.node("Sigmoid", [ids[0]], [ids[1]])
    g.node("Mul", [ids[1], s], [ids[2]])
    g.node("Div", [ids[2], d], [ids[3]])
    g.node("Tanh", [ids[3]], [ids[4]])
    g.node("Ceil", [ids[3]], [ids[5]])
    g.node("Softmax", [ids[4]], [ids[6]])
    g.input, g.output = x, ids[6]
    xin = rng.standard_normal((6, 16)).astype(np.float32)
    want = graph_oracle.run(oracle, g, xin)
    plan = zb.Plan(ctx, g)
    got = plan.run(xin)
    assert np.abs(got - want[ids[6]]).max() <= 1e-5
    assert np.abs(plan.read_tensor(ids[3]) - want[ids[3]]).max() <= 1e-4 * np.abs(want[ids[3]]).max()
    # ceil of nearly equal inputs can differ by one where the input sits on an integer; compare where it does not
    far = np.abs(want[ids[3]] - np.round(want[ids[3]])) > 1e-3
    assert np.array_equal(plan.read_tensor(ids[5])[far], want[ids[5]][far])
    plan.close()


# ------------------------------------------------------------------------------------------------
# Transpose / Slice / Gather: elements are moved, so every dtype is bit-identical to the oracle.
# ------------------------------------------------------------------------------------------------
def same_bytes(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    assert a.tobytes() == b.tobytes()


@pytest.mark.parametrize("shape,perm", [((7,), None), ((5, 9), None), ((3, 4, 5), [1, 2, 0]), ((2, 3, 4, 5), [0, 2, 3, 1]),
                                        ((2, 3, 4, 5), [3, 2, 1, 0]), ((4, 1, 6), [2, 0, 1]), ((2, 64, 17, 9), [0, 2, 3, 1])])
@pytest.mark.parametrize("dt", [np.float32, np.int8, np.uint8, np.int32])
def test_transpose_onnx(ctx, oracle, shape, perm, dt):
    x = np.random.default_rng(len(shape)).integers(-100, 100, shape).astype(dt)
    same_bytes(ctx.transpose_onnx(x, perm), oracle.transpose_onnx(x, perm))
    assert np.array_equal(ctx.transpose_onnx(x, perm), np.transpose(x, perm))


def test_transpose_onnx_errors(zb, ctx):
    x = np.zeros((2, 3), np.float32)
    for perm in ([0, 1, 2], [0, 0], [0, 2]):
        with pytest.raises(zb.ZantError) as e:
            ctx.transpose_onnx(x, perm)
        assert e.value.name == "InvalidPermutation"


SLICES = [
    ((10,), [2], [8], None, None), ((10,), [-3], [100], None, None), ((6, 7), [1, 2], [5, 6], None, [2, 3]),
    ((4, 5, 6), [1], [4], [1], None), ((4, 5, 6), [0, 1], [4, 6], [0, -1], [3, 2]), ((8,), [6], [1], [0], [-2]),
    ((5, 5), [4, 4], [-6, 0], None, [-1, -2]), ((3, 4), [2], [2], [0], None), ((2, 3, 4, 5), [1, 0], [2, 5], [0, 3], [1, 4]),
]


@pytest.mark.parametrize("shape,starts,ends,axes,steps", SLICES)
@pytest.mark.parametrize("dt", [np.float32, np.uint8])
def test_slice_onnx(ctx, oracle, shape, starts, ends, axes, steps, dt):
    x = np.arange(int(np.prod(shape))).reshape(shape).astype(dt)
    got, want = ctx.slice_onnx(x, starts, ends, axes, steps), oracle.slice_onnx(x, starts, ends, axes, steps)
    same_bytes(got, want)
    for lean in (False, True):
        assert ctx.get_slice_output_shape(shape, starts, ends, axes, steps, lean=lean) == oracle.get_slice_output_shape(shape, starts, ends, axes, steps, lean=lean)
    if steps is None or all(s > 0 for s in steps):
        # positive steps: the reference agrees with NumPy slicing
        sl = [slice(None)] * len(shape)
        for i, (s0, e0) in enumerate(zip(starts, ends)):
            ax = axes[i] if axes is not None else i
            sl[ax] = slice(s0, e0, steps[i] if steps is not None else 1)
        assert np.array_equal(got, x[tuple(sl)])


def test_slice_onnx_errors(zb, ctx):
    x = np.zeros((5, 5, 5), np.float32)
    for args, name in ((([1], [4], [5], None), "InvalidSliceIndices"), (([1], [4], None, [0]), "InvalidSliceStep"),
                       (([1, 2], [4], None, None), "InvalidSliceIndices")):
        with pytest.raises(zb.ZantError) as e:
            ctx.slice_onnx(x, *args)
        assert e.value.name == name


@pytest.mark.parametrize("shape,idx_shape,axis", [((9,), (4,), 0), ((3, 3), (2,), 0), ((2, 4), (2, 2), 1), ((5, 6, 7), (3,), -2),
                                                  ((4, 5, 6), (2, 3), 0), ((1000, 64), (128,), 0), ((2, 3, 4, 5), (1,), 3)])
@pytest.mark.parametrize("dt", [np.float32, np.int8])
def test_gather(ctx, oracle, shape, idx_shape, axis, dt):
    rng = np.random.default_rng(sum(shape))
    x = rng.integers(-100, 100, shape).astype(dt)
    idx = rng.integers(0, shape[axis], idx_shape).astype(np.uint64)
    got = ctx.gather(x, idx, axis)
    same_bytes(got, oracle.gather(x, idx, axis))
    assert np.array_equal(got, np.take(x, idx.astype(np.int64), axis=axis))


def test_gather_errors(zb, ctx):
    x = np.zeros((2, 2), np.uint8)
    with pytest.raises(zb.ZantError) as e:
        ctx.gather(x, np.array([2], np.uint64), 0)
    assert e.value.name == "IndexOutOfBounds"
    for axis in (2, -3):
        with pytest.raises(zb.ZantError) as e:
            ctx.gather(x, np.array([0], np.uint64), axis)
        assert e.value.name == "InvalidAxis"


def test_movement_operators_in_a_plan(zb, ctx, oracle):
    import graph_oracle
    g = zb.Graph("moves")
    x = g.tensor("x", zb.F32, (2, 6, 4, 5))
    t = g.tensor("t", zb.F32, (2, 4, 5, 6))
    s = g.tensor("s", zb.F32, (2, 2, 5, 3))
    idx = g.tensor("idx", zb.I32, (2, 2), np.array([[2, 0], [1, 1]], np.int32))
    y = g.tensor("y", zb.F32, (2, 2, 2, 2, 3))
    g.node("Transpose", [x], [t], perm=[0, 2, 3, 1])
    g.node("Slice", [t], [s], starts=[1, 0], ends=[3, 6], slice_axes=[1, 3], steps=[1, 2])
    g.node("Gather", [s, idx], [y], axis=2)
    g.input, g.output = x, y
    xin = np.random.default_rng(8).standard_normal((2, 6, 4, 5)).astype(np.float32)
    want = graph_oracle.run(oracle, g, xin)
    plan = zb.Plan(ctx, g)
    same_bytes(plan.run(xin), want[y])
    ref = np.take(np.transpose(xin, (0, 2, 3, 1))[:, 1:3, :, 0:6:2], np.array([[2, 0], [1, 1]]), axis=2)
    assert np.array_equal(want[y], ref)
    plan.close()


@pytest.mark.parametrize("shape", [(2, 3, 8, 8), (1, 5, 26, 28), (3, 2, 6, 12), (1, 1, 2, 4)])
def test_maxpool_2x2_stride2_float_fast_path(ctx, oracle, shape):
    """The vector form of the 2x2 / stride-2 pool on float planes whose rows are whole float4s, with NaNs and infinities in
    the windows: the reference's comparison chain skips NaNs and starts at -inf."""
    x = rnd(np.random.default_rng(sum(shape)), shape)
    flat = x.reshape(-1)
    flat[::7] = np.nan
    flat[3::11] = -np.inf
    flat[5::13] = np.inf
    x[0, 0, 0:2, 0:2] = np.nan                        # a window of NaNs only
    k, s, d, p = (2, 2), (2, 2), (1, 1), (0, 0, 0, 0)
    got, want = ctx.onnx_maxpool(x, k, s, d, p, "NOTSET", False), oracle.onnx_maxpool(x, k, s, d, p, "NOTSET", False)
    assert got.shape == want.shape and np.array_equal(got.view(np.uint32), want.view(np.uint32))
