"""The tensor-core float path (tcgen05 kind::tf32): Conv, MatMul and Gemm through a context in TF32 mode against the
oracle (the reference's sequential FP32 arithmetic, op_convolution.zig:42-219, op_mat_mul.zig:92-172, op_gemm.zig:91-185).

Two modes, two statements of the 2e-3 tolerance:
  mode 2 (operands split into two TF32 parts, three MMAs per K step): the form the FP32 path uses with 2e-3 in place of 1e-4,
      |y - ref| <= 2e-3 * max(|ref|, 1e-2 * max|ref|)          (floor 1e-1 for the 13-layer detector at 416 x 416, where
      the distance from the reference's summation order alone reaches 1e-4 of the output's scale);
  mode 1 (one MMA per K step on operands rounded to TF32): the error of an output is ~3e-4 of the root sum of squares of its
      products, so it is bounded against the output's scale, |y - ref| <= 2e-3 * max|ref|, and not against outputs that are
      near-cancellations.
The exact FP32 kernels stay the default and stay bit-identical; this file checks that too."""
import numpy as np
import pytest

import graph_oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def within_tf32(got, ref, mode=2, floor=None):
    floor = (1.0 if mode == 1 else 1e-2) if floor is None else floor
    bound = TOL * np.maximum(np.abs(ref), floor * np.abs(ref).max())
    err = np.abs(got - ref)
    return bool(np.all(err <= bound)), float((err / bound).max())


@pytest.fixture(params=[1, 2], ids=["tf32", "tf32x3"])
def tctx(zb, request):
    c = zb.Context(0)
    c.set_tf32(request.param)
    c.mode = request.param
    yield c
    c.close()


CONVS = [
    # N  C   H   W   M  k  stride pad dil
    (2, 3, 32, 32, 16, 3, 1, 1, 1),
    (4, 32, 13, 13, 64, 3, 1, 0, 1),
    (1, 64, 26, 26, 128, 3, 1, 1, 1),
    (2, 128, 14, 14, 300, 1, 1, 0, 1),       # 1x1, three filter tiles of 128 (one partly filled)
    (2, 16, 20, 17, 24, 3, 2, 1, 1),         # stride 2, odd width
    (1, 8, 19, 19, 8, 3, 1, 2, 2),           # dilation 2
    (1, 512, 13, 13, 64, 3, 1, 1, 1),        # K = 4608: a long sum
]


@pytest.mark.parametrize("case", CONVS, ids=[f"conv{i}" for i in range(len(CONVS))])
def test_conv_tf32_within_tolerance(zb, tctx, oracle, case):
    N, C, H, W, M, k, s, p, d = case
    rng = np.random.default_rng(N + C + M)
    x = rng.random((N, C, H, W), dtype=np.float32)                         # activations in [0, 1): sums do not cancel
    w = (rng.standard_normal((M, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = rng.standard_normal(M).astype(np.float32)
    kw = dict(stride=(s, s), pads=(p, p, p, p), dilations=(d, d), group=1, auto_pad="NOTSET")
    want = oracle.Conv(x, w, b, **kw)
    got = tctx.Conv(x, w, b, **kw)
    ok, worst = within_tf32(got, want, tctx.mode)
    assert ok, worst
    assert not np.array_equal(got, want)                                   # it really is the TF32 kernel
    if tctx.mode == 1:
        assert np.abs(got - want).max() > 1e-6 * np.abs(want).max()        # and really the single-pass form


def test_matmul_tf32_and_exact_default(zb, ctx, tctx, oracle):
    rng = np.random.default_rng(9)
    a = rng.random((300, 1600), dtype=np.float32)
    b = (rng.standard_normal((1600, 512)) * 0.03).astype(np.float32)
    want = oracle.mat_mul(a, b)
    ok, worst = within_tf32(tctx.mat_mul(a, b), want, tctx.mode)
    assert ok, worst
    # the default context keeps the reference's arithmetic bit for bit
    assert np.array_equal(ctx.mat_mul(a, b).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("batch", [256, 4096])
def test_small_cnn_fp32_in_tf32_mode(zb, tctx, oracle, batch):
    from zant_b200 import models
    g = models.small_cnn_fp32(batch)
    x = models.small_cnn_input(batch, 31)
    plan = zb.Plan(tctx, g)
    names = plan.step_names()
    assert "Conv(tf32)+Relu" in names and "MatMul(tf32)" in names
    got = plan.run(x)
    plan.close()
    idx = [0, batch // 2 - 1, batch - 1]
    gs = models.small_cnn_fp32(len(idx))
    want = graph_oracle.run(oracle, gs, x[idx])[gs.output]
    ok, worst = within_tf32(got[idx], want, tctx.mode)
    assert ok, worst


@pytest.mark.parametrize("res,batch", [(96, 2), (416, 1)])
def test_tiny_yolo_fp32_in_tf32_mode(zb, tctx, oracle, res, batch):
    from zant_b200 import models
    g = models.tiny_yolo_fp32(batch, res=res)
    x = models.tiny_yolo_input(batch, res)
    want = graph_oracle.run(oracle, g, x)
    plan = zb.Plan(tctx, g)
    names = plan.step_names()
    assert "Conv(tf32)+LeakyRelu" in names
    if res == 416:
        assert "LeakyRelu" not in names and "Conv" not in names      # at 96 x 96 the deepest layers have too few pixels for a tile and stay exact
    got = plan.run(x)
    for name, out, ref in (("head26", got, want[g.output]), ("head13", plan.read_tensor(g.meta["head13"]), want[g.meta["head13"]])):
        ok, worst = within_tf32(out, ref, tctx.mode, floor=1e-1 if (tctx.mode == 2 and res == 416) else None)
        assert ok, (name, worst)
    plan.close()


def test_gemm_node_in_tf32_mode(zb, tctx, oracle):
    """The fully-connected form of Gemm (B transposed, row-vector C) as a plan node."""
    from zant_b200 import F32
    rng = np.random.default_rng(2)
    g = zb.Graph("fc")
    x = g.tensor("x", F32, (1, 1, 256, 320))
    w = g.tensor("w", F32, (1, 1, 100, 320), (rng.standard_normal((1, 1, 100, 320)) * 0.05).astype(np.float32))
    c = g.tensor("c", F32, (1, 1, 1, 100), rng.standard_normal((1, 1, 1, 100)).astype(np.float32))
    y = g.tensor("y", F32, (1, 1, 256, 100))
    g.node("Gemm", [x, w, c], [y], alpha=1.0, beta=1.0, trans_a=0, trans_b=1)
    g.input, g.output = x, y
    xin = rng.random((1, 1, 256, 320), dtype=np.float32)
    want = graph_oracle.run(oracle, g, xin)[g.output]
    plan = zb.Plan(tctx, g)
    assert plan.step_names() == ["Gemm(tf32)"]
    ok, worst = within_tf32(plan.run(xin), want, tctx.mode)
    plan.close()
    assert ok, worst
