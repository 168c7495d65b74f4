"""Host-side behaviour of the product library that needs no GPU: argument checks return the
reference's error names, shape helpers agree with the oracle, compute calls fail loudly."""
import itertools

import numpy as np
import pytest

import golden_cases as gc

CASES = gc.load("reference_goldens.json")
NO_GPU_OPS = ("_error", "get_concatenate_output_shape")
HOST_CASES = [c for c in CASES if c["op"].endswith("_error") or c["op"].startswith("get_concatenate")]


@pytest.fixture(scope="module")
def nogpu(zb):
    return zb.Context(None)


@pytest.mark.parametrize("case", HOST_CASES, ids=[gc.case_id(c) for c in HOST_CASES])
def test_reference_error_cases_without_gpu(zb, nogpu, case):
    gc.run_case(nogpu, case, zb.ZantError)


def test_compute_without_context_fails_loudly(zb, nogpu):
    with pytest.raises(zb.ZantError) as e:
        nogpu.ReLU(np.ones(8, np.float32))
    assert e.value.name == "CudaUnavailable"
    with pytest.raises(zb.ZantError) as e:
        nogpu.qlinearmatmul(np.ones((2, 4), np.int8), 0.1, 0, np.ones((4, 3), np.int8), 0.1, None, 0.1, 0)
    assert e.value.name == "CudaUnavailable"


def test_conv_argument_checks(zb, nogpu):
    x = np.zeros((1, 2, 5, 5), np.float32)
    w = np.zeros((3, 2, 3, 3), np.float32)
    with pytest.raises(zb.ZantError) as e:       # group != 1 (op_convolution.zig:60-65)
        nogpu.conv_lean(x, w, (1, 3, 3, 3), group=2)
    assert e.value.name == "InvalidDimensions"
    with pytest.raises(zb.ZantError) as e:       # NOTSET without pads (op_convolution.zig:111-125)
        nogpu.conv_lean(x, w, (1, 3, 3, 3), auto_pad="NOTSET")
    assert e.value.name == "InvalidPadding"
    with pytest.raises(zb.ZantError) as e:       # wrong output shape (op_convolution.zig:212-217)
        nogpu.conv_lean(x, w, (1, 3, 4, 4))
    assert e.value.name == "InvalidDimensions"
    with pytest.raises(zb.ZantError) as e:       # rank
        nogpu.conv_lean(x[0], w, (1, 3, 3, 3))
    assert e.value.name == "InvalidDimensions"
    with pytest.raises(zb.ZantError) as e:       # valid arguments reach the device requirement
        nogpu.conv_lean(x, w, (1, 3, 3, 3))
    assert e.value.name == "CudaUnavailable"


def test_conv_output_shape_matches_oracle(zb, oracle):
    rng = np.random.default_rng(5)
    n = 0
    for _ in range(400):
        H, W = int(rng.integers(3, 20)), int(rng.integers(3, 20))
        kh, kw = int(rng.integers(1, 5)), int(rng.integers(1, 5))
        stride = [int(rng.integers(1, 4))] if rng.random() < 0.5 else [int(rng.integers(1, 4)), int(rng.integers(1, 4))]
        dil = None if rng.random() < 0.4 else [int(rng.integers(1, 3))] * int(rng.integers(1, 3))
        ap = [None, "VALID", "SAME_UPPER", "SAME_LOWER", "NOTSET"][int(rng.integers(0, 5))]
        pads = None if rng.random() < 0.3 else [int(v) for v in rng.integers(0, 3, 4)]
        xs, ws = (2, 3, H, W), (4, 3, kh, kw)
        try:
            want = oracle.conv_output_shape(xs, ws, stride, pads, dil, ap)
        except oracle.OracleError as e:
            with pytest.raises(zb.ZantError) as z:
                zb.conv_output_shape(xs, ws, stride, pads, dil, ap)
            assert z.value.name == e.name
            continue
        assert zb.conv_output_shape(xs, ws, stride, pads, dil, ap) == want
        n += 1
    assert n > 150


def test_pool_output_shapes_match_oracle(zb, oracle):
    rng = np.random.default_rng(6)
    for _ in range(300):
        xs = (1, 2, int(rng.integers(2, 16)), int(rng.integers(2, 16)))
        k = [int(rng.integers(1, 4)), int(rng.integers(1, 4))]
        s = [int(rng.integers(1, 4)), int(rng.integers(1, 4))]
        d = [int(rng.integers(1, 3)), int(rng.integers(1, 3))]
        pads = [int(v) for v in rng.integers(0, 2, 4)]
        ap = ["NOTSET", "SAME_UPPER", "SAME_LOWER", "VALID"][int(rng.integers(0, 4))]
        ceil = bool(rng.integers(0, 2))
        for fn_o, fn_z, args in ((oracle.get_onnx_maxpool_output_shape, zb.get_onnx_maxpool_output_shape, (xs, k, s, d, pads, ap, ceil)),
                                 (oracle.get_pooling_output_shape, zb.get_pooling_output_shape, (xs, k, s))):
            try:
                want = fn_o(*args)
            except oracle.OracleError as e:
                with pytest.raises(zb.ZantError) as z:
                    fn_z(*args)
                assert z.value.name == e.name
                continue
            assert fn_z(*args) == want


def test_resize_and_concat_shapes(zb, oracle):
    assert zb.get_resize_output_shape((1, 128, 13, 13), [1, 1, 2, 2]) == [1, 128, 26, 26]
    assert zb.get_resize_output_shape((2, 2), None, [3, 3]) == [3, 3]
    assert zb.concat_output_shape([(2, 128, 26, 26), (2, 256, 26, 26)], 1) == [2, 384, 26, 26]
    assert zb.concat_output_shape([(2, 3), (3,)], 0) == oracle.concat_output_shape([(2, 3), (3,)], 0) == [3, 3]


def test_shard_range_partitions_every_sample(zb):
    for total, world in itertools.product((0, 1, 7, 256, 65536, 1000), (1, 2, 3, 4, 8)):
        pos = 0
        for r in range(world):
            b, c = zb.shard_range(total, world, r)
            assert b == pos and c in (total // world, total // world + 1)
            pos += c
        assert pos == total
    with pytest.raises(zb.ZantError):
        zb.shard_range(10, 2, 2)


def test_slice_unsqueeze_shape_helpers_match_oracle(zb, nogpu, oracle):
    """Host-only shape rules of Slice, Unsqueeze and Shape against the oracle over many parameter sets."""
    rng = np.random.default_rng(11)
    for _ in range(300):
        rank = int(rng.integers(1, 5))
        shape = [int(v) for v in rng.integers(1, 9, rank)]
        n = int(rng.integers(1, rank + 1))
        axes = [int(a) - (rank if rng.random() < 0.3 else 0) for a in rng.permutation(rank)[:n]]
        starts = [int(v) for v in rng.integers(-10, 10, n)]
        ends = [int(v) for v in rng.integers(-10, 12, n)]
        steps = [int(v) for v in rng.choice([-3, -2, -1, 1, 2, 3], n)]
        for use_axes, use_steps in itertools.product((False, True), (False, True)):
            if not use_axes and n != rank and False:
                continue
            a = axes if use_axes else None
            s = steps if use_steps else None
            st, en = (starts, ends) if use_axes else (starts[:n], ends[:n])
            for lean in (False, True):
                assert nogpu.get_slice_output_shape(shape, st, en, a, s, lean=lean) == oracle.get_slice_output_shape(shape, st, en, a, s, lean=lean)
        k = int(rng.integers(1, 4))
        orank = rank + k
        ax = [int(v) - (orank if rng.random() < 0.5 else 0) for v in rng.permutation(orank)[:k]]
        assert nogpu.get_unsqueeze_output_shape(shape, ax) == oracle.get_unsqueeze_output_shape(shape, ax)
        s0 = None if rng.random() < 0.3 else int(rng.integers(-6, 6))
        e0 = None if rng.random() < 0.3 else int(rng.integers(-6, 7))
        try:
            want = oracle.shape_onnx(shape, s0, e0).tolist()
        except oracle.OracleError as e:
            with pytest.raises(zb.ZantError) as got:
                nogpu.shape_onnx(shape, s0, e0)
            assert got.value.name == e.name
        else:
            assert nogpu.shape_onnx(shape, s0, e0).tolist() == want
