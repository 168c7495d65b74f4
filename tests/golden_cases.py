"""Runs one case of tests/golden/*.json against an implementation module.

`impl` is either the oracle front end (oracle/zant_oracle.py) or the product package's host
mirror bound to a context: both expose the reference's function names, so the same driver
replays the reference's unit tests against either.
"""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
NP = {"f32": np.float32, "u8": np.uint8, "i8": np.int8, "i32": np.int32}


def load(name):
    with open(os.path.join(HERE, "golden", name)) as f:
        return json.load(f)["cases"]


def case_id(c):
    return f'{c["op"]}@{c["cite"].split("/")[-1]}'


def _expect(c, y):
    y = np.asarray(y)
    assert list(y.shape) == list(c["y_shape"]), (y.shape, c["y_shape"])
    flat = y.reshape(-1)
    atol = c.get("atol", 0)
    if "y" in c:
        exp = np.asarray(c["y"], dtype=np.float64)
        assert flat.size == exp.size
        assert np.all(np.abs(flat.astype(np.float64) - exp) <= atol), (flat, exp)
    for k, v in c.get("y_at", {}).items():
        assert abs(float(flat[int(k)]) - v) <= atol, (k, flat[int(k)], v)


def run_case(impl, c, err_type):
    op = c["op"]

    def arr(key, dt=np.float32):
        if c.get(key) is None:
            return None
        a = np.asarray(c[key], dtype=dt)
        sk = key + "_shape"
        return a.reshape(c[sk]) if sk in c and c[sk] is not None else a

    def raises(fn):
        try:
            fn()
        except err_type as e:
            assert e.name == c["error"], (e.name, c["error"])
            return
        raise AssertionError(f'expected {c["error"]}')

    if op in ("conv_lean", "convolve_tensor_with_bias"):
        y = impl.conv_lean(arr("x"), arr("w"), c["y_shape"], arr("bias"), c["stride"], c["pads"], c["dilations"],
                           c["group"], c["auto_pad"])
        _expect(c, y)
    elif op == "Conv":
        y = impl.Conv(arr("x"), arr("w"), arr("bias"), c["stride"], c["pads"], c["dilations"], c["group"], c["auto_pad"])
        _expect(c, y)
    elif op == "gemm":
        y = impl.gemm(arr("a"), arr("b"), arr("c"), c["alpha"], c["beta"], c["transA"], c["transB"])
        _expect(c, y)
    elif op == "gemm_error":
        raises(lambda: impl.gemm(np.zeros(c["a_shape"], np.float32), np.zeros(c["b_shape"], np.float32)))
    elif op == "mat_mul":
        _expect(c, impl.mat_mul(arr("a"), arr("b")))
    elif op == "mat_mul_error":
        raises(lambda: impl.mat_mul(np.zeros(c["a_shape"], np.float32), np.zeros(c["b_shape"], np.float32)))
    elif op == "onnx_maxpool":
        y = impl.onnx_maxpool(arr("x"), c["kernel"], c["strides"], c["dilations"], c["pads"], c["auto_pad"], c["ceil_mode"])
        _expect(c, y)
    elif op == "ReLU":
        y = impl.ReLU(np.asarray(c["x"], np.float32))
        assert np.array_equal(y, np.asarray(c["y"], np.float32))
    elif op == "leakyReLU":
        y = impl.leakyReLU(np.asarray(c["x"], np.float32), c["slope"])
        assert np.all(np.abs(y.astype(np.float64) - np.asarray(c["y"])) <= c["atol"])
    elif op == "transpose_onnx":
        _expect(c, impl.transpose_onnx(arr("x", NP[c["dtype"]]), c["perm"]))
    elif op == "transpose_onnx_error":
        raises(lambda: impl.transpose_onnx(np.zeros(c["x_shape"], np.float32), c["perm"]))
    elif op == "slice_output_shape":
        assert list(impl.get_slice_output_shape(c["x_shape"], c["starts"], c["ends"], c["axes"], c["steps"])) == c["y"]
    elif op == "slice_output_shape_error":
        raises(lambda: impl.get_slice_output_shape(c["x_shape"], c["starts"], c["ends"], c["axes"], c["steps"]))
    elif op == "gather":
        idx = np.asarray(c["idx"], np.uint64).reshape(c["idx_shape"])
        _expect(c, impl.gather(arr("x", NP[c["dtype"]]), idx, c["axis"]))
    elif op == "gather_error":
        idx = np.asarray(c["idx"], np.uint64).reshape(c["idx_shape"])
        raises(lambda: impl.gather(np.zeros(c["x_shape"], np.uint8), idx, c["axis"]))
    elif op == "unsqueeze_shape":
        assert list(impl.get_unsqueeze_output_shape(c["x_shape"], c["axes"])) == c["y"]
        x = np.arange(int(np.prod(c["x_shape"])), dtype=np.float32).reshape(c["x_shape"])
        y = impl.unsqueeze(x, c["axes"])
        assert list(y.shape) == c["y"] and np.array_equal(y.reshape(-1), x.reshape(-1))
    elif op == "unsqueeze_error":
        raises(lambda: impl.get_unsqueeze_output_shape(c["x_shape"], c["axes"]))
    elif op == "shape_onnx":
        assert impl.shape_onnx(c["x_shape"], c["start"], c["end"]).tolist() == c["y"]
    elif op == "shape_onnx_len":
        assert len(impl.shape_onnx(c["x_shape"], c["start"], c["end"])) == c["n"]
    elif op == "sigmoid":
        y = impl.sigmoid(np.asarray(c["x"], np.float32))
        assert np.all(np.abs(y.astype(np.float64) - np.asarray(c["y"])) < c["atol"])
    elif op == "softmax_rows_sum_to_one":
        y = impl.softmax(arr("x"))
        sums = y.astype(np.float64).sum(axis=1)
        assert np.all(sums > c["lo"]) and np.all(sums < c["hi"])
    elif op == "softmax_equal_entries":
        y = impl.softmax(arr("x"))
        assert np.all(y[:, 0] == y[:, 1])
    elif op == "div":
        y = impl.div(np.asarray(c["a"], np.float32), np.asarray(c["b"], np.float32))
        assert np.array_equal(y, np.asarray(c["y"], np.float32))
    elif op == "tanh_matches_libm":
        import math
        y = impl.tanh(np.asarray(c["x"], np.float32))
        assert np.all(np.abs(y.astype(np.float64) - np.array([math.tanh(v) for v in c["x"]])) <= c["atol"])
    elif op == "ceil":
        y = impl.ceil(np.asarray(c["x"], np.float32))
        assert np.all(np.abs(y.astype(np.float64) - np.asarray(c["y"])) <= c["atol"])
    elif op == "sum_tensors":
        _expect(c, impl.sum_tensors(arr("a"), arr("b")))
    elif op == "add_bias":
        y = impl.add_bias(arr("t"), np.asarray(c["bias"], np.float32))
        assert np.array_equal(y.reshape(-1), np.asarray(c["y"], np.float32))
    elif op == "sum_tensor_list":
        y = impl.sum_tensor_list([np.asarray(t, np.float32) for t in c["tensors"]])
        assert np.array_equal(y.reshape(-1), np.asarray(c["y"], np.float32))
    elif op == "sum_tensor_list_error":
        raises(lambda: impl.sum_tensor_list([]))
    elif op == "reduce_mean":
        y = impl.reduce_mean(arr("x"), c["axes"], c["keepdims"], c["noop"])
        c = dict(c, atol=1e-4)
        _expect(c, y)
    elif op == "concatenate":
        dt = NP[c["dtype"]]
        ts = [np.asarray(t, dt).reshape(s) for t, s in zip(c["tensors"], c["shapes"])]
        _expect(c, impl.concatenate(ts, c["axis"]))
    elif op == "concatenate_error":
        ts = [np.zeros(s, np.float32) for s in c["shapes"]]
        raises(lambda: impl.concatenate(ts, c["axis"]))
    elif op == "get_concatenate_output_shape":
        assert impl.get_concatenate_output_shape(c["shapes"], c["axis"]) == c["y_shape"]
    elif op == "get_concatenate_output_shape_error":
        raises(lambda: impl.get_concatenate_output_shape(c["shapes"], c["axis"]))
    elif op == "resize":
        x = np.asarray(c["x"], NP[c["dtype"]]).reshape(c["x_shape"])
        _expect(c, impl.resize(x, c["mode"], c["scales"], c["sizes"], c["coord_mode"]))
    elif op == "resize_error":
        raises(lambda: impl.resize(np.zeros(c["x_shape"], np.uint8), c["mode"], c["scales"], c["sizes"], "half_pixel"))
    elif op == "reshape":
        x = np.asarray(c["x"], NP[c["dtype"]]).reshape(c["x_shape"])
        _expect(c, impl.reshape(x, c["new_shape"]))
    elif op == "reshape_error":
        raises(lambda: impl.reshape(np.zeros(c["x_shape"], np.uint8), c["new_shape"]))
    else:
        raise AssertionError(f"unknown golden op {op}")
