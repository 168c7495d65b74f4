"""ctypes front end of the CPU oracle (oracle/zant_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the CPU-baseline
legs of bench.py as the checker / timed baseline.  The product package never imports it.

Function names mirror the reference's name table (tensor_math_standard.zig): conv_lean, Conv,
mat_mul, gemm, onnx_maxpool, ReLU, leakyReLU, sum_tensors, sum_tensor_list, add_bias, concatenate,
resize, reshape, reduce_mean; the quantized names follow ONNX.  Inputs and outputs are numpy arrays.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libzant_oracle.so")

F32, I8, U8, I32 = 0, 1, 2, 3
NP_DTYPE = {F32: np.float32, I8: np.int8, U8: np.uint8, I32: np.int32}
AUTO_PAD = {"NOTSET": 0, "SAME_UPPER": 1, "SAME_LOWER": 2, "VALID": 3}
QACT = {None: 0, "none": 0, "relu": 1, "relu6": 2}
SIZE_MAX = (1 << 64) - 1

STATUS_NAMES = {
    0: "OK", -1: "InvalidDimensions", -2: "MemError", -3: "InputTensorDifferentSize",
    -4: "InputTensorDifferentShape", -5: "InputTensorsWrongShape", -6: "OutputTensorDifferentSize",
    -7: "TooSmallOutputType", -8: "InputTensorDimensionMismatch", -9: "WrongStride",
    -10: "IncompatibleBroadcastShapes", -11: "EmptyTensorList", -12: "DivisionError",
    -13: "InvalidPadding", -14: "InvalidAxes", -33: "TensorNotInitialized", -34: "InputArrayWrongType",
    -35: "InputArrayWrongSize", -36: "EmptyTensor", -37: "ZeroSizeTensor", -43: "InvalidSliceIndices",
    -46: "InvalidSliceStep", -49: "AxisOutOfBounds",
    -50: "MismatchedRank", -51: "MismatchedShape", -52: "IndexOutOfBounds", -53: "InvalidAxis", -54: "DuplicateAxis",
    -55: "InvalidInput", -56: "UnsupportedMode", -57: "UnsupportedDimension", -59: "InvalidRank", -60: "InvalidPermutation", -100: "Cuda", -101: "CudaUnavailable",
    -102: "NullPointer", -103: "Unsupported", -104: "ArenaExhausted", -105: "BadHandle",
    -106: "DeviceTimeout", -107: "TooLarge",
}


class OracleError(Exception):
    def __init__(self, status):
        self.status = int(status)
        self.name = STATUS_NAMES.get(self.status, f"status{self.status}")
        super().__init__(self.name)


def build(force=False):
    """Compiles libzant_oracle.so with the Makefile beside this file."""
    src = os.path.join(_HERE, "zant_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libzant_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
    return _lib


def _sz(seq):
    if seq is None:
        return None, 0
    arr = (C.c_size_t * max(len(seq), 1))(*[SIZE_MAX if v == "SIZE_MAX" else int(v) for v in seq])
    return arr, len(seq)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _bytes(s):
    if s is None:
        return None, 0
    b = s.encode() if isinstance(s, str) else bytes(s)
    return C.c_char_p(b), len(b)


def _check(st):
    if st != 0:
        raise OracleError(st)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(np.asarray(a), dtype=dt)


def _dtype_code(a):
    return {np.dtype(np.float32): F32, np.dtype(np.int8): I8, np.dtype(np.uint8): U8, np.dtype(np.int32): I32}[a.dtype]


# ------------------------------------------------------------------ shapes
def conv_output_shape(x_shape, w_shape, stride, pads=None, dilations=None, auto_pad=None):
    xs, xr = _sz(x_shape); ws, wr = _sz(w_shape); st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
    ap, apl = _bytes(auto_pad)
    out = (C.c_size_t * 4)()
    _check(lib().zo_conv_output_shape(xs, C.c_size_t(xr), ws, C.c_size_t(wr), st, C.c_size_t(ns), pd, C.c_size_t(npd),
                                      dl, C.c_size_t(nd), ap, C.c_size_t(apl), out))
    return list(out)


def get_pooling_output_shape(x_shape, kernel, stride):
    xs, xr = _sz(x_shape); k, _ = _sz(kernel); s, _ = _sz(stride)
    out = (C.c_size_t * 4)()
    _check(lib().zo_pooling_output_shape(xs, C.c_size_t(xr), k, s, out))
    return list(out)


def get_onnx_maxpool_output_shape(x_shape, kernel, strides, dilations, pads, auto_pad="NOTSET", ceil_mode=False):
    xs, xr = _sz(x_shape); k, _ = _sz(kernel); s, _ = _sz(strides); d, _ = _sz(dilations); p, _ = _sz(pads)
    out = (C.c_size_t * 4)()
    _check(lib().zo_maxpool_output_shape(xs, C.c_size_t(xr), k, s, d, p, C.c_int32(AUTO_PAD[auto_pad]),
                                         C.c_int32(int(ceil_mode)), out))
    return list(out)


def get_resize_output_shape(x_shape, scales=None, sizes=None):
    xs, r = _sz(x_shape)
    sc = None if scales is None else (C.c_float * len(scales))(*scales)
    sz, nsz = _sz(sizes)
    out = (C.c_size_t * max(r, 1))()
    _check(lib().zo_resize_output_shape(xs, C.c_size_t(r), sc, C.c_size_t(0 if scales is None else len(scales)),
                                        sz, C.c_size_t(nsz), out))
    return list(out)[:r]


def _shape_list(shapes):
    n = len(shapes)
    keep = [_sz(s)[0] for s in shapes]
    ptrs = (C.POINTER(C.c_size_t) * max(n, 1))(*[C.cast(k, C.POINTER(C.c_size_t)) for k in keep])
    ranks = (C.c_size_t * max(n, 1))(*[len(s) for s in shapes])
    return ptrs, ranks, keep


def concat_output_shape(shapes, axis):
    ptrs, ranks, _keep = _shape_list(shapes)
    out = (C.c_size_t * 8)()
    orank = C.c_size_t(0)
    _check(lib().zo_concat_output_shape(ptrs, ranks, C.c_size_t(len(shapes)), C.c_int64(axis), out, C.byref(orank)))
    return list(out)[:orank.value]


def get_concatenate_output_shape(shapes, axis):
    ptrs, ranks, _keep = _shape_list(shapes)
    out = (C.c_size_t * 8)()
    _check(lib().zo_get_concatenate_output_shape(ptrs, ranks, C.c_size_t(len(shapes)), C.c_int64(axis), out))
    return list(out)[:len(shapes[0])]


# ------------------------------------------------------------------ fp32 ops
def conv_lean(x, w, y_shape, bias=None, stride=(1,), pads=None, dilations=None, group=None, auto_pad=None):
    x = _c(x, np.float32); w = _c(w, np.float32); bias = _c(bias, np.float32)
    y = np.zeros(y_shape, np.float32)
    xs, xr = _sz(x.shape); ws, wr = _sz(w.shape); ys, yr = _sz(y.shape)
    st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations); ap, apl = _bytes(auto_pad)
    _check(lib().zo_conv_f32(_p(x), xs, C.c_size_t(xr), _p(w), ws, C.c_size_t(wr), _p(bias),
                             C.c_size_t(0 if bias is None else bias.size), _p(y), ys, C.c_size_t(yr),
                             st, C.c_size_t(ns), pd, C.c_size_t(npd), dl, C.c_size_t(nd),
                             C.c_size_t(0 if group is None else group), ap, C.c_size_t(apl)))
    return y


def Conv(x, w, bias=None, stride=(1,), pads=None, dilations=None, group=None, auto_pad=None):
    x = np.asarray(x); w = np.asarray(w)
    ys = conv_output_shape(x.shape, w.shape, stride, pads, dilations, auto_pad)
    return conv_lean(x, w, ys, bias, stride, pads, dilations, group, auto_pad)


def mat_mul(a, b):
    a = _c(a, np.float32); b = _c(b, np.float32)
    if a.ndim != b.ndim:
        raise OracleError(-4)
    if a.ndim < 2:
        raise OracleError(-5)
    y = np.zeros(a.shape[:-2] + (a.shape[-2], b.shape[-1]), np.float32)
    as_, ar = _sz(a.shape); bs, br = _sz(b.shape); ys, yr = _sz(y.shape)
    _check(lib().zo_mat_mul_f32(_p(a), as_, C.c_size_t(ar), _p(b), bs, C.c_size_t(br), _p(y), ys, C.c_size_t(yr)))
    return y


def gemm(a, b, c=None, alpha=1.0, beta=1.0, transA=False, transB=False):
    a = _c(a, np.float32); b = _c(b, np.float32); c = _c(c, np.float32)
    if a.ndim == 4 and b.ndim == 4:
        rows = a.shape[3] if transA else a.shape[2]
        cols = b.shape[2] if transB else b.shape[3]
        y = np.zeros((a.shape[0], a.shape[1], rows, cols), np.float32)
    else:
        y = np.zeros((1, 1, 1, 1), np.float32)
    as_, ar = _sz(a.shape); bs, br = _sz(b.shape); ys, yr = _sz(y.shape)
    cs, cr = _sz(None if c is None else c.shape)
    _check(lib().zo_gemm_f32(_p(a), as_, C.c_size_t(ar), _p(b), bs, C.c_size_t(br), _p(c), cs, C.c_size_t(cr),
                             C.c_float(alpha), C.c_float(beta), C.c_int32(int(transA)), C.c_int32(int(transB)),
                             _p(y), ys, C.c_size_t(yr)))
    return y


def onnx_maxpool_lean(x, y_shape, kernel, strides, dilations, pads, auto_pad="NOTSET"):
    x = np.ascontiguousarray(x)
    y = np.zeros(y_shape, x.dtype)
    xs, xr = _sz(x.shape); ys, yr = _sz(y.shape)
    k, nk = _sz(kernel); s, ns = _sz(strides); d, nd = _sz(dilations); p, npd = _sz(pads)
    args = (_p(x), xs, C.c_size_t(xr), _p(y), ys, C.c_size_t(yr), k, C.c_size_t(nk), s, C.c_size_t(ns),
            d, C.c_size_t(nd), p, C.c_size_t(npd), C.c_int32(AUTO_PAD[auto_pad]))
    if x.dtype == np.float32:
        _check(lib().zo_maxpool_f32(*args))
    else:
        _check(lib().zo_maxpool_q8(C.c_int32(_dtype_code(x)), *args))
    return y


def onnx_maxpool(x, kernel, strides, dilations, pads, auto_pad="NOTSET", ceil_mode=False):
    x = np.ascontiguousarray(x)
    ys = get_onnx_maxpool_output_shape(x.shape, kernel, strides, dilations, pads, auto_pad, ceil_mode)
    return onnx_maxpool_lean(x, ys, kernel, strides, dilations, pads, auto_pad)


def ReLU(x, out=None):
    """ReLU_standard when `out` is None; lean_ReLU semantics (writes only positives) into `out`."""
    x = _c(x, np.float32)
    zero_first = out is None
    y = np.empty_like(x) if out is None else out
    _check(lib().zo_relu_f32(_p(x), _p(y), C.c_size_t(x.size), C.c_int32(int(zero_first))))
    return y


def leakyReLU(x, slope):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _check(lib().zo_leaky_relu_f32(_p(x), C.c_float(slope), _p(y), C.c_size_t(x.size)))
    return y


def sigmoid(x):
    """TensorMath.sigmoid / sigmoid_lean."""
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _check(lib().zo_sigmoid_f32(_p(x), _p(y), C.c_size_t(x.size)))
    return y


def softmax(x):
    """TensorMath.softmax / lean_softmax on a 2-D tensor (rows are normalised)."""
    x = _c(x, np.float32)
    if x.ndim != 2:
        raise ValueError("softmax takes a 2-D tensor")
    y = np.empty_like(x)
    _check(lib().zo_softmax_f32(_p(x), _p(y), C.c_size_t(x.shape[0]), C.c_size_t(x.shape[1])))
    return y


def tanh(x):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _check(lib().zo_tanh_f32(_p(x), _p(y), C.c_size_t(x.size)))
    return y


def ceil(x):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _check(lib().zo_ceil_f32(_p(x), _p(y), C.c_size_t(x.size)))
    return y


def mul(a, b):
    """TensorMath.mul: element-wise product of tensors of equal size (result takes a's shape)."""
    a, b = _c(a, np.float32), _c(b, np.float32)
    y = np.empty_like(a)
    _check(lib().zo_mul_f32(_p(a), C.c_size_t(a.size), _p(b), C.c_size_t(b.size), _p(y)))
    return y


def div(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    y = np.empty_like(a)
    _check(lib().zo_div_f32(_p(a), C.c_size_t(a.size), _p(b), C.c_size_t(b.size), _p(y)))
    return y


def clip(x, lo, hi):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _check(lib().zo_clip_f32(_p(x), C.c_float(lo), C.c_float(hi), _p(y), C.c_size_t(x.size)))
    return y


def sum_tensors(a, b, return_flag=False):
    a = _c(a, np.float32); b = _c(b, np.float32)
    if a.size == b.size:
        oshape = b.shape
    else:
        oshape = np.broadcast_shapes(a.shape, b.shape) if _broadcastable(a.shape, b.shape) else a.shape
    y = np.zeros(oshape, np.float32)
    as_, ar = _sz(a.shape); bs, br = _sz(b.shape); ys, yr = _sz(y.shape)
    flag = C.c_int32(0)
    _check(lib().zo_sum_tensors_f32(_p(a), as_, C.c_size_t(ar), _p(b), bs, C.c_size_t(br), _p(y), ys, C.c_size_t(yr),
                                    C.byref(flag)))
    return (y, flag.value) if return_flag else y


def _broadcastable(s1, s2):
    try:
        np.broadcast_shapes(s1, s2)
        return True
    except ValueError:
        return False


def sum_tensor_list(tensors):
    ts = [_c(t, np.float32) for t in tensors]
    n = ts[0].size if ts else 0
    for t in ts[1:]:
        if t.size != n:
            raise OracleError(-3)
    y = np.zeros(ts[0].shape if ts else (0,), np.float32)
    ptrs = (C.c_void_p * max(len(ts), 1))(*[t.ctypes.data for t in ts])
    _check(lib().zo_sum_tensor_list_f32(ptrs, C.c_size_t(len(ts)), _p(y), C.c_size_t(n)))
    return y


def add_bias(t, bias):
    t = np.array(t, np.float32, copy=True); bias = _c(bias, np.float32)
    ts, tr = _sz(t.shape); bs, br = _sz(bias.shape)
    _check(lib().zo_add_bias_f32(_p(t), ts, C.c_size_t(tr), _p(bias), bs, C.c_size_t(br)))
    return t


def concatenate(tensors, axis):
    ts = [np.ascontiguousarray(t) for t in tensors]
    if not ts:
        raise OracleError(-11)
    shapes = [t.shape for t in ts]
    oshape = concat_output_shape(shapes, axis)
    y = np.zeros(oshape, ts[0].dtype)
    ptrs, ranks, _keep = _shape_list(shapes)
    data = (C.c_void_p * len(ts))(*[t.ctypes.data for t in ts])
    ys, yr = _sz(y.shape)
    _check(lib().zo_concatenate(C.c_size_t(ts[0].itemsize), data, ptrs, ranks, C.c_size_t(len(ts)), C.c_int64(axis),
                                _p(y), ys, C.c_size_t(yr)))
    return y


def _i64(v):
    if v is None:
        return None
    return (C.c_int64 * len(v))(*[int(a) for a in v])


def transpose_onnx(x, perm=None):
    """TensMath.transpose_onnx: `perm` None reverses the dimensions."""
    x = np.ascontiguousarray(x)
    if perm is not None and (len(perm) != x.ndim or sorted(int(p) for p in perm) != list(range(x.ndim))):
        raise OracleError(-60)
    oshape = [x.shape[i] for i in (perm if perm is not None else range(x.ndim - 1, -1, -1))]
    y = np.zeros(oshape, x.dtype)
    xs, r = _sz(x.shape); ys, yr = _sz(y.shape)
    pm, npm = _sz(perm)
    _check(lib().zo_transpose_onnx(C.c_size_t(x.itemsize), _p(x), xs, C.c_size_t(r), pm, C.c_size_t(npm), _p(y), ys, C.c_size_t(yr)))
    return y


def get_slice_output_shape(x_shape, starts, ends, axes=None, steps=None, lean=False):
    """TensMath.get_slice_output_shape; `lean` = the dimensions lean_slice_onnx gives its output (they
    differ from the shape function's for negative steps)."""
    if len(starts) != len(ends) or (axes is not None and len(axes) != len(starts)) or (steps is not None and len(steps) != len(starts)):
        raise OracleError(-43)
    xs, r = _sz(x_shape)
    out = (C.c_size_t * max(r, 1))()
    _check(lib().zo_slice_output_shape(xs, C.c_size_t(r), _i64(starts), _i64(ends), C.c_size_t(len(starts)), _i64(axes), _i64(steps), out,
                                       C.c_int32(0 if lean else 1)))
    return [int(out[i]) for i in range(r)]


def slice_onnx(x, starts, ends, axes=None, steps=None):
    x = np.ascontiguousarray(x)
    oshape = get_slice_output_shape(x.shape, starts, ends, axes, steps, lean=True)
    y = np.zeros(oshape, x.dtype)
    xs, r = _sz(x.shape); ys, yr = _sz(y.shape)
    _check(lib().zo_slice_onnx(C.c_size_t(x.itemsize), _p(x), xs, C.c_size_t(r), _i64(starts), _i64(ends), C.c_size_t(len(starts)),
                               _i64(axes), _i64(steps), _p(y), ys, C.c_size_t(yr)))
    return y


def gather(x, indices, axis):
    x = np.ascontiguousarray(x)
    idx = np.ascontiguousarray(np.asarray(indices), dtype=np.uint64)
    if x.ndim == 0:
        raise OracleError(-59)
    if axis >= x.ndim or axis < -x.ndim:
        raise OracleError(-53)
    ax = axis + x.ndim if axis < 0 else axis
    oshape = list(x.shape[:ax]) + list(idx.shape) + list(x.shape[ax + 1:])
    y = np.zeros(oshape, x.dtype)
    xs, r = _sz(x.shape); ys, yr = _sz(y.shape); is_, ir = _sz(idx.shape)
    _check(lib().zo_gather(C.c_size_t(x.itemsize), _p(x), xs, C.c_size_t(r), _p(idx), is_, C.c_size_t(ir), C.c_int64(axis),
                           _p(y), ys, C.c_size_t(yr)))
    return y


def get_unsqueeze_output_shape(x_shape, axes):
    xs, r = _sz(x_shape)
    out = (C.c_size_t * max(r + len(axes), 1))()
    _check(lib().zo_unsqueeze_output_shape(xs, C.c_size_t(r), _i64(axes), C.c_size_t(len(axes)), out))
    return [int(out[i]) for i in range(r + len(axes))]


def unsqueeze(x, axes):
    x = np.ascontiguousarray(x)
    return x.reshape(get_unsqueeze_output_shape(x.shape, axes)).copy()


def shape_onnx(x_shape, start=None, end=None):
    """TensMath.shape_onnx on a tensor of shape `x_shape`: int64 values of dimensions [start, end)."""
    xs, r = _sz(x_shape)
    out = (C.c_int64 * max(r, 1))()
    n = C.c_size_t(0)
    _check(lib().zo_shape_onnx(xs, C.c_size_t(r), C.c_int32(start is not None), C.c_int64(start or 0), C.c_int32(end is not None),
                               C.c_int64(end or 0), out, C.byref(n)))
    return np.array([out[i] for i in range(n.value)], np.int64)


def resize(x, mode, scales=None, sizes=None, coord_mode="half_pixel"):
    x = np.ascontiguousarray(x)
    oshape = get_resize_output_shape(x.shape, scales, sizes)
    y = np.zeros(oshape, x.dtype)
    xs, r = _sz(x.shape); ys, yr = _sz(y.shape)
    sc = None if scales is None else (C.c_float * len(scales))(*scales)
    sz, nsz = _sz(sizes); m, ml = _bytes(mode); cm, cml = _bytes(coord_mode)
    _check(lib().zo_resize(C.c_size_t(x.itemsize), _p(x), xs, C.c_size_t(r), m, C.c_size_t(ml), sc,
                           C.c_size_t(0 if scales is None else len(scales)), sz, C.c_size_t(nsz), cm, C.c_size_t(cml),
                           _p(y), ys, C.c_size_t(yr)))
    return y


def reshape(x, new_shape):
    x = np.ascontiguousarray(x)
    y = np.zeros(x.size, x.dtype)
    xs, xr = _sz(x.shape); ns, nr = _sz(new_shape)
    out = (C.c_size_t * max(nr, 1))()
    _check(lib().zo_reshape(C.c_size_t(x.itemsize), _p(x), xs, C.c_size_t(xr), ns, C.c_size_t(nr), _p(y), out))
    return y.reshape(list(out)[:nr])


def reduce_mean_shape(x_shape, axes, keepdims, noop):
    r = len(x_shape)
    if axes is None or len(axes) == 0:
        if noop:
            return list(x_shape)
        return [1] * r if keepdims else [1]
    ax = [a + r if a < 0 else a for a in axes]
    return [1 if i in ax else d for i, d in enumerate(x_shape) if (i not in ax) or keepdims]


def reduce_mean(x, axes=None, keepdims=True, noop_with_empty_axes=False):
    x = _c(x, np.float32)
    y = np.zeros(reduce_mean_shape(x.shape, axes, keepdims, noop_with_empty_axes), np.float32)
    xs, xr = _sz(x.shape); ys, yr = _sz(y.shape)
    ax = None if axes is None else (C.c_int64 * max(len(axes), 1))(*axes)
    _check(lib().zo_reduce_mean_f32(_p(x), xs, C.c_size_t(xr), _p(y), ys, C.c_size_t(yr), ax,
                                    C.c_size_t(0 if axes is None else len(axes)), C.c_int32(int(keepdims)),
                                    C.c_int32(int(noop_with_empty_axes))))
    return y


# ------------------------------------------------------------------ quantized ops
def quantize_linear(x, scale, zp, out_dtype=U8):
    x = _c(x, np.float32)
    y = np.zeros(x.shape, NP_DTYPE[out_dtype])
    _check(lib().zo_quantize_linear(_p(x), C.c_size_t(x.size), C.c_float(scale), C.c_int32(zp), C.c_int32(out_dtype), _p(y)))
    return y


def dequantize_linear(q, scale, zp):
    q = np.ascontiguousarray(q)
    y = np.zeros(q.shape, np.float32)
    _check(lib().zo_dequantize_linear(C.c_int32(_dtype_code(q)), _p(q), C.c_size_t(q.size), C.c_float(scale), C.c_int32(zp), _p(y)))
    return y


def qconv_output_shape(x_shape, w_shape, stride, pads, dilations, auto_pad="NOTSET"):
    xs, _ = _sz(x_shape); ws, _ = _sz(w_shape); st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
    g = (C.c_size_t * 10)()
    _check(lib().zo_qconv_geometry(xs, ws, st, C.c_size_t(ns), pd, C.c_size_t(npd), dl, C.c_size_t(nd),
                                   C.c_int32(AUTO_PAD[auto_pad]), g))
    return [x_shape[0], w_shape[0], g[8], g[9]]


def qlinearconv(x, x_scale, x_zp, w, w_scale, w_zp, y_scale, y_zp, bias=None, y_dtype=I8, stride=(1, 1),
                pads=(0, 0, 0, 0), dilations=(1, 1), group=1, auto_pad="NOTSET", activation=None):
    x = np.ascontiguousarray(x); w = _c(w, np.int8)
    w_scale = np.atleast_1d(_c(w_scale, np.float32))
    w_zp = None if w_zp is None else np.atleast_1d(_c(w_zp, np.int32))
    bias = _c(bias, np.int32)
    ysh = qconv_output_shape(x.shape, w.shape, stride, pads, dilations, auto_pad)
    y = np.zeros(ysh, NP_DTYPE[y_dtype])
    xs, xr = _sz(x.shape); ws, wr = _sz(w.shape); ys, yr = _sz(y.shape)
    st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
    _check(lib().zo_qlinearconv(C.c_int32(_dtype_code(x)), _p(x), xs, C.c_size_t(xr), C.c_float(x_scale), C.c_int32(x_zp),
                                _p(w), ws, C.c_size_t(wr), _p(w_scale), _p(w_zp), C.c_size_t(w_scale.size),
                                C.c_float(y_scale), C.c_int32(y_zp), _p(bias), C.c_size_t(0 if bias is None else bias.size),
                                C.c_int32(y_dtype), _p(y), ys, C.c_size_t(yr), st, C.c_size_t(ns), pd, C.c_size_t(npd),
                                dl, C.c_size_t(nd), C.c_size_t(group), C.c_int32(AUTO_PAD[auto_pad]),
                                C.c_int32(QACT[activation])))
    return y


def qlinearmatmul(a, a_scale, a_zp, b, b_scale, b_zp, y_scale, y_zp, bias=None, y_dtype=I8, activation=None):
    a = np.ascontiguousarray(a); b = _c(b, np.int8)
    b_scale = np.atleast_1d(_c(b_scale, np.float32))
    b_zp = None if b_zp is None else np.atleast_1d(_c(b_zp, np.int32))
    bias = _c(bias, np.int32)
    y = np.zeros((a.shape[0], b.shape[1]), NP_DTYPE[y_dtype])
    as_, ar = _sz(a.shape); bs, br = _sz(b.shape); ys, yr = _sz(y.shape)
    _check(lib().zo_qlinearmatmul(C.c_int32(_dtype_code(a)), _p(a), as_, C.c_size_t(ar), C.c_float(a_scale), C.c_int32(a_zp),
                                  _p(b), bs, C.c_size_t(br), _p(b_scale), _p(b_zp), C.c_size_t(b_scale.size),
                                  C.c_float(y_scale), C.c_int32(y_zp), _p(bias), C.c_size_t(0 if bias is None else bias.size),
                                  C.c_int32(y_dtype), _p(y), ys, C.c_size_t(yr), C.c_int32(QACT[activation])))
    return y


def qlinearadd(a, a_scale, a_zp, b, b_scale, b_zp, y_scale, y_zp, activation=None):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    y = np.zeros(a.shape, a.dtype)
    _check(lib().zo_qlinearadd(C.c_int32(_dtype_code(a)), _p(a), C.c_float(a_scale), C.c_int32(a_zp), _p(b), C.c_float(b_scale),
                               C.c_int32(b_zp), C.c_float(y_scale), C.c_int32(y_zp), _p(y), C.c_size_t(a.size),
                               C.c_int32(QACT[activation])))
    return y


def qlinear_global_avgpool(x, x_scale, x_zp, y_scale, y_zp):
    x = np.ascontiguousarray(x)
    y = np.zeros((x.shape[0], x.shape[1], 1, 1), x.dtype)
    xs, xr = _sz(x.shape)
    _check(lib().zo_qlinear_global_avgpool(C.c_int32(_dtype_code(x)), _p(x), xs, C.c_size_t(xr), C.c_float(x_scale),
                                           C.c_int32(x_zp), C.c_float(y_scale), C.c_int32(y_zp), _p(y)))
    return y


def lut_q8(x, lut):
    x = np.ascontiguousarray(x); lut = _c(lut, np.uint8)
    y = np.zeros(x.shape, x.dtype)
    _check(lib().zo_lut_q8(_p(x), _p(lut), _p(y), C.c_size_t(x.size)))
    return y


def build_leaky_lut(dtype, s_in, zp_in, slope, s_out, zp_out):
    lut = np.zeros(256, np.uint8)
    _check(lib().zo_build_leaky_lut(C.c_int32(dtype), C.c_float(s_in), C.c_int32(zp_in), C.c_float(slope),
                                    C.c_float(s_out), C.c_int32(zp_out), _p(lut)))
    return lut
