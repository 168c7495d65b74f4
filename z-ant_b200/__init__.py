"""zant_b200 — Python binding of libzant_b200.so, the B200 (sm_100a) back end for Z-Ant's
TensorMath inference operators.

This module is a thin ctypes layer over the C ABI declared in include/zant_b200.h.  A `Context`
exposes the operators under the names of the reference's table
(src/Core/Tensor/TensorMath/tensor_math_standard.zig in the Z-Ant tree): conv_lean, Conv, mat_mul,
gemm, onnx_maxpool, ReLU, leakyReLU, sum_tensors, sum_tensor_list, concatenate, resize, reshape,
reduce_mean, plus the ONNX quantized operators.  Arguments may be numpy arrays (host buffers,
staged by the library) or objects with `data_ptr()` such as CUDA torch tensors (used in place).

There is no CPU implementation behind these calls: if the shared library or a B200 is missing the
calls raise.  The directory name contains a hyphen, so the package is loaded by path (see
`__graft_entry__.load_package`) and registers itself as `zant_b200`.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libzant_b200.so")

F32, I8, U8, I32 = 0, 1, 2, 3
NP_DTYPE = {F32: np.float32, I8: np.int8, U8: np.uint8, I32: np.int32}
DTYPE_OF = {np.dtype(np.float32): F32, np.dtype(np.int8): I8, np.dtype(np.uint8): U8, np.dtype(np.int32): I32}
AUTO_PAD = {"NOTSET": 0, "SAME_UPPER": 1, "SAME_LOWER": 2, "VALID": 3}
QACT = {None: 0, "none": 0, "relu": 1, "relu6": 2}
COORD_MODE = {"half_pixel": 0, "align_corners": 1, "asymmetric": 2}
SIZE_MAX = (1 << 64) - 1

OP = dict(Conv=1, MatMul=2, Gemm=3, MaxPool=4, Relu=5, LeakyRelu=6, Add=7, Concat=8, Resize=9, ReduceMean=10,
          Reshape=11, Clip=12, Sigmoid=13, Softmax=14, Tanh=15, Ceil=16, Mul=17, Div=18, Transpose=19, Slice=27, Gather=28,
          QuantizeLinear=20, DequantizeLinear=21, QLinearConv=22, QLinearMatMul=23,
          QLinearAdd=24, QLinearGlobalAveragePool=25, LutQ8=26)


def _i64(v):
    if v is None:
        return None
    return (C.c_int64 * max(len(v), 1))(*[int(a) for a in v])


class ZantError(Exception):
    """A non-zero zant_status; `.name` is the Zig error name the reference would have raised."""

    def __init__(self, status, name, message=""):
        self.status = int(status)
        self.name = name
        super().__init__(f"{name} ({status}): {message}" if message else f"{name} ({status})")


class NodeAttrs(C.Structure):
    _fields_ = [
        ("kernel_shape", C.c_size_t * 2),
        ("strides", C.c_size_t * 2), ("n_strides", C.c_size_t),
        ("dilations", C.c_size_t * 2), ("n_dilations", C.c_size_t),
        ("pads", C.c_size_t * 4), ("n_pads", C.c_size_t),
        ("group", C.c_size_t),
        ("auto_pad", C.c_int32),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("trans_a", C.c_int32), ("trans_b", C.c_int32),
        ("axis", C.c_int64),
        ("axes", C.c_int64 * 4), ("n_axes", C.c_size_t),
        ("keepdims", C.c_int32), ("noop_with_empty_axes", C.c_int32),
        ("scales", C.c_float * 4), ("n_scales", C.c_size_t),
        ("coord_mode", C.c_int32),
        ("x_scale", C.c_float), ("x_zp", C.c_int32),
        ("b_scale", C.c_float), ("b_zp", C.c_int32),
        ("y_scale", C.c_float), ("y_zp", C.c_int32),
        ("activation", C.c_int32),
        ("perm", C.c_int64 * 8), ("n_perm", C.c_size_t),
        ("slice_starts", C.c_int64 * 8), ("slice_ends", C.c_int64 * 8), ("slice_axes", C.c_int64 * 8), ("slice_steps", C.c_int64 * 8),
        ("n_slice", C.c_size_t), ("slice_has_axes", C.c_int32), ("slice_has_steps", C.c_int32),
        ("channels_last", C.c_int32),
    ]


_lib = None


def lib():
    """Loads libzant_b200.so (built in-tree by `build()`); raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(nvcc, sm_100a). There is no CPU fallback.")
        _lib = C.CDLL(LIB_PATH)
        _lib.zant_b200_version.restype = C.c_char_p
        _lib.zant_b200_status_name.restype = C.c_char_p
        _lib.zant_b200_last_error.restype = C.c_char_p
        _lib.zant_b200_ctx_stream.restype = C.c_void_p
        _lib.zant_b200_ctx_launch_count.restype = C.c_uint64
        _lib.zant_b200_plan_arena_bytes.restype = C.c_size_t
        _lib.zant_b200_plan_tensor_ptr.restype = C.c_void_p
        _lib.zant_b200_plan_step_name.restype = C.c_char_p
    return _lib


def build(verbose=False):
    from importlib import util
    spec = util.spec_from_file_location("zant_b200_build", os.path.join(_HERE, "_build.py"))
    mod = util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(verbose=verbose)


def version():
    return lib().zant_b200_version().decode()


def device_count():
    return int(lib().zant_b200_device_count())


def check(status):
    if status != 0:
        L = lib()
        raise ZantError(status, L.zant_b200_status_name(C.c_int32(status)).decode(), L.zant_b200_last_error().decode())


# ----------------------------------------------------------------------------------------- helpers
def _sz(seq):
    if seq is None:
        return None, 0
    vals = [SIZE_MAX if v == "SIZE_MAX" else int(v) for v in seq]
    return (C.c_size_t * max(len(vals), 1))(*vals), len(vals)


def _bytes(s):
    if s is None:
        return None, 0
    b = s.encode() if isinstance(s, str) else bytes(s)
    return C.c_char_p(b), len(b)


def _ptr(a):
    if a is None:
        return None
    if hasattr(a, "data_ptr"):
        return C.c_void_p(a.data_ptr())
    return a.ctypes.data_as(C.c_void_p)


def _host(a, dt=None):
    """numpy arrays are made contiguous (and cast when dt is given); device tensors pass through."""
    if a is None or hasattr(a, "data_ptr"):
        return a
    return np.ascontiguousarray(np.asarray(a), dtype=dt)


def _shape(a):
    return tuple(a.shape)


def _dtype_code(a):
    if hasattr(a, "data_ptr"):
        import torch
        return {torch.float32: F32, torch.int8: I8, torch.uint8: U8, torch.int32: I32}[a.dtype]
    return DTYPE_OF[a.dtype]


def _shape_list(shapes):
    n = len(shapes)
    keep = [_sz(s)[0] for s in shapes]
    ptrs = (C.POINTER(C.c_size_t) * max(n, 1))(*[C.cast(k, C.POINTER(C.c_size_t)) for k in keep])
    ranks = (C.c_size_t * max(n, 1))(*[len(s) for s in shapes])
    return ptrs, ranks, keep


def _numel(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


# ----------------------------------------------------------------------------------------- shape helpers (no GPU needed)
def conv_output_shape(x_shape, w_shape, stride, pads=None, dilations=None, auto_pad=None):
    xs, xr = _sz(x_shape); ws, wr = _sz(w_shape); st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
    ap, apl = _bytes(auto_pad)
    out = (C.c_size_t * 4)()
    check(lib().zant_b200_conv_output_shape(xs, C.c_size_t(xr), ws, C.c_size_t(wr), st, C.c_size_t(ns), pd, C.c_size_t(npd),
                                            dl, C.c_size_t(nd), ap, C.c_size_t(apl), out))
    return list(out)


def get_pooling_output_shape(x_shape, kernel, stride):
    xs, xr = _sz(x_shape); k, _ = _sz(kernel); s, _ = _sz(stride)
    out = (C.c_size_t * 4)()
    check(lib().zant_b200_pooling_output_shape(xs, C.c_size_t(xr), k, s, out))
    return list(out)


def get_onnx_maxpool_output_shape(x_shape, kernel, strides, dilations, pads, auto_pad="NOTSET", ceil_mode=False):
    xs, xr = _sz(x_shape); k, _ = _sz(kernel); s, _ = _sz(strides); d, _ = _sz(dilations); p, _ = _sz(pads)
    out = (C.c_size_t * 4)()
    check(lib().zant_b200_maxpool_output_shape(xs, C.c_size_t(xr), k, s, d, p, C.c_int32(AUTO_PAD[auto_pad]),
                                               C.c_int32(int(ceil_mode)), out))
    return list(out)


def get_resize_output_shape(x_shape, scales=None, sizes=None):
    xs, r = _sz(x_shape)
    sc = None if scales is None else (C.c_float * max(len(scales), 1))(*scales)
    sz, nsz = _sz(sizes)
    out = (C.c_size_t * max(r, 1))()
    check(lib().zant_b200_resize_output_shape(xs, C.c_size_t(r), sc, C.c_size_t(0 if scales is None else len(scales)),
                                              sz, C.c_size_t(nsz), out))
    return list(out)[:r]


def concat_output_shape(shapes, axis):
    ptrs, ranks, _keep = _shape_list(shapes)
    out = (C.c_size_t * 8)()
    orank = C.c_size_t(0)
    check(lib().zant_b200_concat_output_shape(ptrs, ranks, C.c_size_t(len(shapes)), C.c_int64(axis), out, C.byref(orank)))
    return list(out)[:orank.value]


def get_concatenate_output_shape(shapes, axis):
    ptrs, ranks, _keep = _shape_list(shapes)
    out = (C.c_size_t * 8)()
    check(lib().zant_b200_get_concatenate_output_shape(ptrs, ranks, C.c_size_t(len(shapes)), C.c_int64(axis), out))
    return list(out)[:len(shapes[0])]


def shard_range(total, world, rank):
    b, c = C.c_size_t(0), C.c_size_t(0)
    check(lib().zant_b200_shard_range(C.c_size_t(total), C.c_size_t(world), C.c_size_t(rank), C.byref(b), C.byref(c)))
    return b.value, c.value


def reduce_mean_shape(x_shape, axes, keepdims, noop):
    r = len(x_shape)
    if axes is None or len(axes) == 0:
        if noop:
            return list(x_shape)
        return [1] * r if keepdims else [1]
    ax = [a + r if a < 0 else a for a in axes]
    return [1 if i in ax else d for i, d in enumerate(x_shape) if (i not in ax) or keepdims]


# ----------------------------------------------------------------------------------------- context
class Context:
    """One device + one stream.  `device=None` builds a context-less object whose compute calls
    fail with CudaUnavailable after argument validation (used by the host-logic tests)."""

    def __init__(self, device=0, arena_bytes=0):
        self._h = C.c_void_p(None)
        self.device = device
        if device is not None:
            check(lib().zant_b200_ctx_create(C.c_int32(device), C.c_size_t(arena_bytes), C.byref(self._h)))

    # -- housekeeping
    def close(self):
        if self._h:
            lib().zant_b200_ctx_destroy(self._h)
            self._h = C.c_void_p(None)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def synchronize(self):
        check(lib().zant_b200_ctx_synchronize(self._h))

    @property
    def stream(self):
        return lib().zant_b200_ctx_stream(self._h)

    def set_stream(self, cuda_stream_ptr):
        check(lib().zant_b200_ctx_set_stream(self._h, C.c_void_p(cuda_stream_ptr)))

    def set_tf32(self, mode=1):
        """Float contractions: 0 = exact FP32 kernels, 1 = tensor cores (TF32, one pass), 2 = tensor cores with split operands."""
        check(lib().zant_b200_ctx_set_tf32(self._h, C.c_int32(int(mode))))

    def set_arena_limit(self, max_bytes):
        """Caps the staging arena of host-pointer calls (0 = grow on demand)."""
        check(lib().zant_b200_ctx_set_arena_limit(self._h, C.c_size_t(int(max_bytes))))

    def selftest_bounded_wait(self, budget_us=50):
        """Launches the bounded-wait self test; the next synchronize() raises DeviceTimeout once."""
        check(lib().zant_b200_selftest_bounded_wait(self._h, C.c_uint32(int(budget_us))))

    def measure_int8_peak(self, iters=20000):
        """Attainable int8 tensor rate (TOP/s) from the resident-tile tcgen05 probe."""
        v = C.c_double(0.0)
        check(lib().zant_b200_measure_int8_peak(self._h, C.c_int32(iters), C.byref(v)))
        return v.value

    def measure_int8_peak_sustained(self, seconds=2.0):
        out = C.c_double(0.0)
        check(lib().zant_b200_measure_int8_peak_sustained(self._h, C.c_double(float(seconds)), C.byref(out)))
        return out.value

    def launch_count(self):
        return int(lib().zant_b200_ctx_launch_count(self._h))

    def reset_launch_count(self):
        lib().zant_b200_ctx_reset_launch_count(self._h)

    def _out(self, out, shape, dt):
        return np.zeros(shape, NP_DTYPE[dt] if isinstance(dt, int) else dt) if out is None else out

    # -- fp32 operators (names of tensor_math_standard.zig)
    def conv_lean(self, x, w, y_shape, bias=None, stride=(1,), pads=None, dilations=None, group=None, auto_pad=None, out=None):
        x = _host(x, np.float32); w = _host(w, np.float32); bias = _host(bias, np.float32)
        y = self._out(out, y_shape, F32)
        xs, xr = _sz(_shape(x)); ws, wr = _sz(_shape(w)); ys, yr = _sz(y_shape)
        st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations); ap, apl = _bytes(auto_pad)
        check(lib().zant_b200_conv_f32(self._h, _ptr(x), xs, C.c_size_t(xr), _ptr(w), ws, C.c_size_t(wr), _ptr(bias),
                                       C.c_size_t(0 if bias is None else _numel(_shape(bias))), _ptr(y), ys, C.c_size_t(yr),
                                       st, C.c_size_t(ns), pd, C.c_size_t(npd), dl, C.c_size_t(nd),
                                       C.c_size_t(0 if group is None else group), ap, C.c_size_t(apl)))
        return y

    def Conv(self, x, w, bias=None, stride=(1,), pads=None, dilations=None, group=None, auto_pad=None):
        ys = conv_output_shape(_shape(x), _shape(w), stride, pads, dilations, auto_pad)
        return self.conv_lean(x, w, ys, bias, stride, pads, dilations, group, auto_pad)

    def mat_mul(self, a, b, out=None):
        a = _host(a, np.float32); b = _host(b, np.float32)
        sa, sb = _shape(a), _shape(b)
        yshape = tuple(sa[:-2]) + (sa[-2], sb[-1]) if len(sa) >= 2 and len(sb) >= 2 else (1, 1)
        y = self._out(out, yshape, F32)
        as_, ar = _sz(sa); bs, br = _sz(sb); ys, yr = _sz(yshape)
        check(lib().zant_b200_mat_mul_f32(self._h, _ptr(a), as_, C.c_size_t(ar), _ptr(b), bs, C.c_size_t(br), _ptr(y), ys, C.c_size_t(yr)))
        return y

    def gemm(self, a, b, c=None, alpha=1.0, beta=1.0, transA=False, transB=False, out=None):
        a = _host(a, np.float32); b = _host(b, np.float32); c = _host(c, np.float32)
        sa, sb = _shape(a), _shape(b)
        if len(sa) == 4 and len(sb) == 4:
            yshape = (sa[0], sa[1], sa[3] if transA else sa[2], sb[2] if transB else sb[3])
        else:
            yshape = (1, 1, 1, 1)
        y = self._out(out, yshape, F32)
        as_, ar = _sz(sa); bs, br = _sz(sb); ys, yr = _sz(yshape)
        cs, cr = _sz(None if c is None else _shape(c))
        check(lib().zant_b200_gemm_f32(self._h, _ptr(a), as_, C.c_size_t(ar), _ptr(b), bs, C.c_size_t(br), _ptr(c), cs, C.c_size_t(cr),
                                       C.c_float(alpha), C.c_float(beta), C.c_int32(int(transA)), C.c_int32(int(transB)),
                                       _ptr(y), ys, C.c_size_t(yr)))
        return y

    def gemm_lean(self, a, b, c=None, alpha=1.0, beta=1.0, transA=False, transB=False, out=None):
        """gemm_lean as generated code calls it: operands of rank 2..4, the last two dimensions are multiplied."""
        a = _host(a, np.float32); b = _host(b, np.float32); c = _host(c, np.float32)
        sa, sb = _shape(a), _shape(b)
        yshape = tuple(sa[:-2]) + (sa[-1] if transA else sa[-2], sb[-2] if transB else sb[-1])
        y = self._out(out, yshape, F32)
        as_, ar = _sz(sa); bs, br = _sz(sb); ys, yr = _sz(yshape)
        cs, cr = _sz(None if c is None else _shape(c))
        check(lib().zant_b200_gemm_lean_f32(self._h, _ptr(a), as_, C.c_size_t(ar), _ptr(b), bs, C.c_size_t(br), _ptr(c), cs, C.c_size_t(cr),
                                            C.c_float(alpha), C.c_float(beta), C.c_int32(int(transA)), C.c_int32(int(transB)),
                                            _ptr(y), ys, C.c_size_t(yr)))
        return y

    def onnx_maxpool_lean(self, x, y_shape, kernel, strides, dilations, pads, auto_pad="NOTSET", out=None):
        x = _host(x)
        dt = _dtype_code(x)
        y = self._out(out, y_shape, dt)
        xs, xr = _sz(_shape(x)); ys, yr = _sz(y_shape)
        k, nk = _sz(kernel); s, ns = _sz(strides); d, nd = _sz(dilations); p, npd = _sz(pads)
        tail = (xs, C.c_size_t(xr), _ptr(y), ys, C.c_size_t(yr), k, C.c_size_t(nk), s, C.c_size_t(ns), d, C.c_size_t(nd),
                p, C.c_size_t(npd), C.c_int32(AUTO_PAD[auto_pad]))
        if dt == F32:
            check(lib().zant_b200_maxpool_f32(self._h, _ptr(x), *tail))
        else:
            check(lib().zant_b200_maxpool_q8(self._h, C.c_int32(dt), _ptr(x), *tail))
        return y

    def onnx_maxpool(self, x, kernel, strides, dilations, pads, auto_pad="NOTSET", ceil_mode=False):
        ys = get_onnx_maxpool_output_shape(_shape(x), kernel, strides, dilations, pads, auto_pad, ceil_mode)
        return self.onnx_maxpool_lean(x, ys, kernel, strides, dilations, pads, auto_pad)

    def ReLU(self, x, out=None):
        x = _host(x, np.float32)
        y = self._out(out, _shape(x), F32)
        check(lib().zant_b200_relu_f32(self._h, _ptr(x), _ptr(y), C.c_size_t(_numel(_shape(x)))))
        return y

    def leakyReLU(self, x, slope, out=None):
        x = _host(x, np.float32)
        y = self._out(out, _shape(x), F32)
        check(lib().zant_b200_leaky_relu_f32(self._h, _ptr(x), C.c_float(slope), _ptr(y), C.c_size_t(_numel(_shape(x)))))
        return y

    def clip(self, x, lo, hi, out=None):
        x = _host(x, np.float32)
        y = self._out(out, _shape(x), F32)
        check(lib().zant_b200_clip_f32(self._h, _ptr(x), C.c_float(lo), C.c_float(hi), _ptr(y), C.c_size_t(_numel(_shape(x)))))
        return y

    def _unary(self, fn, x, out=None):
        x = _host(x, np.float32)
        y = self._out(out, _shape(x), F32)
        check(fn(self._h, _ptr(x), _ptr(y), C.c_size_t(_numel(_shape(x)))))
        return y

    def sigmoid(self, x, out=None):
        return self._unary(lib().zant_b200_sigmoid_f32, x, out)

    def tanh(self, x, out=None):
        return self._unary(lib().zant_b200_tanh_f32, x, out)

    def ceil(self, x, out=None):
        return self._unary(lib().zant_b200_ceil_f32, x, out)

    def softmax(self, x, out=None):
        x = _host(x, np.float32)
        sh = _shape(x)
        if len(sh) != 2:
            raise ZantError(-1, "InvalidDimensions", "softmax takes a 2-D tensor")
        y = self._out(out, sh, F32)
        check(lib().zant_b200_softmax_f32(self._h, _ptr(x), _ptr(y), C.c_size_t(sh[0]), C.c_size_t(sh[1])))
        return y

    def _binary(self, fn, a, b, out=None):
        a = _host(a, np.float32); b = _host(b, np.float32)
        y = self._out(out, _shape(a), F32)
        check(fn(self._h, _ptr(a), C.c_size_t(_numel(_shape(a))), _ptr(b), C.c_size_t(_numel(_shape(b))), _ptr(y)))
        return y

    def mul(self, a, b, out=None):
        return self._binary(lib().zant_b200_mul_f32, a, b, out)

    def div(self, a, b, out=None):
        return self._binary(lib().zant_b200_div_f32, a, b, out)

    def sum_tensors(self, a, b, out=None):
        a = _host(a, np.float32); b = _host(b, np.float32)
        sa, sb = _shape(a), _shape(b)
        if _numel(sa) == _numel(sb):
            yshape = sb
        else:
            try:
                yshape = tuple(np.broadcast_shapes(sa, sb))
            except ValueError:
                yshape = sa
        y = self._out(out, yshape, F32)
        as_, ar = _sz(sa); bs, br = _sz(sb); ys, yr = _sz(yshape)
        check(lib().zant_b200_sum_tensors_f32(self._h, _ptr(a), as_, C.c_size_t(ar), _ptr(b), bs, C.c_size_t(br), _ptr(y), ys, C.c_size_t(yr)))
        return y

    def add_bias(self, t, bias):
        """add_bias of the reference (lib_elementWise_math.zig:22-45) is a broadcast Add of a 1-D
        bias over the last dimension; it is served by the same kernel as sum_tensors."""
        t = _host(t, np.float32); bias = _host(bias, np.float32)
        if _numel(_shape(t)) == 0 or _numel(_shape(bias)) == 0:
            raise ZantError(-36, "EmptyTensor")
        if len(_shape(bias)) != 1:
            raise ZantError(-5, "InputTensorsWrongShape")
        if _shape(bias)[0] != _shape(t)[-1]:
            raise ZantError(-8, "InputTensorDimensionMismatch")
        if _numel(_shape(t)) == _numel(_shape(bias)):
            return self.sum_tensors(t, bias.reshape(_shape(t)))
        return self.sum_tensors(t, bias)

    def sum_tensor_list(self, tensors, out=None):
        ts = [_host(t, np.float32) for t in tensors]
        n = _numel(_shape(ts[0])) if ts else 0
        for t in ts[1:]:
            if _numel(_shape(t)) != n:
                raise ZantError(-3, "InputTensorDifferentSize")
        y = self._out(out, _shape(ts[0]) if ts else (0,), F32)
        ptrs = (C.c_void_p * max(len(ts), 1))(*[_ptr(t).value for t in ts])
        check(lib().zant_b200_sum_tensor_list_f32(self._h, ptrs, C.c_size_t(len(ts)), _ptr(y), C.c_size_t(n)))
        return y

    def concatenate(self, tensors, axis, out=None):
        ts = [_host(t) for t in tensors]
        if not ts:
            raise ZantError(-11, "EmptyTensorList")
        shapes = [_shape(t) for t in ts]
        oshape = concat_output_shape(shapes, axis)
        dt = _dtype_code(ts[0])
        y = self._out(out, oshape, dt)
        ptrs, ranks, _keep = _shape_list(shapes)
        data = (C.c_void_p * len(ts))(*[_ptr(t).value for t in ts])
        ys, yr = _sz(oshape)
        check(lib().zant_b200_concatenate(self._h, C.c_int32(dt), data, ptrs, ranks, C.c_size_t(len(ts)), C.c_int64(axis),
                                          _ptr(y), ys, C.c_size_t(yr)))
        return y

    def get_concatenate_output_shape(self, shapes, axis):
        return get_concatenate_output_shape(shapes, axis)

    def get_unsqueeze_output_shape(self, x_shape, axes):
        xs, r = _sz(x_shape)
        out = (C.c_size_t * max(r + len(axes), 1))()
        check(lib().zant_b200_unsqueeze_output_shape(xs, C.c_size_t(r), _i64(axes), C.c_size_t(len(axes)), out))
        return [int(out[i]) for i in range(r + len(axes))]

    def unsqueeze(self, x, axes, out=None):
        x = _host(x)
        sh = _shape(x)
        oshape = self.get_unsqueeze_output_shape(sh, axes)
        dt = _dtype_code(x)
        y = self._out(out, oshape, dt)
        xs, r = _sz(sh); ys, yr = _sz(oshape)
        check(lib().zant_b200_unsqueeze(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(r), _i64(axes), C.c_size_t(len(axes)), _ptr(y), ys, C.c_size_t(yr)))
        return y

    def shape_onnx(self, x_shape, start=None, end=None):
        xs, r = _sz(x_shape)
        out = (C.c_int64 * max(r, 1))()
        n = C.c_size_t(0)
        check(lib().zant_b200_shape_onnx(xs, C.c_size_t(r), C.c_int32(start is not None), C.c_int64(start or 0), C.c_int32(end is not None),
                                         C.c_int64(end or 0), out, C.byref(n)))
        return np.array([out[i] for i in range(n.value)], np.int64)

    def transpose_onnx(self, x, perm=None, out=None):
        x = _host(x)
        sh = _shape(x)
        if perm is not None and len(perm) == len(sh) and sorted(int(p) for p in perm) == list(range(len(sh))):
            oshape = [sh[int(p)] for p in perm]
        else:
            oshape = list(reversed(sh))       # a bad perm is reported by the library
        dt = _dtype_code(x)
        y = self._out(out, oshape, dt)
        xs, r = _sz(sh); ys, yr = _sz(oshape); pm, npm = _sz(perm)
        check(lib().zant_b200_transpose_onnx(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(r), pm, C.c_size_t(npm), _ptr(y), ys, C.c_size_t(yr)))
        return y

    def get_slice_output_shape(self, x_shape, starts, ends, axes=None, steps=None, lean=False):
        n = len(starts)
        if len(ends) != n or (axes is not None and len(axes) != n) or (steps is not None and len(steps) != n):
            raise ZantError(-43, "InvalidSliceIndices")
        xs, r = _sz(x_shape)
        out = (C.c_size_t * max(r, 1))()
        fn = lib().zant_b200_slice_lean_dims if lean else lib().zant_b200_slice_output_shape
        check(fn(xs, C.c_size_t(r), _i64(starts), _i64(ends), C.c_size_t(n), _i64(axes), _i64(steps), out))
        return [int(out[i]) for i in range(r)]

    def slice_onnx(self, x, starts, ends, axes=None, steps=None, out=None):
        x = _host(x)
        sh = _shape(x)
        oshape = self.get_slice_output_shape(sh, starts, ends, axes, steps, lean=True)
        dt = _dtype_code(x)
        y = self._out(out, oshape, dt)
        xs, r = _sz(sh); ys, yr = _sz(oshape)
        check(lib().zant_b200_slice_onnx(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(r), _i64(starts), _i64(ends), C.c_size_t(len(starts)),
                                         _i64(axes), _i64(steps), _ptr(y), ys, C.c_size_t(yr)))
        return y

    def gather(self, x, indices, axis, out=None):
        x = _host(x)
        sh = _shape(x)
        idx = np.ascontiguousarray(np.asarray(indices), dtype=np.uint64)
        nd = len(sh)
        ax = axis + nd if -nd <= axis < 0 else (axis if 0 <= axis < nd else 0)
        oshape = (list(sh[:ax]) + list(idx.shape) + list(sh[ax + 1:])) if nd else [1]
        dt = _dtype_code(x)
        y = self._out(out, oshape, dt)
        xs, r = _sz(sh); ys, yr = _sz(oshape); is_, ir = _sz(idx.shape)
        check(lib().zant_b200_gather(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(r), idx.ctypes.data_as(C.c_void_p), is_, C.c_size_t(ir),
                                     C.c_int64(axis), _ptr(y), ys, C.c_size_t(yr)))
        return y

    def resize(self, x, mode, scales=None, sizes=None, coord_mode="half_pixel", out=None):
        x = _host(x)
        dt = _dtype_code(x)
        oshape = get_resize_output_shape(_shape(x), scales, sizes)
        y = self._out(out, oshape, dt)
        xs, r = _sz(_shape(x)); ys, yr = _sz(oshape)
        sc = None if scales is None else (C.c_float * max(len(scales), 1))(*scales)
        sz, nsz = _sz(sizes); m, ml = _bytes(mode); cm, cml = _bytes(coord_mode)
        check(lib().zant_b200_resize(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(r), m, C.c_size_t(ml), sc,
                                     C.c_size_t(0 if scales is None else len(scales)), sz, C.c_size_t(nsz), cm, C.c_size_t(cml),
                                     _ptr(y), ys, C.c_size_t(yr)))
        return y

    def reshape(self, x, new_shape):
        x = _host(x)
        dt = _dtype_code(x)
        y = np.zeros(_numel(_shape(x)), NP_DTYPE[dt])
        xs, xr = _sz(_shape(x)); ns, nr = _sz(new_shape)
        out = (C.c_size_t * max(nr, 1))()
        check(lib().zant_b200_reshape(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(xr), ns, C.c_size_t(nr), _ptr(y), out))
        return y.reshape(list(out)[:nr])

    def reduce_mean(self, x, axes=None, keepdims=True, noop_with_empty_axes=False, out=None):
        x = _host(x, np.float32)
        yshape = reduce_mean_shape(_shape(x), axes, keepdims, noop_with_empty_axes)
        y = self._out(out, yshape, F32)
        xs, xr = _sz(_shape(x)); ys, yr = _sz(yshape)
        ax = None if axes is None else (C.c_int64 * max(len(axes), 1))(*axes)
        check(lib().zant_b200_reduce_mean_f32(self._h, _ptr(x), xs, C.c_size_t(xr), _ptr(y), ys, C.c_size_t(yr), ax,
                                              C.c_size_t(0 if axes is None else len(axes)), C.c_int32(int(keepdims)),
                                              C.c_int32(int(noop_with_empty_axes))))
        return y

    # -- quantized operators
    def quantize_linear(self, x, scale, zp, out_dtype=U8, out=None):
        x = _host(x, np.float32)
        y = self._out(out, _shape(x), out_dtype)
        check(lib().zant_b200_quantize_linear(self._h, _ptr(x), C.c_size_t(_numel(_shape(x))), C.c_float(scale), C.c_int32(zp),
                                              C.c_int32(out_dtype), _ptr(y)))
        return y

    def dequantize_linear(self, q, scale, zp, out=None):
        q = _host(q)
        y = self._out(out, _shape(q), F32)
        check(lib().zant_b200_dequantize_linear(self._h, C.c_int32(_dtype_code(q)), _ptr(q), C.c_size_t(_numel(_shape(q))),
                                                C.c_float(scale), C.c_int32(zp), _ptr(y)))
        return y

    def qlinearconv(self, x, x_scale, x_zp, w, w_scale, w_zp, y_scale, y_zp, bias=None, y_dtype=I8, stride=(1, 1),
                    pads=(0, 0, 0, 0), dilations=(1, 1), group=1, auto_pad="NOTSET", activation=None, y_shape=None, out=None):
        x = _host(x); w = _host(w, np.int8)
        w_scale = np.atleast_1d(np.ascontiguousarray(w_scale, np.float32))
        w_zp = None if w_zp is None else np.atleast_1d(np.ascontiguousarray(w_zp, np.int32))
        bias = _host(bias, np.int32)
        if y_shape is None:
            y_shape = qconv_output_shape(_shape(x), _shape(w), stride, pads, dilations, auto_pad)
        y = self._out(out, y_shape, y_dtype)
        xs, xr = _sz(_shape(x)); ws, wr = _sz(_shape(w)); ys, yr = _sz(y_shape)
        st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
        check(lib().zant_b200_qlinearconv(self._h, C.c_int32(_dtype_code(x)), _ptr(x), xs, C.c_size_t(xr), C.c_float(x_scale),
                                          C.c_int32(x_zp), _ptr(w), ws, C.c_size_t(wr), _ptr(w_scale), _ptr(w_zp),
                                          C.c_size_t(w_scale.size), C.c_float(y_scale), C.c_int32(y_zp), _ptr(bias),
                                          C.c_size_t(0 if bias is None else bias.size), C.c_int32(y_dtype), _ptr(y), ys,
                                          C.c_size_t(yr), st, C.c_size_t(ns), pd, C.c_size_t(npd), dl, C.c_size_t(nd),
                                          C.c_size_t(group), C.c_int32(AUTO_PAD[auto_pad]), C.c_int32(QACT[activation])))
        return y

    def qlinearconv_nhwc(self, x, x_scale, x_zp, w, w_scale, w_zp, y_scale, y_zp, bias=None, y_dtype=I8, stride=(1, 1),
                         pads=(0, 0, 0, 0), dilations=(1, 1), group=1, auto_pad="NOTSET", activation=None, out=None):
        """QLinearConv on channels-last tensors (zant_b200_qlinearconv_nhwc): x [N,H,W,C] -> y [N,OH,OW,M],
        w in the ONNX [M,C,KH,KW] order; everything else as qlinearconv."""
        x = _host(x); w = _host(w, np.int8)
        w_scale = np.atleast_1d(np.ascontiguousarray(w_scale, np.float32))
        w_zp = None if w_zp is None else np.atleast_1d(np.ascontiguousarray(w_zp, np.int32))
        bias = _host(bias, np.int32)
        n, h, wd, c = _shape(x)
        yn, ym, yh, yw = qconv_output_shape((n, c, h, wd), _shape(w), stride, pads, dilations, auto_pad)
        y_shape = (yn, yh, yw, ym)
        y = self._out(out, y_shape, y_dtype)
        xs, xr = _sz(_shape(x)); ws, wr = _sz(_shape(w)); ys, yr = _sz(y_shape)
        st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
        check(lib().zant_b200_qlinearconv_nhwc(self._h, C.c_int32(_dtype_code(x)), _ptr(x), xs, C.c_size_t(xr), C.c_float(x_scale),
                                               C.c_int32(x_zp), _ptr(w), ws, C.c_size_t(wr), _ptr(w_scale), _ptr(w_zp),
                                               C.c_size_t(w_scale.size), C.c_float(y_scale), C.c_int32(y_zp), _ptr(bias),
                                               C.c_size_t(0 if bias is None else bias.size), C.c_int32(y_dtype), _ptr(y), ys,
                                               C.c_size_t(yr), st, C.c_size_t(ns), pd, C.c_size_t(npd), dl, C.c_size_t(nd),
                                               C.c_size_t(group), C.c_int32(AUTO_PAD[auto_pad]), C.c_int32(QACT[activation])))
        return y

    def qlinearmatmul(self, a, a_scale, a_zp, b, b_scale, b_zp, y_scale, y_zp, bias=None, y_dtype=I8, activation=None, out=None):
        a = _host(a); b = _host(b, np.int8)
        b_scale = np.atleast_1d(np.ascontiguousarray(b_scale, np.float32))
        b_zp = None if b_zp is None else np.atleast_1d(np.ascontiguousarray(b_zp, np.int32))
        bias = _host(bias, np.int32)
        yshape = (_shape(a)[0], _shape(b)[1])
        y = self._out(out, yshape, y_dtype)
        as_, ar = _sz(_shape(a)); bs, br = _sz(_shape(b)); ys, yr = _sz(yshape)
        check(lib().zant_b200_qlinearmatmul(self._h, C.c_int32(_dtype_code(a)), _ptr(a), as_, C.c_size_t(ar), C.c_float(a_scale),
                                            C.c_int32(a_zp), _ptr(b), bs, C.c_size_t(br), _ptr(b_scale), _ptr(b_zp),
                                            C.c_size_t(b_scale.size), C.c_float(y_scale), C.c_int32(y_zp), _ptr(bias),
                                            C.c_size_t(0 if bias is None else bias.size), C.c_int32(y_dtype), _ptr(y), ys,
                                            C.c_size_t(yr), C.c_int32(QACT[activation])))
        return y

    def qlinearadd(self, a, a_scale, a_zp, b, b_scale, b_zp, y_scale, y_zp, activation=None, out=None):
        a = _host(a); b = _host(b)
        dt = _dtype_code(a)
        y = self._out(out, _shape(a), dt)
        check(lib().zant_b200_qlinearadd(self._h, C.c_int32(dt), _ptr(a), C.c_float(a_scale), C.c_int32(a_zp), _ptr(b),
                                         C.c_float(b_scale), C.c_int32(b_zp), C.c_float(y_scale), C.c_int32(y_zp), _ptr(y),
                                         C.c_size_t(_numel(_shape(a))), C.c_int32(QACT[activation])))
        return y

    def qlinear_global_avgpool(self, x, x_scale, x_zp, y_scale, y_zp, out=None):
        x = _host(x)
        dt = _dtype_code(x)
        y = self._out(out, (_shape(x)[0], _shape(x)[1], 1, 1), dt)
        xs, xr = _sz(_shape(x))
        check(lib().zant_b200_qlinear_global_avgpool(self._h, C.c_int32(dt), _ptr(x), xs, C.c_size_t(xr), C.c_float(x_scale),
                                                     C.c_int32(x_zp), C.c_float(y_scale), C.c_int32(y_zp), _ptr(y)))
        return y

    def lut_q8(self, x, lut, out=None):
        x = _host(x); lut = np.ascontiguousarray(lut, np.uint8)
        y = self._out(out, _shape(x), _dtype_code(x))
        check(lib().zant_b200_lut_q8(self._h, _ptr(x), _ptr(lut), _ptr(y), C.c_size_t(_numel(_shape(x)))))
        return y


def qlinearconv_noalloc(x, x_scale, x_zp, w, w_scale, w_zp, y_scale, y_zp, out, bias=None, stride=(1, 1), pads=(0, 0, 0, 0),
                        dilations=(1, 1), group=1, auto_pad="NOTSET", activation=None, stream=None):
    """QLinearConv without any device allocation (zant_b200_qlinearconv_noalloc): no Context is
    involved; x, w, bias and `out` are device tensors (objects with data_ptr()), `stream` is a raw
    cudaStream_t value or None for the default stream.  Asynchronous."""
    w_scale = np.atleast_1d(np.ascontiguousarray(w_scale, np.float32))
    w_zp = None if w_zp is None else np.atleast_1d(np.ascontiguousarray(w_zp, np.int32))
    xs, xr = _sz(_shape(x)); ws, wr = _sz(_shape(w)); ys, yr = _sz(_shape(out))
    st, ns = _sz(stride); pd, npd = _sz(pads); dl, nd = _sz(dilations)
    check(lib().zant_b200_qlinearconv_noalloc(
        C.c_void_p(stream), C.c_int32(_dtype_code(x)), _ptr(x), xs, C.c_size_t(xr), C.c_float(x_scale), C.c_int32(x_zp),
        _ptr(w), ws, C.c_size_t(wr), _ptr(w_scale), _ptr(w_zp), C.c_size_t(w_scale.size), C.c_float(y_scale), C.c_int32(y_zp),
        _ptr(bias), C.c_size_t(0 if bias is None else _numel(_shape(bias))), C.c_int32(_dtype_code(out)), _ptr(out), ys,
        C.c_size_t(yr), st, C.c_size_t(ns), pd, C.c_size_t(npd), dl, C.c_size_t(nd), C.c_size_t(group),
        C.c_int32(AUTO_PAD[auto_pad]), C.c_int32(QACT[activation])))
    return out


def debug_fail_alloc(nth):
    """Test hook: the `nth` next device allocation of the library fails (0 disarms)."""
    check(lib().zant_b200_debug_fail_alloc(C.c_int32(int(nth))))


def qconv_output_shape(x_shape, w_shape, stride, pads, dilations, auto_pad="NOTSET"):
    """ONNX output shape of QLinearConv (explicit pads unless auto_pad says otherwise)."""
    sh = stride[0] if len(stride) > 0 else 1
    sw = stride[1] if len(stride) > 1 else sh
    dh = dilations[0] if dilations is not None and len(dilations) > 0 else 1
    dw = dilations[1] if dilations is not None and len(dilations) > 1 else dh
    dkh, dkw = (w_shape[2] - 1) * dh + 1, (w_shape[3] - 1) * dw + 1
    H, W = x_shape[2], x_shape[3]
    if auto_pad in ("SAME_UPPER", "SAME_LOWER"):
        return [x_shape[0], w_shape[0], -(-H // sh), -(-W // sw)]
    ph = pw = 0
    if auto_pad == "NOTSET" and pads is not None and len(pads) >= 4:
        ph, pw = pads[0] + pads[2], pads[1] + pads[3]
    return [x_shape[0], w_shape[0], (H + ph - dkh) // sh + 1, (W + pw - dkw) // sw + 1]


# ----------------------------------------------------------------------------------------- graph description + plan
class Graph:
    """A frozen inference graph: tensors (activations and initializers) and nodes in execution
    order — what the reference's code generator would have unrolled into a predict() body."""

    def __init__(self, name=""):
        self.name = name
        self.tensors = []   # dict(name, dtype, shape, data)
        self.nodes = []     # dict(op, inputs, outputs, attrs)
        self.input = None
        self.output = None
        self.meta = {}

    def tensor(self, name, dtype, shape, data=None):
        if data is not None:
            data = np.ascontiguousarray(data, NP_DTYPE[dtype]).reshape(shape)
        self.tensors.append(dict(name=name, dtype=dtype, shape=[int(s) for s in shape], data=data))
        return len(self.tensors) - 1

    def node(self, op, inputs, outputs, **attrs):
        self.nodes.append(dict(op=op, inputs=list(inputs), outputs=list(outputs), attrs=attrs))
        return len(self.nodes) - 1

    def id_of(self, name):
        for i, t in enumerate(self.tensors):
            if t["name"] == name:
                return i
        raise KeyError(name)


def _fill_attrs(attrs):
    a = NodeAttrs()
    a.auto_pad = -1
    for k, v in attrs.items():
        if k == "kernel_shape":
            a.kernel_shape[0], a.kernel_shape[1] = v
        elif k == "strides":
            for i, s in enumerate(v): a.strides[i] = s
            a.n_strides = len(v)
        elif k == "dilations":
            for i, s in enumerate(v): a.dilations[i] = s
            a.n_dilations = len(v)
        elif k == "pads":
            for i, s in enumerate(v): a.pads[i] = s
            a.n_pads = len(v)
        elif k == "auto_pad":
            a.auto_pad = -1 if v is None else AUTO_PAD[v]
        elif k == "axes":
            for i, s in enumerate(v): a.axes[i] = s
            a.n_axes = len(v)
        elif k == "scales":
            for i, s in enumerate(v): a.scales[i] = s
            a.n_scales = len(v)
        elif k == "perm":
            if v is not None:
                for i, s in enumerate(v): a.perm[i] = s
                a.n_perm = len(v)
        elif k in ("starts", "ends", "slice_axes", "steps"):
            if v is not None:
                arr = {"starts": a.slice_starts, "ends": a.slice_ends, "slice_axes": a.slice_axes, "steps": a.slice_steps}[k]
                for i, s in enumerate(v): arr[i] = s
                a.n_slice = len(v)
                if k == "slice_axes": a.slice_has_axes = 1
                if k == "steps": a.slice_has_steps = 1
        elif k == "coord_mode":
            a.coord_mode = COORD_MODE[v]
        elif k == "activation":
            a.activation = QACT[v]
        elif k in ("alpha", "beta", "x_scale", "b_scale", "y_scale"):
            setattr(a, k, float(v))
        elif k in ("group", "trans_a", "trans_b", "axis", "keepdims", "noop_with_empty_axes", "x_zp", "b_zp", "y_zp", "channels_last"):
            setattr(a, k, int(v))
        else:
            raise KeyError(f"unknown node attribute {k}")
    return a


class Plan:
    """Run-time form of a Graph on one Context (the analogue of a generated predict())."""

    def __init__(self, ctx, graph, fuse=True):
        self.ctx = ctx
        self.graph = graph
        self._h = C.c_void_p(None)
        L = lib()
        check(L.zant_b200_plan_create(ctx._h, C.byref(self._h)))
        try:
            for t in graph.tensors:
                sh, r = _sz(t["shape"])
                tid = C.c_int32(-1)
                check(L.zant_b200_plan_tensor(self._h, C.c_int32(t["dtype"]), sh, C.c_size_t(r), _ptr(t["data"]), C.byref(tid)))
            for n in graph.nodes:
                ins = (C.c_int32 * max(len(n["inputs"]), 1))(*n["inputs"])
                outs = (C.c_int32 * max(len(n["outputs"]), 1))(*n["outputs"])
                a = _fill_attrs(n["attrs"])
                check(L.zant_b200_plan_node(self._h, C.c_int32(OP[n["op"]]), ins, C.c_size_t(len(n["inputs"])), outs,
                                            C.c_size_t(len(n["outputs"])), C.byref(a)))
            check(L.zant_b200_plan_finalize(self._h, C.c_int32(graph.input), C.c_int32(graph.output), C.c_int32(int(fuse))))
        except Exception:
            L.zant_b200_plan_destroy(self._h)
            self._h = C.c_void_p(None)
            raise
        self.in_shape = graph.tensors[graph.input]["shape"]
        self.out_shape = graph.tensors[graph.output]["shape"]
        self.in_dtype = graph.tensors[graph.input]["dtype"]
        self.out_dtype = graph.tensors[graph.output]["dtype"]

    def close(self):
        if self._h:
            lib().zant_b200_plan_destroy(self._h)
            self._h = C.c_void_p(None)

    def run(self, x, out=None):
        """predict(): numpy in -> numpy out, or device tensors in place (asynchronous)."""
        x = _host(x, NP_DTYPE[self.in_dtype]) if not hasattr(x, "data_ptr") else x
        y = np.zeros(self.out_shape, NP_DTYPE[self.out_dtype]) if out is None else out
        check(lib().zant_b200_plan_run(self._h, _ptr(x), _ptr(y)))
        return y

    def read_tensor(self, tid):
        if isinstance(tid, str):
            tid = self.graph.id_of(tid)
        t = self.graph.tensors[tid]
        y = np.zeros(t["shape"], NP_DTYPE[t["dtype"]])
        check(lib().zant_b200_plan_read_tensor(self._h, C.c_int32(tid), _ptr(y)))
        return y

    def step_names(self):
        L = lib()
        return [L.zant_b200_plan_step_name(self._h, C.c_int32(i)).decode() for i in range(L.zant_b200_plan_step_count(self._h))]

    def step_costs(self):
        """[(macs, bytes)] per step: the algorithmic work behind the roofline figures."""
        L = lib()
        out = []
        for i in range(L.zant_b200_plan_step_count(self._h)):
            m, b = C.c_double(0), C.c_double(0)
            check(L.zant_b200_plan_step_cost(self._h, C.c_int32(i), C.byref(m), C.byref(b)))
            out.append((m.value, b.value))
        return out

    def use_graph(self, enable=True):
        """Replays all steps as one captured CUDA graph per run (batch-1 latency)."""
        check(lib().zant_b200_plan_use_graph(self._h, C.c_int32(int(enable))))

    def profile(self, enable=True):
        check(lib().zant_b200_plan_profile(self._h, C.c_int32(int(enable))))

    def profile_read(self):
        """(per-step summed milliseconds, number of runs) recorded since the last read."""
        n = lib().zant_b200_plan_step_count(self._h)
        ms = (C.c_float * max(n, 1))()
        runs = C.c_int32(0)
        check(lib().zant_b200_plan_profile_read(self._h, ms, C.byref(runs)))
        return list(ms)[:n], runs.value

    @property
    def arena_bytes(self):
        return int(lib().zant_b200_plan_arena_bytes(self._h))

    @property
    def launches_per_run(self):
        return int(lib().zant_b200_plan_launches_per_run(self._h))


class _ShardContext(Context):
    """Context of one shard of a ShardedPredict (owned by the multi handle, not closed by itself)."""

    def __init__(self, handle):
        self._h = handle

    def close(self):
        self._h = C.c_void_p(None)


class ShardedPredict:
    """predict() over several GPUs of one machine (zant_b200_multi_* / zant_b200_predict_sharded):
    `make_graph(batch)` builds the graph of one shard; the global batch is split by shard_range, every
    device runs its own plan on its own context, stream and worker thread, and writes its slice of
    the output.  No collective."""

    def __init__(self, make_graph, global_batch, devices=None, fuse=True, arena_bytes=0):
        L = lib()
        L.zant_b200_multi_size.restype = C.c_size_t
        L.zant_b200_multi_ctx.restype = C.c_void_p
        self._h = C.c_void_p(None)
        devs = None if not devices else (C.c_int32 * len(devices))(*devices)
        check(L.zant_b200_multi_create(devs, C.c_size_t(0 if not devices else len(devices)), C.c_size_t(arena_bytes), C.byref(self._h)))
        self.world = int(L.zant_b200_multi_size(self._h))
        self.global_batch = int(global_batch)
        self.plans, self.contexts = [], []
        try:
            for i in range(self.world):
                _b, count = shard_range(self.global_batch, self.world, i)
                ctx = _ShardContext(C.c_void_p(L.zant_b200_multi_ctx(self._h, C.c_size_t(i))))
                self.contexts.append(ctx)
                if count == 0:
                    self.plans.append(None)
                    continue
                plan = Plan(ctx, make_graph(count), fuse=fuse)
                self.plans.append(plan)
                check(L.zant_b200_multi_set_plan(self._h, C.c_size_t(i), plan._h))
        except Exception:
            self.close()
            raise
        first = next(p for p in self.plans if p is not None)
        self.sample_in = tuple(first.in_shape[1:]); self.sample_out = tuple(first.out_shape[1:])
        self.in_dtype, self.out_dtype = first.in_dtype, first.out_dtype

    def run(self, x, out=None, return_status=False):
        """x: host array (numpy, or a CPU torch tensor, pinned or not) of the global batch."""
        x = _host(x, NP_DTYPE[self.in_dtype]) if not hasattr(x, "data_ptr") else x
        y = np.zeros((self.global_batch,) + self.sample_out, NP_DTYPE[self.out_dtype]) if out is None else out
        st = (C.c_int32 * self.world)()
        rc = lib().zant_b200_predict_sharded(self._h, _ptr(x), _ptr(y), C.c_size_t(self.global_batch), st)
        if return_status:
            return y, rc, list(st)
        check(rc)
        return y

    def close(self):
        for p in self.plans:
            if p is not None:
                p.close()
        self.plans = []
        if self._h:
            lib().zant_b200_multi_destroy(self._h)
            self._h = C.c_void_p(None)
