"""Writes tests/golden/reference_goldens.json.

The vectors below were transcribed by hand from the unit tests of the Z-Ant tree (the file and
line range of the Zig test is given in every case's "cite").  The Z-Ant sources are Zig and cannot
be executed with the toolchains available to this repository, so nothing here is *computed* by the
reference: inputs and expected outputs are the literals its tests assert.  Re-run this script after
editing a case:  python tests/golden/make_reference_goldens.py
"""
import json
import os

T = "tests/Core/Tensor/TensorMath/"
ones55 = [1.0] * 25
same_upper_55 = [4, 6, 6, 6, 4, 6, 9, 9, 9, 6, 6, 9, 9, 9, 6, 6, 9, 9, 9, 6, 4, 6, 6, 6, 4]
seq16 = [float(i) for i in range(1, 17)]
seq9 = [float(i) for i in range(1, 10)]

cases = []


def add(**kw):
    cases.append(kw)


# ----------------------------------------------------------------------------- Conv
add(op="convolve_tensor_with_bias", cite=T + "test_op_convolution.zig:8-140",
    x_shape=[2, 2, 3, 3],
    x=[2, 2, 3, 4, 5, 6, 7, 8, 9, 8, 8, 7, 6, 5, 4, 3, 2, 1,
       2, 3, 4, 5, 6, 7, 8, 9, 10, 10, 9, 8, 7, 6, 5, 4, 3, 2],
    w_shape=[2, 2, 2, 2],
    w=[-1, 0, 0, 1, 1, -1, -1, 1, 0, 0, 0, 0, 0, 0, 0, 0],
    bias=[1, 1], stride=[1, 1], pads=None, dilations=None, group=None, auto_pad="VALID",
    note="the Zig test calls convolve_tensor_with_bias directly (no padding); conv_lean with "
         "auto_pad VALID runs the identical code on an unpadded copy",
    y_shape=[2, 2, 2, 2],
    y=[3, 5, 5, 5, 1, 1, 1, 1, 5, 5, 5, 5, 1, 1, 1, 1])
add(op="conv_lean", cite=T + "test_op_convolution.zig:654-709",
    x_shape=[1, 1, 5, 5], x=ones55, w_shape=[1, 1, 3, 3], w=[1.0] * 9, bias=None,
    stride=[1], pads=[0, 0, 0, 0], dilations=None, group=None, auto_pad=None,
    y_shape=[1, 1, 3, 3], y=[9.0] * 9)
add(op="conv_lean", cite=T + "test_op_convolution.zig:711-812",
    x_shape=[1, 1, 5, 5], x=ones55, w_shape=[1, 1, 3, 3], w=[1.0] * 9, bias=None,
    stride=[1], pads=None, dilations=None, group=None, auto_pad="SAME_UPPER",
    y_shape=[1, 1, 5, 5], y=same_upper_55)
add(op="conv_lean", cite=T + "test_op_convolution.zig:814-874",
    x_shape=[1, 1, 5, 5], x=ones55, w_shape=[1, 1, 2, 2], w=[1.0] * 4, bias=[1.0],
    stride=[1], pads=None, dilations=[2], group=None, auto_pad=None,
    y_shape=[1, 1, 3, 3], y=[5.0] * 9)
# The same three through the allocating wrapper Conv (OnnxConv): the output shape is computed.
add(op="Conv", cite=T + "test_op_convolution.zig:876-930",
    x_shape=[1, 1, 5, 5], x=ones55, w_shape=[1, 1, 3, 3], w=[1.0] * 9, bias=None,
    stride=[1], pads=[0, 0, 0, 0], dilations=None, group=None, auto_pad=None,
    y_shape=[1, 1, 3, 3], y=[9.0] * 9)
add(op="Conv", cite=T + "test_op_convolution.zig:932-988",
    x_shape=[1, 1, 5, 5], x=ones55, w_shape=[1, 1, 3, 3], w=[1.0] * 9, bias=None,
    stride=[1], pads=None, dilations=None, group=None, auto_pad="SAME_UPPER",
    y_shape=[1, 1, 5, 5], y=same_upper_55)
add(op="Conv", cite=T + "test_op_convolution.zig:990-1043",
    x_shape=[1, 1, 5, 5], x=ones55, w_shape=[1, 1, 2, 2], w=[1.0] * 4, bias=[1.0],
    stride=[1], pads=None, dilations=[2], group=None, auto_pad=None,
    y_shape=[1, 1, 3, 3], y=[5.0] * 9)

# ----------------------------------------------------------------------------- Gemm
add(op="gemm", cite=T + "test_op_gemm.zig:14-37",
    a_shape=[1, 1, 2, 2], a=[1, 2, 4, 5], b_shape=[1, 1, 2, 2], b=[1, 2, 4, 5], c_shape=None, c=None,
    alpha=1, beta=1, transA=False, transB=False, y_shape=[1, 1, 2, 2], y_at={"0": 9, "1": 12})
add(op="gemm", cite=T + "test_op_gemm.zig:39-69",
    a_shape=[1, 1, 2, 2], a=[1, 2, 4, 5], b_shape=[1, 1, 2, 1], b=[1, 4], c_shape=[1, 1, 2, 1], c=[1, 4],
    alpha=1, beta=1, transA=False, transB=False, y_shape=[1, 1, 2, 1], y_at={"0": 10, "1": 28})
add(op="gemm", cite=T + "test_op_gemm.zig:71-107",
    a_shape=[1, 1, 3, 3], a=seq9, b_shape=[1, 1, 3, 2], b=[1, 2, 4, 5, 7, 8], c_shape=[1, 1, 1, 2], c=[1, 2],
    alpha=1, beta=1, transA=False, transB=False, y_shape=[1, 1, 3, 2], y_at={"0": 31, "5": 128})
add(op="gemm", cite=T + "test_op_gemm.zig:109-144",
    a_shape=[1, 1, 3, 3], a=seq9, b_shape=[1, 1, 2, 3], b=[1, 4, 7, 2, 5, 8], c_shape=[1, 1, 1, 2], c=[1, 2],
    alpha=2, beta=3, transA=False, transB=True, y_shape=[1, 1, 3, 2], y_at={"0": 63, "5": 258})
add(op="gemm", cite=T + "test_op_gemm.zig:146-193",
    a_shape=[1, 1, 3, 2], a=[1, 2, 4, 5, 7, 8], b_shape=[1, 1, 2, 3], b=[1, 4, 7, 2, 5, 8],
    c_shape=[1, 1, 2, 1], c=[1, 2],
    alpha=2, beta=3, transA=True, transB=True, y_shape=[1, 1, 2, 2], y_at={"0": 135, "1": 159, "2": 162, "3": 192})
add(op="gemm_error", cite=T + "test_op_gemm.zig:280-297",
    a_shape=[1, 2, 2], b_shape=[1, 2, 2], error="InputTensorsWrongShape")
add(op="gemm_error", cite=T + "test_op_gemm.zig:299-316",
    a_shape=[2, 1, 2, 2], b_shape=[1, 2, 2, 2], error="InputTensorDifferentShape")
add(op="gemm_error", cite=T + "test_op_gemm.zig:318-335",
    a_shape=[4, 4, 2, 2], b_shape=[4, 4, 3, 2], error="InputTensorDimensionMismatch")

# ----------------------------------------------------------------------------- MatMul
add(op="mat_mul", cite=T + "test_op_mat_mul.zig:9-32",
    a_shape=[2, 2], a=[1, 2, 4, 5], b_shape=[2, 2], b=[1, 2, 4, 5], y_shape=[2, 2], y_at={"0": 9, "1": 12})
add(op="mat_mul_error", cite=T + "test_op_mat_mul.zig:34-49",
    a_shape=[2, 2], b_shape=[3, 2], error="InputTensorsWrongShape")
add(op="mat_mul_error", cite=T + "test_op_mat_mul.zig:51-64",
    a_shape=[2, 2], b_shape=[4, 1], error="InputTensorsWrongShape")

# ----------------------------------------------------------------------------- MaxPool
add(op="onnx_maxpool", cite=T + "test_op_pooling.zig:156-202",
    x_shape=[1, 1, 4, 4], x=seq16, kernel=[2, 2], strides=[2, 2], dilations=[1, 1], pads=[0, 0, 0, 0],
    auto_pad="NOTSET", ceil_mode=False, y_shape=[1, 1, 2, 2], y=[6, 8, 14, 16])
add(op="onnx_maxpool", cite=T + "test_op_pooling.zig:204-254",
    x_shape=[1, 1, 3, 3], x=seq9, kernel=[2, 2], strides=[1, 1], dilations=[1, 1], pads=[0, 0, 0, 0],
    auto_pad="SAME_UPPER", ceil_mode=False, y_shape=[1, 1, 3, 3], y=[5, 6, 6, 8, 9, 9, 8, 9, 9])
add(op="onnx_maxpool", cite=T + "test_op_pooling.zig:256-304",
    x_shape=[1, 1, 4, 4], x=seq16, kernel=[2, 2], strides=[1, 1], dilations=[2, 2], pads=[0, 0, 0, 0],
    auto_pad="NOTSET", ceil_mode=False, y_shape=[1, 1, 2, 2], y=[11, 12, 15, 16])
add(op="onnx_maxpool", cite=T + "test_op_pooling.zig:306-351",
    x_shape=[1, 1, 3, 3], x=seq9, kernel=[2, 2], strides=[2, 2], dilations=[1, 1], pads=[0, 0, 0, 0],
    auto_pad="NOTSET", ceil_mode=True, y_shape=[1, 1, 2, 2], y=[5, 6, 8, 9])
add(op="onnx_maxpool", cite=T + "test_op_pooling.zig:353-416",
    x_shape=[1, 1, 3, 3], x=seq9, kernel=[2, 2], strides=[1, 1], dilations=[1, 1], pads=[1, 1, 1, 1],
    auto_pad="NOTSET", ceil_mode=False, y_shape=[1, 1, 4, 4],
    y=[1, 2, 3, 3, 4, 5, 6, 6, 7, 8, 9, 9, 7, 8, 9, 9])

# ----------------------------------------------------------------------------- activations
A = "tests/Model/test_activation_function.zig"
add(op="ReLU", cite=A + ":13-35", x=[1, -2, -4, 5], y=[1, 0, 0, 5],
    note="the Zig test asserts sign/zero only; the values follow from lean_ReLU")
add(op="ReLU", cite=A + ":37-58", x=[-1, -2, -4, -5], y=[0, 0, 0, 0])
add(op="ReLU", cite=A + ":60-81", x=[1, 2, 4, 5], y=[1, 2, 4, 5])
add(op="leakyReLU", cite=A + ":265-287", x=[1, -2, -4, 5], slope=0.01, y=[1, -0.02, -0.04, 5], atol=1e-5)
add(op="leakyReLU", cite=A + ":289-310", x=[-1, -2, -4, -5], slope=0.01, y=[-0.01, -0.02, -0.04, -0.05], atol=1e-5)
add(op="leakyReLU", cite=A + ":312-333", x=[1, 2, 4, 5], slope=0.01, y=[1, 2, 4, 5], atol=0)

add(op="sigmoid", cite=A + ":210-227", x=[0.0, 2.0, -2.0], y=[0.5, 0.880797, 0.119203], atol=1e-6,
    note="the Zig test runs on f64; the f32 kernel meets the same 1e-6 bound")
add(op="softmax_rows_sum_to_one", cite=A + ":126-151", x_shape=[2, 2], x=[1.0, 2.0, 4.0, 5.0], lo=0.9, hi=1.1)
add(op="softmax_equal_entries", cite=A + ":153-175", x_shape=[2, 2], x=[0.0, 0.0, 0.0, 0.0])

# ----------------------------------------------------------------------------- element-wise
E = T + "test_lib_elementWise_math.zig"
add(op="div", cite=E + ":234-262", a=[2, 4, 6, 8, 10, 12], b=[1, 2, 3, 4, 5, 6], y=[2, 2, 2, 2, 2, 2],
    note="the Zig test divides u8 tensors; the quotients are exact, so the f32 operator gives the same values")
add(op="tanh_matches_libm", cite=E + ":387-409", x=[0.0, 1.0, -1.0, 0.5, -0.5, 2.0], atol=1e-6)
add(op="ceil", cite=E + ":411-434", x=[0.0, 1.2, -1.2, 0.5, -0.5, 2.0], y=[0.0, 2.0, -1.0, 1.0, 0.0, 2.0], atol=1e-6)
add(op="sum_tensors", cite=E + ":10-32", a_shape=[2, 2], a=[1, 2, 4, 5], b_shape=[2, 2], b=[1, 2, 4, 5],
    y_shape=[2, 2], y_at={"0": 2, "1": 4})
add(op="add_bias", cite=E + ":90-115", t_shape=[2, 3], t=[1, 2, 3, 4, 5, 6], bias=[1, 1, 1], y=[2, 3, 4, 5, 6, 7])
add(op="sum_tensor_list", cite=E + ":265-299",
    tensors=[[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], y=[15, 18, 21, 24])
add(op="sum_tensor_list", cite=E + ":301-322", tensors=[[1, 2, 3, 4]], y=[1, 2, 3, 4])
add(op="sum_tensor_list_error", cite=E + ":324-329", tensors=[], error="EmptyTensorList")

# ----------------------------------------------------------------------------- reductions
R = T + "test_lib_reduction_math.zig"
add(op="reduce_mean", cite=R + ":24-38", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], axes=[0], keepdims=True, noop=False,
    y_shape=[1, 3], y=[2.5, 3.5, 4.5])
add(op="reduce_mean", cite=R + ":40-54", x_shape=[2, 2, 2], x=[1, 2, 3, 4, 5, 6, 7, 8], axes=[1, 2], keepdims=False,
    noop=False, y_shape=[2], y=[2.5, 6.5])
add(op="reduce_mean", cite=R + ":56-68", x_shape=[2, 2], x=[1, 2, 3, 4], axes=None, keepdims=True, noop=False,
    y_shape=[1, 1], y=[2.5])
add(op="reduce_mean", cite=R + ":70-86", x_shape=[2, 2], x=[1, 2, 3, 4], axes=None, keepdims=True, noop=True,
    y_shape=[2, 2], y=[1, 2, 3, 4])
add(op="reduce_mean", cite=R + ":88-105", x_shape=[2, 3, 2], x=[float(i) for i in range(1, 13)], axes=[-1],
    keepdims=False, noop=False, y_shape=[2, 3], y=[1.5, 3.5, 5.5, 7.5, 9.5, 11.5])
add(op="reduce_mean", cite=R + ":122-150", x_shape=[2, 3, 4], x=[float(i) for i in range(1, 25)], axes=[0, 2],
    keepdims=True, noop=False, y_shape=[1, 3, 1], y=[8.5, 12.5, 16.5])
add(op="reduce_mean", cite=R + ":152-180", x_shape=[2, 2, 2, 2], x=seq16, axes=[1], keepdims=False, noop=False,
    y_shape=[2, 2, 2], y_at={"0": 3.0, "1": 4.0, "2": 5.0})

# ----------------------------------------------------------------------------- shape ops
S = T + "test_lib_shape_math.zig"
add(op="concatenate", cite=S + ":9-51", dtype="f32", shapes=[[2, 2], [2, 2]], tensors=[[1, 2, 3, 4], [5, 6, 7, 8]],
    axis=0, y_shape=[4, 2], y=[1, 2, 3, 4, 5, 6, 7, 8])
add(op="concatenate", cite=S + ":53-94", dtype="f32", shapes=[[2, 2], [2, 2]], tensors=[[1, 2, 3, 4], [5, 6, 7, 8]],
    axis=1, y_shape=[2, 4], y=[1, 2, 5, 6, 3, 4, 7, 8])
add(op="concatenate", cite=S + ":96-137", dtype="f32", shapes=[[2, 2], [2, 2]], tensors=[[1, 2, 3, 4], [5, 6, 7, 8]],
    axis=-1, y_shape=[2, 4], y=[1, 2, 5, 6, 3, 4, 7, 8])
add(op="concatenate", cite=S + ":139-189", dtype="f32", shapes=[[2, 2, 2], [2, 2, 3]],
    tensors=[[1, 2, 3, 4, 5, 6, 7, 8], [9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20]],
    axis=2, y_shape=[2, 2, 5],
    y=[1, 2, 9, 10, 11, 3, 4, 12, 13, 14, 5, 6, 15, 16, 17, 7, 8, 18, 19, 20])
add(op="concatenate_error", cite=S + ":2182-2200", shapes=[[2, 2], [2, 3]], axis=0, error="MismatchedShape")
add(op="concatenate", cite=S + ":2202-2228", dtype="f32", shapes=[[2, 2], [2, 3]],
    tensors=[[1, 2, 3, 4], [5, 6, 7, 8, 9, 10]], axis=1, y_shape=[2, 5], y=[1, 2, 5, 6, 7, 3, 4, 8, 9, 10])
add(op="concatenate_error", cite=S + ":2230-2256", shapes=[[2, 2], [2, 2]], axis=2, error="AxisOutOfBounds")
add(op="concatenate_error", cite=S + ":2230-2256", shapes=[[2, 2], [2, 2]], axis=-3, error="AxisOutOfBounds")
add(op="get_concatenate_output_shape", cite=S + ":781-796", shapes=[[2, 3], [3, 3], [1, 3]], axis=0, y_shape=[6, 3])
add(op="get_concatenate_output_shape", cite=S + ":798-810", shapes=[[2, 3], [2, 2]], axis=1, y_shape=[2, 5])
add(op="get_concatenate_output_shape", cite=S + ":812-818", shapes=[[2, 3], [2, 2]], axis=-1, y_shape=[2, 5])
add(op="get_concatenate_output_shape_error", cite=S + ":820-822", shapes=[], axis=0, error="EmptyTensorList")
add(op="get_concatenate_output_shape_error", cite=S + ":824-829", shapes=[[2, 3], [3, 4]], axis=0, error="MismatchedShape")
add(op="get_concatenate_output_shape_error", cite=S + ":831-836", shapes=[[2, 3], [2, 3, 4]], axis=0, error="MismatchedRank")
add(op="get_concatenate_output_shape_error", cite=S + ":838-839", shapes=[[2, 3], [2, 2]], axis=2, error="AxisOutOfBounds")
add(op="get_concatenate_output_shape_error", cite=S + ":840-841", shapes=[[2, 3], [2, 2]], axis=-3, error="AxisOutOfBounds")
add(op="resize", cite=S + ":480-500", dtype="u8", x_shape=[4], x=[1, 2, 3, 4], mode="nearest", scales=[2.0],
    sizes=None, coord_mode="half_pixel", y_shape=[8], y_at={"0": 1, "1": 1, "2": 2, "3": 2})
add(op="resize", cite=S + ":502-518", dtype="u8", x_shape=[2, 2], x=[1, 2, 3, 4], mode="nearest", scales=[2.0, 2.0],
    sizes=None, coord_mode="half_pixel", y_shape=[4, 4], y_at={})
add(op="resize", cite=S + ":574-594", dtype="u8", x_shape=[2, 2], x=[1, 2, 3, 4], mode="nearest", scales=None,
    sizes=[3, 3], coord_mode="half_pixel", y_shape=[3, 3], y_at={})
add(op="resize_error", cite=S + ":596-613", x_shape=[2, 2], mode="invalid_mode", scales=[2.0, 2.0], sizes=None,
    error="UnsupportedMode")
add(op="resize_error", cite=S + ":615-620", x_shape=[2, 2], mode="nearest", scales=[2.0, 2.0], sizes=[3, 3],
    error="InvalidInput")
add(op="resize_error", cite=S + ":622-627", x_shape=[2, 2], mode="nearest", scales=None, sizes=None,
    error="InvalidInput")
NEG1 = "SIZE_MAX"
add(op="reshape", cite=S + ":904-927", dtype="u8", x_shape=[1, 1, 2, 3], x=[1, 2, 4, 4, 5, 6], new_shape=[1, 1, 3, 2],
    y_shape=[1, 1, 3, 2], y=[1, 2, 4, 4, 5, 6])
add(op="reshape", cite=S + ":1690-1721", dtype="u8", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], new_shape=[3, 2],
    y_shape=[3, 2], y=[1, 2, 3, 4, 5, 6])
add(op="reshape", cite=S + ":1723-1757", dtype="u8", x_shape=[2, 2, 2], x=[1, 2, 3, 4, 5, 6, 7, 8], new_shape=[2, 4],
    y_shape=[2, 4], y=[1, 2, 3, 4, 5, 6, 7, 8])
add(op="reshape_error", cite=S + ":1759-1776", x_shape=[2, 3], new_shape=[2, 4], error="InputArrayWrongSize")
add(op="reshape", cite=S + ":1778-1806", dtype="u8", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], new_shape=[1, 6],
    y_shape=[1, 6], y=[1, 2, 3, 4, 5, 6])
add(op="reshape", cite=S + ":1808-1836", dtype="u8", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], new_shape=[3, NEG1],
    y_shape=[3, 2], y=[1, 2, 3, 4, 5, 6])
add(op="reshape", cite=S + ":1838-1866", dtype="u8", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], new_shape=[0, NEG1],
    y_shape=[2, 3], y=[1, 2, 3, 4, 5, 6])
add(op="reshape_error", cite=S + ":1868-1885", x_shape=[2, 3], new_shape=[NEG1, NEG1], error="InvalidInput")

# ----------------------------------------------------------------------------- transpose / slice / gather
add(op="transpose_onnx", cite=S + ":1172-1206", dtype="f32", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], perm=None,
    y_shape=[3, 2], y=[1, 4, 2, 5, 3, 6])
add(op="transpose_onnx", cite=S + ":1208-1255", dtype="f32", x_shape=[2, 2, 3], x=list(range(1, 13)), perm=[2, 1, 0],
    y_shape=[3, 2, 2], y=[1, 7, 4, 10, 2, 8, 5, 11, 3, 9, 6, 12])
add(op="transpose_onnx_error", cite=S + ":1257-1285", x_shape=[2, 3], perm=[0, 1, 2], error="InvalidPermutation")
add(op="slice_output_shape", cite=S + ":1033-1048", x_shape=[5, 5, 5], starts=[1, 1, 1], ends=[4, 4, 4], axes=None, steps=None, y=[3, 3, 3])
add(op="slice_output_shape", cite=S + ":1050-1059", x_shape=[5, 5, 5], starts=[1, 1, 1], ends=[4, 4, 4], axes=None, steps=[2, 2, 2], y=[2, 2, 2])
add(op="slice_output_shape", cite=S + ":1061-1076", x_shape=[5, 5, 5], starts=[-3, -3, -3], ends=[-1, -1, -1], axes=None, steps=None, y=[2, 2, 2])
add(op="slice_output_shape", cite=S + ":1078-1102", x_shape=[5, 5, 5], starts=[1], ends=[4], axes=[1], steps=None, y=[5, 3, 5])
add(op="slice_output_shape", cite=S + ":1104-1133", x_shape=[5, 5, 5], starts=[4, 4, 4], ends=[1, 1, 1], axes=None, steps=[-1, -1, -1], y=[4, 4, 4],
    note="the shape function counts (start - end) / |step| + 1 for a negative step")
add(op="slice_output_shape_error", cite=S + ":1135-1145", x_shape=[5, 5, 5], starts=[1, 2], ends=[4], axes=None, steps=None, error="InvalidSliceIndices")
add(op="slice_output_shape_error", cite=S + ":1147-1153", x_shape=[5, 5, 5], starts=[1, 2], ends=[4, 5], axes=[1], steps=None, error="InvalidSliceIndices")
add(op="slice_output_shape_error", cite=S + ":1155-1161", x_shape=[5, 5, 5], starts=[1], ends=[4], axes=None, steps=[0], error="InvalidSliceStep")
add(op="slice_output_shape_error", cite=S + ":1163-1169", x_shape=[5, 5, 5], starts=[1], ends=[4], axes=[5], steps=None, error="InvalidSliceIndices")
add(op="gather", cite=S + ":929-975", dtype="u8", x_shape=[3, 3], x=[1, 2, 3, 4, 5, 6, 7, 8, 9], idx_shape=[2], idx=[0, 2], axis=0,
    y_shape=[2, 3], y=[1, 2, 3, 7, 8, 9])
add(op="gather", cite=S + ":977-1025", dtype="u8", x_shape=[2, 4], x=[10, 20, 30, 40, 50, 60, 70, 80], idx_shape=[2, 2], idx=[1, 3, 0, 2], axis=1,
    y_shape=[2, 2, 2], y=[20, 40, 10, 30, 60, 80, 50, 70])
add(op="gather", cite=S + ":1887-1916", dtype="u8", x_shape=[2, 3], x=[1, 2, 3, 4, 5, 6], idx_shape=[1], idx=[1], axis=-2,
    y_shape=[1, 3], y=[4, 5, 6])
add(op="gather", cite=S + ":1941-1988", dtype="u8", x_shape=[3, 3], x=[1, 2, 3, 4, 5, 6, 7, 8, 9], idx_shape=[2, 2], idx=[0, 2, 1, 1], axis=0,
    y_shape=[2, 2, 3], y=[1, 2, 3, 7, 8, 9, 4, 5, 6, 4, 5, 6])
add(op="gather_error", cite=S + ":1918-1939", x_shape=[2, 2], idx_shape=[1], idx=[2], axis=0, error="IndexOutOfBounds")
add(op="gather_error", cite=S + ":1027-1031", x_shape=[3, 3], idx_shape=[2], idx=[0, 2], axis=5, error="InvalidAxis",
    note="the Zig test passes an axis beyond the rank")

# ----------------------------------------------------------------------------- unsqueeze / shape
add(op="unsqueeze_shape", cite=S + ":2016-2048", x_shape=[2, 3], axes=[1], y=[2, 1, 3])
add(op="unsqueeze_shape", cite=S + ":2050-2083", x_shape=[2, 2], axes=[0, 2], y=[1, 2, 1, 2])
add(op="unsqueeze_shape", cite=S + ":2085-2117", x_shape=[2, 3], axes=[-1], y=[2, 3, 1])
add(op="unsqueeze_shape", cite=S + ":2119-2146", x_shape=[1, 1], axes=[0, 2, 3], y=[1, 1, 1, 1, 1],
    note="the Zig test checks the rank (5); every dimension is 1")
add(op="unsqueeze_error", cite=S + ":1644-1666", x_shape=[2, 3], axes=[3], error="AxisOutOfBounds")
add(op="unsqueeze_error", cite=S + ":1668-1688", x_shape=[2, 3], axes=[0, 0], error="DuplicateAxis")
add(op="unsqueeze_error", cite=S + ":2148-2180", x_shape=[2, 2], axes=[5], error="AxisOutOfBounds")
add(op="unsqueeze_error", cite=S + ":2148-2180", x_shape=[2, 2], axes=[-5], error="AxisOutOfBounds")
add(op="shape_onnx", cite=S + ":1324-1350", x_shape=[2, 2, 3], start=None, end=None, y=[2, 2, 3])
add(op="shape_onnx", cite=S + ":1352-1376", x_shape=[2, 2, 3], start=1, end=3, y=[2, 3])
add(op="shape_onnx", cite=S + ":1378-1402", x_shape=[2, 2, 3], start=-2, end=None, y=[2, 3])
add(op="shape_onnx", cite=S + ":1404-1430", x_shape=[4], start=None, end=None, y=[4])
add(op="shape_onnx", cite=S + ":1404-1430", x_shape=[4], start=-5, end=5, y=[4])
add(op="shape_onnx_len", cite=S + ":1521-1606", x_shape=[2, 3, 4, 5], start=1, end=None, n=3)
add(op="shape_onnx_len", cite=S + ":1521-1606", x_shape=[2, 3, 4, 5, 6], start=1, end=3, n=2)
add(op="shape_onnx_len", cite=S + ":1521-1606", x_shape=[2, 3, 4, 5], start=-2, end=-1, n=1)
add(op="shape_onnx_len", cite=S + ":1521-1606", x_shape=[2, 3, 4], start=2, end=1, n=0)
add(op="shape_onnx_len", cite=S + ":1521-1606", x_shape=[], start=None, end=None, n=0)
add(op="shape_onnx_len", cite=S + ":1521-1606", x_shape=[2, 3, 4], start=-5, end=5, n=3)

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_goldens.json")
    with open(out, "w") as f:
        json.dump({"source": "Z-Ant unit tests (literals transcribed by hand)", "cases": cases}, f, indent=1)
    print(f"wrote {len(cases)} cases to {out}")
