//! Drop-in replacement for src/Core/Tensor/TensorMath/tensor_math_standard.zig (Z-Ant) for the
//! operators a generated predict() calls: the same `pub` names and parameter lists, each body
//! unpacks Tensor(T) into (pointer, shape pointer, rank) and calls libzant_b200.so.
//! Point `zant.core.tensor.math_standard` (src/Core/Tensor/tensor.zig:6-7) at this file and link
//! the generated library with -lzant_b200.  Not compiled by this repository (no Zig toolchain);
//! tests/test_zig_shim.py checks every name and parameter count against the reference's table.
//!
//! Conventions
//!  * every lean function returns `!void`, also mul_lean / div_lean / tanh_lean / ceil_lean, which
//!    return plain `void` in the reference: the generator appends ` catch return;` to every
//!    emitted call (src/codeGen/math_handler.zig:107), which only compiles against an error union;
//!  * allocating functions (concatenate, resize, the get_*_output_shape helpers) allocate their
//!    result with the package allocator exactly as the reference does; the caller frees it;
//!  * the code generator fixes `T = f32` (src/codeGen/skeleton.zig:112-117); data-moving
//!    functions (reshape, concatenate, resize, transpose, slice, gather, unsqueeze) also take
//!    i8 / u8 / i32 tensors.
const std = @import("std");
const zant = @import("../../../zant.zig");
const Tensor = zant.core.tensor.Tensor;
const pkg_allocator = zant.utils.allocator.allocator;
const TensorMathError = zant.utils.error_handler.TensorMathError;
const TensorError = zant.utils.error_handler.TensorError;

/// Failures of the device back end that have no name in the reference's error sets.
pub const B200Error = error{ Cuda, CudaUnavailable, NullPointer, Unsupported, ArenaExhausted, BadHandle, DeviceTimeout, TooLarge, UnknownStatus };

pub const Ctx = opaque {};
pub const AutoPadType = enum(i32) { NOTSET = 0, SAME_UPPER = 1, SAME_LOWER = 2, VALID = 3 };

// zant_dtype of include/zant_b200.h
fn dtypeOf(comptime T: type) i32 {
    return switch (T) {
        f32 => 0,
        i8 => 1,
        u8 => 2,
        i32 => 3,
        else => @compileError("zant_b200: element type not supported by the device back end"),
    };
}

// ------------------------------------------------------------------------------------------
// C ABI (include/zant_b200.h)
// ------------------------------------------------------------------------------------------
extern fn zant_b200_ctx_create(device: i32, arena_bytes: usize, out: *?*Ctx) i32;
extern fn zant_b200_set_log(f: ?*const fn ([*c]u8) callconv(.C) void) void;
extern fn zant_b200_conv_output_shape(xs: [*]const usize, xr: usize, ws: [*]const usize, wr: usize, stride: [*]const usize, n_stride: usize, pads: ?[*]const usize, n_pads: usize, dil: ?[*]const usize, n_dil: usize, auto_pad: ?[*]const u8, auto_pad_len: usize, out: *[4]usize) i32;
extern fn zant_b200_pooling_output_shape(xs: [*]const usize, xr: usize, kernel: *const [2]usize, stride: *const [2]usize, out: *[4]usize) i32;
extern fn zant_b200_maxpool_output_shape(xs: [*]const usize, xr: usize, k: [*]const usize, s: [*]const usize, d: [*]const usize, p: [*]const usize, auto_pad: i32, ceil_mode: i32, out: *[4]usize) i32;
extern fn zant_b200_resize_output_shape(xs: [*]const usize, rank: usize, scales: ?[*]const f32, n_scales: usize, sizes: ?[*]const usize, n_sizes: usize, out: [*]usize) i32;
extern fn zant_b200_concat_output_shape(shapes: [*]const [*]const usize, ranks: [*]const usize, n: usize, axis: i64, out: [*]usize, out_rank: *usize) i32;
extern fn zant_b200_get_concatenate_output_shape(shapes: [*]const [*]const usize, ranks: [*]const usize, n: usize, axis: i64, out: [*]usize) i32;
extern fn zant_b200_slice_output_shape(xs: [*]const usize, xr: usize, starts: [*]const i64, ends: [*]const i64, n: usize, axes: ?[*]const i64, steps: ?[*]const i64, out: [*]usize) i32;
extern fn zant_b200_unsqueeze_output_shape(xs: [*]const usize, xr: usize, axes: [*]const i64, n_axes: usize, out: [*]usize) i32;
extern fn zant_b200_shape_onnx(xs: [*]const usize, xr: usize, has_start: i32, start: i64, has_end: i32, end: i64, out: [*]i64, out_len: *usize) i32;
extern fn zant_b200_conv_f32(ctx: ?*Ctx, x: [*]const f32, xs: [*]const usize, xr: usize, w: [*]const f32, ws: [*]const usize, wr: usize, bias: ?[*]const f32, bias_len: usize, y: [*]f32, ys: [*]const usize, yr: usize, stride: [*]const usize, n_stride: usize, pads: ?[*]const usize, n_pads: usize, dil: ?[*]const usize, n_dil: usize, group: usize, auto_pad: ?[*]const u8, auto_pad_len: usize) i32;
extern fn zant_b200_mat_mul_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, y: [*]f32, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_gemm_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, c: ?[*]const f32, cs: ?[*]const usize, cr: usize, alpha: f32, beta: f32, ta: i32, tb: i32, y: [*]f32, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_gemm_lean_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, c: ?[*]const f32, cs: ?[*]const usize, cr: usize, alpha: f32, beta: f32, ta: i32, tb: i32, y: [*]f32, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_maxpool_f32(ctx: ?*Ctx, x: [*]const f32, xs: [*]const usize, xr: usize, y: [*]f32, ys: [*]const usize, yr: usize, k: [*]const usize, nk: usize, s: [*]const usize, ns: usize, d: [*]const usize, nd: usize, p: [*]const usize, np: usize, auto_pad: i32) i32;
extern fn zant_b200_relu_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_leaky_relu_f32(ctx: ?*Ctx, x: [*]const f32, slope: f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_sigmoid_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_softmax_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, rows: usize, cols: usize) i32;
extern fn zant_b200_tanh_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_ceil_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_mul_f32(ctx: ?*Ctx, a: [*]const f32, na: usize, b: [*]const f32, nb: usize, y: [*]f32) i32;
extern fn zant_b200_div_f32(ctx: ?*Ctx, a: [*]const f32, na: usize, b: [*]const f32, nb: usize, y: [*]f32) i32;
extern fn zant_b200_sum_tensors_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, y: [*]f32, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_sum_tensor_list_f32(ctx: ?*Ctx, tensors: [*]const [*]const f32, n_tensors: usize, y: [*]f32, n: usize) i32;
extern fn zant_b200_concatenate(ctx: ?*Ctx, dtype: i32, tensors: [*]const *const anyopaque, shapes: [*]const [*]const usize, ranks: [*]const usize, n: usize, axis: i64, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_resize(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, rank: usize, mode: [*]const u8, mode_len: usize, scales: ?[*]const f32, n_scales: usize, sizes: ?[*]const usize, n_sizes: usize, coord: [*]const u8, coord_len: usize, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_reduce_mean_f32(ctx: ?*Ctx, x: [*]const f32, xs: [*]const usize, xr: usize, y: [*]f32, ys: [*]const usize, yr: usize, axes: ?[*]const i64, n_axes: usize, keepdims: i32, noop: i32) i32;
extern fn zant_b200_reshape(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, new_shape: [*]const usize, new_rank: usize, y: *anyopaque, ys_out: [*]usize) i32;
extern fn zant_b200_transpose_onnx(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, perm: ?[*]const usize, np: usize, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_slice_onnx(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, starts: [*]const i64, ends: [*]const i64, n: usize, axes: ?[*]const i64, steps: ?[*]const i64, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_unsqueeze(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, axes: [*]const i64, na: usize, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_gather(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, indices: [*]const usize, is: [*]const usize, ir: usize, axis: i64, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_quantize_linear(ctx: ?*Ctx, x: [*]const f32, n: usize, scale: f32, zp: i32, out_dtype: i32, y: *anyopaque) i32;
extern fn zant_b200_dequantize_linear(ctx: ?*Ctx, in_dtype: i32, q: *const anyopaque, n: usize, scale: f32, zp: i32, y: [*]f32) i32;
extern fn zant_b200_qlinearconv(ctx: ?*Ctx, x_dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, x_scale: f32, x_zp: i32, w: [*]const i8, ws: [*]const usize, wr: usize, w_scale: [*]const f32, w_zp: ?[*]const i32, n_w_scale: usize, y_scale: f32, y_zp: i32, bias: ?[*]const i32, bias_len: usize, y_dtype: i32, y: *anyopaque, ys: [*]const usize, yr: usize, stride: [*]const usize, n_stride: usize, pads: ?[*]const usize, n_pads: usize, dil: ?[*]const usize, n_dil: usize, group: usize, auto_pad: i32, activation: i32) i32;
extern fn zant_b200_qlinearmatmul(ctx: ?*Ctx, a_dtype: i32, a: *const anyopaque, as: [*]const usize, ar: usize, a_scale: f32, a_zp: i32, b: [*]const i8, bs: [*]const usize, br: usize, b_scale: [*]const f32, b_zp: ?[*]const i32, n_b_scale: usize, y_scale: f32, y_zp: i32, bias: ?[*]const i32, bias_len: usize, y_dtype: i32, y: *anyopaque, ys: [*]const usize, yr: usize, activation: i32) i32;

// ------------------------------------------------------------------------------------------
// Context, log hook, status -> Zig error
// ------------------------------------------------------------------------------------------
var ctx: ?*Ctx = null;
fn context() ?*Ctx {
    if (ctx == null) _ = zant_b200_ctx_create(0, 0, &ctx);
    return ctx; // null when no B200 is present: every call then fails with CudaUnavailable
}

/// op_convolution.zig:37-41: the C callback that receives one line per logged event.
pub fn setLogFunctionC(func: ?*const fn ([*c]u8) callconv(.C) void) void {
    zant_b200_set_log(func);
}

/// Status code -> the Zig error the reference function would have returned
/// (src/Utils/errorHandler.zig:36-84); every code of zant_status has an arm.
fn check(status: i32) !void {
    return switch (status) {
        0 => {},
        -1 => TensorMathError.InvalidDimensions,
        -2 => TensorMathError.MemError,
        -3 => TensorMathError.InputTensorDifferentSize,
        -4 => TensorMathError.InputTensorDifferentShape,
        -5 => TensorMathError.InputTensorsWrongShape,
        -6 => TensorMathError.OutputTensorDifferentSize,
        -7 => TensorMathError.TooSmallOutputType,
        -8 => TensorMathError.InputTensorDimensionMismatch,
        -9 => TensorMathError.WrongStride,
        -10 => TensorMathError.IncompatibleBroadcastShapes,
        -11 => TensorMathError.EmptyTensorList,
        -12 => TensorMathError.DivisionError,
        -13 => TensorMathError.InvalidPadding,
        -14 => TensorMathError.InvalidAxes,
        -33 => TensorError.TensorNotInitialized,
        -34 => TensorError.InputArrayWrongType,
        -35 => TensorError.InputArrayWrongSize,
        -36 => TensorError.EmptyTensor,
        -37 => TensorError.ZeroSizeTensor,
        -43 => TensorError.InvalidSliceIndices,
        -46 => TensorError.InvalidSliceStep,
        -49 => TensorError.AxisOutOfBounds,
        -50 => TensorError.MismatchedRank,
        -51 => TensorError.MismatchedShape,
        -52 => TensorError.IndexOutOfBounds,
        -53 => TensorError.InvalidAxis,
        -54 => TensorError.DuplicateAxis,
        -55 => TensorError.InvalidInput,
        -56 => TensorError.UnsupportedMode,
        -57 => TensorError.UnsupportedDimension,
        -59 => TensorError.InvalidRank,
        -60 => TensorError.InvalidPermutation,
        -100 => B200Error.Cuda,
        -101 => B200Error.CudaUnavailable,
        -102 => B200Error.NullPointer,
        -103 => B200Error.Unsupported,
        -104 => B200Error.ArenaExhausted,
        -105 => B200Error.BadHandle,
        -106 => B200Error.DeviceTimeout,
        -107 => B200Error.TooLarge,
        else => B200Error.UnknownStatus,
    };
}

// ------------------------------------------------------------------------------------------
// Shape helpers used at code-generation time (host only)
// ------------------------------------------------------------------------------------------
pub fn get_convolution_output_shape(input_shape: []const usize, kernel_shape: []const usize, stride: []const usize, pads: ?[]const usize, dilations: ?[]const usize, auto_pad: ?[]const u8) ![4]usize {
    var out: [4]usize = undefined;
    try check(zant_b200_conv_output_shape(input_shape.ptr, input_shape.len, kernel_shape.ptr, kernel_shape.len, stride.ptr, stride.len, if (pads) |p| p.ptr else null, if (pads) |p| p.len else 0, if (dilations) |d| d.ptr else null, if (dilations) |d| d.len else 0, if (auto_pad) |a| a.ptr else null, if (auto_pad) |a| a.len else 0, &out));
    return out;
}

pub fn get_pooling_output_shape(input_shape: []const usize, kernel: [2]usize, stride: [2]usize) ![4]usize {
    var out: [4]usize = undefined;
    try check(zant_b200_pooling_output_shape(input_shape.ptr, input_shape.len, &kernel, &stride, &out));
    return out;
}

pub fn get_onnx_maxpool_output_shape(input_shape: []const usize, kernel_shape: []const usize, strides: []const usize, dilations: []const usize, pads: []const usize, auto_pad: AutoPadType, ceil_mode: bool) ![]usize {
    var out4: [4]usize = undefined;
    try check(zant_b200_maxpool_output_shape(input_shape.ptr, input_shape.len, kernel_shape.ptr, strides.ptr, dilations.ptr, pads.ptr, @intFromEnum(auto_pad), @intFromBool(ceil_mode), &out4));
    const out = try pkg_allocator.alloc(usize, 4);
    @memcpy(out, &out4);
    return out;
}

pub fn get_resize_output_shape(input_shape: []const usize, scales: ?[]const f32, sizes: ?[]const usize) ![]usize {
    const out = try pkg_allocator.alloc(usize, input_shape.len);
    errdefer pkg_allocator.free(out);
    try check(zant_b200_resize_output_shape(input_shape.ptr, input_shape.len, if (scales) |s| s.ptr else null, if (scales) |s| s.len else 0, if (sizes) |s| s.ptr else null, if (sizes) |s| s.len else 0, out.ptr));
    return out;
}

pub fn get_concatenate_output_shape(tensors: []const []const usize, axis: isize) ![]usize {
    if (tensors.len == 0) return TensorMathError.EmptyTensorList;
    const ptrs = try pkg_allocator.alloc([*]const usize, tensors.len);
    defer pkg_allocator.free(ptrs);
    const ranks = try pkg_allocator.alloc(usize, tensors.len);
    defer pkg_allocator.free(ranks);
    for (tensors, 0..) |s, i| {
        ptrs[i] = s.ptr;
        ranks[i] = s.len;
    }
    const out = try pkg_allocator.alloc(usize, tensors[0].len);
    errdefer pkg_allocator.free(out);
    try check(zant_b200_get_concatenate_output_shape(ptrs.ptr, ranks.ptr, tensors.len, @intCast(axis), out.ptr));
    return out;
}

pub fn get_slice_output_shape(input_shape: []const usize, starts: []const i64, ends: []const i64, axes: ?[]const i64, steps: ?[]const i64) ![]usize {
    if (starts.len != ends.len) return TensorError.InvalidSliceIndices;
    const out = try pkg_allocator.alloc(usize, input_shape.len);
    errdefer pkg_allocator.free(out);
    try check(zant_b200_slice_output_shape(input_shape.ptr, input_shape.len, starts.ptr, ends.ptr, starts.len, if (axes) |a| a.ptr else null, if (steps) |s| s.ptr else null, out.ptr));
    return out;
}

pub fn get_unsqueeze_output_shape(input_shape: []const usize, axes: []const i64) ![]usize {
    const out = try pkg_allocator.alloc(usize, input_shape.len + axes.len);
    errdefer pkg_allocator.free(out);
    try check(zant_b200_unsqueeze_output_shape(input_shape.ptr, input_shape.len, axes.ptr, axes.len, out.ptr));
    return out;
}

pub fn get_shape_output_shape(input_shape: []const usize, start: ?i64, end: ?i64) ![]usize {
    const vals = try pkg_allocator.alloc(i64, @max(input_shape.len, 1));
    defer pkg_allocator.free(vals);
    var n: usize = 0;
    try check(zant_b200_shape_onnx(input_shape.ptr, input_shape.len, @intFromBool(start != null), start orelse 0, @intFromBool(end != null), end orelse 0, vals.ptr, &n));
    const out = try pkg_allocator.alloc(usize, 1);
    out[0] = n;
    return out;
}

pub fn get_transpose_output_shape(input_shape: []const usize, perm: ?[]const usize) ![]usize {
    const rank = input_shape.len;
    if (perm) |p| if (p.len != rank) return TensorError.InvalidPermutation;
    const out = try pkg_allocator.alloc(usize, rank);
    errdefer pkg_allocator.free(out);
    for (0..rank) |i| {
        const src = if (perm) |p| p[i] else rank - 1 - i;
        if (src >= rank) return TensorError.InvalidPermutation;
        out[i] = input_shape[src];
    }
    return out;
}
