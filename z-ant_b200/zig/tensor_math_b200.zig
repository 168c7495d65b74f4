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

// ------------------------------------------------------------------------------------------
// FP32 operators
// ------------------------------------------------------------------------------------------
pub fn conv_lean(comptime T: type, input: *Tensor(T), kernel: *Tensor(T), output: *Tensor(T), bias: ?*const Tensor(T), stride: []const usize, pads: ?[]const usize, dilations: ?[]const usize, group: ?usize, auto_pad: ?[]const u8) !void {
    comptime std.debug.assert(T == f32);
    try check(zant_b200_conv_f32(context(), input.data.ptr, input.shape.ptr, input.shape.len, kernel.data.ptr, kernel.shape.ptr, kernel.shape.len, if (bias) |b| b.data.ptr else null, if (bias) |b| b.size else 0, output.data.ptr, output.shape.ptr, output.shape.len, stride.ptr, stride.len, if (pads) |p| p.ptr else null, if (pads) |p| p.len else 0, if (dilations) |d| d.ptr else null, if (dilations) |d| d.len else 0, group orelse 0, if (auto_pad) |a| a.ptr else null, if (auto_pad) |a| a.len else 0));
}

/// OnnxConv (op_convolution.zig:647-745): allocates the output, then conv_lean.
pub fn Conv(comptime T: type, input: *Tensor(T), kernel: *Tensor(T), bias: ?*const Tensor(T), stride: []const usize, pads: ?[]const usize, dilations: ?[]const usize, group: ?usize, auto_pad: ?[]const u8) !Tensor(T) {
    var shape = try get_convolution_output_shape(input.shape, kernel.shape, stride, pads, dilations, auto_pad);
    var output = try Tensor(T).fromShape(&pkg_allocator, &shape);
    errdefer output.deinit();
    try conv_lean(T, input, kernel, &output, bias, stride, pads, dilations, group, auto_pad);
    return output;
}

pub fn mat_mul_lean(comptime T: type, A: *const Tensor(T), B: *const Tensor(T), Y: *Tensor(T)) !void {
    try check(zant_b200_mat_mul_f32(context(), A.data.ptr, A.shape.ptr, A.shape.len, B.data.ptr, B.shape.ptr, B.shape.len, Y.data.ptr, Y.shape.ptr, Y.shape.len));
}
pub const lean_matmul = mat_mul_lean;

/// gemm_lean as generated code calls it: operands of rank 2..4 (hardcoded_sentiment_it.zig:137).
pub fn gemm_lean(comptime T: type, A: *Tensor(T), B: *Tensor(T), C: ?*Tensor(T), alpha: T, beta: T, transA: bool, transB: bool, result: *Tensor(T)) !void {
    try check(zant_b200_gemm_lean_f32(context(), A.data.ptr, A.shape.ptr, A.shape.len, B.data.ptr, B.shape.ptr, B.shape.len, if (C) |c| c.data.ptr else null, if (C) |c| c.shape.ptr else null, if (C) |c| c.shape.len else 0, alpha, beta, @intFromBool(transA), @intFromBool(transB), result.data.ptr, result.shape.ptr, result.shape.len));
}

pub fn onnx_maxpool_lean(comptime T: type, input: *Tensor(T), output: *Tensor(T), kernel_shape: []const usize, strides: []const usize, dilations: []const usize, pads: []const usize, auto_pad: AutoPadType) !void {
    try check(zant_b200_maxpool_f32(context(), input.data.ptr, input.shape.ptr, input.shape.len, output.data.ptr, output.shape.ptr, output.shape.len, kernel_shape.ptr, kernel_shape.len, strides.ptr, strides.len, dilations.ptr, dilations.len, pads.ptr, pads.len, @intFromEnum(auto_pad)));
}

pub fn ReLU_lean(comptime T: type, input: *Tensor(T), output: *Tensor(T)) !void {
    try check(zant_b200_relu_f32(context(), input.data.ptr, output.data.ptr, input.size));
}

pub fn leakyReLU_lean(comptime T: type, input: *Tensor(T), slope: T, output: *Tensor(T)) !void {
    try check(zant_b200_leaky_relu_f32(context(), input.data.ptr, slope, output.data.ptr, input.size));
}

pub fn sigmoid_lean(comptime T: type, input: *Tensor(T), output: *Tensor(T)) !void {
    try check(zant_b200_sigmoid_f32(context(), input.data.ptr, output.data.ptr, input.size));
}

pub fn softmax_lean(comptime T: type, input: *Tensor(T), output: *Tensor(T)) !void {
    try check(zant_b200_softmax_f32(context(), input.data.ptr, output.data.ptr, input.shape[0], input.shape[1]));
}

pub fn tanh_lean(comptime T: type, input: *Tensor(T), result: *Tensor(T)) !void {
    try check(zant_b200_tanh_f32(context(), input.data.ptr, result.data.ptr, input.size));
}

pub fn ceil_lean(comptime T: type, input: *Tensor(T), result: *Tensor(T)) !void {
    try check(zant_b200_ceil_f32(context(), input.data.ptr, result.data.ptr, input.size));
}

pub fn mul_lean(comptime T: type, lhs: *Tensor(T), rhs: *Tensor(T), result: *Tensor(T)) !void {
    try check(zant_b200_mul_f32(context(), lhs.data.ptr, lhs.size, rhs.data.ptr, rhs.size, result.data.ptr));
}

pub fn div_lean(comptime T: type, lhs: *Tensor(T), rhs: *Tensor(T), result: *Tensor(T)) !void {
    try check(zant_b200_div_f32(context(), lhs.data.ptr, lhs.size, rhs.data.ptr, rhs.size, result.data.ptr));
}

pub fn sum_tensors_lean(comptime inputType: type, comptime outputType: type, t1: *Tensor(inputType), t2: *Tensor(inputType), outputTensor: *Tensor(outputType)) !void {
    comptime std.debug.assert(inputType == f32 and outputType == f32);
    try check(zant_b200_sum_tensors_f32(context(), t1.data.ptr, t1.shape.ptr, t1.shape.len, t2.data.ptr, t2.shape.ptr, t2.shape.len, outputTensor.data.ptr, outputTensor.shape.ptr, outputTensor.shape.len));
}

pub fn sum_tensor_list_lean(comptime inputType: type, comptime outputType: type, tensors: []const *Tensor(inputType), outputTensor: *Tensor(outputType)) !void {
    comptime std.debug.assert(inputType == f32 and outputType == f32);
    if (tensors.len == 0) return TensorMathError.EmptyTensorList;
    const ptrs = try pkg_allocator.alloc([*]const f32, tensors.len);
    defer pkg_allocator.free(ptrs);
    for (tensors, 0..) |t, i| {
        if (t.size != outputTensor.size) return TensorMathError.InputTensorDifferentSize;
        ptrs[i] = t.data.ptr;
    }
    try check(zant_b200_sum_tensor_list_f32(context(), ptrs.ptr, tensors.len, outputTensor.data.ptr, outputTensor.size));
}

/// add_bias (lib_elementWise_math.zig:22-45): tensor[.., j] += bias[j], in place.
pub fn add_bias(comptime T: type, tensor: *Tensor(T), bias: *Tensor(T)) !void {
    if (tensor.size == 0 or bias.size == 0) return TensorError.EmptyTensor;
    if (bias.shape.len != 1) return TensorMathError.InputTensorsWrongShape;
    if (bias.shape[0] != tensor.shape[tensor.shape.len - 1]) return TensorMathError.InputTensorDimensionMismatch;
    try check(zant_b200_sum_tensors_f32(context(), tensor.data.ptr, tensor.shape.ptr, tensor.shape.len, bias.data.ptr, bias.shape.ptr, bias.shape.len, tensor.data.ptr, tensor.shape.ptr, tensor.shape.len));
}

pub fn reduce_mean_lean(comptime T: type, input_tensor: *Tensor(T), output_tensor: *Tensor(T), axes: ?[]const i64, keepdims: bool, noop_with_empty_axes: bool) !void {
    try check(zant_b200_reduce_mean_f32(context(), input_tensor.data.ptr, input_tensor.shape.ptr, input_tensor.shape.len, output_tensor.data.ptr, output_tensor.shape.ptr, output_tensor.shape.len, if (axes) |a| a.ptr else null, if (axes) |a| a.len else 0, @intFromBool(keepdims), @intFromBool(noop_with_empty_axes)));
}

// ------------------------------------------------------------------------------------------
// Shape operators (any element type the back end moves: f32, i8, u8, i32)
// ------------------------------------------------------------------------------------------
/// reshape_lean (lib_shape_math.zig:1139-1209): 0 copies the input dimension (unless allowZero),
/// maxInt(usize) stands for -1; the data is copied unchanged into `output`.
pub fn reshape_lean(comptime T: type, input: *Tensor(T), newShape: []const usize, allowZero: ?bool, output: *Tensor(T)) !void {
    if (newShape.len > 8) return TensorError.UnsupportedDimension;
    // with allowZero a literal 0 is a dimension of size zero: the tensor is empty, nothing to copy
    if (allowZero orelse false) for (newShape) |d| if (d == 0) return;
    var resolved: [8]usize = undefined;
    try check(zant_b200_reshape(context(), dtypeOf(T), input.data.ptr, input.shape.ptr, input.shape.len, newShape.ptr, newShape.len, output.data.ptr, &resolved));
}

/// reshape_lean_f32 (lib_shape_math.zig:1102-1137): the new shape arrives as floats (-1 = infer).
pub fn reshape_lean_f32(comptime T: type, input: *Tensor(T), newShape: []f32, allowZero: ?bool, output: *Tensor(T)) !void {
    if (newShape.len > 8) return TensorError.UnsupportedDimension;
    var as_usize: [8]usize = undefined;
    for (newShape, 0..) |d, i| as_usize[i] = if (d < 0) std.math.maxInt(usize) else @intFromFloat(d);
    try reshape_lean(T, input, as_usize[0..newShape.len], allowZero, output);
}

/// concatenate (lib_shape_math.zig:463-580): allocates the result with `allocator`.
pub fn concatenate(comptime T: type, allocator: *const std.mem.Allocator, tensors: []const Tensor(T), axis: isize) !Tensor(T) {
    if (tensors.len == 0) return TensorMathError.EmptyTensorList;
    const n = tensors.len;
    const datas = try allocator.alloc(*const anyopaque, n);
    defer allocator.free(datas);
    const shapes = try allocator.alloc([*]const usize, n);
    defer allocator.free(shapes);
    const ranks = try allocator.alloc(usize, n);
    defer allocator.free(ranks);
    var max_rank: usize = 0;
    for (tensors, 0..) |t, i| {
        datas[i] = t.data.ptr;
        shapes[i] = t.shape.ptr;
        ranks[i] = t.shape.len;
        max_rank = @max(max_rank, t.shape.len);
    }
    const out_shape = try allocator.alloc(usize, max_rank);
    defer allocator.free(out_shape);
    var out_rank: usize = 0;
    try check(zant_b200_concat_output_shape(shapes.ptr, ranks.ptr, n, @intCast(axis), out_shape.ptr, &out_rank));
    var output = try Tensor(T).fromShape(allocator, out_shape[0..out_rank]);
    errdefer output.deinit();
    try check(zant_b200_concatenate(context(), dtypeOf(T), datas.ptr, shapes.ptr, ranks.ptr, n, @intCast(axis), output.data.ptr, output.shape.ptr, output.shape.len));
    return output;
}

/// resize (lib_shape_math.zig:22-76): "nearest" on the device; the result is allocated here.
pub fn resize(comptime T: type, t: *Tensor(T), comptime mode: []const u8, scales: ?[]const f32, sizes: ?[]const usize, coordinate_transformation_mode: []const u8) !Tensor(T) {
    const out_shape = try get_resize_output_shape(t.shape, scales, sizes);
    defer pkg_allocator.free(out_shape);
    var output = try Tensor(T).fromShape(&pkg_allocator, out_shape);
    errdefer output.deinit();
    try check(zant_b200_resize(context(), dtypeOf(T), t.data.ptr, t.shape.ptr, t.shape.len, mode.ptr, mode.len, if (scales) |s| s.ptr else null, if (scales) |s| s.len else 0, if (sizes) |s| s.ptr else null, if (sizes) |s| s.len else 0, coordinate_transformation_mode.ptr, coordinate_transformation_mode.len, output.data.ptr, output.shape.ptr, output.shape.len));
    return output;
}

pub fn transpose_onnx_lean(comptime T: type, input: *Tensor(T), perm: ?[]const usize, output: *Tensor(T)) !void {
    try check(zant_b200_transpose_onnx(context(), dtypeOf(T), input.data.ptr, input.shape.ptr, input.shape.len, if (perm) |p| p.ptr else null, if (perm) |p| p.len else 0, output.data.ptr, output.shape.ptr, output.shape.len));
}

pub fn slice_onnx_lean(comptime T: type, input: *Tensor(T), starts: []const i64, ends: []const i64, axes: ?[]const i64, steps: ?[]const i64, output: *Tensor(T)) !void {
    if (starts.len != ends.len) return TensorError.InvalidSliceIndices;
    try check(zant_b200_slice_onnx(context(), dtypeOf(T), input.data.ptr, input.shape.ptr, input.shape.len, starts.ptr, ends.ptr, starts.len, if (axes) |a| a.ptr else null, if (steps) |s| s.ptr else null, output.data.ptr, output.shape.ptr, output.shape.len));
}
/// The generator emits this spelling (src/codeGen/math_handler.zig:973).
pub const lean_slice_onnx = slice_onnx_lean;

/// gather_lean = lean_gather (lib_shape_math.zig:1279-1330); `indices` stays on the host.
pub fn gather_lean(comptime T: type, data: *Tensor(T), indices: *Tensor(usize), selected_axis: isize, output: *Tensor(T)) !void {
    try check(zant_b200_gather(context(), dtypeOf(T), data.data.ptr, data.shape.ptr, data.shape.len, indices.data.ptr, indices.shape.ptr, indices.shape.len, @intCast(selected_axis), output.data.ptr, output.shape.ptr, output.shape.len));
}

pub fn unsqueeze_lean(comptime T: type, data: *Tensor(T), axes: *Tensor(i64), output: *Tensor(T)) !void {
    try check(zant_b200_unsqueeze(context(), dtypeOf(T), data.data.ptr, data.shape.ptr, data.shape.len, axes.data.ptr, axes.size, output.data.ptr, output.shape.ptr, output.shape.len));
}

/// shape_onnx_lean = lean_shape_onnx (lib_shape_math.zig:1869-1901): host-only, writes the
/// dimensions [start, end) of the input's shape into `output`.
pub fn shape_onnx_lean(comptime InputT: type, comptime OutputT: type, input: *const Tensor(InputT), start: ?i64, end: ?i64, output: *Tensor(OutputT)) !void {
    var dims: [8]i64 = undefined;
    if (input.shape.len > 8) return TensorError.UnsupportedDimension;
    var n: usize = 0;
    try check(zant_b200_shape_onnx(input.shape.ptr, input.shape.len, @intFromBool(start != null), start orelse 0, @intFromBool(end != null), end orelse 0, &dims, &n));
    if (output.size < n) return TensorMathError.OutputTensorDifferentSize;
    for (0..n) |i| {
        output.data[i] = switch (@typeInfo(OutputT)) {
            .Float => @floatFromInt(dims[i]),
            else => @intCast(dims[i]),
        };
    }
}

// ------------------------------------------------------------------------------------------
// Quantized operators.  The reference has none (src/Core/Quantization/quantization.zig is empty);
// the names follow its `<op>_lean` style and the argument order is that of the ONNX operators
// (x, x_scale, x_zero_point, w, w_scale, w_zero_point, y_scale, y_zero_point, B).  Scales and zero
// points are one-element tensors, or one element per output channel for the weights.
// ------------------------------------------------------------------------------------------
pub fn quantizelinear_lean(comptime OutT: type, x: *Tensor(f32), y_scale: *const Tensor(f32), y_zero_point: ?*const Tensor(OutT), y: *Tensor(OutT)) !void {
    const zp: i32 = if (y_zero_point) |z| @intCast(z.data[0]) else 0;
    try check(zant_b200_quantize_linear(context(), x.data.ptr, x.size, y_scale.data[0], zp, dtypeOf(OutT), y.data.ptr));
}

pub fn dequantizelinear_lean(comptime InT: type, x: *Tensor(InT), x_scale: *const Tensor(f32), x_zero_point: ?*const Tensor(InT), y: *Tensor(f32)) !void {
    const zp: i32 = if (x_zero_point) |z| @intCast(z.data[0]) else 0;
    try check(zant_b200_dequantize_linear(context(), dtypeOf(InT), x.data.ptr, x.size, x_scale.data[0], zp, y.data.ptr));
}

pub fn qlinearconv_lean(comptime XT: type, comptime YT: type, x: *Tensor(XT), x_scale: *const Tensor(f32), x_zero_point: *const Tensor(XT), w: *Tensor(i8), w_scale: *const Tensor(f32), w_zero_point: ?*const Tensor(i32), y_scale: *const Tensor(f32), y_zero_point: *const Tensor(YT), bias: ?*const Tensor(i32), output: *Tensor(YT), stride: []const usize, pads: ?[]const usize, dilations: ?[]const usize, group: ?usize, auto_pad: AutoPadType) !void {
    try check(zant_b200_qlinearconv(context(), dtypeOf(XT), x.data.ptr, x.shape.ptr, x.shape.len, x_scale.data[0], @intCast(x_zero_point.data[0]), w.data.ptr, w.shape.ptr, w.shape.len, w_scale.data.ptr, if (w_zero_point) |z| z.data.ptr else null, w_scale.size, y_scale.data[0], @intCast(y_zero_point.data[0]), if (bias) |b| b.data.ptr else null, if (bias) |b| b.size else 0, dtypeOf(YT), output.data.ptr, output.shape.ptr, output.shape.len, stride.ptr, stride.len, if (pads) |p| p.ptr else null, if (pads) |p| p.len else 0, if (dilations) |d| d.ptr else null, if (dilations) |d| d.len else 0, group orelse 1, @intFromEnum(auto_pad), 0));
}

pub fn qlinearmatmul_lean(comptime AT: type, comptime YT: type, a: *Tensor(AT), a_scale: *const Tensor(f32), a_zero_point: *const Tensor(AT), b: *Tensor(i8), b_scale: *const Tensor(f32), b_zero_point: ?*const Tensor(i32), y_scale: *const Tensor(f32), y_zero_point: *const Tensor(YT), output: *Tensor(YT)) !void {
    try check(zant_b200_qlinearmatmul(context(), dtypeOf(AT), a.data.ptr, a.shape.ptr, a.shape.len, a_scale.data[0], @intCast(a_zero_point.data[0]), b.data.ptr, b.shape.ptr, b.shape.len, b_scale.data.ptr, if (b_zero_point) |z| z.data.ptr else null, b_scale.size, y_scale.data[0], @intCast(y_zero_point.data[0]), null, 0, dtypeOf(YT), output.data.ptr, output.shape.ptr, output.shape.len, 0));
}

extern fn zant_b200_lut_q8(ctx: ?*Ctx, x: *const anyopaque, lut: *const [256]u8, y: *anyopaque, n: usize) i32;

pub const QActivation = enum { relu, leaky_relu, clip };

/// Relu / LeakyRelu / Clip between two quantized tensors (QDQ graphs): dequantise, activate, requantise,
///   y = sat(rne(f(float(q - x_zp) * x_scale) / y_scale) + y_zp),
/// evaluated once per code into a 256-entry table on the host and applied on the device.  `alpha` is the LeakyRelu
/// slope or the Clip minimum, `beta` the Clip maximum.  No reference counterpart (the reference has no quantized ops).
pub fn qlinear_activation_lean(comptime T: type, input: *Tensor(T), x_scale: f32, x_zp: i32, kind: QActivation, alpha: f32, beta: f32, y_scale: f32, y_zp: i32, output: *Tensor(T)) !void {
    comptime std.debug.assert(T == i8 or T == u8);
    var lut: [256]u8 = undefined;
    const lo: i32 = if (T == u8) 0 else -128;
    const hi: i32 = if (T == u8) 255 else 127;
    for (0..256) |code| {
        const q: i32 = if (T == u8) @intCast(code) else @as(i32, @as(i8, @bitCast(@as(u8, @intCast(code)))));
        const x: f32 = @as(f32, @floatFromInt(q - x_zp)) * x_scale;
        const a: f32 = switch (kind) {
            .relu => if (x > 0) x else 0,
            .leaky_relu => if (x <= 0) alpha * x else x,
            .clip => @min(@max(x, alpha), beta),
        };
        const v: f32 = @min(@max(a / y_scale, -512.0), 511.0);
        // @round is half-away-from-zero; the back end rounds half to even
        var r: f32 = @floor(v);
        const d = v - r;
        if (d > 0.5 or (d == 0.5 and @mod(r, 2.0) != 0)) r += 1;
        const t: i32 = @min(@max(@as(i32, @intFromFloat(r)) + y_zp, lo), hi);
        lut[code] = @bitCast(@as(i8, @truncate(t)));
    }
    try check(zant_b200_lut_q8(context(), input.data.ptr, &lut, output.data.ptr, input.size));
}
