//! Drop-in replacement for src/Core/Tensor/TensorMath/tensor_math_standard.zig (Z-Ant) for the
//! operators a generated predict() calls: the same `pub` names and parameter lists, each body
//! unpacks Tensor(T) into (pointer, shape pointer, rank) and calls libzant_b200.so.
//! Point `zant.core.tensor.math_standard` (src/Core/Tensor/tensor.zig:6-7) at this file and link
//! the generated library with -lzant_b200.  Not compiled by this repository (no Zig toolchain).
const std = @import("std");
const zant = @import("../../../zant.zig");
const Tensor = zant.core.tensor.Tensor;
const TensorMathError = zant.utils.error_handler.TensorMathError;
const TensorError = zant.utils.error_handler.TensorError;

pub const Ctx = opaque {};
extern fn zant_b200_ctx_create(device: i32, arena_bytes: usize, out: *?*Ctx) i32;
extern fn zant_b200_conv_f32(ctx: ?*Ctx, x: [*]const f32, xs: [*]const usize, xr: usize, w: [*]const f32, ws: [*]const usize, wr: usize, bias: ?[*]const f32, bias_len: usize, y: [*]f32, ys: [*]const usize, yr: usize, stride: [*]const usize, n_stride: usize, pads: ?[*]const usize, n_pads: usize, dil: ?[*]const usize, n_dil: usize, group: usize, auto_pad: ?[*]const u8, auto_pad_len: usize) i32;
extern fn zant_b200_mat_mul_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, y: [*]f32, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_gemm_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, c: ?[*]const f32, cs: ?[*]const usize, cr: usize, alpha: f32, beta: f32, ta: i32, tb: i32, y: [*]f32, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_maxpool_f32(ctx: ?*Ctx, x: [*]const f32, xs: [*]const usize, xr: usize, y: [*]f32, ys: [*]const usize, yr: usize, k: [*]const usize, nk: usize, s: [*]const usize, ns: usize, d: [*]const usize, nd: usize, p: [*]const usize, np: usize, auto_pad: i32) i32;
extern fn zant_b200_relu_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_leaky_relu_f32(ctx: ?*Ctx, x: [*]const f32, slope: f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_sigmoid_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_softmax_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, rows: usize, cols: usize) i32;
extern fn zant_b200_tanh_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_ceil_f32(ctx: ?*Ctx, x: [*]const f32, y: [*]f32, n: usize) i32;
extern fn zant_b200_mul_f32(ctx: ?*Ctx, a: [*]const f32, na: usize, b: [*]const f32, nb: usize, y: [*]f32) i32;
extern fn zant_b200_div_f32(ctx: ?*Ctx, a: [*]const f32, na: usize, b: [*]const f32, nb: usize, y: [*]f32) i32;
extern fn zant_b200_transpose_onnx(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, perm: ?[*]const usize, np: usize, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_slice_onnx(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, starts: [*]const i64, ends: [*]const i64, n: usize, axes: ?[*]const i64, steps: ?[*]const i64, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_unsqueeze(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, axes: [*]const i64, na: usize, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_shape_onnx(xs: [*]const usize, xr: usize, has_start: i32, start: i64, has_end: i32, end: i64, out: [*]i64, out_len: *usize) i32;
extern fn zant_b200_gather(ctx: ?*Ctx, dtype: i32, x: *const anyopaque, xs: [*]const usize, xr: usize, indices: [*]const usize, is: [*]const usize, ir: usize, axis: i64, y: *anyopaque, ys: [*]const usize, yr: usize) i32;
extern fn zant_b200_sum_tensors_f32(ctx: ?*Ctx, a: [*]const f32, as: [*]const usize, ar: usize, b: [*]const f32, bs: [*]const usize, br: usize, y: [*]f32, ys: [*]const usize, yr: usize) i32;

pub const AutoPadType = enum { NOTSET, SAME_UPPER, SAME_LOWER, VALID };

var ctx: ?*Ctx = null;
fn context() ?*Ctx {
    if (ctx == null) _ = zant_b200_ctx_create(0, 0, &ctx);
    return ctx; // null when no B200 is present: every call then fails with CudaUnavailable
}

/// Status code -> the Zig error the reference function would have returned.
fn check(status: i32) !void {
    return switch (status) {
        0 => {},
        -1 => TensorMathError.InvalidDimensions,
        -4 => TensorMathError.InputTensorDifferentShape,
        -5 => TensorMathError.InputTensorsWrongShape,
        -6 => TensorMathError.OutputTensorDifferentSize,
        -8 => TensorMathError.InputTensorDimensionMismatch,
        -10 => TensorMathError.IncompatibleBroadcastShapes,
        -11 => TensorMathError.EmptyTensorList,
        -13 => TensorMathError.InvalidPadding,
        -14 => TensorMathError.InvalidAxes,
        -35 => TensorError.InputArrayWrongSize,
        -55 => TensorError.InvalidInput,
        else => TensorMathError.MemError, // CUDA / backend failures
    };
}

pub fn conv_lean(comptime T: type, input: *Tensor(T), kernel: *Tensor(T), output: *Tensor(T), bias: ?*const Tensor(T), stride: []const usize, pads: ?[]const usize, dilations: ?[]const usize, group: ?usize, auto_pad: ?[]const u8) !void {
    comptime std.debug.assert(T == f32);
    try check(zant_b200_conv_f32(context(), input.data.ptr, input.shape.ptr, input.shape.len, kernel.data.ptr, kernel.shape.ptr, kernel.shape.len, if (bias) |b| b.data.ptr else null, if (bias) |b| b.size else 0, output.data.ptr, output.shape.ptr, output.shape.len, stride.ptr, stride.len, if (pads) |p| p.ptr else null, if (pads) |p| p.len else 0, if (dilations) |d| d.ptr else null, if (dilations) |d| d.len else 0, group orelse 0, if (auto_pad) |a| a.ptr else null, if (auto_pad) |a| a.len else 0));
}

pub fn mat_mul_lean(comptime T: type, A: *const Tensor(T), B: *const Tensor(T), Y: *Tensor(T)) !void {
    try check(zant_b200_mat_mul_f32(context(), A.data.ptr, A.shape.ptr, A.shape.len, B.data.ptr, B.shape.ptr, B.shape.len, Y.data.ptr, Y.shape.ptr, Y.shape.len));
}

pub fn gemm_lean(comptime T: type, A: *Tensor(T), B: *Tensor(T), C: ?*Tensor(T), alpha: T, beta: T, transA: bool, transB: bool, result: *Tensor(T)) !void {
    try check(zant_b200_gemm_f32(context(), A.data.ptr, A.shape.ptr, A.shape.len, B.data.ptr, B.shape.ptr, B.shape.len, if (C) |c| c.data.ptr else null, if (C) |c| c.shape.ptr else null, if (C) |c| c.shape.len else 0, alpha, beta, @intFromBool(transA), @intFromBool(transB), result.data.ptr, result.shape.ptr, result.shape.len));
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

pub fn tanh_lean(comptime T: type, input: *Tensor(T), output: *Tensor(T)) !void {
    try check(zant_b200_tanh_f32(context(), input.data.ptr, output.data.ptr, input.size));
}

pub fn ceil_lean(comptime T: type, input: *Tensor(T), output: *Tensor(T)) !void {
    try check(zant_b200_ceil_f32(context(), input.data.ptr, output.data.ptr, input.size));
}

pub fn mul_lean(comptime T: type, lhs: *Tensor(T), rhs: *Tensor(T), result: *Tensor(T)) !void {
    try check(zant_b200_mul_f32(context(), lhs.data.ptr, lhs.size, rhs.data.ptr, rhs.size, result.data.ptr));
}

pub fn div_lean(comptime T: type, lhs: *Tensor(T), rhs: *Tensor(T), result: *Tensor(T)) !void {
    try check(zant_b200_div_f32(context(), lhs.data.ptr, lhs.size, rhs.data.ptr, rhs.size, result.data.ptr));
}

pub fn sum_tensors_lean(comptime inT: type, comptime outT: type, t1: *Tensor(inT), t2: *Tensor(inT), out: *Tensor(outT)) !void {
    try check(zant_b200_sum_tensors_f32(context(), t1.data.ptr, t1.shape.ptr, t1.shape.len, t2.data.ptr, t2.shape.ptr, t2.shape.len, out.data.ptr, out.shape.ptr, out.shape.len));
}
// concatenate, resize, reduce_mean_lean, reshape_lean and the quantized names
// (qlinearconv_lean, qlinearmatmul_lean, quantizelinear_lean, dequantizelinear_lean) follow the
// same pattern against zant_b200_concatenate / _resize / _reduce_mean_f32 / _reshape / _qlinear*.
