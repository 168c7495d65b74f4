"""Emits the Zig source of a generated model that runs on this back end.

The reference's code generator writes, per model, `lib_<model>.zig` (one TensorMath call per node inside
an exported `predict`, src/codeGen/predict.zig:23-70) and `static_parameters.zig` (the initializers).
This emitter writes the same two files for a zant_b200.Graph, but `predict` hands the whole graph to
the plan API once (`zant_b200_plan_tensor / _node / _finalize`), where chains such as
QuantizeLinear -> QLinearConv -> Relu -> MaxPool are recognised and fused, and then only calls
`zant_b200_plan_run`.  The exported signature and its silent return on a wrong shape are the
reference's (predict.zig:34-40, tests/CodeGen/test_model.template.zig).

The output is text: it is not compiled here (there is no Zig toolchain on the build machine).
"""
import numpy as np

from . import F32, I8, I32, OP, U8, _fill_attrs

_ZIG_T = {F32: "f32", I8: "i8", U8: "u8", I32: "i32"}


def _ident(name):
    out = "".join(ch if ch.isalnum() else "_" for ch in name)
    return out if out and not out[0].isdigit() else "t_" + out


def _array_literal(arr, zig_t, per_line=12):
    flat = np.asarray(arr).reshape(-1)
    if zig_t == "f32":
        items = [np.format_float_scientific(np.float32(v), unique=True) if np.isfinite(v) else "0" for v in flat]
    else:
        items = [str(int(v)) for v in flat]
    lines = [", ".join(items[i:i + per_line]) for i in range(0, len(items), per_line)]
    return "[_]" + zig_t + "{\n    " + ",\n    ".join(lines) + ",\n}"


def emit_static_parameters(graph):
    """static_parameters.zig: one array per initializer and its shape."""
    out = ["// Initializers of the model, as the reference's static_parameters.zig holds them.", ""]
    for t in graph.tensors:
        if t["data"] is None:
            continue
        name, zt = _ident(t["name"]), _ZIG_T[t["dtype"]]
        out.append(f"pub const shape_{name} = [_]usize{{ {', '.join(str(d) for d in t['shape'])} }};")
        out.append(f"pub const array_{name} align(16) = {_array_literal(t['data'], zt)};")
        out.append("")
    return "\n".join(out)


_ATTR_FIELDS = ("kernel_shape", "strides", "n_strides", "dilations", "n_dilations", "pads", "n_pads", "group", "auto_pad", "alpha", "beta",
                "trans_a", "trans_b", "axis", "axes", "n_axes", "keepdims", "noop_with_empty_axes", "scales", "n_scales", "coord_mode",
                "x_scale", "x_zp", "b_scale", "b_zp", "y_scale", "y_zp", "activation", "perm", "n_perm", "slice_starts", "slice_ends",
                "slice_axes", "slice_steps", "n_slice", "slice_has_axes", "slice_has_steps", "channels_last")


def _attrs_literal(attrs):
    """A Zig struct literal for zant_node_attrs holding exactly what the Python binding would pass."""
    a = _fill_attrs(attrs)
    parts = []
    for f in _ATTR_FIELDS:
        v = getattr(a, f)
        if hasattr(v, "__len__"):
            vals = list(v)
            if any(vals):
                parts.append(f".{f} = .{{ {', '.join(repr(float(x)) if isinstance(x, float) else str(int(x)) for x in vals)} }}")
        elif isinstance(v, float):
            if v != 0.0:
                parts.append(f".{f} = {np.format_float_scientific(np.float32(v), unique=True)}")
        elif int(v) != 0:
            parts.append(f".{f} = {int(v)}")
    return ".{ " + ", ".join(parts) + " }" if parts else ".{}"


def emit_lib(graph, model_name="model", fuse=True):
    """lib_<model>.zig: registers the graph with the plan API on first use and exports predict()."""
    tin, tout = graph.tensors[graph.input], graph.tensors[graph.output]
    in_t, out_t = _ZIG_T[tin["dtype"]], _ZIG_T[tout["dtype"]]
    n_out = int(np.prod(tout["shape"]))
    L = []
    w = L.append
    w(f"// lib_{model_name}.zig: {len(graph.nodes)} nodes, {len(graph.tensors)} tensors; computes on libzant_b200.so.")
    w('const std = @import("std");')
    w('const param = @import("static_parameters.zig");')
    w("")
    w("const Ctx = opaque {};")
    w("const Plan = opaque {};")
    w("const NodeAttrs = extern struct {")
    w("    kernel_shape: [2]usize = .{ 0, 0 }, strides: [2]usize = .{ 0, 0 }, n_strides: usize = 0,")
    w("    dilations: [2]usize = .{ 0, 0 }, n_dilations: usize = 0, pads: [4]usize = .{ 0, 0, 0, 0 }, n_pads: usize = 0,")
    w("    group: usize = 0, auto_pad: i32 = -1, alpha: f32 = 0, beta: f32 = 0, trans_a: i32 = 0, trans_b: i32 = 0,")
    w("    axis: i64 = 0, axes: [4]i64 = .{ 0, 0, 0, 0 }, n_axes: usize = 0, keepdims: i32 = 0, noop_with_empty_axes: i32 = 0,")
    w("    scales: [4]f32 = .{ 0, 0, 0, 0 }, n_scales: usize = 0, coord_mode: i32 = 0,")
    w("    x_scale: f32 = 0, x_zp: i32 = 0, b_scale: f32 = 0, b_zp: i32 = 0, y_scale: f32 = 0, y_zp: i32 = 0, activation: i32 = 0,")
    w("    perm: [8]i64 = [_]i64{0} ** 8, n_perm: usize = 0,")
    w("    slice_starts: [8]i64 = [_]i64{0} ** 8, slice_ends: [8]i64 = [_]i64{0} ** 8, slice_axes: [8]i64 = [_]i64{0} ** 8,")
    w("    slice_steps: [8]i64 = [_]i64{0} ** 8, n_slice: usize = 0, slice_has_axes: i32 = 0, slice_has_steps: i32 = 0,")
    w("    channels_last: i32 = 0,")
    w("};")
    w("extern fn zant_b200_ctx_create(device: i32, arena_bytes: usize, out: *?*Ctx) i32;")
    w("extern fn zant_b200_plan_create(ctx: ?*Ctx, out: *?*Plan) i32;")
    w("extern fn zant_b200_plan_tensor(plan: ?*Plan, dtype: i32, shape: [*]const usize, rank: usize, data: ?*const anyopaque, id: *i32) i32;")
    w("extern fn zant_b200_plan_node(plan: ?*Plan, op: i32, inputs: [*]const i32, n_in: usize, outputs: [*]const i32, n_out: usize, attrs: *const NodeAttrs) i32;")
    w("extern fn zant_b200_plan_finalize(plan: ?*Plan, input_id: i32, output_id: i32, fuse: i32) i32;")
    w("extern fn zant_b200_plan_run(plan: ?*Plan, input: *const anyopaque, output: *anyopaque) i32;")
    w("")
    w("var ctx: ?*Ctx = null;")
    w("var plan: ?*Plan = null;")
    w(f"var output_buffer: [{n_out}]{out_t} align(16) = undefined;")
    w(f"const input_shape_expected = [_]u32{{ {', '.join(str(d) for d in tin['shape'])} }};")
    w("")
    w("fn buildPlan() bool {")
    w("    if (zant_b200_ctx_create(0, 0, &ctx) != 0) return false;")
    w("    if (zant_b200_plan_create(ctx, &plan) != 0) return false;")
    w(f"    var id: [{len(graph.tensors)}]i32 = undefined;")
    for i, t in enumerate(graph.tensors):
        shape = ", ".join(str(d) for d in t["shape"])
        data = f"@ptrCast(&param.array_{_ident(t['name'])})" if t["data"] is not None else "null"
        w(f"    if (zant_b200_plan_tensor(plan, {t['dtype']}, &[_]usize{{ {shape} }}, {len(t['shape'])}, {data}, &id[{i}]) != 0) return false; // {t['name']}")
    for n in graph.nodes:
        ins = ", ".join(f"id[{t}]" if t >= 0 else "-1" for t in n["inputs"])
        outs = ", ".join(f"id[{t}]" for t in n["outputs"])
        attrs = "NodeAttrs" + _attrs_literal(n["attrs"])[1:]
        w(f"    if (zant_b200_plan_node(plan, {OP[n['op']]}, &[_]i32{{ {ins} }}, {len(n['inputs'])}, &[_]i32{{ {outs} }}, {len(n['outputs'])}, "
          f"&{attrs}) != 0) return false; // {n['op']}")
    w(f"    return zant_b200_plan_finalize(plan, id[{graph.input}], id[{graph.output}], {1 if fuse else 0}) == 0;")
    w("}")
    w("")
    w("pub export fn predict(")
    w(f"    input: [*]{in_t},")
    w("    input_shape: [*]u32,")
    w("    shape_len: u32,")
    w(f"    result: *[*]{out_t},")
    w(") void {")
    w("    // wrong rank or shape: return without touching the result, as the reference's generated code does")
    w("    if (shape_len != input_shape_expected.len) return;")
    w("    for (input_shape_expected, 0..) |dim, i| {")
    w("        if (input_shape[i] != dim) return;")
    w("    }")
    w("    if (plan == null and !buildPlan()) return;")
    w("    if (zant_b200_plan_run(plan, @ptrCast(input), @ptrCast(&output_buffer)) != 0) return;")
    w("    result.* = &output_buffer;")
    w("}")
    return "\n".join(L) + "\n"
