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


# ------------------------------------------------------------------------------------------------
# Chain recognition (the generator-side view of what zant_b200_plan_finalize fuses)
# ------------------------------------------------------------------------------------------------
def fusion_groups(graph, tf32=False):
    """Groups of consecutive nodes that the plan runs as one step: [(first node, count, label)].

    The rules are those of the plan's fusion pass: QLinearConv -> [Relu | LeakyRelu | Clip on the same scale as the
    convolution's output] -> [MaxPool 2x2, stride 2, no padding], every interior tensor read by exactly one node and not
    the graph output; in TF32 mode also Conv -> Relu | LeakyRelu.  Whether the pool really joins the group is decided at
    finalize time by the kernel that takes the convolution (it needs the implicit-GEMM tiling), so groups that end in
    MaxPool are an upper bound: the plan may leave the pool as a step of its own.  The whole example CNN in QLinear form
    (12 nodes) is recognised by the plan as four fused steps and is reported here as one group."""
    readers = {}
    for n in graph.nodes:
        for t in n["inputs"]:
            if t >= 0:
                readers[t] = readers.get(t, 0) + 1

    def only_feeds_next(t):
        return readers.get(t, 0) == 1 and t != graph.output and graph.tensors[t]["data"] is None

    def pool2x2(a):
        return (tuple(a.get("kernel_shape", ())) == (2, 2) and tuple(a.get("strides", ())) == (2, 2) and not any(a.get("pads", (0,) * 4))
                and tuple(a.get("dilations", (1, 1))) == (1, 1) and a.get("auto_pad") in (None, "NOTSET", "VALID"))

    ops = [n["op"] for n in graph.nodes]
    small_cnn = ["QuantizeLinear", "QLinearConv", "Relu", "MaxPool", "QLinearConv", "Relu", "MaxPool", "Reshape", "QLinearMatMul", "Relu",
                 "QLinearMatMul", "DequantizeLinear"]
    groups, i = [], 0
    while i < len(graph.nodes):
        if ops[i:i + 12] == small_cnn and graph.tensors[graph.nodes[i]["inputs"][0]]["shape"][1:] == [1, 28, 28]:
            groups.append((i, 12, "example CNN chain: 4 fused kernels"))
            i += 12
            continue
        n = graph.nodes[i]
        j, cur, label = i + 1, n["outputs"][0], None
        if n["op"] == "QLinearConv" and graph.tensors[cur]["dtype"] in (I8, U8):
            label = "QLinearConv"
            if j < len(graph.nodes) and only_feeds_next(cur):
                a = graph.nodes[j]
                if (a["op"] in ("Relu", "LeakyRelu", "Clip") and a["inputs"] == [cur] and a["attrs"].get("x_scale") == n["attrs"].get("y_scale")
                        and a["attrs"].get("x_zp", 0) == n["attrs"].get("y_zp", 0)):
                    label += "+" + a["op"]
                    cur = a["outputs"][0]
                    j += 1
            if not n["attrs"].get("channels_last") and j < len(graph.nodes) and only_feeds_next(cur):
                p = graph.nodes[j]
                si, so = graph.tensors[cur]["shape"], graph.tensors[p["outputs"][0]]["shape"]
                if p["op"] == "MaxPool" and p["inputs"] == [cur] and pool2x2(p["attrs"]) and len(si) == 4 and so == [si[0], si[1], si[2] // 2, si[3] // 2]:
                    label += "+MaxPool"
                    j += 1
        elif tf32 and n["op"] == "Conv" and j < len(graph.nodes) and only_feeds_next(cur):
            a = graph.nodes[j]
            if a["op"] in ("Relu", "LeakyRelu") and a["inputs"] == [cur] and graph.tensors[a["outputs"][0]]["dtype"] == F32:
                label = "Conv+" + a["op"]
                j += 1
        if label is not None and j - i > 1:
            groups.append((i, j - i, label))
            i = j
        else:
            i += 1
    return groups


# ------------------------------------------------------------------------------------------------
# Reference-style emission: one tensMath call per node, as src/codeGen/math_handler.zig writes them, including the
# operators whose emitters the reference leaves as stubs (LeakyRelu :65-66, Resize :83-84, Flatten :59-60,
# GlobalAveragePool via ReduceMean, Add of two activations :140-156) and the quantized operators.
# ------------------------------------------------------------------------------------------------
def _usize_slice(vals):
    return "&[_]usize{ " + ", ".join(str(int(v)) for v in vals) + " }"


def _f(v):
    return np.format_float_scientific(np.float32(v), unique=True)


def emit_node_call(graph, node):
    """The Zig statement (without the trailing ` catch return;`) that runs one node through the tensMath module."""
    op, a = node["op"], node["attrs"]
    t = lambda i: "tensor_" + _ident(graph.tensors[i]["name"])     # noqa: E731
    ins = [t(i) if i >= 0 else None for i in node["inputs"]]
    out = t(node["outputs"][0])
    in_t = _ZIG_T[graph.tensors[node["inputs"][0]]["dtype"]]
    out_t = _ZIG_T[graph.tensors[node["outputs"][0]]["dtype"]]
    ap = a.get("auto_pad")
    if op == "Conv":
        bias = f"&{ins[2]}" if len(ins) > 2 and ins[2] else "null"
        pads = _usize_slice(a["pads"]) if a.get("pads") is not None else "null"
        dil = _usize_slice(a["dilations"]) if a.get("dilations") is not None else "null"
        return (f'tensMath.conv_lean(T, &{ins[0]}, @constCast(&{ins[1]}), &{out}, {bias}, {_usize_slice(a.get("strides", (1,)))}, {pads}, {dil}, '
                f'{a.get("group", 1) or 1}, {chr(34) + ap + chr(34) if ap else "null"})')
    if op == "MatMul":
        return f"tensMath.mat_mul_lean(T, &{ins[0]}, @constCast(&{ins[1]}), &{out})"
    if op == "Gemm":
        c = f"@constCast(&{ins[2]})" if len(ins) > 2 and ins[2] else "null"
        return (f"tensMath.gemm_lean(T, &{ins[0]}, @constCast(&{ins[1]}), {c}, {_f(a.get('alpha', 1.0))}, {_f(a.get('beta', 1.0))}, "
                f"{'true' if a.get('trans_a') else 'false'}, {'true' if a.get('trans_b') else 'false'}, &{out})")
    if op == "MaxPool":
        return (f"tensMath.onnx_maxpool_lean({in_t}, &{ins[0]}, &{out}, {_usize_slice(a['kernel_shape'])}, {_usize_slice(a.get('strides', (1, 1)))}, "
                f"{_usize_slice(a.get('dilations', (1, 1)))}, {_usize_slice(a.get('pads', (0, 0, 0, 0)))}, tensMath.AutoPadType.{ap or 'NOTSET'})")
    if op == "Relu" and in_t == "f32":
        return f"tensMath.ReLU_lean(T, &{ins[0]}, &{out})"
    if op == "LeakyRelu" and in_t == "f32":           # a stub in the reference's generator
        return f"tensMath.leakyReLU_lean(T, &{ins[0]}, {_f(a['alpha'])}, &{out})"
    if op in ("Relu", "LeakyRelu", "Clip"):          # between two quantized tensors: requantising activation
        kind = {"Relu": ".relu", "LeakyRelu": ".leaky_relu", "Clip": ".clip"}[op]
        return (f"tensMath.qlinear_activation_lean({in_t}, &{ins[0]}, {_f(a['x_scale'])}, {int(a['x_zp'])}, {kind}, {_f(a.get('alpha', 0.0))}, "
                f"{_f(a.get('beta', 0.0))}, {_f(a['y_scale'])}, {int(a['y_zp'])}, &{out})")
    if op in ("Sigmoid", "Softmax", "Tanh", "Ceil"):
        return f"tensMath.{op.lower()}_lean(T, &{ins[0]}, &{out})"
    if op in ("Mul", "Div"):
        return f"tensMath.{op.lower()}_lean(T, &{ins[0]}, @constCast(&{ins[1]}), &{out})"
    if op == "Add":                                   # also between two activations, which the reference cannot emit
        return f"tensMath.sum_tensors_lean(T, T, &{ins[0]}, @constCast(&{ins[1]}), &{out})"
    if op == "Concat":
        return (f"blk: {{ const list = [_]Tensor({out_t}){{ {', '.join(ins)} }}; const r = tensMath.concatenate({out_t}, &allocator, &list, {int(a['axis'])}) catch return; "
                f"@memcpy({out}.data, r.data); var rr = r; rr.deinit(); break :blk; }}")
    if op == "Resize":                                # a stub in the reference's generator
        scales = "&[_]f32{ " + ", ".join(_f(v) for v in a["scales"]) + " }"
        return (f'blk: {{ var r = tensMath.resize({out_t}, &{ins[0]}, "nearest", {scales}, null, "{a.get("coord_mode", "half_pixel")}") catch return; '
                f"@memcpy({out}.data, r.data); r.deinit(); break :blk; }}")
    if op == "ReduceMean":                            # GlobalAveragePool is ReduceMean over H and W
        axes = "&[_]i64{ " + ", ".join(str(int(v)) for v in a.get("axes", ())) + " }" if a.get("axes") else "null"
        return (f"tensMath.reduce_mean_lean(T, &{ins[0]}, &{out}, {axes}, {'true' if a.get('keepdims', 1) else 'false'}, "
                f"{'true' if a.get('noop_with_empty_axes') else 'false'})")
    if op == "Reshape":                               # Flatten is a Reshape to [N, -1]
        return f"tensMath.reshape_lean({out_t}, &{ins[0]}, {_usize_slice(graph.tensors[node['outputs'][0]]['shape'])}, false, &{out})"
    if op == "Transpose":
        perm = _usize_slice(a["perm"]) if a.get("perm") is not None else "null"
        return f"tensMath.transpose_onnx_lean({out_t}, &{ins[0]}, {perm}, &{out})"
    if op == "QuantizeLinear":
        return f"tensMath.quantizelinear_lean({out_t}, &{ins[0]}, &scalar_f32({_f(a['y_scale'])}), &scalar({out_t}, {int(a['y_zp'])}), &{out})"
    if op == "DequantizeLinear":
        return f"tensMath.dequantizelinear_lean({in_t}, &{ins[0]}, &scalar_f32({_f(a['x_scale'])}), &scalar({in_t}, {int(a['x_zp'])}), &{out})"
    if op == "QLinearConv":
        wz = f"&{ins[3]}" if len(ins) > 3 and ins[3] else "null"
        bias = f"&{ins[4]}" if len(ins) > 4 and ins[4] else "null"
        return (f"tensMath.qlinearconv_lean({in_t}, {out_t}, &{ins[0]}, &scalar_f32({_f(a['x_scale'])}), &scalar({in_t}, {int(a['x_zp'])}), @constCast(&{ins[1]}), "
                f"&{ins[2]}, {wz}, &scalar_f32({_f(a['y_scale'])}), &scalar({out_t}, {int(a['y_zp'])}), {bias}, &{out}, {_usize_slice(a.get('strides', (1, 1)))}, "
                f"{_usize_slice(a.get('pads', (0, 0, 0, 0)))}, {_usize_slice(a.get('dilations', (1, 1)))}, {a.get('group', 1) or 1}, tensMath.AutoPadType.{ap or 'NOTSET'})")
    if op == "QLinearMatMul":
        wz = f"&{ins[3]}" if len(ins) > 3 and ins[3] else "null"
        return (f"tensMath.qlinearmatmul_lean({in_t}, {out_t}, &{ins[0]}, &scalar_f32({_f(a['x_scale'])}), &scalar({in_t}, {int(a['x_zp'])}), @constCast(&{ins[1]}), "
                f"&{ins[2]}, {wz}, &scalar_f32({_f(a['y_scale'])}), &scalar({out_t}, {int(a['y_zp'])}), &{out})")
    raise NotImplementedError(f"no reference-style emitter for {op} on {in_t}: use the plan form (emit_lib)")


def emit_predict_calls(graph, model_name="model"):
    """The body of a reference-style predict(): one statement per node in graph order, each followed by ` catch return;`
    exactly as src/codeGen/math_handler.zig:107 appends it, with the fused groups the plan form would build named in
    comments.  Tensors are the `tensor_<name>` globals of the generated library (src/codeGen/predict.zig:110-142)."""
    groups = {first: (count, label) for first, count, label in fusion_groups(graph)}
    lines = [f"// predict() body of {model_name}: {len(graph.nodes)} nodes, reference-style calls into the tensMath module"]
    i = 0
    while i < len(graph.nodes):
        if i in groups:
            count, label = groups[i]
            lines.append(f"    // nodes {i}..{i + count - 1} form one fused step in the plan form: {label}")
        n = graph.nodes[i]
        call = emit_node_call(graph, n)
        lines.append(f"    {call}{'' if call.startswith('blk:') else ' catch return;'}  // {n['op']}")
        i += 1
    return "\n".join(lines) + "\n"
