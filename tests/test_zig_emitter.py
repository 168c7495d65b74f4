"""The Zig emitter: text of lib_<model>.zig and static_parameters.zig for a Graph (not compiled here)."""
import re

import numpy as np
import pytest

import __graft_entry__ as ge


@pytest.fixture(scope="module")
def pkg():
    zb = ge.load_package()
    from zant_b200 import models, zig_emitter
    return zb, models, zig_emitter


def test_emitted_library_registers_every_tensor_and_node(pkg):
    zb, models, ze = pkg
    scales = dict(relu1=0.02, relu2=0.03, relu3=0.05, logits=0.1)
    g = models.small_cnn_int8(4, act_scales=scales)
    lib = ze.emit_lib(g, "small_cnn_int8")
    assert lib.count("zant_b200_plan_tensor(plan,") == len(g.tensors)
    assert lib.count("zant_b200_plan_node(plan,") == len(g.nodes)
    for n in g.nodes:
        assert f"// {n['op']}" in lib
    # the reference's exported signature and its silent return on a wrong shape
    assert re.search(r"pub export fn predict\(\s*input: \[\*\]f32,\s*input_shape: \[\*\]u32,\s*shape_len: u32,\s*result: \*\[\*\]f32,\s*\) void", lib)
    assert "input_shape_expected = [_]u32{ 4, 1, 28, 28 }" in lib
    assert "if (input_shape[i] != dim) return;" in lib
    assert lib.count("{") == lib.count("}") and lib.count("(") == lib.count(")")
    # quantisation parameters travel in the node attributes
    q = next(n for n in g.nodes if n["op"] == "QLinearConv")
    assert ".y_scale = " in lib and ".x_scale = " in lib
    assert q["attrs"]["x_zp"] == 0 or f".x_zp = {q['attrs']['x_zp']}" in lib


def test_static_parameters_hold_the_initializers(pkg):
    zb, models, ze = pkg
    g = models.small_cnn_fp32(1)
    text = ze.emit_static_parameters(g)
    for t in g.tensors:
        if t["data"] is not None:
            assert f"pub const array_{t['name']} align(16) = [_]f32{{" in text
            assert f"pub const shape_{t['name']} = [_]usize{{ {', '.join(str(d) for d in t['shape'])} }};" in text
    # the numbers survive the text form exactly
    b1 = g.tensors[g.id_of("W1")]["data"].reshape(-1)
    block = text.split("pub const array_W1 align(16) = [_]f32{")[1].split("};")[0]
    parsed = np.array([float(v) for v in block.replace("\n", " ").split(",") if v.strip()], np.float32)
    assert np.array_equal(parsed, b1)


def test_reference_style_calls_cover_the_stubbed_operators(pkg):
    """One tensMath call per node, in the reference's own call style, for graphs that hold the operators the reference's
    generator only has stubs for (LeakyRelu, Resize, activation + activation Add via Concat's neighbours) and the quantized
    operators; every emitted name must exist in the Zig module that stands in for tensor_math_standard.zig."""
    zb, models, ze = pkg
    import os
    shim = open(os.path.join(os.path.dirname(ze.__file__), "zig", "tensor_math_b200.zig")).read()
    for g in (models.tiny_yolo_fp32(1, res=64), models.small_cnn_fp32(2), models.small_cnn_int8(2)):
        text = ze.emit_predict_calls(g, g.name)
        assert text.count("// ") >= len(g.nodes)
        for name in set(re.findall(r"tensMath\.(\w+)\(", text)):
            assert re.search(r"pub (?:fn|const) " + name + r"\b", shim), name
        assert sum(1 for line in text.splitlines() if re.search(r"  // \w+$", line)) == len(g.nodes)
        assert all(" catch return;" in line for line in text.splitlines() if "tensMath." in line)
    yolo = ze.emit_predict_calls(models.tiny_yolo_fp32(1, res=64))
    assert "tensMath.leakyReLU_lean(T," in yolo and "tensMath.resize(f32," in yolo and "tensMath.concatenate(f32," in yolo
    q = ze.emit_predict_calls(models.small_cnn_int8(2))
    assert "tensMath.qlinearconv_lean(u8, i8," in q and "tensMath.quantizelinear_lean(u8," in q and "tensMath.dequantizelinear_lean(i8," in q


def test_fusion_groups_follow_the_plan_rules(pkg):
    zb, models, ze = pkg
    assert ze.fusion_groups(models.small_cnn_int8(3)) == [(0, 12, "example CNN chain: 4 fused kernels")]
    f = models.tiny_yolo_fp32(1, res=64)
    scales = {t["name"]: 0.05 for t in f.tensors if t["data"] is None}
    q = models.tiny_yolo_int8(f, scales)
    groups = ze.fusion_groups(q)
    labels = [g[2] for g in groups]
    assert labels.count("QLinearConv+LeakyRelu+MaxPool") == 4          # four backbone stages; the fifth activation is also read by the Concat
    assert "QLinearConv+LeakyRelu" in labels                            # the stride-1 pool stays outside its group
    covered = sum(g[1] for g in groups)
    assert covered >= 2 * len([n for n in q.nodes if n["op"] == "LeakyRelu"])
    assert ze.fusion_groups(f, tf32=True)[0][2] == "Conv+LeakyRelu" and ze.fusion_groups(f) == []
    # a tensor with a second reader is not fused away
    g = models.small_cnn_fp32(1)
    assert ze.fusion_groups(g) == []
