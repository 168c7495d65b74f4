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
