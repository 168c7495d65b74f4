"""ONNX ingest: wire-format reader and writer, Graph construction, and the resulting plans."""
import os
import sys

import numpy as np
import pytest

import graph_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

# Two small model files of the reference (datasets/models/mnist-8/mnist-8.onnx, datasets/models/debug_model/debug_model.onnx)
# are kept as fixtures beside the golden vectors, so that these tests run wherever the repository does.
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def pkg():
    zb = ge.load_package()
    from zant_b200 import models, onnx_ingest
    return zb, models, onnx_ingest


def test_round_trip_keeps_the_graph(pkg, oracle):
    """Graph -> ONNX bytes -> Graph: same nodes, shapes and weights, and the same oracle result."""
    zb, models, oi = pkg
    g = models.small_cnn_fp32(3)
    data = oi.write_model(g)
    m = oi.read_model(data)
    assert [n["op"] for n in m["nodes"]] == [n["op"] for n in g.nodes]
    assert set(m["initializers"]) >= {"W1", "B1", "W2", "B2", "W3", "B3", "W4", "B4"}
    assert np.array_equal(m["initializers"]["W2"], g.tensors[g.id_of("W2")]["data"])
    g2 = oi.to_graph(m)
    assert [n["op"] for n in g2.nodes] == [n["op"] for n in g.nodes]
    for n1, n2 in zip(g.nodes, g2.nodes):
        assert g.tensors[n1["outputs"][0]]["shape"] == g2.tensors[n2["outputs"][0]]["shape"]
    x = models.small_cnn_input(3)
    y1 = graph_oracle.run(oracle, g, x)[g.output]
    y2 = graph_oracle.run(oracle, g2, x)[g2.output]
    assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32))


def test_batch_override_and_errors(pkg):
    zb, models, oi = pkg
    m = oi.read_model(oi.write_model(models.small_cnn_fp32(1)))
    g = oi.to_graph(m, batch=5)
    assert g.tensors[g.input]["shape"] == [5, 1, 28, 28] and g.tensors[g.output]["shape"] == [5, 10]
    m["nodes"][1]["op"] = "Erf"
    with pytest.raises(ValueError):
        oi.to_graph(m)
    with pytest.raises(ValueError):
        oi.read_model(b"\x08\x08")            # a ModelProto without a graph


def test_reads_the_references_mnist_model(pkg, oracle):
    """The MNIST model the reference ships: decoded, shapes inferred, run by the oracle."""
    zb, models, oi = pkg
    m = oi.read_model(os.path.join(GOLDEN, "mnist-8.onnx"))
    ops = [n["op"] for n in m["nodes"]]
    assert ops.count("Conv") == 2 and ops.count("MaxPool") == 2 and "MatMul" in ops
    g = oi.to_graph(m, batch=2)
    assert g.tensors[g.input]["shape"] == [2, 1, 28, 28] and g.tensors[g.output]["shape"] == [2, 10]
    x = np.random.default_rng(0).random((2, 1, 28, 28), dtype=np.float32)
    y = graph_oracle.run(oracle, g, x)[g.output]
    assert y.shape == (2, 10) and np.isfinite(y).all() and len(np.unique(y)) == 20


def test_reads_the_references_debug_model(pkg, oracle):
    """The reference's debug model (Gemm, Relu, Gemm, Relu, Softmax on a symbolic batch)."""
    zb, models, oi = pkg
    g = oi.to_graph(oi.read_model(os.path.join(GOLDEN, "debug_model.onnx")), batch=3)
    assert [n["op"] for n in g.nodes] == ["Gemm", "Relu", "Gemm", "Relu", "Softmax"]
    x = np.random.default_rng(1).random(g.tensors[g.input]["shape"], dtype=np.float32)
    y = graph_oracle.run(oracle, g, x)[g.output]
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("name,batch", [("mnist-8.onnx", 1), ("mnist-8.onnx", 6), ("debug_model.onnx", 3)])
def test_reference_models_run_as_plans(pkg, oracle, name, batch):
    """The reference's own model files through ingest -> Plan on the GPU against the oracle running the same graph
    (the call sequence of a generated predict(), src/codeGen/hardcoded/hardcoded_mnist8.zig:140-288)."""
    zb, models, oi = pkg
    g = oi.to_graph(oi.read_model(os.path.join(GOLDEN, name)), batch=batch)
    x = np.random.default_rng(7).random(g.tensors[g.input]["shape"], dtype=np.float32)
    want = graph_oracle.run(oracle, g, x)
    ctx = zb.Context(0)
    try:
        for fuse in (False, True):
            plan = zb.Plan(ctx, g, fuse=fuse)
            got = plan.run(x)
            ref = want[g.output]
            tol = 1e-4 * np.maximum(np.abs(ref), 1e-2 * np.abs(ref).max())       # the FP32 contract
            assert np.all(np.abs(got - ref) <= tol)
            if name.startswith("mnist"):                                          # no transcendental op: bit-identical
                assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
            plan.close()
    finally:
        ctx.close()


@pytest.mark.gpu
def test_ingested_model_runs_as_a_plan(pkg, oracle):
    zb, models, oi = pkg
    ctx = zb.Context(0)
    g = oi.to_graph(oi.read_model(oi.write_model(models.small_cnn_fp32(4))))
    x = models.small_cnn_input(4)
    want = graph_oracle.run(oracle, g, x)[g.output]
    plan = zb.Plan(ctx, g)
    got = plan.run(x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    plan.close()
    ctx.close()
