"""ONNX ingest: wire-format reader and writer, Graph construction, and the resulting plans."""
import os
import sys

import numpy as np
import pytest

import graph_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

# the reference checkout, where one sits beside this repository (or where ZANT_REFERENCE_MODELS points); the test that
# reads its model files is skipped elsewhere
REFERENCE_MODELS = os.environ.get("ZANT_REFERENCE_MODELS", os.path.join(os.path.dirname(ROOT), "reference", "datasets", "models"))


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


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_MODELS, "mnist-8", "mnist-8.onnx")), reason="reference model files are not on this machine")
def test_reads_the_references_mnist_model(pkg, oracle):
    """The MNIST model the reference ships: decoded, shapes inferred, run by the oracle."""
    zb, models, oi = pkg
    m = oi.read_model(os.path.join(REFERENCE_MODELS, "mnist-8", "mnist-8.onnx"))
    ops = [n["op"] for n in m["nodes"]]
    assert ops.count("Conv") == 2 and ops.count("MaxPool") == 2 and "MatMul" in ops
    g = oi.to_graph(m, batch=2)
    assert g.tensors[g.input]["shape"] == [2, 1, 28, 28] and g.tensors[g.output]["shape"] == [2, 10]
    x = np.random.default_rng(0).random((2, 1, 28, 28), dtype=np.float32)
    y = graph_oracle.run(oracle, g, x)[g.output]
    assert y.shape == (2, 10) and np.isfinite(y).all() and len(np.unique(y)) == 20


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
