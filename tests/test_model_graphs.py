"""The synthetic graphs of the benchmark configurations build on the CPU and the oracle runs them."""
import numpy as np

import graph_oracle


def test_graph_builders_and_oracle(zb, oracle):
    from zant_b200 import models
    g = models.mobilenetv2_int8(1, res=32, classes=10)
    assert sum(1 for n in g.nodes if n["op"] == "QLinearConv") == 1 + 16 * 3 + 2 + 1   # stem, 16 expanded + 1 unexpanded block, head
    assert sum(1 for n in g.nodes if n["op"] == "QLinearAdd") == 10
    y = graph_oracle.run(oracle, g, models.mobilenetv2_input(1, 32))[g.output]
    assert y.shape == (1, 10)
    f = models.tiny_yolo_fp32(1, res=32)
    vals = graph_oracle.run(oracle, f, models.tiny_yolo_input(1, 32))
    assert vals[f.output].shape == (1, 255, 2, 2) and vals[f.meta["head13"]].shape == (1, 255, 1, 1)
    sc = models.act_scales_from({f.tensors[i]["name"]: v for i, v in vals.items() if f.tensors[i]["data"] is None and i != f.input})
    q = models.tiny_yolo_int8(f, sc)
    out = graph_oracle.run(oracle, q, models.tiny_yolo_input(1, 32))[q.output]
    assert np.abs(out - vals[f.output]).max() <= 0.25 * np.abs(vals[f.output]).max()
    assert models.mobilenetv2_int8(1).meta["macs_per_image"] > 2.9e8
