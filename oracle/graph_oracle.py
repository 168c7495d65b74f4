"""Executes a zant_b200 Graph node by node with the CPU oracle (checker for plan-level parity)."""
import numpy as np

NP = {0: np.float32, 1: np.int8, 2: np.uint8, 3: np.int32}


def run(zo, g, x):
    """Returns {tensor id: numpy array} for every tensor of graph `g` on input `x`."""
    val = {}
    for i, t in enumerate(g.tensors):
        if t["data"] is not None:
            val[i] = t["data"]
    val[g.input] = np.ascontiguousarray(x, NP[g.tensors[g.input]["dtype"]])
    for n in g.nodes:
        op, a = n["op"], n["attrs"]
        ins = [val[i] if i >= 0 else None for i in n["inputs"]]
        out_t = g.tensors[n["outputs"][0]]
        oshape, odt = out_t["shape"], out_t["dtype"]
        if op == "Conv":
            y = zo.conv_lean(ins[0], ins[1], oshape, ins[2] if len(ins) > 2 else None, a.get("strides", (1,)),
                             a.get("pads"), a.get("dilations"), a.get("group"), a.get("auto_pad"))
        elif op == "MatMul":
            y = zo.mat_mul(ins[0], ins[1])
        elif op == "Gemm":
            # gemm_lean multiplies the last two dimensions whatever the rank (op_gemm.zig:128, :150-156); the
            # restated function takes the reference's [b,c,rows,cols] form, so lower ranks get leading ones
            def four_d(t):
                return None if t is None else t.reshape((1,) * (4 - t.ndim) + tuple(t.shape))
            y = zo.gemm(four_d(ins[0]), four_d(ins[1]), four_d(ins[2]) if len(ins) > 2 else None, a.get("alpha", 1.0), a.get("beta", 1.0),
                        bool(a.get("trans_a", 0)), bool(a.get("trans_b", 0)))
        elif op == "MaxPool":
            y = zo.onnx_maxpool_lean(ins[0], oshape, a["kernel_shape"], a.get("strides", (1, 1)), a.get("dilations", (1, 1)),
                                     a.get("pads", (0, 0, 0, 0)), a.get("auto_pad") or "NOTSET")
        elif op in ("Relu", "LeakyRelu", "Clip"):
            if ins[0].dtype == np.float32:
                y = zo.ReLU(ins[0]) if op == "Relu" else zo.leakyReLU(ins[0], a["alpha"]) if op == "LeakyRelu" else zo.clip(ins[0], a["alpha"], a["beta"])
            else:
                dt = {np.dtype(np.int8): 1, np.dtype(np.uint8): 2}[ins[0].dtype]
                f = zo.dequantize_linear(ins[0], a["x_scale"], a["x_zp"])
                f = zo.ReLU(f) if op == "Relu" else zo.leakyReLU(f, a["alpha"]) if op == "LeakyRelu" else zo.clip(f, a["alpha"], a["beta"])
                y = zo.quantize_linear(f, a["y_scale"], a["y_zp"], dt)
        elif op == "Add":
            y = zo.sum_tensors(ins[0], ins[1])
        elif op in ("Sigmoid", "Tanh", "Ceil"):
            y = {"Sigmoid": zo.sigmoid, "Tanh": zo.tanh, "Ceil": zo.ceil}[op](ins[0])
        elif op == "Softmax":
            y = zo.softmax(ins[0])
        elif op == "Transpose":
            y = zo.transpose_onnx(ins[0], a.get("perm"))
        elif op == "Slice":
            y = zo.slice_onnx(ins[0], a["starts"], a["ends"], a.get("slice_axes"), a.get("steps"))
        elif op == "Gather":
            y = zo.gather(ins[0], ins[1], a["axis"])
        elif op in ("Mul", "Div"):
            y = (zo.mul if op == "Mul" else zo.div)(ins[0], ins[1]).reshape(oshape)
        elif op == "Concat":
            y = zo.concatenate(ins, a["axis"])
        elif op == "Resize":
            y = zo.resize(ins[0], "nearest", list(a["scales"]), None, a.get("coord_mode", "half_pixel"))
        elif op == "ReduceMean":
            y = zo.reduce_mean(ins[0], a.get("axes"), bool(a.get("keepdims", 1)), bool(a.get("noop_with_empty_axes", 0)))
        elif op == "Reshape":
            y = ins[0].reshape(oshape)
        elif op == "QuantizeLinear":
            y = zo.quantize_linear(ins[0], a["y_scale"], a["y_zp"], odt)
        elif op == "DequantizeLinear":
            y = zo.dequantize_linear(ins[0], a["x_scale"], a["x_zp"])
        elif op == "QLinearConv":
            y = zo.qlinearconv(ins[0], a["x_scale"], a["x_zp"], ins[1], ins[2], ins[3] if len(ins) > 3 else None,
                               a["y_scale"], a["y_zp"], ins[4] if len(ins) > 4 else None, odt, a.get("strides", (1, 1)),
                               a.get("pads", (0, 0, 0, 0)), a.get("dilations", (1, 1)), a.get("group", 1) or 1,
                               a.get("auto_pad") or "NOTSET", a.get("activation"))
        elif op == "QLinearMatMul":
            y = zo.qlinearmatmul(ins[0], a["x_scale"], a["x_zp"], ins[1], ins[2], ins[3] if len(ins) > 3 else None,
                                 a["y_scale"], a["y_zp"], ins[4] if len(ins) > 4 else None, odt, a.get("activation"))
        elif op == "QLinearAdd":
            y = zo.qlinearadd(ins[0], a["x_scale"], a["x_zp"], ins[1], a["b_scale"], a["b_zp"], a["y_scale"], a["y_zp"], a.get("activation"))
        elif op == "QLinearGlobalAveragePool":
            y = zo.qlinear_global_avgpool(ins[0], a["x_scale"], a["x_zp"], a["y_scale"], a["y_zp"])
        elif op == "LutQ8":
            y = zo.lut_q8(ins[0], ins[1])
        else:
            raise NotImplementedError(op)
        y = np.asarray(y).reshape(oshape)
        assert y.dtype == NP[odt], (op, y.dtype, odt)
        val[n["outputs"][0]] = y
    return val


def calibrate(zo, fp32_graph, calib_x):
    """Activation scales from the oracle (CPU counterpart of models.calibrate_on_gpu)."""
    import zant_b200.models as models
    vals = run(zo, fp32_graph, calib_x)
    return models.act_scales_from({n: vals[fp32_graph.id_of(n)] for n in fp32_graph.meta["calib_tensors"]})
