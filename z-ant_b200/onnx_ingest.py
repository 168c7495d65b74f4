"""ONNX model files -> zant_b200.Graph, without the onnx / protobuf packages.

The reference reads .onnx files with its own protobuf wire reader (src/onnx/protobuf.zig:31-210) into
message structs (src/onnx/onnx.zig: ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto,
ValueInfoProto) and hands them to its code generator.  This module does the same in Python for the
operators the back end implements: `read_model` decodes the wire format into plain dictionaries,
`to_graph` turns them into a Graph with every tensor shape inferred (the plan needs them all up
front, like the generator's static memory plan), folding nodes whose inputs are all initializers.
`write_model` serialises a float Graph back to ONNX bytes; the tests use it to make model files.
"""
import struct

import numpy as np

from . import F32, I8, I32, U8, Graph, conv_output_shape, get_onnx_maxpool_output_shape, concat_output_shape, \
    get_resize_output_shape, reduce_mean_shape

# TensorProto.DataType values used here
_ONNX_F32, _ONNX_U8, _ONNX_I8, _ONNX_I32, _ONNX_I64 = 1, 2, 3, 6, 7
_NP_OF = {_ONNX_F32: np.float32, _ONNX_U8: np.uint8, _ONNX_I8: np.int8, _ONNX_I32: np.int32, _ONNX_I64: np.int64}
_DT_OF = {_ONNX_F32: F32, _ONNX_U8: U8, _ONNX_I8: I8, _ONNX_I32: I32}


# ------------------------------------------------------------------------------------------------
# protobuf wire format
# ------------------------------------------------------------------------------------------------
def _varint(buf, pos):
    result, shift = 0, 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def _fields(buf):
    """Yields (field number, wire type, value) of one message; length-delimited values are bytes."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            val, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            n, pos = _varint(buf, pos)
            val, pos = buf[pos:pos + n], pos + n
        elif wt == 5:
            val, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        yield num, wt, val


def _str(v):
    return bytes(v).decode()


def _signed(v):
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(val, wt):
    if wt == 0:
        return [_signed(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_signed(v))
    return out


def _tensor(buf):
    dims, dtype, name, raw = [], _ONNX_F32, "", None
    floats, i32s, i64s = [], [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += _packed_varints(val, wt)
        elif num == 2:
            dtype = val
        elif num == 4:
            floats += list(struct.unpack(f"<{len(val) // 4}f", val)) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num == 5:
            i32s += _packed_varints(val, wt)
        elif num == 7:
            i64s += _packed_varints(val, wt)
        elif num == 8:
            name = _str(val)
        elif num == 9:
            raw = bytes(val)
    np_dt = _NP_OF.get(dtype)
    if np_dt is None:
        raise ValueError(f"initializer {name}: unsupported ONNX data type {dtype}")
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(np_dt).newbyteorder("<")).astype(np_dt)
    elif dtype == _ONNX_F32:
        arr = np.asarray(floats, np.float32)
    elif dtype == _ONNX_I64:
        arr = np.asarray(i64s, np.int64)
    else:
        arr = np.asarray(i32s, np.int64).astype(np_dt)      # uint8 / int8 / int32 travel in int32_data
    return name, arr.reshape([int(d) for d in dims])


def _attribute(buf):
    name, out = "", {}
    for num, wt, val in _fields(buf):
        if num == 1:
            name = _str(val)
        elif num == 2:
            out["f"] = struct.unpack("<f", val)[0]
        elif num == 3:
            out["i"] = _signed(val)
        elif num == 4:
            out["s"] = bytes(val)
        elif num == 5:
            out["t"] = _tensor(val)[1]
        elif num == 7:
            out.setdefault("floats", [])
            out["floats"] += list(struct.unpack(f"<{len(val) // 4}f", val)) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num == 8:
            out.setdefault("ints", [])
            out["ints"] += _packed_varints(val, wt)
    for key in ("ints", "floats", "t", "s", "i", "f"):
        if key in out:
            return name, (_str(out[key]) if key == "s" else out[key])
    return name, None


def _value_info(buf):
    name, elem, shape = "", _ONNX_F32, None
    for num, _wt, val in _fields(buf):
        if num == 1:
            name = _str(val)
        elif num == 2:                                         # TypeProto
            for n2, _w2, v2 in _fields(val):
                if n2 == 1:                                    # tensor_type
                    for n3, _w3, v3 in _fields(v2):
                        if n3 == 1:
                            elem = v3
                        elif n3 == 2:                          # TensorShapeProto
                            shape = []
                            for n4, _w4, v4 in _fields(v3):
                                if n4 == 1:
                                    dim = None
                                    for n5, w5, v5 in _fields(v4):
                                        if n5 == 1 and w5 == 0:
                                            dim = _signed(v5)
                                    shape.append(dim)          # None: symbolic (dim_param)
    return name, elem, shape


def read_model(data):
    """`data`: bytes or a path.  Returns dict(nodes, initializers, inputs, outputs, value_info)."""
    if not isinstance(data, (bytes, bytearray, memoryview)):
        with open(data, "rb") as f:
            data = f.read()
    graph = None
    for num, _wt, val in _fields(memoryview(data)):
        if num == 7:
            graph = val
    if graph is None:
        raise ValueError("no GraphProto in the model")
    model = dict(nodes=[], initializers={}, inputs=[], outputs=[], value_info={})
    for num, _wt, val in _fields(graph):
        if num == 1:
            node = dict(inputs=[], outputs=[], op="", name="", attrs={})
            for n2, _w2, v2 in _fields(val):
                if n2 == 1:
                    node["inputs"].append(_str(v2))
                elif n2 == 2:
                    node["outputs"].append(_str(v2))
                elif n2 == 3:
                    node["name"] = _str(v2)
                elif n2 == 4:
                    node["op"] = _str(v2)
                elif n2 == 5:
                    k, v = _attribute(v2)
                    node["attrs"][k] = v
            model["nodes"].append(node)
        elif num == 5:
            name, arr = _tensor(val)
            model["initializers"][name] = arr
        elif num in (11, 12, 13):
            name, elem, shape = _value_info(val)
            if num == 11:
                model["inputs"].append(name)
            elif num == 12:
                model["outputs"].append(name)
            model["value_info"][name] = (elem, shape)
    return model


# ------------------------------------------------------------------------------------------------
# model -> Graph
# ------------------------------------------------------------------------------------------------
def _pads4(a, rank=2):
    p = a.get("pads")
    return [0, 0, 0, 0] if p is None else [int(v) for v in p]


def to_graph(model, batch=None, name="onnx"):
    """Builds a Graph from `read_model` output.  The graph input is the one model input that is not an
    initializer; a symbolic or differing leading dimension is replaced by `batch` when given."""
    init = dict(model["initializers"])
    g = Graph(name)
    ids, shapes, dtypes = {}, {}, {}

    def const_id(nm):
        if nm not in ids:
            arr = init[nm]
            if arr.dtype == np.int64:
                arr = arr.astype(np.int32)
            dt = {np.dtype(np.float32): F32, np.dtype(np.int8): I8, np.dtype(np.uint8): U8, np.dtype(np.int32): I32}[arr.dtype]
            ids[nm] = g.tensor(nm, dt, arr.shape, arr)
            shapes[nm], dtypes[nm] = list(arr.shape), dt
        return ids[nm]

    def act(nm, dt, shape):
        ids[nm] = g.tensor(nm, dt, shape)
        shapes[nm], dtypes[nm] = [int(s) for s in shape], dt
        return ids[nm]

    def ref(nm):
        return const_id(nm) if nm in init else ids[nm]

    def shape_of(nm):
        return list(init[nm].shape) if nm in init and nm not in shapes else shapes[nm]

    graph_inputs = [n for n in model["inputs"] if n not in init]
    if len(graph_inputs) != 1:
        raise ValueError(f"expected one graph input, found {graph_inputs}")
    elem, shp = model["value_info"][graph_inputs[0]]
    shp = [batch if (i == 0 and batch is not None) else d for i, d in enumerate(shp)]
    if any(d is None for d in shp):
        raise ValueError("the input shape has symbolic dimensions: pass batch=")
    g.input = act(graph_inputs[0], _DT_OF[elem], shp)

    def scalar(nm):
        return init[nm].reshape(-1)[0]

    for nd in model["nodes"]:
        op, a, ins, outs = nd["op"], nd["attrs"], [i for i in nd["inputs"]], nd["outputs"]
        present = [i for i in ins if i]
        # constant folding of shape plumbing on initializers
        if present and all(i in init for i in present) and op in ("Reshape", "Flatten", "Transpose", "Unsqueeze", "Identity"):
            x = init[ins[0]]
            if op == "Reshape":
                tgt = [int(v) for v in init[ins[1]].reshape(-1)]
                tgt = [x.shape[i] if v == 0 else v for i, v in enumerate(tgt)]
                init[outs[0]] = x.reshape(tgt)
            elif op == "Flatten":
                ax = int(a.get("axis", 1))
                init[outs[0]] = x.reshape(int(np.prod(x.shape[:ax])), -1)
            elif op == "Transpose":
                init[outs[0]] = np.ascontiguousarray(np.transpose(x, a.get("perm")))
            elif op == "Unsqueeze":
                axes = a.get("axes") if "axes" in a else [int(v) for v in init[ins[1]].reshape(-1)]
                init[outs[0]] = np.expand_dims(x, tuple(int(v) for v in axes))
            else:
                init[outs[0]] = x
            continue
        xs = shape_of(ins[0])
        xdt = dtypes[ins[0]] if ins[0] in dtypes else _DT_OF.get({np.dtype(np.float32): 1, np.dtype(np.uint8): 2, np.dtype(np.int8): 3, np.dtype(np.int32): 6}[init[ins[0]].dtype])
        if op == "Conv":
            ws = shape_of(ins[1])
            strides = [int(v) for v in a.get("strides", [1, 1])]
            dil = [int(v) for v in a.get("dilations", [1, 1])]
            auto_pad = a.get("auto_pad", "NOTSET")
            pads = _pads4(a)
            os_ = conv_output_shape(xs, ws, strides, pads, dil, auto_pad)
            y = act(outs[0], F32, os_)
            g.node("Conv", [ref(ins[0]), ref(ins[1]), ref(ins[2]) if len(ins) > 2 and ins[2] else -1], [y], strides=strides, pads=pads,
                   dilations=dil, group=int(a.get("group", 1)), auto_pad=auto_pad)
        elif op == "MaxPool":
            k = [int(v) for v in a["kernel_shape"]]
            strides = [int(v) for v in a.get("strides", [1, 1])]
            dil = [int(v) for v in a.get("dilations", [1, 1])]
            auto_pad = a.get("auto_pad", "NOTSET")
            pads = _pads4(a)
            os_ = get_onnx_maxpool_output_shape(xs, k, strides, dil, pads, auto_pad, bool(a.get("ceil_mode", 0)))
            y = act(outs[0], xdt, os_)
            g.node("MaxPool", [ref(ins[0])], [y], kernel_shape=k, strides=strides, dilations=dil, pads=pads, auto_pad=auto_pad)
        elif op in ("Relu", "Sigmoid", "Tanh", "Ceil", "LeakyRelu", "Clip"):
            y = act(outs[0], xdt, xs)
            if op == "LeakyRelu":
                g.node(op, [ref(ins[0])], [y], alpha=float(a.get("alpha", 0.01)))
            elif op == "Clip":
                lo = float(scalar(ins[1])) if len(ins) > 1 and ins[1] else float(a.get("min", -3.4e38))
                hi = float(scalar(ins[2])) if len(ins) > 2 and ins[2] else float(a.get("max", 3.4e38))
                g.node(op, [ref(ins[0])], [y], alpha=lo, beta=hi)
            else:
                g.node(op, [ref(ins[0])], [y])
        elif op == "Softmax":
            if len(xs) != 2:
                raise ValueError("Softmax: only 2-D inputs (rows are normalised)")
            g.node(op, [ref(ins[0])], [act(outs[0], F32, xs)])
        elif op in ("Add", "Mul", "Div"):
            bs = shape_of(ins[1])
            os_ = list(np.broadcast_shapes(tuple(xs), tuple(bs))) if op == "Add" else xs
            g.node(op, [ref(ins[0]), ref(ins[1])], [act(outs[0], F32, os_)])
        elif op == "MatMul":
            bs = shape_of(ins[1])
            g.node(op, [ref(ins[0]), ref(ins[1])], [act(outs[0], F32, xs[:-1] + [bs[-1]])])
        elif op == "Gemm":
            bs = shape_of(ins[1])
            ta, tb = int(a.get("transA", 0)), int(a.get("transB", 0))
            m = xs[1] if ta else xs[0]
            n = bs[0] if tb else bs[1]
            g.node(op, [ref(ins[0]), ref(ins[1]), ref(ins[2]) if len(ins) > 2 and ins[2] else -1], [act(outs[0], F32, [m, n])],
                   alpha=float(a.get("alpha", 1.0)), beta=float(a.get("beta", 1.0)), trans_a=ta, trans_b=tb)
        elif op in ("Reshape", "Flatten"):
            if op == "Reshape":
                tgt = [int(v) for v in init[ins[1]].reshape(-1)]
                tgt = [xs[i] if v == 0 else v for i, v in enumerate(tgt)]
                if -1 in tgt:
                    tgt[tgt.index(-1)] = int(np.prod(xs)) // int(-np.prod(tgt))
                elif int(np.prod(tgt)) != int(np.prod(xs)) and len(tgt) > 1 and int(np.prod(xs)) % int(np.prod(tgt[1:])) == 0:
                    tgt[0] = int(np.prod(xs)) // int(np.prod(tgt[1:]))     # a literal batch dimension under a batch override
            else:
                ax = int(a.get("axis", 1))
                tgt = [int(np.prod(xs[:ax])), int(np.prod(xs[ax:]))]
            g.node("Reshape", [ref(ins[0])], [act(outs[0], xdt, tgt)])
        elif op == "Concat":
            os_ = concat_output_shape([shape_of(i) for i in ins], int(a["axis"]))
            g.node(op, [ref(i) for i in ins], [act(outs[0], xdt, os_)], axis=int(a["axis"]))
        elif op == "Transpose":
            perm = [int(v) for v in a["perm"]] if "perm" in a else list(range(len(xs) - 1, -1, -1))
            g.node(op, [ref(ins[0])], [act(outs[0], xdt, [xs[p] for p in perm])], perm=perm)
        elif op == "Resize":
            scales = [float(v) for v in init[ins[2]].reshape(-1)]
            os_ = get_resize_output_shape(xs, scales, None)
            g.node(op, [ref(ins[0])], [act(outs[0], xdt, os_)], scales=scales,
                   coord_mode=a.get("coordinate_transformation_mode", "half_pixel"))
        elif op == "ReduceMean":
            axes = [int(v) for v in a["axes"]] if "axes" in a else None
            keep = int(a.get("keepdims", 1))
            os_ = reduce_mean_shape(xs, axes, bool(keep), False)
            g.node(op, [ref(ins[0])], [act(outs[0], F32, os_)], axes=axes or [], keepdims=keep)
        elif op == "QuantizeLinear":
            zp = init[ins[2]] if len(ins) > 2 and ins[2] else np.zeros(1, np.uint8)
            g.node(op, [ref(ins[0])], [act(outs[0], U8 if zp.dtype == np.uint8 else I8, xs)], y_scale=float(scalar(ins[1])), y_zp=int(zp.reshape(-1)[0]))
        elif op == "DequantizeLinear":
            zp = int(scalar(ins[2])) if len(ins) > 2 and ins[2] else 0
            g.node(op, [ref(ins[0])], [act(outs[0], F32, xs)], x_scale=float(scalar(ins[1])), x_zp=zp)
        else:
            raise ValueError(f"ONNX operator {op} is not supported by this back end")
    g.output = ids[model["outputs"][0]]
    return g


# ------------------------------------------------------------------------------------------------
# Graph -> ONNX bytes (float graphs; enough to make model files for tests)
# ------------------------------------------------------------------------------------------------
def _enc_varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _enc(num, wt, payload):
    key = _enc_varint((num << 3) | wt)
    if wt == 0:
        return key + _enc_varint(payload)
    if wt == 5:
        return key + payload
    return key + _enc_varint(len(payload)) + payload


def _enc_tensor(name, arr):
    arr = np.ascontiguousarray(arr)
    code = {np.dtype(np.float32): _ONNX_F32, np.dtype(np.int64): _ONNX_I64, np.dtype(np.int32): _ONNX_I32,
            np.dtype(np.int8): _ONNX_I8, np.dtype(np.uint8): _ONNX_U8}[arr.dtype]
    out = b"".join(_enc(1, 0, int(d)) for d in arr.shape)
    out += _enc(2, 0, code) + _enc(8, 2, name.encode()) + _enc(9, 2, arr.astype(arr.dtype.newbyteorder("<")).tobytes())
    return out


def _enc_attr(name, v):
    out = _enc(1, 2, name.encode())
    if isinstance(v, float):
        return out + _enc(2, 5, struct.pack("<f", v)) + _enc(20, 0, 1)
    if isinstance(v, int):
        return out + _enc(3, 0, v) + _enc(20, 0, 2)
    if isinstance(v, str):
        return out + _enc(4, 2, v.encode()) + _enc(20, 0, 3)
    return out + b"".join(_enc(8, 0, int(i)) for i in v) + _enc(20, 0, 7)


def _enc_value_info(name, dtype, shape):
    dims = b"".join(_enc(1, 2, _enc(1, 0, int(d))) for d in shape)
    ttype = _enc(1, 0, {F32: _ONNX_F32, U8: _ONNX_U8, I8: _ONNX_I8, I32: _ONNX_I32}[dtype]) + _enc(2, 2, dims)
    return _enc(1, 2, name.encode()) + _enc(2, 2, _enc(1, 2, ttype))


_ATTR_NAMES = dict(strides="strides", pads="pads", dilations="dilations", group="group", auto_pad="auto_pad", kernel_shape="kernel_shape",
                   alpha="alpha", beta="beta", trans_a="transA", trans_b="transB", axis="axis", perm="perm", keepdims="keepdims")


def write_model(graph):
    """Serialises a float Graph (Conv, Relu, LeakyRelu, MaxPool, Add, MatMul, Gemm, Reshape, Concat, Transpose,
    Sigmoid, Tanh, Softmax, Mul, Div) to ONNX bytes.  Reshape targets become int64 initializers."""
    body = b""
    names = [t["name"] for t in graph.tensors]
    extra_init = []
    for i, n in enumerate(graph.nodes):
        ins = [names[t] if t >= 0 else "" for t in n["inputs"]]
        attrs = dict(n["attrs"])
        if n["op"] == "Reshape":
            tgt = f"__shape_{i}"
            extra_init.append((tgt, np.asarray(graph.tensors[n["outputs"][0]]["shape"], np.int64)))
            ins.append(tgt)
        node = b"".join(_enc(1, 2, s.encode()) for s in ins) + b"".join(_enc(2, 2, names[t].encode()) for t in n["outputs"])
        node += _enc(3, 2, f"node{i}".encode()) + _enc(4, 2, n["op"].encode())
        for k, v in attrs.items():
            if v is None or k not in _ATTR_NAMES:
                continue
            node += _enc(5, 2, _enc_attr(_ATTR_NAMES[k], v if not isinstance(v, (tuple, list)) else list(v)))
        body += _enc(1, 2, node)
    body += _enc(2, 2, (graph.name or "graph").encode())
    for t in graph.tensors:
        if t["data"] is not None:
            body += _enc(5, 2, _enc_tensor(t["name"], t["data"]))
    for nm, arr in extra_init:
        body += _enc(5, 2, _enc_tensor(nm, arr))
    ti, to = graph.tensors[graph.input], graph.tensors[graph.output]
    body += _enc(11, 2, _enc_value_info(ti["name"], ti["dtype"], ti["shape"]))
    body += _enc(12, 2, _enc_value_info(to["name"], to["dtype"], to["shape"]))
    opset = _enc(1, 2, b"") + _enc(2, 0, 13)
    return _enc(1, 0, 8) + _enc(2, 2, b"zant_b200") + _enc(7, 2, body) + _enc(8, 2, opset)
