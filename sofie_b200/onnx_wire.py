"""Protobuf-free reader and writer for the subset of the ONNX wire format the dense-contraction
path needs (ModelProto > GraphProto > NodeProto / TensorProto / ValueInfoProto / AttributeProto).

Field numbers follow the ONNX schema the reference vendors (src/SOFIE_parsers/onnx_proto3):
Model.graph=7, Model.ir_version=1, Model.opset_import=8; Graph.node=1, name=2, initializer=5,
input=11, output=12; Node.input=1, output=2, name=3, op_type=4, attribute=5; Tensor.dims=1,
data_type=2, float_data=4, int32_data=5, int64_data=7, name=8, raw_data=9; Attribute.name=1, f=2,
i=3, s=4, t=5, floats=7, ints=8, type=20; ValueInfo.name=1, type=2; Type.tensor_type=1;
Type.Tensor.elem_type=1, shape=2; Shape.dim=1; Dim.dim_value=1, dim_param=2.
"""
from __future__ import annotations

import struct

import numpy as np

# ONNX TensorProto.DataType
FLOAT, UINT8, INT8, INT32, INT64, BFLOAT16, FLOAT8E4M3FN = 1, 2, 3, 6, 7, 16, 17
NP_DTYPES = {FLOAT: np.float32, UINT8: np.uint8, INT8: np.int8, INT32: np.int32, INT64: np.int64}
DT_OF_NP = {np.dtype(v): k for k, v in NP_DTYPES.items()}


# ------------------------------------------------------------------------------------ writer
def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _ld(field: int, payload: bytes) -> bytes:
    return _key(field, 2) + _varint(len(payload)) + payload


def _vi(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(v)


def _s(field: int, text: str) -> bytes:
    return _ld(field, text.encode())


def tensor(name: str, arr: np.ndarray, data_type: int | None = None) -> bytes:
    arr = np.ascontiguousarray(arr)
    dt = data_type if data_type is not None else DT_OF_NP[arr.dtype]
    out = b"".join(_vi(1, d) for d in arr.shape) + _vi(2, dt) + _s(8, name) + _ld(9, arr.tobytes())
    return out


def attr_int(name, v):
    return _s(1, name) + _vi(3, int(v)) + _vi(20, 2)


def attr_float(name, v):
    return _s(1, name) + _key(2, 5) + struct.pack("<f", float(v)) + _vi(20, 1)


def attr_ints(name, vs):
    return _s(1, name) + b"".join(_vi(8, int(v)) for v in vs) + _vi(20, 7)


def attr_tensor(name, tensor_name, arr):
    """AttributeProto of type TENSOR (field 5 = t, type 4), as a Constant node's `value`."""
    return _s(1, name) + _ld(5, tensor(tensor_name, np.asarray(arr))) + _vi(20, 4)


def attr_str(name, v):
    return _s(1, name) + _ld(4, v.encode()) + _vi(20, 3)


def node(op_type, inputs, outputs, attrs=(), name=""):
    out = b"".join(_s(1, i) for i in inputs) + b"".join(_s(2, o) for o in outputs)
    if name:
        out += _s(3, name)
    out += _s(4, op_type) + b"".join(_ld(5, a) for a in attrs)
    return out


def value_info(name, elem_type, shape):
    dims = b""
    for d in shape:
        dims += _ld(1, _s(2, d) if isinstance(d, str) else _vi(1, int(d)))
    ttype = _vi(1, elem_type) + _ld(2, dims)
    return _s(1, name) + _ld(2, _ld(1, ttype))


def model(graph_name, nodes, inputs, outputs, initializers, opset=13):
    g = b"".join(_ld(1, n) for n in nodes) + _s(2, graph_name) + b"".join(_ld(5, t) for t in initializers)
    g += b"".join(_ld(11, i) for i in inputs) + b"".join(_ld(12, o) for o in outputs)
    return _vi(1, 8) + _s(2, "sofie_b200") + _ld(7, g) + _ld(8, _s(1, "") + _vi(2, opset))


# ------------------------------------------------------------------------------------ reader
def _read_varint(buf, pos):
    v, shift = 0, 0
    while True:
        b = buf[pos]
        pos += 1
        v |= (b & 0x7F) << shift
        if not b & 0x80:
            return v, pos
        shift += 7


def fields(buf):
    """Yield (field_number, wire_type, value) of one message; length-delimited values are bytes."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _read_varint(buf, pos)
        f, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _read_varint(buf, pos)
        elif wt == 1:
            v, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            ln, pos = _read_varint(buf, pos)
            v, pos = buf[pos:pos + ln], pos + ln
        elif wt == 5:
            v, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        yield f, wt, v


def _signed(v):
    return v - (1 << 64) if v >= 1 << 63 else v


def _packed_varints(b):
    out, pos = [], 0
    while pos < len(b):
        v, pos = _read_varint(b, pos)
        out.append(_signed(v))
    return out


def read_tensor(buf):
    dims, dt, name, raw, floats, i32, i64 = [], FLOAT, "", None, [], [], []
    for f, wt, v in fields(buf):
        if f == 1:
            dims += _packed_varints(v) if wt == 2 else [_signed(v)]
        elif f == 2:
            dt = v
        elif f == 8:
            name = bytes(v).decode()
        elif f == 9:
            raw = bytes(v)
        elif f == 4:
            floats += list(struct.unpack(f"<{len(v) // 4}f", v)) if wt == 2 else [struct.unpack("<f", v)[0]]
        elif f == 5:
            i32 += _packed_varints(v) if wt == 2 else [_signed(v)]
        elif f == 7:
            i64 += _packed_varints(v) if wt == 2 else [_signed(v)]
    npdt = NP_DTYPES.get(dt, np.uint8)
    if raw is not None:
        arr = np.frombuffer(raw, dtype=npdt).copy()
    elif dt == FLOAT:
        arr = np.array(floats, np.float32)
    elif dt == INT64:
        arr = np.array(i64, np.int64)
    else:
        arr = np.array(i32, npdt)
    return name, arr.reshape(dims) if dims else arr, dt


def read_attribute(buf):
    name, val, ints, floats = "", None, [], []
    for f, wt, v in fields(buf):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            val = struct.unpack("<f", v)[0]
        elif f == 3:
            val = _signed(v)
        elif f == 4:
            val = bytes(v).decode()
        elif f == 5:
            val = read_tensor(v)
        elif f == 7:
            floats += list(struct.unpack(f"<{len(v) // 4}f", v)) if wt == 2 else [struct.unpack("<f", v)[0]]
        elif f == 8:
            ints += _packed_varints(v) if wt == 2 else [_signed(v)]
    if ints:
        val = ints
    elif floats:
        val = floats
    return name, val


def read_value_info(buf):
    name, elem, shape = "", 0, []
    for f, _, v in fields(buf):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            for f2, _, v2 in fields(v):
                if f2 == 1:  # tensor_type
                    for f3, _, v3 in fields(v2):
                        if f3 == 1:
                            elem = v3
                        elif f3 == 2:
                            for f4, _, v4 in fields(v3):
                                if f4 == 1:
                                    d = None
                                    for f5, _, v5 in fields(v4):
                                        d = _signed(v5) if f5 == 1 else bytes(v5).decode()
                                    shape.append(d)
    return name, elem, shape


def read_model(data: bytes):
    """Return dict(nodes=[dict(op, inputs, outputs, attrs)], initializers={name: array}, inputs, outputs)."""
    graph = None
    for f, _, v in fields(data):
        if f == 7:
            graph = v
    if graph is None:
        raise ValueError("no graph in ONNX model")
    out = dict(nodes=[], initializers={}, init_types={}, inputs=[], outputs=[])
    for f, _, v in fields(graph):
        if f == 1:
            n = dict(op="", inputs=[], outputs=[], attrs={}, name="")
            for f2, _, v2 in fields(v):
                if f2 == 1:
                    n["inputs"].append(bytes(v2).decode())
                elif f2 == 2:
                    n["outputs"].append(bytes(v2).decode())
                elif f2 == 3:
                    n["name"] = bytes(v2).decode()
                elif f2 == 4:
                    n["op"] = bytes(v2).decode()
                elif f2 == 5:
                    k, val = read_attribute(v2)
                    n["attrs"][k] = val
            out["nodes"].append(n)
        elif f == 5:
            name, arr, dt = read_tensor(v)
            out["initializers"][name] = arr
            out["init_types"][name] = dt
        elif f == 11:
            out["inputs"].append(read_value_info(v))
        elif f == 12:
            out["outputs"].append(read_value_info(v))
    return out


# ------------------------------------------------------------------------------------ Model -> ONNX
def e4m3_bytes(x: np.ndarray, scale: float) -> np.ndarray:
    """E4M3 bit patterns of x / scale: fp32 division, round to nearest even, saturating at +-448 (the
    quantisation the library applies on the device)."""
    import ml_dtypes
    q = (np.asarray(x, np.float32) / np.float32(scale)).astype(np.float32)
    return np.clip(q, -448.0, 448.0).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)


def model_to_onnx(m, fp8_scales=None, batch_param=None) -> bytes:
    """Serialise a sofie_b200.configs.Model as an ONNX file (batch_param: write the first input dimension as the named
    parameter instead of a number, as exporters do for a dynamic batch axis). The FP8 chain (Fp8Gemm layers) needs its calibrated
    activation scales: it is written as QuantizeLinear to FLOAT8E4M3FN, one custom Fp8Gemm node per layer with
    E4M3 weights and static scales as attributes, and a final Cast from bfloat16 to float."""
    nodes, inits = [], []
    w = m.weights
    used = set()
    fp8_layers = [L for L in m.layers if L["op"] == "Fp8Gemm"]
    fp8_dynamic = isinstance(fp8_scales, str) and fp8_scales == "dynamic"   # scales from amax at run time
    if fp8_layers and not fp8_dynamic and (fp8_scales is None or len(fp8_scales) != len(fp8_layers)):
        raise ValueError("the FP8 chain needs one calibrated activation scale per Fp8Gemm layer (or fp8_scales='dynamic')")
    fp8_i = 0

    def init(name, arr=None):
        if name not in used:
            used.add(name)
            inits.append(tensor(name, w[name] if arr is None else arr))
        return name

    def scalar(name, val, dt):
        return init(name, np.array(val, dt))

    for i, L in enumerate(m.layers):
        op = L["op"]
        if op == "Gemm":
            ins = [L["A"], init(L["B"])] + ([init(L["C"])] if L.get("C") else [])
            nodes.append(node("Gemm", ins, [L["Y"]], [attr_float("alpha", L.get("alpha", 1.0)),
                                                      attr_float("beta", L.get("beta", 1.0)),
                                                      attr_int("transB", L.get("transB", 0))]))
            if L.get("relu"):
                # Gemm+Relu is written as two nodes; the parser fuses them as the reference does
                nodes[-1] = node("Gemm", ins, [L["Y"] + "_pre"], [attr_float("alpha", L.get("alpha", 1.0)),
                                                                  attr_float("beta", L.get("beta", 1.0)),
                                                                  attr_int("transB", L.get("transB", 0))])
                nodes.append(node("Relu", [L["Y"] + "_pre"], [L["Y"]]))
        elif op == "Conv":
            ins = [L["X"], init(L["W"])] + ([init(L["B"])] if L.get("B") else [])
            nodes.append(node("Conv", ins, [L["Y"]], [attr_ints("kernel_shape", L["kernel"]), attr_ints("pads", L["pads"]),
                                                      attr_ints("strides", L["strides"]), attr_int("group", L.get("group", 1)),
                                                      attr_ints("dilations", L.get("dilations", (1,) * len(L["kernel"])))]))
        elif op == "ConvTranspose":
            ins = [L["X"], init(L["W"])] + ([init(L["B"])] if L.get("B") else [])
            nodes.append(node("ConvTranspose", ins, [L["Y"]],
                              [attr_ints("kernel_shape", L["kernel"]), attr_ints("pads", L["pads"]), attr_ints("strides", L["strides"]),
                               attr_ints("output_padding", L.get("output_padding", (0, 0))), attr_int("group", 1),
                               attr_ints("dilations", (1, 1))]))
        elif op == "Relu":
            nodes.append(node("Relu", [L["X"]], [L["Y"]]))
        elif op == "MaxPool":
            nodes.append(node("MaxPool", [L["X"]], [L["Y"]], [attr_ints("kernel_shape", L["kernel"]),
                                                              attr_ints("pads", L["pads"]), attr_ints("strides", L["strides"])]))
        elif op == "Flatten":
            nodes.append(node("Flatten", [L["X"]], [L["Y"]], [attr_int("axis", L.get("axis", 1))]))
        elif op == "Softmax":
            nodes.append(node("Softmax", [L["X"]], [L["Y"]], [attr_int("axis", L.get("axis", -1))]))
        elif op == "QuantizeLinear":
            nodes.append(node("QuantizeLinear", [L["X"], scalar(f"qs{i}", L["scale"], np.float32),
                                                 scalar(f"qz{i}", L["zp"], np.uint8)], [L["Y"]]))
        elif op == "DequantizeLinear":
            nodes.append(node("DequantizeLinear", [L["X"], scalar(f"ds{i}", L["scale"], np.float32),
                                                   scalar(f"dz{i}", L["zp"], np.uint8)], [L["Y"]]))
        elif op == "QLinearMatMul":
            ins = [L["A"], scalar(f"as{i}", L["a_scale"], np.float32), scalar(f"az{i}", L["a_zp"], np.uint8),
                   init(L["B"]), init(L["w_scale"]), init(f"wz{i}", np.zeros(w[L["w_scale"]].shape, np.int8)),
                   scalar(f"ys{i}", L["y_scale"], np.float32), scalar(f"yz{i}", L["y_zp"], np.uint8)]
            out = L["Y"] + "_pre" if L.get("relu") else L["Y"]
            nodes.append(node("QLinearMatMul", ins, [out]))
            if L.get("relu"):
                nodes.append(node("Relu", [out], [L["Y"]]))
        elif op == "QLinearConv":
            ins = [L["X"], scalar(f"xs{i}", L["x_scale"], np.float32), scalar(f"xz{i}", L["x_zp"], np.uint8),
                   init(L["W"]), init(L["w_scale"]), init(f"wz{i}", np.zeros(w[L["w_scale"]].shape, np.int8)),
                   scalar(f"ys{i}", L["y_scale"], np.float32), scalar(f"yz{i}", L["y_zp"], np.uint8)]
            out = L["Y"] + "_pre" if L.get("relu") else L["Y"]
            nodes.append(node("QLinearConv", ins, [out], [attr_ints("kernel_shape", L["kernel"]), attr_ints("pads", L["pads"]),
                                                          attr_ints("strides", L["strides"])]))
            if L.get("relu"):
                nodes.append(node("Relu", [out], [L["Y"]]))
        elif op == "Fp8Gemm" and fp8_dynamic:
            # DynamicQuantizeE4M3 in front of every layer; the layer reads its scale as a fourth input and writes bfloat16
            last = fp8_i + 1 == len(fp8_layers)
            src, sc = L["A"] + "_q", L["A"] + "_scale"
            prev = L["A"] if fp8_i == 0 else L["A"] + "_bf16"
            nodes.append(node("DynamicQuantizeE4M3", [prev], [src, sc]))
            wq = L["B"] + "_e4m3"
            inits.append(tensor(wq, e4m3_bytes(w[L["B"]], L["w_scale"]), FLOAT8E4M3FN))
            ins = [src, wq, init(L["C"]) if L.get("C") else "", sc]
            out = L["Y"] + "_bf16"
            nodes.append(node("Fp8Gemm", ins, [out], [attr_float("w_scale", L["w_scale"]), attr_int("relu", int(bool(L.get("relu"))))]))
            if last:
                nodes.append(node("Cast", [out], [L["Y"]], [attr_int("to", FLOAT)]))
            fp8_i += 1
        elif op == "Fp8Gemm":
            a_scale = float(fp8_scales[fp8_i])
            last = fp8_i + 1 == len(fp8_layers)
            out_scale = 0.0 if last else float(fp8_scales[fp8_i + 1])
            src = L["A"] + "_q"
            if fp8_i == 0:
                inits.append(tensor(f"fp8s{i}", np.array(a_scale, np.float32)))
                inits.append(tensor(f"fp8z{i}", np.zeros((), np.uint8), FLOAT8E4M3FN))
                nodes.append(node("QuantizeLinear", [L["A"], f"fp8s{i}", f"fp8z{i}"], [src]))
            wq = L["B"] + "_e4m3"
            inits.append(tensor(wq, e4m3_bytes(w[L["B"]], L["w_scale"]), FLOAT8E4M3FN))
            ins = [src, wq] + ([init(L["C"])] if L.get("C") else [])
            out = L["Y"] + ("_bf16" if last else "_q")
            nodes.append(node("Fp8Gemm", ins, [out], [attr_float("a_scale", a_scale), attr_float("w_scale", L["w_scale"]),
                                                    attr_float("out_scale", out_scale), attr_int("relu", int(bool(L.get("relu"))))]))
            if last:
                nodes.append(node("Cast", [out], [L["Y"]], [attr_int("to", FLOAT)]))
            fp8_i += 1
        elif op in ("Sigmoid", "Tanh", "Selu", "Neg", "Exp", "Log", "Sqrt", "Reciprocal", "Abs"):
            nodes.append(node(op, [L["X"]], [L["Y"]]))
        elif op in ("LeakyRelu", "Elu"):
            nodes.append(node(op, [L["X"]], [L["Y"]], [attr_float("alpha", L.get("alpha", 0.01 if op == "LeakyRelu" else 1.0))]))
        elif op in ("Add", "Sub", "Mul", "Div"):
            nodes.append(node(op, [init(n) if n in w else n for n in (L["A"], L["B"])], [L["Y"]]))
        elif op == "BatchNormalization":
            ins = [L["X"], init(L["scale"]), init(L["bias"]), init(L["mean"]), init(L["var"])]
            out = L["Y"] + "_pre" if L.get("relu") else L["Y"]
            nodes.append(node(op, ins, [out], [attr_float("epsilon", L.get("epsilon", 1e-5))]))
            if L.get("relu"):
                # BatchNormalization + Relu is written as two nodes; the parser fuses them as the reference does
                nodes.append(node("Relu", [out], [L["Y"]]))
        else:
            raise NotImplementedError(f"no ONNX serialisation for {op}")
    inputs = [value_info(m.input_name, FLOAT, ([batch_param] + list(m.input_shape[1:])) if batch_param else m.input_shape)]
    outputs = [value_info(m.output_name, FLOAT, [])]
    return model(m.name, nodes, inputs, outputs, inits)
