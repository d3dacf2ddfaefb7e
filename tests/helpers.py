"""Shared test helpers: the golden fixtures of the reference, two interchangeable back ends
(the CPU oracle and the CUDA path through the C ABI) and the error metrics the tests use."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_fixtures():
    manifest = json.loads((GOLDEN / "reference_fixtures.json").read_text())
    arrays = np.load(GOLDEN / "reference_fixtures.npz")
    return manifest, arrays


def rel_err(y, ref):
    """max_i |y_i - ref_i| / max_i |ref_i|: the error of a tensor relative to the tensor's own scale.
    This is the metric behind the fp32 tolerance of 1e-5. A per-element ratio is not usable: two
    correct fp32 evaluations of the same dot product (OpenBLAS's blocked order, a double
    accumulator) already differ by ~1e-6 absolute, which is 1e-4 of an output that cancels to 0.01."""
    y = np.asarray(y, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    assert y.shape == ref.shape, (y.shape, ref.shape)
    if ref.size == 0:
        return 0.0
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


class OracleBackend:
    """numpy in / numpy out through oracle/sofie_oracle.c."""

    def __init__(self):
        from oracle import cpu_oracle
        self.o = cpu_oracle

    def gemm(self, A, B, C=None, **kw):
        return self.o.gemm_f32(A, B, C, **kw)

    def conv(self, X, W, B=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), group=1):
        return self.o.conv2d_f32(X, W, B, pad=pad, stride=stride, dil=dil, group=group)

    def conv_transpose(self, X, W, B=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0)):
        return self.o.conv_transpose2d_f32(X, W, B, pad=pad, stride=stride, dil=dil, out_pad=out_pad)

    def einsum(self, equation, A, B):
        return self.o.einsum_f32(equation, A, B)

    def relu(self, X):
        return self.o.relu_f32(X)

    def pool(self, X, mode, kernel, stride, pads, count_include_pad=0):
        return self.o.pool2d_f32(X, mode, kernel, stride, pads, count_include_pad)

    def pool3d(self, X, mode, kernel, stride, pads, count_include_pad=0):
        return self.o.pool3d_f32(X, mode, kernel, stride, pads, count_include_pad)

    def softmax(self, X, axis):
        return self.o.softmax_f32(X, axis)

    def unary(self, X, op, alpha):
        return self.o.unary_f32(X, op, alpha)

    def binary(self, A, B, op):
        return self.o.binary_f32(A, B, op)


class CudaBackend:
    """numpy in / numpy out through libSOFIE_cuda (C ABI) on cuda:0."""

    def __init__(self, device="cuda:0"):
        import torch
        from sofie_b200 import ops
        self.t, self.ops, self.dev = torch, ops, device

    def _d(self, a):
        return None if a is None else self.t.from_numpy(np.ascontiguousarray(a)).to(self.dev)

    def gemm(self, A, B, C=None, **kw):
        return self.ops.gemm_f32(self._d(A), self._d(B), self._d(C), **kw).cpu().numpy()

    def conv(self, X, W, B=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), group=1):
        return self.ops.conv2d_f32(self._d(X), self._d(W), self._d(B), pad=pad, stride=stride, dil=dil,
                                   group=group).cpu().numpy()

    def conv_transpose(self, X, W, B=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0)):
        return self.ops.conv_transpose2d_f32(self._d(X), self._d(W), self._d(B), pad=pad, stride=stride, dil=dil,
                                             out_pad=out_pad).cpu().numpy()

    def einsum(self, equation, A, B):
        return self.ops.einsum_f32(equation, self._d(A), self._d(B)).cpu().numpy()

    def relu(self, X):
        return self.ops.relu_f32(self._d(X)).cpu().numpy()

    def pool(self, X, mode, kernel, stride, pads, count_include_pad=0):
        return self.ops.pool2d_f32(self._d(X), mode=mode, kernel=kernel, stride=stride, pads=pads,
                                   count_include_pad=count_include_pad).cpu().numpy()

    def pool3d(self, X, mode, kernel, stride, pads, count_include_pad=0):
        return self.ops.pool3d_f32(self._d(X), mode=mode, kernel=kernel, stride=stride, pads=pads,
                                   count_include_pad=count_include_pad).cpu().numpy()

    def softmax(self, X, axis):
        return self.ops.softmax_f32(self._d(X), axis).cpu().numpy()

    def unary(self, X, op, alpha):
        return self.ops.unary_f32(self._d(X), op, alpha).cpu().numpy()

    def binary(self, A, B, op):
        return self.ops.binary_f32(self._d(A), self._d(B), op).cpu().numpy()


def conv_attrs(attrs, kshape):
    """ONNX Conv attributes -> (pad_h, pad_w), strides, dilations, group following the reference's
    rules: no pads attribute means pad 1 (ROperator_Conv.hxx:136-139), SAME_* means k/2 after the
    averaging of asymmetric pads (ROperator_Conv.hxx:140-158,387-410)."""
    kh, kw = attrs.get("kernel_shape", kshape)
    auto = attrs.get("auto_pad", "NOTSET")
    if auto == "NOTSET":
        pads = attrs.get("pads", [1, 1, 1, 1])
    elif auto in ("SAME_UPPER", "SAME_LOWER"):
        pads = [kh // 2, kw // 2, kh // 2, kw // 2]
        if kh % 2 == 1:
            pads[0 if auto == "SAME_UPPER" else 2] += 1
        if kw % 2 == 1:
            pads[1 if auto == "SAME_UPPER" else 3] += 1
    else:
        pads = [0, 0, 0, 0]
    pad = ((pads[0] + pads[2]) // 2, (pads[1] + pads[3]) // 2) if (pads[0] != pads[2] or pads[1] != pads[3]) \
        else (pads[0], pads[1])
    return pad, tuple(attrs.get("strides", [1, 1])), tuple(attrs.get("dilations", [1, 1])), attrs.get("group", 1)


def run_fixture(name, manifest, arrays, backend):
    """Evaluate one golden fixture's graph with the given back end; returns the flat output."""
    entry = manifest[name]
    t = {i: arrays[f"{name}/in/{i}"] for i in entry["inputs"]}
    for key in arrays.files:
        if key.startswith(f"{name}/w/"):
            t[key[len(name) + 3:]] = arrays[key]
    out = None
    for n in entry["nodes"]:
        op, a, ins = n["op"], n["attrs"], n["inputs"]
        if op == "Gemm":
            y = backend.gemm(t[ins[0]], t[ins[1]], t[ins[2]] if len(ins) > 2 else None, transA=a.get("transA", 0),
                             transB=a.get("transB", 0), alpha=a.get("alpha", 1.0), beta=a.get("beta", 1.0))
        elif op == "Einsum":
            if a["equation"].replace(" ", "") == "ik,kj->ij":
                y = backend.gemm(t[ins[0]], t[ins[1]], None, beta=0.0)
            else:
                y = backend.einsum(a["equation"], t[ins[0]], t[ins[1]])
        elif op == "Relu":
            y = backend.relu(t[ins[0]])
        elif op == "Conv":
            W = t[ins[1]]
            pad, stride, dil, group = conv_attrs(a, W.shape[2:])
            y = backend.conv(t[ins[0]], W, t[ins[2]] if len(ins) > 2 else None, pad=pad, stride=stride, dil=dil, group=group)
        elif op == "ConvTranspose":
            X, W = t[ins[0]], t[ins[1]]
            one_d = X.ndim == 3  # a 1-D transposed convolution is the 2-D one with a height of 1
            if one_d:
                X, W = X[:, :, None, :], W[:, :, None, :]
            nd = 1 if one_d else 2
            lift = (lambda v, fill: (fill, v[0]) if one_d else tuple(v))
            pads = a.get("pads", [0] * (2 * nd))
            # asymmetric pads are averaged, as the reference does (ROperator_ConvTranspose.icc:332-346)
            pad = lift([(pads[i] + pads[i + nd]) // 2 if pads[i] != pads[i + nd] else pads[i] for i in range(nd)], 0)
            y = backend.conv_transpose(X, W, t[ins[2]] if len(ins) > 2 else None, pad=pad,
                                       stride=lift(a.get("strides", [1] * nd), 1), dil=lift(a.get("dilations", [1] * nd), 1),
                                       out_pad=lift(a.get("output_padding", [0] * nd), 0))
            if one_d:
                y = y[:, :, 0, :]
        elif op in ("MaxPool", "AveragePool"):
            X = t[ins[0]]
            if X.ndim == 5:
                y = backend.pool3d(X, 0 if op == "MaxPool" else 1, tuple(a["kernel_shape"]), tuple(a.get("strides", [1, 1, 1])),
                                   tuple(a.get("pads", [0] * 6)), a.get("count_include_pad", 0))
            elif X.ndim == 3:   # a 1-D pooling is the 2-D one with a height of 1
                p1 = a.get("pads", [0, 0])
                y = backend.pool(X[:, :, None, :], 0 if op == "MaxPool" else 1, (1, a["kernel_shape"][0]), (1, a.get("strides", [1])[0]),
                                 (0, p1[0], 0, p1[1]), a.get("count_include_pad", 0))[:, :, 0, :]
            else:
                y = backend.pool(X, 0 if op == "MaxPool" else 1, tuple(a["kernel_shape"]),
                                 tuple(a.get("strides", [1, 1])), tuple(a.get("pads", [0, 0, 0, 0])),
                                 a.get("count_include_pad", 0))
        elif op == "Softmax":
            y = backend.softmax(t[ins[0]], a.get("axis", -1))
        elif op in UNARY_FIXTURE_OPS:
            y = backend.unary(t[ins[0]], op, a.get("alpha", 0.01 if op == "LeakyRelu" else 1.0))
        elif op in ("Add", "Sub", "Mul", "Div"):
            y = backend.binary(t[ins[0]], t[ins[1]], op)
        elif op == "Constant":
            y = arrays[a["value"]["tensor"]]
        elif op == "Identity":
            y = t[ins[0]]
        else:
            raise NotImplementedError(op)
        t[n["outputs"][0]] = y
        out = y
    return np.asarray(out).ravel()


UNARY_FIXTURE_OPS = ("Sigmoid", "Tanh", "LeakyRelu", "Selu", "Elu", "Neg", "Exp", "Log", "Sqrt", "Reciprocal", "Abs", "Erf", "Swish", "Cos", "Sin")

FIXTURE_CASES = ["Linear_16", "Linear_32", "Linear_64", "ConvWithPadding", "ConvWithoutPadding",
                 "ConvWithAutopadSameLower", "ConvWithStridesPadding", "ConvWithStridesNoPadding", "MaxPool2d", "MaxPool3d", "AvgPool",
                 "Softmax1d", "Softmax2d", "Softmax3d", "Softmax4d", "Einsum_matmul",
                 "LinearWithSelu", "LinearWithSigmoid", "LinearWithLeakyRelu", "Add", "Sub", "Mul", "Div", "Neg", "Exp", "Log",
                 "Elu", "Tanh", "Sqrt", "Reciprocal",
                 "AddBroadcast1", "AddBroadcast2", "AddBroadcast3", "AddBroadcast4", "AddBroadcast5", "AddBroadcast7",
                 "ConvTranspose1d", "ConvTranspose2d", "ConvTransposeBias2d", "ConvTransposeBias2dBatched", "MaxPool1d",
                 "Einsum_3", "Einsum_4", "Einsum_dotprod", "Erf", "Abs", "Cos", "Sin", "Constant"]
# fixtures the test-side ONNX writer can re-encode (it has no tensor-valued attributes)
REENCODABLE_CASES = [n for n in FIXTURE_CASES if n != "Constant"]


def fixture_onnx_bytes(name):
    """The fixture model exactly as the reference's tests hold it (tests/golden/onnx/<name>.onnx, copied byte for byte by
    tests/golden/make_golden.py): what the C++ parser is tested on."""
    return (GOLDEN / "onnx" / f"{name}.onnx").read_bytes()


def fixture_to_onnx(name, manifest, arrays):
    """Re-serialise one golden fixture (nodes, attributes, weights, input shapes) as ONNX bytes with this repository's
    own writer: a test of the writer (the parser itself is tested on the reference's bytes, fixture_onnx_bytes)."""
    from sofie_b200 import onnx_wire as ow
    entry = manifest[name]
    nodes = []
    for n in entry["nodes"]:
        attrs = []
        for k, v in n["attrs"].items():
            if isinstance(v, str):
                attrs.append(ow.attr_str(k, v))
            elif isinstance(v, float):
                attrs.append(ow.attr_float(k, v))
            elif isinstance(v, int):
                attrs.append(ow.attr_int(k, v))
            else:
                attrs.append(ow.attr_ints(k, v))
        nodes.append(ow.node(n["op"], n["inputs"], n["outputs"], attrs))
    inits = [ow.tensor(key[len(name) + 3:], arrays[key]) for key in arrays.files if key.startswith(f"{name}/w/")]
    inputs = [ow.value_info(i, ow.FLOAT, arrays[f"{name}/in/{i}"].shape) for i in entry["inputs"]]
    outputs = [ow.value_info(entry["nodes"][-1]["outputs"][0], ow.FLOAT, [])]
    return ow.model(name, nodes, inputs, outputs, inits)


FUNCTOR_MAIN = r"""
#include "{header}"
#include "SOFIE/SOFIEHelpers.hxx"
#include <cstdio>
#include <thread>
#include <vector>
int main(int argc, char **argv)
{{
   if (argc != 4) return 2;
   const unsigned nslots = 3;
   try {{
      auto f = SofieFunctor<{nfeat}, SOFIE_{name}::Session>(nslots, argv[1]);
      // Sessions are movable: they can be kept in a std::vector, as the reference's functor keeps them
      std::vector<SOFIE_{name}::Session> sessions;
      sessions.emplace_back(argv[1]);
      sessions.emplace_back(argv[1]);
      const long rows = std::atol(argv[3]);
      std::vector<float> x(rows * {nfeat});
      std::FILE *fp = std::fopen(argv[2], "rb");
      if (!fp || std::fread(x.data(), sizeof(float), x.size(), fp) != x.size()) return 3;
      std::fclose(fp);
      std::vector<double> y(rows);
      std::vector<std::thread> pool;
      for (unsigned s = 0; s < nslots; s++)
         pool.emplace_back([&, s] {{
            for (long i = s; i < rows; i += nslots) {{
               const float *r = x.data() + i * {nfeat};
               y[i] = f(s, {args});
            }}
         }});
      for (auto &t : pool) t.join();
      for (long i = 0; i < rows; i++) std::printf("%.9g\n", y[i]);
      float first[{nfeat}];
      for (int k = 0; k < {nfeat}; k++) first[k] = x[k];
      std::printf("%.9g\n", (double)sessions[1].infer(first)[0]);
   }} catch (const std::exception &e) {{
      std::fprintf(stderr, "%s\n", e.what());
      return 1;
   }}
   return 0;
}}
"""


def build_functor_program(model, name, nfeat):
    """Emits `model` (batch 1, nfeat input features) and builds a small program that evaluates it through
    SofieFunctor from three threads. Returns (program, weight file)."""
    import subprocess
    from sofie_b200 import _build, generated, onnx_wire
    hxx = generated.emit(onnx_wire.model_to_onnx(model), name)
    lib = _build.build()
    src = hxx.with_name(name + "_functor.cxx")
    src.write_text(FUNCTOR_MAIN.format(header=hxx.name, name=name, nfeat=nfeat, args=", ".join(f"r[{i}]" for i in range(nfeat))))
    exe = hxx.with_name(name + "_functor")
    cmd = ["g++", "-std=c++17", "-O2", "-pthread", "-I", str(generated.ROOT / "include"), "-I", str(generated.HOST / "inc"),
           "-I", str(hxx.parent), str(src), "-o", str(exe), "-L", str(lib.parent), "-lSOFIE_cuda", f"-Wl,-rpath,{lib.parent}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling the functor program failed:\n{r.stdout}")
    return exe, hxx.with_suffix(".dat")


def tiny_regressor(nfeat=4):
    """Gemm nfeat -> 8 + Relu, Gemm 8 -> 1 on a single row: the shape of model SofieFunctor is used with."""
    from sofie_b200 import configs
    rng = np.random.default_rng(11)
    m = configs.Model("regressor", "x", (1, nfeat), [])
    m.weights["w0"] = rng.standard_normal((8, nfeat)).astype(np.float32)
    m.weights["b0"] = rng.standard_normal(8).astype(np.float32)
    m.weights["w1"] = rng.standard_normal((1, 8)).astype(np.float32)
    m.weights["b1"] = rng.standard_normal(1).astype(np.float32)
    m.layers.append(dict(op="Gemm", A="x", B="w0", C="b0", Y="h", transB=1, relu=True))
    m.layers.append(dict(op="Gemm", A="h", B="w1", C="b1", Y="y", transB=1))
    m.output_name = "y"
    return m


def conv1d_model_onnx(batch=3, length=10, seed=11):
    """The shape of the reference's 1-D convolution test model (test/Conv1dModelGenerator.py, TestSofieModels.cxx Conv1d_B1):
    Conv1d 2->4, kernel 2, pad 1, Relu; Conv1d 4->8, kernel 3, pad 1, two groups, Relu. Returns (onnx bytes, weights, input)."""
    from sofie_b200 import onnx_wire as ow
    rng = np.random.default_rng(seed)
    w0 = (rng.standard_normal((4, 2, 2)) * 0.5).astype(np.float32)
    b0 = rng.uniform(-0.1, 0.1, 4).astype(np.float32)
    w1 = (rng.standard_normal((8, 2, 3)) * 0.4).astype(np.float32)
    b1 = rng.uniform(-0.1, 0.1, 8).astype(np.float32)
    x = rng.standard_normal((batch, 2, length)).astype(np.float32)
    nodes = [ow.node("Conv", ["x", "w0", "b0"], ["c0"], [ow.attr_ints("kernel_shape", [2]), ow.attr_ints("pads", [1, 1]), ow.attr_ints("strides", [1])]),
             ow.node("Relu", ["c0"], ["r0"]),
             ow.node("Conv", ["r0", "w1", "b1"], ["c1"], [ow.attr_ints("kernel_shape", [3]), ow.attr_ints("pads", [1, 1]), ow.attr_int("group", 2)]),
             ow.node("Relu", ["c1"], ["y"])]
    g = ow.model("conv1d", nodes, [ow.value_info("x", ow.FLOAT, list(x.shape))], [ow.value_info("y", ow.FLOAT, [])],
                 [ow.tensor("w0", w0), ow.tensor("b0", b0), ow.tensor("w1", w1), ow.tensor("b1", b1)])
    return g, dict(w0=w0, b0=b0, w1=w1, b1=b1), x


SHARDED_MAIN = r"""
#include "{header}"
#include "SOFIE/SOFIEHelpers.hxx"
#include <cstdio>
#include <cstdlib>
#include <vector>
// usage: prog <weights> <input file> <batch> <floats per sample> <device> [<device> ...]; prints one output value per line
int main(int argc, char **argv)
{{
   if (argc < 6) return 2;
   try {{
      const long batch = std::atol(argv[3]), per = std::atol(argv[4]);
      std::vector<int> devices;
      for (int i = 5; i < argc; i++) devices.push_back(std::atoi(argv[i]));
      SofieSharded<SOFIE_{name}::Session> net(argv[1], devices, (size_t)batch, (size_t)per);
      std::vector<float> x(batch * per);
      std::FILE *fp = std::fopen(argv[2], "rb");
      if (!fp || std::fread(x.data(), sizeof(float), x.size(), fp) != x.size()) return 3;
      std::fclose(fp);
      std::vector<float> y = net.infer((size_t)batch, x.data());
      std::vector<float> y7 = net.infer(7, x.data());                      // a batch smaller than the number of shards' worth
      for (float v : y) std::printf("%.9g\n", v);
      std::printf("#\n");
      for (float v : y7) std::printf("%.9g\n", v);
      try {{ net.infer((size_t)batch + devices.size(), x.data()); return 5; }} catch (const std::runtime_error &) {{ }}
   }} catch (const std::exception &e) {{
      std::fprintf(stderr, "%s\n", e.what());
      return 4;
   }}
   return 0;
}}
"""


def build_sharded_program(model, name):
    """Emits `model` with a run-time batch parameter and builds a program that runs it through SofieSharded."""
    import subprocess
    from sofie_b200 import _build, generated, onnx_wire
    hxx = generated.emit(onnx_wire.model_to_onnx(model, batch_param="bs"), name)
    lib = _build.build()
    src = hxx.with_name(name + "_sharded.cxx")
    src.write_text(SHARDED_MAIN.format(header=hxx.name, name=name))
    exe = hxx.with_name(name + "_sharded")
    cmd = ["g++", "-std=c++17", "-O2", "-pthread", "-I", str(generated.ROOT / "include"), "-I", str(generated.HOST / "inc"),
           "-I", str(hxx.parent), str(src), "-o", str(exe), "-L", str(lib.parent), "-lSOFIE_cuda", f"-Wl,-rpath,{lib.parent}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling the sharded program failed:\n{r.stdout}")
    return exe, hxx.with_suffix(".dat")
