"""The five benchmark configurations as seeded synthetic models.

No public dataset is involved: these seeded definitions are the benchmark. Each configuration
has a fixed seed; one numpy PCG64 generator per configuration draws, in this order, the weights
layer by layer (weight then bias / scales of a layer), then the input. A model is a list of
layer records using ONNX operator vocabulary (Gemm, Conv, Relu, MaxPool, Flatten, QuantizeLinear,
QLinearMatMul, QLinearConv, DequantizeLinear, plus the FP8 Gemm chain) and a dict of numpy
weights. The same records feed the ONNX writer (and through it the C++ generator) and the CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

SEEDS = {"C1": 20260001, "C2": 20260002, "C3": 20260003, "C4": 20260004, "C5": 20260005}


@dataclass
class Model:
    name: str
    input_name: str
    input_shape: tuple
    layers: list
    weights: dict = field(default_factory=dict)
    output_name: str = ""
    flops_per_sample: int = 0  # 2*M*N*K per GEMM, 2*oH*oW*Cout*Cin*kH*kW per conv; everything else 0

    def batch(self) -> int:
        return self.input_shape[0]


def _rng(key: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(SEEDS[key]))


# ------------------------------------------------------------------------------------ C1
def mlp_f32(batch=1024, dims=(64, 128, 128, 10), key="C1", with_input=True):
    """fp32 MLP of Gemm(transB=1)+Relu layers, last layer without Relu. Kaiming-uniform weights
    (bound sqrt(6/fan_in)), bias U(-0.1, 0.1), input N(0,1)."""
    rng = _rng(key)
    m = Model(f"mlp_f32_b{batch}", "x", (batch, dims[0]), [])
    prev = "x"
    for i in range(len(dims) - 1):
        k, n = dims[i], dims[i + 1]
        bound = np.sqrt(6.0 / k)
        m.weights[f"W{i}"] = rng.uniform(-bound, bound, size=(n, k)).astype(np.float32)
        m.weights[f"b{i}"] = rng.uniform(-0.1, 0.1, size=(n,)).astype(np.float32)
        last = i == len(dims) - 2
        m.layers.append(dict(op="Gemm", A=prev, B=f"W{i}", C=f"b{i}", Y=f"y{i}", transB=1, alpha=1.0, beta=1.0,
                             relu=not last))
        prev = f"y{i}"
        m.flops_per_sample += 2 * k * n
    m.output_name = prev
    x = rng.standard_normal((batch, dims[0])).astype(np.float32) if with_input else None
    return m, x


# ------------------------------------------------------------------------------------ C2
def cnn_f32(batch=256, key="C2", hw=32, chans=(3, 16, 32, 64), classes=10, with_input=True):
    """fp32 CNN: Conv 3->16 + Relu; Conv 16->32 + Relu; MaxPool 2x2; Conv 32->64 + Relu; MaxPool 2x2;
    Flatten; Gemm ->10. 3x3, stride 1, pad 1. Kaiming-normal weights (std sqrt(2/fan_in)),
    bias U(-0.1, 0.1), input N(0,1)."""
    rng = _rng(key)
    m = Model(f"cnn_f32_b{batch}", "x", (batch, chans[0], hw, hw), [])
    prev, h = "x", hw
    pool_after = {1, 2}
    for i in range(3):
        cin, cout = chans[i], chans[i + 1]
        fan_in = cin * 9
        m.weights[f"cw{i}"] = (rng.standard_normal((cout, cin, 3, 3)) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        m.weights[f"cb{i}"] = rng.uniform(-0.1, 0.1, size=(cout,)).astype(np.float32)
        m.layers.append(dict(op="Conv", X=prev, W=f"cw{i}", B=f"cb{i}", Y=f"c{i}", pads=(1, 1, 1, 1), strides=(1, 1),
                             kernel=(3, 3), group=1))
        m.layers.append(dict(op="Relu", X=f"c{i}", Y=f"r{i}"))
        prev = f"r{i}"
        m.flops_per_sample += 2 * h * h * cout * cin * 9
        if i in pool_after:
            m.layers.append(dict(op="MaxPool", X=prev, Y=f"p{i}", kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0)))
            prev = f"p{i}"
            h //= 2
    feat = chans[3] * h * h
    m.layers.append(dict(op="Flatten", X=prev, Y="flat", axis=1))
    m.weights["fw"] = (rng.standard_normal((classes, feat)) * np.sqrt(2.0 / feat)).astype(np.float32)
    m.weights["fb"] = rng.uniform(-0.1, 0.1, size=(classes,)).astype(np.float32)
    m.layers.append(dict(op="Gemm", A="flat", B="fw", C="fb", Y="logits", transB=1, alpha=1.0, beta=1.0, relu=False))
    m.flops_per_sample += 2 * feat * classes
    m.output_name = "logits"
    x = rng.standard_normal((batch, chans[0], hw, hw)).astype(np.float32) if with_input else None
    return m, x


# ------------------------------------------------------------------------------------ C3
def mlp_i8(batch=8192, dims=(512, 1024, 1024, 256), key="C3", act_scale=0.02, act_zp=128, with_input=True):
    """int8 MLP: QuantizeLinear -> QLinearMatMul x3 -> DequantizeLinear. Activations uint8 with scale
    0.02 and zero point 128 everywhere; weights int8 U{-127..127} stored [K,N] as ONNX does, with
    per-output-channel scales U(0.001, 0.01) and zero point 0."""
    rng = _rng(key)
    m = Model(f"mlp_i8_b{batch}", "x", (batch, dims[0]), [])
    m.layers.append(dict(op="QuantizeLinear", X="x", Y="q0", scale=act_scale, zp=act_zp))
    prev = "q0"
    for i in range(len(dims) - 1):
        k, n = dims[i], dims[i + 1]
        m.weights[f"W{i}"] = rng.integers(-127, 128, size=(k, n), dtype=np.int64).astype(np.int8)
        m.weights[f"s{i}"] = rng.uniform(0.001, 0.01, size=(n,)).astype(np.float32)
        m.layers.append(dict(op="QLinearMatMul", A=prev, B=f"W{i}", Y=f"q{i + 1}", a_scale=act_scale, a_zp=act_zp,
                             w_scale=f"s{i}", y_scale=act_scale, y_zp=act_zp, relu=False))
        prev = f"q{i + 1}"
        m.flops_per_sample += 2 * k * n
    m.layers.append(dict(op="DequantizeLinear", X=prev, Y="y", scale=act_scale, zp=act_zp))
    m.output_name = "y"
    x = rng.standard_normal((batch, dims[0])).astype(np.float32) if with_input else None
    return m, x


# ------------------------------------------------------------------------------------ C4
def gemm_chain_fp8(rows=65536, width=4096, layers=4, key="C4", with_input=True):
    """FP8 E4M3 Gemm chain: `layers` layers of K = N = width on `rows` rows. Weights N(0, 0.02) stored
    [N,K], bias N(0, 0.02), input N(0,1). fp32 accumulation, bf16 output with bias and Relu
    (no Relu after the last layer). Per-tensor scales = amax/448; weight scales are computed here,
    activation scales are calibrated by the caller on the seeded input (static scales)."""
    rng = _rng(key)
    m = Model(f"gemm_chain_fp8_m{rows}", "x", (rows, width), [])
    prev = "x"
    for i in range(layers):
        w = (rng.standard_normal((width, width)) * 0.02).astype(np.float32)
        m.weights[f"W{i}"] = w
        m.weights[f"b{i}"] = (rng.standard_normal((width,)) * 0.02).astype(np.float32)
        m.layers.append(dict(op="Fp8Gemm", A=prev, B=f"W{i}", C=f"b{i}", Y=f"y{i}", relu=i < layers - 1,
                             w_scale=float(np.abs(w).max() / 448.0)))
        prev = f"y{i}"
        m.flops_per_sample += 2 * width * width
    m.output_name = prev
    x = rng.standard_normal((rows, width)).astype(np.float32) if with_input else None
    return m, x


def calibrate_fp8_scales(model, x):
    """Static per-tensor activation scales (amax / 448) of the FP8 chain: one fp32 pass of the chain
    over the given (seeded) input at model-build time. Returns one scale per Fp8Gemm layer input."""
    scales = []
    cur = np.asarray(x, np.float32)
    for L in model.layers:
        if L["op"] != "Fp8Gemm":
            continue
        scales.append(float(np.abs(cur).max() / 448.0) or 1.0)
        cur = cur @ model.weights[L["B"]].T + model.weights[L["C"]]
        if L["relu"]:
            cur = np.maximum(cur, 0)
    return scales


# ------------------------------------------------------------------------------------ elementwise family
def resblock_f32(batch=8, chans=16, hw=16, key="C2", with_input=True):
    """Residual block: Conv 8->C + BatchNormalization + Relu; Conv C->C + BatchNormalization; Add(skip); LeakyRelu;
    MaxPool 2x2; Mul by a per-channel constant; Flatten; Gemm -> 10; Sigmoid. Seeded like C2."""
    rng = np.random.Generator(np.random.PCG64(SEEDS[key] + 77))
    m = Model(f"resblock_b{batch}", "x", (batch, 8, hw, hw), [])

    def bn(prefix):
        m.weights[prefix + "_g"] = rng.uniform(0.5, 1.5, chans).astype(np.float32)
        m.weights[prefix + "_b"] = rng.uniform(-0.2, 0.2, chans).astype(np.float32)
        m.weights[prefix + "_m"] = (rng.standard_normal(chans) * 0.1).astype(np.float32)
        m.weights[prefix + "_v"] = rng.uniform(0.5, 2.0, chans).astype(np.float32)
        return dict(scale=prefix + "_g", bias=prefix + "_b", mean=prefix + "_m", var=prefix + "_v", epsilon=1e-5)

    for i, cin in enumerate((8, chans)):
        m.weights[f"w{i}"] = (rng.standard_normal((chans, cin, 3, 3)) * np.sqrt(2.0 / (cin * 9))).astype(np.float32)
        m.weights[f"b{i}"] = rng.uniform(-0.1, 0.1, chans).astype(np.float32)
    m.layers.append(dict(op="Conv", X="x", W="w0", B="b0", Y="c0", pads=(1, 1, 1, 1), strides=(1, 1), kernel=(3, 3)))
    m.layers.append(dict(op="BatchNormalization", X="c0", Y="n0", relu=True, **bn("bn0")))
    m.layers.append(dict(op="Conv", X="n0", W="w1", B="b1", Y="c1", pads=(1, 1, 1, 1), strides=(1, 1), kernel=(3, 3)))
    m.layers.append(dict(op="BatchNormalization", X="c1", Y="n1", **bn("bn1")))
    m.layers.append(dict(op="Add", A="n1", B="n0", Y="s"))
    m.layers.append(dict(op="LeakyRelu", X="s", Y="a", alpha=0.1))
    m.layers.append(dict(op="MaxPool", X="a", Y="p", kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0)))
    m.weights["gain"] = rng.uniform(0.5, 1.5, (chans, 1, 1)).astype(np.float32)
    m.layers.append(dict(op="Mul", A="p", B="gain", Y="g"))
    m.layers.append(dict(op="Flatten", X="g", Y="f", axis=1))
    k = chans * (hw // 2) ** 2
    m.weights["fw"] = (rng.standard_normal((10, k)) * np.sqrt(1.0 / k)).astype(np.float32)
    m.weights["fb"] = rng.uniform(-0.1, 0.1, 10).astype(np.float32)
    m.layers.append(dict(op="Gemm", A="f", B="fw", C="fb", Y="l", transB=1))
    m.layers.append(dict(op="Sigmoid", X="l", Y="y"))
    m.output_name = "y"
    m.flops_per_sample = 2 * hw * hw * chans * 9 * (8 + chans) + 2 * k * 10
    x = rng.standard_normal((batch, 8, hw, hw)).astype(np.float32) if with_input else None
    return m, x


def upsample_f32(batch=4, hw=12, key="C2", with_input=True, channels=(8, 6)):
    """Decoder-style stack: Conv 3->8 + Relu; ConvTranspose 8->6, 2x2 stride 2; Relu; ConvTranspose 6->3, 3x3 stride 2 pad 1
    output_padding 1, with bias; Tanh. Seeded like C2. `channels` widens the two hidden layers (8 and 6 by default)."""
    rng = np.random.Generator(np.random.PCG64(SEEDS[key] + 79))
    c0, c1 = channels
    m = Model(f"upsample_b{batch}" + ("" if channels == (8, 6) else f"_c{c0}_{c1}"), "x", (batch, 3, hw, hw), [])
    m.weights["w0"] = (rng.standard_normal((c0, 3, 3, 3)) * np.sqrt(2.0 / 27)).astype(np.float32)
    m.weights["b0"] = rng.uniform(-0.1, 0.1, c0).astype(np.float32)
    m.weights["t1"] = (rng.standard_normal((c0, c1, 2, 2)) * np.sqrt(2.0 / c0)).astype(np.float32)
    m.weights["t2"] = (rng.standard_normal((c1, 3, 3, 3)) * np.sqrt(2.0 / (14 if c1 == 6 else 2.25 * c1))).astype(np.float32)
    m.weights["tb2"] = rng.uniform(-0.1, 0.1, 3).astype(np.float32)
    m.layers.append(dict(op="Conv", X="x", W="w0", B="b0", Y="c0", pads=(1, 1, 1, 1), strides=(1, 1), kernel=(3, 3)))
    m.layers.append(dict(op="Relu", X="c0", Y="r0"))
    m.layers.append(dict(op="ConvTranspose", X="r0", W="t1", Y="u1", pads=(0, 0, 0, 0), strides=(2, 2), kernel=(2, 2),
                         output_padding=(0, 0)))
    m.layers.append(dict(op="Relu", X="u1", Y="r1"))
    m.layers.append(dict(op="ConvTranspose", X="r1", W="t2", B="tb2", Y="u2", pads=(1, 1, 1, 1), strides=(2, 2), kernel=(3, 3),
                         output_padding=(1, 1)))
    m.layers.append(dict(op="Tanh", X="u2", Y="y"))
    m.output_name = "y"
    m.flops_per_sample = 2 * hw * hw * (c0 * 27 + c0 * c1 * 4 + 4 * c1 * 3 * 9)
    x = rng.standard_normal((batch, 3, hw, hw)).astype(np.float32) if with_input else None
    return m, x


def volume_f32(batch=3, dhw=(6, 8, 10), key="C2", with_input=True):
    """A small 3-D network: Conv3d 2->8 (3x3x3, pad 1) + Relu; MaxPool3d 2x2x2; Conv3d 8->4 (2x3x1, stride (1,2,1), group 2) with bias."""
    rng = np.random.Generator(np.random.PCG64(SEEDS[key] + 131))
    D, H, W = dhw
    m = Model(f"volume_b{batch}", "x", (batch, 2, D, H, W), [])
    m.weights["w0"] = (rng.standard_normal((8, 2, 3, 3, 3)) * np.sqrt(2.0 / 54)).astype(np.float32)
    m.weights["b0"] = rng.uniform(-0.1, 0.1, 8).astype(np.float32)
    m.weights["w1"] = (rng.standard_normal((4, 4, 2, 3, 1)) * np.sqrt(2.0 / 24)).astype(np.float32)
    m.weights["b1"] = rng.uniform(-0.1, 0.1, 4).astype(np.float32)
    m.layers.append(dict(op="Conv", X="x", W="w0", B="b0", Y="c0", pads=(1, 1, 1, 1, 1, 1), strides=(1, 1, 1), kernel=(3, 3, 3)))
    m.layers.append(dict(op="Relu", X="c0", Y="r0"))
    m.layers.append(dict(op="MaxPool", X="r0", Y="p0", pads=(0, 0, 0, 0, 0, 0), strides=(2, 2, 2), kernel=(2, 2, 2)))
    m.layers.append(dict(op="Conv", X="p0", W="w1", B="b1", Y="y", pads=(0, 0, 0, 0, 0, 0), strides=(1, 2, 1), kernel=(2, 3, 1), group=2))
    m.output_name = "y"
    m.flops_per_sample = 2 * D * H * W * 8 * 54
    x = rng.standard_normal((batch, 2, D, H, W)).astype(np.float32) if with_input else None
    return m, x


def mlp_activations_f32(batch=64, key="C1", with_input=True):
    """Gemm 32->48 + Selu; Gemm 48->48 + Tanh; Sub of a constant row; Gemm 48->24 + Elu; Div by a constant; Sigmoid."""
    rng = np.random.Generator(np.random.PCG64(SEEDS[key] + 78))
    m = Model(f"mlp_act_b{batch}", "x", (batch, 32), [])
    dims = (32, 48, 48, 24)
    acts = ("Selu", "Tanh", "Elu")
    prev = "x"
    for i in range(3):
        k, n = dims[i], dims[i + 1]
        m.weights[f"w{i}"] = (rng.standard_normal((n, k)) * np.sqrt(1.0 / k)).astype(np.float32)
        m.weights[f"b{i}"] = rng.uniform(-0.1, 0.1, n).astype(np.float32)
        m.layers.append(dict(op="Gemm", A=prev, B=f"w{i}", C=f"b{i}", Y=f"g{i}", transB=1))
        m.layers.append(dict(op=acts[i], X=f"g{i}", Y=f"a{i}", **({"alpha": 1.0} if acts[i] == "Elu" else {})))
        prev = f"a{i}"
        if i == 1:
            m.weights["shift"] = rng.uniform(-0.5, 0.5, (n,)).astype(np.float32)
            m.layers.append(dict(op="Sub", A=prev, B="shift", Y="sh"))
            prev = "sh"
    m.weights["den"] = rng.uniform(0.5, 2.0, (24,)).astype(np.float32)
    m.layers.append(dict(op="Div", A=prev, B="den", Y="d"))
    m.layers.append(dict(op="Sigmoid", X="d", Y="y"))
    m.output_name = "y"
    m.flops_per_sample = 2 * sum(dims[i] * dims[i + 1] for i in range(3))
    x = rng.standard_normal((batch, 32)).astype(np.float32) if with_input else None
    return m, x


# ------------------------------------------------------------------------------------ C5
# Fixed activation scales of the calorimeter CNN: input energies are clipped at 8 (scale 8/255);
# the scales after each layer were chosen once so that the seeded activations use the uint8 range.
CALO_SCALES = dict(x=8.0 / 255.0, c0=0.01, c1=0.063, c2=0.56, c3=6.4, f0=100.0, f1=800.0)


def cnn_i8(batch=16384, key="C5", hw=64, chans=(1, 32, 64, 64, 128), hidden=256, classes=2, with_input=True):
    """int8 calorimeter-image CNN: QuantizeLinear; 4 x (QLinearConv 3x3 pad 1 + Relu + MaxPool 2x2);
    Flatten; QLinearMatMul 2048->256 (+Relu) -> 2; DequantizeLinear. Input energies Exp(1) with 95%
    of the cells zeroed. uint8 activations with zero point 0, int8 weights U{-127..127}, per-output-
    channel weight scales U(0.001, 0.01)."""
    rng = _rng(key)
    m = Model(f"cnn_i8_b{batch}", "x", (batch, chans[0], hw, hw), [])
    sc = CALO_SCALES
    m.layers.append(dict(op="QuantizeLinear", X="x", Y="q", scale=sc["x"], zp=0))
    prev, prev_scale, h = "q", sc["x"], hw
    for i in range(4):
        cin, cout = chans[i], chans[i + 1]
        m.weights[f"cw{i}"] = rng.integers(-127, 128, size=(cout, cin, 3, 3), dtype=np.int64).astype(np.int8)
        m.weights[f"cs{i}"] = rng.uniform(0.001, 0.01, size=(cout,)).astype(np.float32)
        m.layers.append(dict(op="QLinearConv", X=prev, W=f"cw{i}", Y=f"c{i}", x_scale=prev_scale, x_zp=0,
                             w_scale=f"cs{i}", y_scale=sc[f"c{i}"], y_zp=0, pads=(1, 1, 1, 1), strides=(1, 1),
                             kernel=(3, 3), relu=True))
        m.layers.append(dict(op="MaxPool", X=f"c{i}", Y=f"p{i}", kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0)))
        m.flops_per_sample += 2 * h * h * cout * cin * 9
        prev, prev_scale, h = f"p{i}", sc[f"c{i}"], h // 2
    feat = chans[4] * h * h
    m.layers.append(dict(op="Flatten", X=prev, Y="flat", axis=1))
    dims = (feat, hidden, classes)
    prev = "flat"
    for i in range(2):
        k, n = dims[i], dims[i + 1]
        m.weights[f"fw{i}"] = rng.integers(-127, 128, size=(k, n), dtype=np.int64).astype(np.int8)
        m.weights[f"fs{i}"] = rng.uniform(0.001, 0.01, size=(n,)).astype(np.float32)
        # the last layer's zero point is 128 so that both signs of the two logits survive
        y_zp = 0 if i == 0 else 128
        m.layers.append(dict(op="QLinearMatMul", A=prev, B=f"fw{i}", Y=f"f{i}", a_scale=prev_scale, a_zp=0,
                             w_scale=f"fs{i}", y_scale=sc[f"f{i}"], y_zp=y_zp, relu=i == 0))
        m.flops_per_sample += 2 * k * n
        prev, prev_scale = f"f{i}", sc[f"f{i}"]
    m.layers.append(dict(op="DequantizeLinear", X=prev, Y="y", scale=prev_scale, zp=128))
    m.output_name = "y"
    x = None
    if with_input:
        x = calo_input(rng, batch, chans[0], hw)
    return m, x


def calo_input(rng, batch, chans, hw):
    """Exp(1) energies with 95 % of the cells zeroed, drawn in chunks to bound host memory."""
    x = np.empty((batch, chans, hw, hw), np.float32)
    step = 1024
    for b0 in range(0, batch, step):
        b1 = min(batch, b0 + step)
        e = rng.exponential(1.0, size=(b1 - b0, chans, hw, hw)).astype(np.float32)
        keep = rng.random(size=e.shape) < 0.05
        x[b0:b1] = e * keep
    return x


BUILDERS = {"C1": mlp_f32, "C2": cnn_f32, "C3": mlp_i8, "C4": gemm_chain_fp8, "C5": cnn_i8}
