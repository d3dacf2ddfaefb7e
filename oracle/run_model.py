"""Evaluate a sofie_b200.configs.Model on the CPU with the oracle, operator by operator, in the
reference's layouts (row-major, NCHW). TEST INFRASTRUCTURE ONLY: used by tests, the smoke check and
the benchmark's CPU-baseline leg."""
from __future__ import annotations

import numpy as np

from . import cpu_oracle as o


def calibrate_fp8_scales(model, x):
    """Static FP8 activation scales; the model-build step of the product computes them the same way."""
    from sofie_b200 import configs
    return configs.calibrate_fp8_scales(model, x)


def run(model, x, fp8_scales=None, return_all=False):
    t = {model.input_name: np.asarray(x)}
    w = model.weights
    fp8_i = 0
    for L in model.layers:
        op = L["op"]
        if op == "Gemm":
            t[L["Y"]] = o.gemm_f32(t[L["A"]], w[L["B"]], w.get(L.get("C")), transB=L.get("transB", 0),
                                   alpha=L.get("alpha", 1.0), beta=L.get("beta", 1.0), relu=L.get("relu", False))
        elif op == "Conv" and len(L["kernel"]) == 3:
            p = L["pads"]
            t[L["Y"]] = o.conv3d_f32(t[L["X"]], w[L["W"]], w.get(L.get("B")), pad=(p[0], p[1], p[2]), stride=L["strides"],
                                     dil=L.get("dilations", (1, 1, 1)), group=L.get("group", 1))
        elif op == "Conv":
            p, s = L["pads"], L["strides"]
            t[L["Y"]] = o.conv2d_f32(t[L["X"]], w[L["W"]], w.get(L.get("B")), pad=(p[0], p[1]), stride=s,
                                     group=L.get("group", 1))
        elif op == "ConvTranspose":
            p, s = L["pads"], L["strides"]
            t[L["Y"]] = o.conv_transpose2d_f32(t[L["X"]], w[L["W"]], w.get(L.get("B")), pad=(p[0], p[1]), stride=s,
                                               out_pad=L.get("output_padding", (0, 0)))
        elif op == "Relu":
            t[L["Y"]] = o.relu_f32(t[L["X"]])
        elif op == "MaxPool":
            X = t[L["X"]]
            if X.ndim == 5:
                t[L["Y"]] = o.pool3d_f32(X, 0, L["kernel"], L["strides"], L["pads"])
            elif X.dtype == np.uint8:
                t[L["Y"]] = o.maxpool2d_u8(X, L["kernel"], L["strides"])
            else:
                t[L["Y"]] = o.pool2d_f32(X, 0, L["kernel"], L["strides"], L["pads"])
        elif op == "Flatten":
            X = t[L["X"]]
            t[L["Y"]] = X.reshape(X.shape[0], -1)
        elif op == "Softmax":
            t[L["Y"]] = o.softmax_f32(t[L["X"]], L.get("axis", -1))
        elif op in o.UNARY_OPS:
            t[L["Y"]] = o.unary_f32(t[L["X"]], op, L.get("alpha", 0.01 if op == "LeakyRelu" else 1.0))
        elif op in o.BINARY_OPS:
            a = w[L["A"]] if L["A"] in w else t[L["A"]]
            b = w[L["B"]] if L["B"] in w else t[L["B"]]
            t[L["Y"]] = o.binary_f32(a, b, op)
        elif op == "BatchNormalization":
            t[L["Y"]] = o.batchnorm_f32(t[L["X"]], w[L["scale"]], w[L["bias"]], w[L["mean"]], w[L["var"]], L.get("epsilon", 1e-5),
                                        bool(L.get("relu")))
        elif op == "QuantizeLinear":
            t[L["Y"]] = o.quantize_u8(t[L["X"]], L["scale"], L["zp"])
        elif op == "DequantizeLinear":
            t[L["Y"]] = o.dequantize_u8(t[L["X"]], L["scale"], L["zp"])
        elif op == "QLinearMatMul":
            t[L["Y"]] = o.qlinear_matmul(t[L["A"]], L["a_scale"], L["a_zp"], w[L["B"]], w[L["w_scale"]], L["y_scale"],
                                         L["y_zp"], w_is_nk=False, relu=L.get("relu", False))
        elif op == "QLinearConv":
            p, s = L["pads"], L["strides"]
            t[L["Y"]] = o.qlinear_conv2d(t[L["X"]], L["x_scale"], L["x_zp"], w[L["W"]], w[L["w_scale"]], L["y_scale"],
                                         L["y_zp"], pad=(p[0], p[1]), stride=s, relu=L.get("relu", False))
        elif op == "Fp8Gemm":
            A = t[L["A"]]
            if isinstance(fp8_scales, str) and fp8_scales == "dynamic":
                # scale computed from the tensor itself: max|x| / 448 in float32, 1 for an all-zero tensor
                amax = np.float32(np.abs(np.asarray(A, np.float32)).max()) if A.size else np.float32(0)
                a_scale = float(amax / np.float32(448.0)) if amax > 0 else 1.0
            else:
                a_scale = fp8_scales[fp8_i]
            fp8_i += 1
            Aq = o.quantize_e4m3(A, a_scale)
            Wq = o.quantize_e4m3(w[L["B"]], L["w_scale"])
            bits = o.gemm_e4m3(Aq, a_scale, Wq, L["w_scale"], w.get(L.get("C")), relu=L["relu"])
            t[L["Y"]] = o.bf16_bits_to_f32(bits)  # bf16 values held as fp32
        else:
            raise ValueError(f"oracle has no operator {op}")
    return t if return_all else t[model.output_name]
