"""Test infrastructure: a Python mirror of the emitted Session for models described by sofie_b200.configs.Model.

It does what the generated C++ Session does -- plan once (operator fusion, NHWC layout between
convolutions, weight repacking, requantisation tables), upload weights once, then run infer() as
a fixed sequence of libSOFIE_cuda calls -- but drives the C ABI from Python, so that tests can reach
the intermediate tensors of a model and force layouts the generator would not choose. The product's
planner is the C++ generator (sofie_b200/host); nothing outside tests/ imports this file.
torch supplies device memory, streams and graph capture only.

Reference behaviour mirrored: Session construction loads weights, infer(float*) returns a new
vector (src/SOFIE_core/src/RModel.cxx:744-910).
"""
from __future__ import annotations

import numpy as np
import torch

from sofie_b200 import capi, ops
from sofie_b200.capi import LAYOUT_NCHW, LAYOUT_NHWC

# Largest batch that goes to the fused MLP kernel: it computes with fp32 FMA out of shared memory, which beats one
# tensor-core GEMM launch per layer only while those launches are latency bound (measured cross-over between 2048
# and 4096 rows for 64-128-128-10).
MLP_FUSED_MAX_ROWS = 2048


class Step:
    """One fused launch: a callable taking the tensor table."""

    def __init__(self, name, fn, flops=0):
        self.name, self.fn, self.flops = name, fn, flops


class Session:
    def __init__(self, model, device=0, fp8_scales=None, use_graph=True, nhwc=True):
        if not torch.cuda.is_available():
            raise RuntimeError("the mirror Session needs a CUDA device: there is no CPU path")
        self.model = model
        self.dev = torch.device("cuda", device)
        self.use_graph = use_graph
        self.nhwc = nhwc
        self.fp8_scales = fp8_scales
        self.w = {}
        self.steps: list[Step] = []
        self.layout = {model.input_name: LAYOUT_NCHW}
        self.shape = {model.input_name: tuple(model.input_shape)}  # logical (NCHW / row-major) shapes
        self.graph = None
        self.static_in = None
        self.static_out = None
        self.out_dtype = torch.float32
        with torch.cuda.device(self.dev):
            self._plan()
        self.launches_per_infer = len(self.steps)

    # ------------------------------------------------------------------ planning
    def _up(self, arr):
        return torch.from_numpy(np.ascontiguousarray(arr)).to(self.dev)

    def _consumers(self, name):
        return [L for L in self.model.layers if name in (L.get("X"), L.get("A"), L.get("B") if L["op"] in ops.BINARY_OPS else None)]

    def _plan(self):
        layers = self.model.layers
        mw = self.model.weights
        i = 0
        fp8_i = 0
        while i < len(layers):
            L = layers[i]
            op = L["op"]
            if op == "Gemm":
                chain = self._mlp_chain(i)
                if len(chain) >= 2:
                    self._plan_mlp(chain)
                    i += len(chain)
                else:
                    self._plan_gemm(L)
                    i += 1
            elif op in ("Conv", "QLinearConv"):
                # fuse Conv [+ Relu] [+ MaxPool 2x2 stride 2 no pad] when each intermediate has one consumer
                j, relu, pool, out = i + 1, bool(L.get("relu", False)), 0, L["Y"]
                bn = None
                if op == "Conv" and j < len(layers) and layers[j]["op"] == "BatchNormalization" and layers[j]["X"] == out and \
                        len(self._consumers(out)) == 1:
                    # inference BatchNormalization behind a convolution: folded into its weights and bias
                    bn, out, j = layers[j], layers[j]["Y"], j + 1
                    relu = bool(bn.get("relu", False))
                if op == "Conv" and not relu and j < len(layers) and layers[j]["op"] == "Relu" and layers[j]["X"] == out and \
                        len(self._consumers(out)) == 1:
                    relu, out, j = True, layers[j]["Y"], j + 1
                if j < len(layers) and layers[j]["op"] == "MaxPool" and layers[j]["X"] == out and \
                        len(self._consumers(out)) == 1 and tuple(layers[j]["kernel"]) == (2, 2) and \
                        tuple(layers[j]["strides"]) == (2, 2) and not any(layers[j]["pads"]):
                    pool, out, j = 2, layers[j]["Y"], j + 1
                self._plan_conv(L, relu, pool, out, quant=(op == "QLinearConv"), bn=bn)
                i = j
            elif op == "Relu":
                x, y = L["X"], L["Y"]
                self.layout[y], self.shape[y] = self.layout[x], self.shape[x]
                self.steps.append(Step(f"relu:{y}", lambda t, x=x, y=y: t.__setitem__(y, ops.relu_f32(t[x]))))
                i += 1
            elif op == "MaxPool":
                self._plan_pool(L)
                i += 1
            elif op == "ConvTranspose":
                self._plan_conv_transpose(L)
                i += 1
            elif op == "Flatten":
                x, y = L["X"], L["Y"]
                # a flattened NHWC tensor keeps its memory; consumers permute their weights instead
                self.layout[y], self.shape[y] = self.layout[x], self.shape[x]
                self.steps.append(Step(f"alias:{y}", lambda t, x=x, y=y: t.__setitem__(y, t[x].reshape(t[x].shape[0], -1))))
                self.steps[-1].is_alias = True
                i += 1
            elif op == "Softmax":
                x, y, ax = L["X"], L["Y"], L.get("axis", -1)
                self.layout[y], self.shape[y] = self.layout[x], self.shape[x]
                self.steps.append(Step(f"softmax:{y}", lambda t, x=x, y=y, ax=ax: t.__setitem__(y, ops.softmax_f32(t[x], ax))))
                i += 1
            elif op in ops.UNARY_OPS:
                x, y = L["X"], L["Y"]
                alpha = L.get("alpha", {"LeakyRelu": 0.01, "Elu": 1.0}.get(op, 0.0))
                self.layout[y], self.shape[y] = self.layout[x], self.shape[x]
                self.steps.append(Step(f"{op.lower()}:{y}", lambda t, x=x, y=y, op=op, alpha=alpha: t.__setitem__(y, ops.unary_f32(t[x], op, alpha))))
                i += 1
            elif op in ops.BINARY_OPS:
                self._plan_binary(L)
                i += 1
            elif op == "BatchNormalization":
                self._plan_batchnorm(L)
                i += 1
            elif op == "QuantizeLinear":
                self._plan_quantize(L)
                i += 1
            elif op == "DequantizeLinear":
                x, y, s, zp = L["X"], L["Y"], L["scale"], L["zp"]
                self.layout[y], self.shape[y] = self.layout[x], self.shape[x]
                self.steps.append(Step(f"dequant:{y}", lambda t, x=x, y=y, s=s, zp=zp: t.__setitem__(y, ops.dequantize_u8(t[x], s, zp))))
                i += 1
            elif op == "QLinearMatMul":
                # a DequantizeLinear with the product's zero point as the only reader: the product writes the floats
                dq = layers[i + 1] if i + 1 < len(layers) else None
                if dq is not None and dq["op"] == "DequantizeLinear" and dq["X"] == L["Y"] and dq["zp"] == L["y_zp"] and \
                        L["Y"] != self.model.output_name and len(self._consumers(L["Y"])) == 1:
                    self._plan_qmatmul(L, dequant=dq)
                    i += 2
                else:
                    self._plan_qmatmul(L)
                    i += 1
            elif op == "Fp8Gemm":
                nxt = layers[i + 1] if i + 1 < len(layers) and layers[i + 1]["op"] == "Fp8Gemm" else None
                self._plan_fp8(L, fp8_i, first=(fp8_i == 0), nxt=nxt)
                fp8_i += 1
                i += 1
            else:
                raise NotImplementedError(f"operator {op} is outside the dense-contraction path")
        del mw

    def _nhwc_ok(self, name, depth=0):
        if name == self.model.output_name or depth > 8:
            return False
        cons = self._consumers(name)
        if not cons:
            return False
        for L in cons:
            op = L["op"]
            if op in ("Conv", "QLinearConv"):
                if L.get("group", 1) != 1:
                    return False
            elif op in ("Relu", "MaxPool", "BatchNormalization") or op in ops.UNARY_OPS:
                if not self._nhwc_ok(L["Y"], depth + 1):
                    return False
            elif op == "Flatten":
                nxt = self._consumers(L["Y"])
                if L["Y"] == self.model.output_name or not nxt or \
                        any(n["op"] not in ("Gemm", "QLinearMatMul") for n in nxt):
                    return False
            else:
                return False
        return True

    def _flatten_perm(self, src_name, K):
        """Column permutation that maps a weight's K axis from (c,h,w) order to the (h,w,c) order of an
        NHWC activation, or None when the activation is not NHWC / not 4-D."""
        shp = self.shape.get(src_name)
        if self.layout.get(src_name) != LAYOUT_NHWC or shp is None or len(shp) != 4:
            return None
        _, c, h, w = shp
        assert c * h * w == K
        return np.arange(K).reshape(c, h, w).transpose(1, 2, 0).reshape(-1)

    def _mlp_chain(self, i):
        """Consecutive Gemm layers starting at layer i that the fused MLP kernel takes in one launch: each feeds only
        the next, plain x W^T + b (alpha = beta = 1 or no bias), widths <= 256, weights within shared memory, and a
        batch of at most MLP_FUSED_MAX_ROWS rows."""
        layers, mw = self.model.layers, self.model.weights
        chain, dims = [], []
        j = i
        while j < len(layers) and len(chain) < capi.MLP_MAX_LAYERS:
            L = layers[j]
            if L["op"] != "Gemm" or L.get("alpha", 1.0) != 1.0 or (L.get("C") and L.get("beta", 1.0) != 1.0):
                break
            if chain and L["A"] != chain[-1]["Y"]:
                break
            W = mw[L["B"]]
            N, K = (W.shape if L.get("transB", 0) else W.shape[::-1])
            if not chain:
                shp = self.shape.get(L["A"])
                if shp is None or len(shp) != 2 or shp[0] > MLP_FUSED_MAX_ROWS or self._flatten_perm(L["A"], K) is not None:
                    break
                dims = [K]
            if (L.get("C") and mw[L["C"]].shape != (N,)) or not ops.mlp_fits(dims + [N]):
                break
            dims.append(N)
            chain.append(L)
            if L["Y"] == self.model.output_name or len(self._consumers(L["Y"])) != 1:
                break
            j += 1
        return chain

    def _plan_mlp(self, chain):
        mw = self.model.weights
        names = []
        for L in chain:
            self.w[L["B"]] = self._up(mw[L["B"]])  # kept in the model's own layout; the kernel transposes while staging
            if L.get("C"):
                self.w[L["C"]] = self._up(mw[L["C"]])
            names.append((L["B"], L.get("C")))
        relu = [bool(L.get("relu", False)) for L in chain]
        nk = [bool(L.get("transB", 0)) for L in chain]
        a, y = chain[0]["A"], chain[-1]["Y"]
        N_out = mw[chain[-1]["B"]].shape[0 if nk[-1] else 1]
        self.layout[y], self.shape[y] = LAYOUT_NCHW, (self.shape[a][0], N_out)
        flops = sum(2 * int(np.prod(mw[L["B"]].shape)) for L in chain)

        def run(t):
            t[y] = ops.mlp_f32(t[a], [self.w[b] for b, _ in names], [self.w[c] if c else None for _, c in names], relu, nk)
        self.steps.append(Step(f"mlp:{y}", run, flops=flops))

    def _plan_gemm(self, L):
        mw = self.model.weights
        a, b, c, y = L["A"], L["B"], L.get("C"), L["Y"]
        transB = L.get("transB", 0)
        W = mw[b]
        Wnk = W if transB else W.T  # [N,K]
        perm = self._flatten_perm(a, Wnk.shape[1])
        if perm is not None:
            Wnk = Wnk[:, perm]
        self.w[b] = self._up(Wnk)
        if c:
            self.w[c] = self._up(mw[c])
        alpha, beta, relu = L.get("alpha", 1.0), L.get("beta", 1.0), L.get("relu", False)
        N, K = Wnk.shape
        self.layout[y], self.shape[y] = LAYOUT_NCHW, (self.shape[a][0], N)

        def run(t, a=a, b=b, c=c, y=y):
            A = t[a].reshape(t[a].shape[0], -1)
            t[y] = ops.gemm_f32(A, self.w[b], self.w[c] if c else None, transB=1, alpha=alpha, beta=beta, relu=relu)
        self.steps.append(Step(f"gemm:{y}", run, flops=2 * N * K))

    def _plan_conv(self, L, relu, pool, out, quant, bn=None):
        mw = self.model.weights
        x, wname, bname = L["X"], L["W"], L.get("B")
        W = mw[wname]
        Cout, Cg, kH, kW = W.shape
        group = L.get("group", 1)
        N, C, H, Wd = self.shape[x]
        pads, strides = L["pads"], L["strides"]
        assert pads[0] == pads[2] and pads[1] == pads[3], "asymmetric pads are outside the reference's support"
        oH, oW = ops.conv_out_hw(H, Wd, kH, kW, (pads[0], pads[1]), strides)
        if pool == 2:
            oH, oW = oH // 2, oW // 2
        # NHWC output when the result stays inside the runner: every consumer is a convolution, a
        # pool, a Relu or a Flatten feeding a matmul (whose weight is permuted instead); model
        # outputs keep the reference's NCHW order
        y_layout = LAYOUT_NHWC if (self.nhwc and group == 1 and self._nhwc_ok(out)) else LAYOUT_NCHW
        x_layout = self.layout[x]
        packed = x_layout == LAYOUT_NHWC and group == 1
        self.layout[out], self.shape[out] = y_layout, (N, Cout, oH, oW)
        flops = 2 * self.shape[out][2] * self.shape[out][3] * (4 if pool == 2 else 1) * Cout * Cg * kH * kW
        if quant:
            self.w[wname] = ops.qconv2d_pack_i8(self._up(W)) if packed else self._up(W)
            mult, corr = ops.qlinear_prepare(W.reshape(Cout, -1), True, L["x_scale"], 0, mw[L["w_scale"]], L["y_scale"],
                                             mw.get(bname) if bname else None, self.dev)
            self.w[wname + ":mult"], self.w[wname + ":bias"] = mult, (corr if bname else None)
            x_zp, y_zp = L["x_zp"], L["y_zp"]

            def run(t):
                t[out] = ops.qlinear_conv2d(t[x], self.w[wname], self.w[wname + ":mult"], self.w[wname + ":bias"],
                                            shape=(t[x].shape[0], C, H, Wd), pad=(pads[0], pads[1]), stride=strides,
                                            x_zp=x_zp, y_zp=y_zp, relu=relu, pool=pool, x_layout=x_layout,
                                            y_layout=y_layout, w_packed=packed, kernel=(kH, kW))
        else:
            Bv = mw[bname] if bname else None
            if bn is not None:
                # w' = w * s, b' = (b - mean) * s + beta with s = gamma * float(1 / sqrt(var + eps))
                v = (mw[bn["var"]].astype(np.float32) + np.float32(bn.get("epsilon", 1e-5))).astype(np.float32)
                s_ = (mw[bn["scale"]].astype(np.float32) * (1.0 / np.sqrt(v.astype(np.float64))).astype(np.float32)).astype(np.float32)
                W = (W * s_[:, None, None, None]).astype(np.float32)
                b0 = Bv.astype(np.float32) if Bv is not None else np.zeros(Cout, np.float32)
                Bv = ((b0 - mw[bn["mean"]].astype(np.float32)) * s_ + mw[bn["bias"]].astype(np.float32)).astype(np.float32)
                wname, bname = f"{wname}:bn:{out}", f"{out}:bnbias"
            self.w[wname] = ops.conv2d_pack_f32(self._up(W)) if packed else self._up(W)
            if bname:
                self.w[bname] = self._up(Bv)

            def run(t):
                t[out] = ops.conv2d_f32(t[x], self.w[wname], self.w[bname] if bname else None,
                                        shape=(t[x].shape[0], C, H, Wd), pad=(pads[0], pads[1]), stride=strides,
                                        group=group, relu=relu, pool=pool, x_layout=x_layout, y_layout=y_layout,
                                        w_packed=packed, kernel=(kH, kW))
        self.steps.append(Step(f"conv:{out}", run, flops=flops))

    def _plan_binary(self, L):
        """Add / Sub / Mul / Div with numpy-style broadcasting; an operand may be a constant of the model."""
        a, b, y, op = L["A"], L["B"], L["Y"], L["op"]
        mw = self.model.weights

        def operand(name):
            if name in mw:
                self.w[name] = self._up(np.ascontiguousarray(mw[name], np.float32))
                return tuple(mw[name].shape), True
            if self.layout.get(name, LAYOUT_NCHW) != LAYOUT_NCHW:
                raise ValueError(f"{op}: operand {name} must be NCHW")
            return tuple(self.shape[name]), False

        (sa, ca), (sb, cb) = operand(a), operand(b)
        out = tuple(np.broadcast_shapes(sa, sb))
        self.layout[y], self.shape[y] = LAYOUT_NCHW, out

        def run(t):
            A = self.w[a] if ca else t[a]
            B = self.w[b] if cb else t[b]
            # the batch dimension of an activation follows the batch actually given to infer()
            t[y] = ops.binary_f32(A, B, op)
        self.steps.append(Step(f"{op.lower()}:{y}", run))

    def _plan_batchnorm(self, L):
        """Inference BatchNormalization; gamma / sqrt(var + eps) is folded on the host with the roundings
        of the reference's Initialize (float sum, double reciprocal square root, float product)."""
        x, y = L["X"], L["Y"]
        mw = self.model.weights
        eps = np.float32(L.get("epsilon", 1e-5))
        v = (mw[L["var"]].astype(np.float32) + eps).astype(np.float32)
        inv = (1.0 / np.sqrt(v.astype(np.float64))).astype(np.float32)
        key = f"bn:{y}"
        self.w[key + ":scale"] = self._up((mw[L["scale"]].astype(np.float32) * inv).astype(np.float32))
        self.w[key + ":bias"] = self._up(mw[L["bias"]].astype(np.float32))
        self.w[key + ":mean"] = self._up(mw[L["mean"]].astype(np.float32))
        shp = self.shape[x]
        Cc = shp[1]
        HW = int(np.prod(shp[2:], dtype=np.int64)) if len(shp) > 2 else 1
        layout = self.layout[x]
        relu = bool(L.get("relu", False))
        self.layout[y], self.shape[y] = layout, shp

        def run(t):
            t[y] = ops.batchnorm_f32(t[x], self.w[key + ":scale"], self.w[key + ":bias"], self.w[key + ":mean"],
                                     t[x].shape[0], Cc, HW, layout=layout, relu=relu)
        self.steps.append(Step(f"batchnorm:{y}", run))

    def _plan_pool(self, L):
        x, y = L["X"], L["Y"]
        N, C, H, Wd = self.shape[x]
        k, s, p = L["kernel"], L["strides"], L["pads"]
        lay = self.layout[x]
        oH = -(-(H + p[0] + p[2] - k[0] + 1) // s[0])
        oW = -(-(Wd + p[1] + p[3] - k[1] + 1) // s[1])
        self.layout[y], self.shape[y] = lay, (N, C, oH, oW)

        def run(t):
            X = t[x]
            shp = (X.shape[0], C, H, Wd)
            if X.dtype == torch.uint8:
                t[y] = ops.maxpool2d_u8(X, kernel=k, stride=s, layout=lay, shape=shp)
            else:
                t[y] = ops.pool2d_f32(X, mode=0, kernel=k, stride=s, pads=p, layout=lay, shape=shp)
        self.steps.append(Step(f"maxpool:{y}", run))

    def _plan_conv_transpose(self, L):
        mw = self.model.weights
        x, y, wn, bn = L["X"], L["Y"], L["W"], L.get("B")
        N, C, H, Wd = self.shape[x]
        W = mw[wn]
        p, s, op_ = L["pads"], L["strides"], L.get("output_padding", (0, 0))
        if L.get("group", 1) != 1 or p[0] != p[2] or p[1] != p[3]:
            raise NotImplementedError("ConvTranspose: group 1 and symmetric pads only")
        self.w[wn] = self._up(W)
        if bn:
            self.w[bn] = self._up(mw[bn])
        oH = s[0] * (H - 1) + W.shape[2] + op_[0] - 2 * p[0]
        oW = s[1] * (Wd - 1) + W.shape[3] + op_[1] - 2 * p[1]
        self.layout[y], self.shape[y] = LAYOUT_NCHW, (N, W.shape[1], oH, oW)

        def run(t):
            t[y] = ops.conv_transpose2d_f32(t[x], self.w[wn], self.w[bn] if bn else None, pad=(p[0], p[1]), stride=tuple(s),
                                            out_pad=tuple(op_))
        self.steps.append(Step(f"convtr:{y}", run, flops=2 * H * Wd * C * int(np.prod(W.shape[1:]))))

    def _plan_quantize(self, L):
        x, y, s, zp = L["X"], L["Y"], L["scale"], L["zp"]
        self.layout[y], self.shape[y] = self.layout[x], self.shape[x]
        self.steps.append(Step(f"quant:{y}", lambda t: t.__setitem__(y, ops.quantize_u8(t[x], s, zp))))

    def _plan_qmatmul(self, L, dequant=None):
        mw = self.model.weights
        a, b, y = L["A"], L["B"], L["Y"]
        Wkn = mw[b]  # ONNX order [K,N]
        Wnk = np.ascontiguousarray(Wkn.T)
        perm = self._flatten_perm(a, Wnk.shape[1])
        if perm is not None:
            Wnk = np.ascontiguousarray(Wnk[:, perm])
        N, K = Wnk.shape
        self.w[b] = self._up(Wnk)
        mult, corr = ops.qlinear_prepare(Wnk, True, L["a_scale"], L["a_zp"], mw[L["w_scale"]], L["y_scale"], None, self.dev)
        self.w[b + ":mult"], self.w[b + ":corr"] = mult, corr
        y_zp, relu = L["y_zp"], L.get("relu", False)
        self.layout[y], self.shape[y] = LAYOUT_NCHW, (self.shape[a][0], N)

        if dequant is not None:
            yf, dq_scale = dequant["Y"], dequant["scale"]
            self.layout[yf], self.shape[yf] = LAYOUT_NCHW, (self.shape[a][0], N)

            def run_f32(t):
                A = t[a].reshape(t[a].shape[0], -1)
                t[yf] = ops.qlinear_matmul_f32(A, self.w[b], self.w[b + ":mult"], self.w[b + ":corr"], dq_scale, w_is_nk=True,
                                               y_zp=y_zp, relu=relu)
            self.steps.append(Step(f"qmatmul:{yf}", run_f32, flops=2 * N * K))
            return

        def run(t):
            A = t[a].reshape(t[a].shape[0], -1)
            t[y] = ops.qlinear_matmul(A, self.w[b], self.w[b + ":mult"], self.w[b + ":corr"], w_is_nk=True, y_zp=y_zp,
                                      relu=relu)
        self.steps.append(Step(f"qmatmul:{y}", run, flops=2 * N * K))

    def _plan_fp8(self, L, idx, first, nxt):
        if self.fp8_scales is None:
            raise ValueError("the FP8 chain needs calibrated activation scales (fp8_scales)")
        mw = self.model.weights
        a, b, c, y = L["A"], L["B"], L.get("C"), L["Y"]
        W = mw[b]
        N, K = W.shape
        self.w[b] = ops.quantize_e4m3(self._up(W), L["w_scale"])
        if c:
            self.w[c] = self._up(mw[c])
        a_scale, w_scale, relu = self.fp8_scales[idx], L["w_scale"], L["relu"]
        q_scale = self.fp8_scales[idx + 1] if nxt is not None else 0.0
        self.layout[y], self.shape[y] = LAYOUT_NCHW, (self.shape[a][0], N)
        if first:
            self.steps.append(Step(f"quant_e4m3:{a}", lambda t: t.__setitem__(a + ":q", ops.quantize_e4m3(t[a], a_scale))))

        if nxt is None:
            # last layer of the chain: bf16 result widened to float in the GEMM's own epilogue (Fp8Gemm + Cast)
            def run_last(t):
                t[y] = ops.gemm_e4m3_f32(t[a + ":q"], self.w[b], self.w[c] if c else None, a_scale=a_scale, w_scale=w_scale, relu=relu)
            self.steps.append(Step(f"fp8gemm:{y}", run_last, flops=2 * N * K))
            return

        def run(t):
            _, Yq = ops.gemm_e4m3(t[a + ":q"], self.w[b], self.w[c] if c else None, a_scale=a_scale, w_scale=w_scale,
                                  relu=relu, q_scale=q_scale, want_bf16=False)
            t[y + ":q"] = Yq
        self.steps.append(Step(f"fp8gemm:{y}", run, flops=2 * N * K))

    # ------------------------------------------------------------------ execution
    def _run_steps(self, x_dev):
        t = {self.model.input_name: x_dev}
        for s in self.steps:
            s.fn(t)
        return t

    def kernel_launches(self):
        return sum(1 for s in self.steps if not getattr(s, "is_alias", False))

    def infer_device(self, x_dev, return_all=False):
        """Run on an input already resident on the device; returns device tensor(s). No graph."""
        with torch.cuda.device(self.dev):
            t = self._run_steps(x_dev)
        return t if return_all else t[self.model.output_name]

    def capture(self, x_dev):
        """Capture the infer() kernel sequence for this input shape into a CUDA graph."""
        with torch.cuda.device(self.dev):
            self.static_in = x_dev.clone()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):  # warm-up outside capture: attribute setup, allocator
                    self._run_steps(self.static_in)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.static_out = self._run_steps(self.static_in)[self.model.output_name]
        return self.graph

    def replay(self):
        self.graph.replay()
        return self.static_out

    def infer(self, x_host: np.ndarray) -> np.ndarray:
        """End to end, as the emitted Session::infer: host input -> device, kernels, host output."""
        with torch.cuda.device(self.dev):
            xh = torch.from_numpy(np.ascontiguousarray(x_host))
            if self.use_graph:
                if self.graph is None or tuple(self.static_in.shape) != tuple(xh.shape):
                    self.capture(xh.to(self.dev))
                self.static_in.copy_(xh, non_blocking=True)
                self.graph.replay()
                return self.static_out.cpu().numpy()
            return self._run_steps(xh.to(self.dev))[self.model.output_name].cpu().numpy()

    def output_to_nchw(self, name, tensor):
        """Bring an intermediate tensor to the reference's NCHW order for comparisons."""
        if self.layout.get(name) == LAYOUT_NHWC and tensor.dim() == 4:
            return tensor.permute(0, 3, 1, 2).contiguous()
        return tensor
