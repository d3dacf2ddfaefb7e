"""Operator-level calls into libSOFIE_cuda on torch CUDA tensors.

torch is used for device memory and streams only; every computation below is one call through
the C ABI (include/sofie_cuda.h). Names follow the ONNX / SOFIE operators they implement
(reference: src/SOFIE_core/inc/SOFIE/ROperator_{Gemm,Conv,Relu,Pool,Softmax}.hxx).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import capi
from .capi import LAYOUT_NCHW, LAYOUT_NHWC


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t) -> C.c_void_p:
    if t is None:
        return C.c_void_p(0)
    assert t.is_cuda and t.is_contiguous(), "tensors passed to libSOFIE_cuda must be contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


def set_engine(engine: int) -> None:
    capi.call("sofie_cuda_set_engine", engine)


def last_engine() -> int:
    return capi.load().sofie_cuda_last_engine()


def gemm_f32(A, B, C_=None, *, transA=0, transB=0, alpha=1.0, beta=1.0, relu=False, out=None):
    """ONNX Gemm / MatMul: Y = alpha*op(A)*op(B) + beta*broadcast(C), optional Relu."""
    M = A.shape[1] if transA else A.shape[0]
    K = A.shape[0] if transA else A.shape[1]
    N = B.shape[0] if transB else B.shape[1]
    assert (B.shape[1] if transB else B.shape[0]) == K
    bias_kind = 0
    if C_ is not None:
        bias_kind = 1 if C_.numel() == N else 2
        assert C_.numel() in (N, M * N)
    Y = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=A.device)
    d = capi.GemmF32Desc(M, N, K, int(transA), int(transB), float(alpha), float(beta), bias_kind, int(relu))
    capi.call("sofie_cuda_gemm_f32", _stream(), C.byref(d), _p(A), _p(B), _p(C_), _p(Y))
    return Y


def conv_out_hw(H, W, kH, kW, pad, stride, dil=(1, 1)):
    oH = (H + 2 * pad[0] - (dil[0] * (kH - 1) + 1)) // stride[0] + 1
    oW = (W + 2 * pad[1] - (dil[1] * (kW - 1) + 1)) // stride[1] + 1
    return oH, oW


def conv2d_f32(X, W, bias=None, *, shape=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), group=1, relu=False, pool=0,
               x_layout=LAYOUT_NCHW, y_layout=LAYOUT_NCHW, w_packed=False, kernel=None, out=None):
    """ONNX Conv (+Relu, +MaxPool 2x2). `shape` = (N, C, H, W) of the logical input."""
    N, Cin, H, Wd = shape if shape is not None else X.shape
    if w_packed:
        Cout, kH, kW = W.shape[0], kernel[0], kernel[1]
    else:
        Cout, kH, kW = W.shape[0], W.shape[2], W.shape[3]
    oH, oW = conv_out_hw(H, Wd, kH, kW, pad, stride, dil)
    if pool == 2:
        oH, oW = oH // 2, oW // 2
    yshape = (N, oH, oW, Cout) if y_layout == LAYOUT_NHWC else (N, Cout, oH, oW)
    Y = out if out is not None else torch.empty(yshape, dtype=torch.float32, device=X.device)
    d = capi.Conv2dDesc(N, Cin, H, Wd, Cout, kH, kW, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1], group,
                        x_layout, y_layout, int(w_packed), int(relu), pool)
    capi.call("sofie_cuda_conv2d_f32", _stream(), C.byref(d), _p(X), _p(W), _p(bias), _p(Y))
    return Y


def conv2d_pack_f32(W):
    Cout, Cin, kH, kW = W.shape
    P = torch.empty((Cout, kH, kW, Cin), dtype=torch.float32, device=W.device)
    d = capi.Conv2dDesc(0, Cin, 1, 1, Cout, kH, kW, 0, 0, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0)
    capi.call("sofie_cuda_conv2d_pack_f32", _stream(), C.byref(d), _p(W), _p(P))
    return P


def relu_f32(X, out=None):
    Y = out if out is not None else torch.empty_like(X)
    capi.call("sofie_cuda_relu_f32", _stream(), _p(X), _p(Y), X.numel())
    return Y


def pool2d_f32(X, *, mode=0, kernel=(2, 2), stride=(2, 2), pads=(0, 0, 0, 0), count_include_pad=0,
               layout=LAYOUT_NCHW, shape=None):
    N, Cc, H, W = shape if shape is not None else X.shape
    oH = -(-(H + pads[0] + pads[2] - kernel[0] + 1) // stride[0])
    oW = -(-(W + pads[1] + pads[3] - kernel[1] + 1) // stride[1])
    yshape = (N, oH, oW, Cc) if layout == LAYOUT_NHWC else (N, Cc, oH, oW)
    Y = torch.empty(yshape, dtype=torch.float32, device=X.device)
    d = capi.Pool2dDesc(mode, N, Cc, H, W, kernel[0], kernel[1], stride[0], stride[1], (capi.i32 * 4)(*pads),
                        count_include_pad, layout)
    capi.call("sofie_cuda_pool2d_f32", _stream(), C.byref(d), _p(X), _p(Y))
    return Y


def pool3d_f32(X, *, mode=0, kernel=(2, 2, 2), stride=(2, 2, 2), pads=(0, 0, 0, 0, 0, 0), count_include_pad=0):
    """MaxPool (mode 0) / AveragePool (mode 1) of [N, C, D, H, W]; pads = (d, h, w begin, d, h, w end)."""
    N, Cc, D, H, W = X.shape
    o = [-(-(e + pads[i] + pads[i + 3] - kernel[i] + 1) // stride[i]) for i, e in enumerate((D, H, W))]
    Y = torch.empty((N, Cc, *o), dtype=torch.float32, device=X.device)
    d = capi.Pool3dDesc(mode, N, Cc, D, H, W, *kernel, *stride, (capi.i32 * 6)(*pads), count_include_pad)
    capi.call("sofie_cuda_pool3d_f32", _stream(), C.byref(d), _p(X), _p(Y))
    return Y


def conv3d_f32(X, W, bias=None, *, pad=(0, 0, 0), stride=(1, 1, 1), dil=(1, 1, 1), group=1, relu=False):
    """X [N, C, D, H, W], W [Cout, C/group, kD, kH, kW] -> [N, Cout, oD, oH, oW]."""
    N, Cin, D, H, Wd = X.shape
    Cout, _, kD, kH, kW = W.shape
    o = [(e + 2 * pad[i] - (dil[i] * (k - 1) + 1)) // stride[i] + 1 for i, (e, k) in enumerate(((D, kD), (H, kH), (Wd, kW)))]
    Y = torch.empty((N, Cout, *[max(v, 0) for v in o]), dtype=torch.float32, device=X.device)
    d = capi.Conv3dDesc(N, Cin, D, H, Wd, Cout, kD, kH, kW, *pad, *stride, *dil, group, int(relu))
    capi.call("sofie_cuda_conv3d_f32", _stream(), C.byref(d), _p(X), _p(W), _p(bias) if bias is not None else None, _p(Y))
    return Y


def softmax_f32(X, axis=-1):
    axis = axis % X.dim()
    outer = int(np.prod(X.shape[:axis], dtype=np.int64))
    inner = int(np.prod(X.shape[axis + 1:], dtype=np.int64))
    Y = torch.empty_like(X)
    capi.call("sofie_cuda_softmax_f32", _stream(), _p(X), _p(Y), outer, X.shape[axis], inner)
    return Y


def conv_transpose2d_f32(X, W, bias=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0), relu=False, product_form=False):
    """ONNX ConvTranspose, group 1: X [N, C, H, W], W [C, Cout, kH, kW] -> [N, Cout, oH, oW]. product_form: the entry
    point that lowers to one tensor-core GEMM plus a gather (shapes with at least 16 input channels, a multiple of 4)."""
    N, Cin, H, Wd = X.shape
    _, Cout, kH, kW = W.shape
    oH = stride[0] * (H - 1) + dil[0] * (kH - 1) + 1 + out_pad[0] - 2 * pad[0]
    oW = stride[1] * (Wd - 1) + dil[1] * (kW - 1) + 1 + out_pad[1] - 2 * pad[1]
    Y = torch.empty((N, Cout, max(oH, 0), max(oW, 0)), dtype=torch.float32, device=X.device)
    d = capi.ConvTranspose2dDesc(N, Cin, H, Wd, Cout, kH, kW, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1], out_pad[0],
                                 out_pad[1], int(relu))
    b = _p(bias) if bias is not None else None
    if product_form:
        nbytes = capi.load().sofie_cuda_conv_transpose2d_f32_gemm_scratch(C.byref(d))
        scratch = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=X.device)
        capi.call("sofie_cuda_conv_transpose2d_f32_gemm", _stream(), C.byref(d), _p(X), _p(W), b, _p(Y), _p(scratch), nbytes)
    else:
        capi.call("sofie_cuda_conv_transpose2d_f32", _stream(), C.byref(d), _p(X), _p(W), b, _p(Y))
    return Y


def einsum_plan(equation, shape_a, shape_b):
    """Two-operand Einsum without ellipsis -> (output shape, n_out, n_sum, extents, strides in A, strides in B):
    the output labels first, in output order, then every other label in order of first appearance."""
    eq = equation.replace(" ", "")
    lhs, out = eq.split("->") if "->" in eq else (eq, None)
    la, lb = lhs.split(",")
    if "." in eq or len(la) != len(shape_a) or len(lb) != len(shape_b):
        raise ValueError(f"Einsum {equation}: two operands, one label per axis, no ellipsis")
    if out is None:   # implicit form: the labels that appear once, sorted
        out = "".join(sorted(c for c in set(la + lb) if (la + lb).count(c) == 1))
    size = {}
    for labels, shape in ((la, shape_a), (lb, shape_b)):
        for c, n in zip(labels, shape):
            if size.setdefault(c, int(n)) != int(n):
                raise ValueError(f"Einsum {equation}: label {c} has two extents")
    if len(set(la)) != len(la) or len(set(lb)) != len(lb) or len(set(out)) != len(out) or any(c not in size for c in out):
        raise ValueError(f"Einsum {equation}: repeated labels within one operand are not supported")
    summed = [c for c in dict.fromkeys(la + lb) if c not in out]
    labels = list(out) + summed
    if len(labels) > 8:
        raise ValueError("Einsum: at most 8 labels")

    def strides(lab, shape):
        st, dense = {}, 1
        for c, n in zip(reversed(lab), reversed(shape)):
            st[c] = dense
            dense *= int(n)
        return [st.get(c, 0) for c in labels]
    return tuple(size[c] for c in out), len(out), len(summed), [size[c] for c in labels], strides(la, shape_a), strides(lb, shape_b)


def einsum_f32(equation, A, B):
    out_shape, n_out, n_sum, extent, sa, sb = einsum_plan(equation, tuple(A.shape), tuple(B.shape))
    Y = torch.empty(out_shape, dtype=torch.float32, device=A.device)
    pad = lambda v: (C.c_int64 * 8)(*(list(v) + [0] * (8 - len(v))))
    d = capi.EinsumDesc(n_out, n_sum, pad(extent), pad(sa), pad(sb))
    capi.call("sofie_cuda_einsum_f32", _stream(), C.byref(d), _p(A), _p(B), _p(Y))
    return Y


def mlp_desc(M, dims, relu, w_is_nk):
    L = len(dims) - 1
    return capi.MlpDesc(M, L, (capi.i32 * 9)(*(list(dims) + [0] * (8 - L))), (capi.i32 * 8)(*([int(r) for r in relu] + [0] * (8 - L))),
                        (capi.i32 * 8)(*([int(n) for n in w_is_nk] + [0] * (8 - L))))


def mlp_fits(dims):
    """Whether a chain of layers with these widths is within what the fused MLP kernel takes (host arithmetic)."""
    if not 2 <= len(dims) <= capi.MLP_MAX_LAYERS + 1 or max(dims) > capi.MLP_MAX_WIDTH or min(dims) < 1:
        return False
    d = mlp_desc(0, dims, [0] * (len(dims) - 1), [0] * (len(dims) - 1))
    return capi.load().sofie_cuda_mlp_f32_smem(C.byref(d)) <= capi.MLP_MAX_SMEM


def mlp_f32(X, weights, biases, relu, w_is_nk):
    """Fused chain of Gemm (+ Relu) layers; weights[l] is [N, K] when w_is_nk[l] else [K, N]."""
    L = len(weights)
    dims = [X.shape[1]] + [(W.shape[0] if nk else W.shape[1]) for W, nk in zip(weights, w_is_nk)]
    Y = torch.empty((X.shape[0], dims[-1]), dtype=torch.float32, device=X.device)
    d = mlp_desc(X.shape[0], dims, relu, w_is_nk)
    Wp = (C.c_void_p * L)(*[_p(W) for W in weights])
    Bp = (C.c_void_p * L)(*[(_p(b) if b is not None else None) for b in biases])
    capi.call("sofie_cuda_mlp_f32", _stream(), C.byref(d), _p(X), Wp, Bp, _p(Y))
    return Y


UNARY_OPS = {"Sigmoid": 0, "Tanh": 1, "LeakyRelu": 2, "Selu": 3, "Elu": 4, "Neg": 5, "Exp": 6, "Log": 7, "Sqrt": 8,
             "Reciprocal": 9, "Abs": 10, "Erf": 11, "Swish": 12, "Cos": 13, "Sin": 14}
BINARY_OPS = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3}


def unary_f32(X, op, alpha=0.0):
    Y = torch.empty_like(X)
    capi.call("sofie_cuda_unary_f32", _stream(), UNARY_OPS[op], float(alpha), _p(X), _p(Y), X.numel())
    return Y


def binary_strides(a_shape, b_shape):
    """Output shape and the rank-4 shape / element strides (0 along broadcast dimensions) of A op B."""
    out = tuple(torch.broadcast_shapes(tuple(a_shape), tuple(b_shape)))
    if len(out) > 4:
        raise ValueError("binary operators are built for rank <= 4")

    def strides(shape):
        shape = (1,) * (len(out) - len(shape)) + tuple(shape)
        st, dense = [], 1
        for d in reversed(shape):
            st.append(0 if d == 1 else dense)
            dense *= d
        return [0] * (4 - len(out)) + list(reversed(st))

    return out, [1] * (4 - len(out)) + list(out), strides(a_shape), strides(b_shape)


def binary_f32(A, B, op):
    out, shape4, sa, sb = binary_strides(A.shape, B.shape)
    Y = torch.empty(out, dtype=torch.float32, device=A.device)
    i64 = C.c_int64 * 4
    d = capi.BinaryDesc(BINARY_OPS[op], i64(*shape4), i64(*sa), i64(*sb))
    capi.call("sofie_cuda_binary_f32", _stream(), C.byref(d), _p(A), _p(B), _p(Y))
    return Y


def batchnorm_f32(X, scale, bias, mean, N, Cc, HW, layout=LAYOUT_NCHW, relu=False):
    """scale is the folded gamma / sqrt(var + eps)."""
    Y = torch.empty_like(X)
    d = capi.BatchNormDesc(N, Cc, HW, layout, int(relu))
    capi.call("sofie_cuda_batchnorm_f32", _stream(), C.byref(d), _p(X), _p(scale), _p(bias), _p(mean), _p(Y))
    return Y


def nchw_to_nhwc(X):
    N, Cc, H, W = X.shape
    Y = torch.empty((N, H, W, Cc), dtype=X.dtype, device=X.device)
    fn = "sofie_cuda_nchw_to_nhwc_f32" if X.dtype == torch.float32 else "sofie_cuda_nchw_to_nhwc_u8"
    capi.call(fn, _stream(), _p(X), _p(Y), N, Cc, H, W)
    return Y


def nhwc_to_nchw(X):
    N, H, W, Cc = X.shape
    Y = torch.empty((N, Cc, H, W), dtype=X.dtype, device=X.device)
    fn = "sofie_cuda_nhwc_to_nchw_f32" if X.dtype == torch.float32 else "sofie_cuda_nhwc_to_nchw_u8"
    capi.call(fn, _stream(), _p(X), _p(Y), N, Cc, H, W)
    return Y


def transpose2d(X):
    rows, cols = X.shape
    Y = torch.empty((cols, rows), dtype=X.dtype, device=X.device)
    fn = "sofie_cuda_transpose_f32" if X.dtype == torch.float32 else "sofie_cuda_transpose_i8"
    capi.call(fn, _stream(), _p(X), _p(Y), rows, cols)
    return Y


# ---------------------------------------------------------------- int8 -------------------------
def quantize_u8(X, scale, zp):
    Y = torch.empty(X.shape, dtype=torch.uint8, device=X.device)
    capi.call("sofie_cuda_quantize_u8", _stream(), _p(X), _p(Y), X.numel(), float(scale), int(zp))
    return Y


def dequantize_u8(X, scale, zp):
    Y = torch.empty(X.shape, dtype=torch.float32, device=X.device)
    capi.call("sofie_cuda_dequantize_u8", _stream(), _p(X), _p(Y), X.numel(), float(scale), int(zp))
    return Y


def qlinear_prepare(W_host: np.ndarray, w_is_nk: bool, a_scale, a_zp, w_scale_host: np.ndarray, y_scale,
                    bias_host: np.ndarray | None, device, n_out=None, rows_per_n=None):
    """Per-output-channel requantisation multiplier and int32 correction, computed on the host."""
    W_host = np.ascontiguousarray(W_host, dtype=np.int8)
    w_scale_host = np.ascontiguousarray(w_scale_host, dtype=np.float32)
    if n_out is None:
        n_out = W_host.shape[0] if w_is_nk else W_host.shape[1]
    if rows_per_n is None:
        rows_per_n = W_host.size // n_out
    mult = torch.empty(n_out, dtype=torch.float32, device=device)
    corr = torch.empty(n_out, dtype=torch.int32, device=device)
    bias_p = C.c_void_p(0)
    if bias_host is not None:
        bias_host = np.ascontiguousarray(bias_host, dtype=np.int32)
        bias_p = bias_host.ctypes.data_as(C.c_void_p)
    capi.call("sofie_cuda_qlinear_prepare", _stream(), n_out, rows_per_n, W_host.ctypes.data_as(C.c_void_p),
              int(w_is_nk), float(a_scale), int(a_zp), w_scale_host.ctypes.data_as(C.c_void_p), float(y_scale),
              bias_p, _p(mult), _p(corr))
    return mult, corr


def qlinear_matmul(A, W, mult, corr, *, w_is_nk=True, y_zp=0, relu=False):
    M, K = A.shape
    N = W.shape[0] if w_is_nk else W.shape[1]
    Y = torch.empty((M, N), dtype=torch.uint8, device=A.device)
    d = capi.QGemmDesc(M, N, K, int(w_is_nk), int(y_zp), int(relu))
    capi.call("sofie_cuda_qlinear_matmul", _stream(), C.byref(d), _p(A), _p(W), _p(mult), _p(corr), _p(Y))
    return Y


def qlinear_matmul_f32(A, W, mult, corr, y_scale, *, w_is_nk=True, y_zp=0, relu=False):
    """QLinearMatMul + DequantizeLinear (same zero point) in one pass: float32 (q - y_zp) * y_scale."""
    M, K = A.shape
    N = W.shape[0] if w_is_nk else W.shape[1]
    Y = torch.empty((M, N), dtype=torch.float32, device=A.device)
    d = capi.QGemmDesc(M, N, K, int(w_is_nk), int(y_zp), int(relu))
    capi.call("sofie_cuda_qlinear_matmul_f32", _stream(), C.byref(d), _p(A), _p(W), _p(mult), _p(corr), float(y_scale), _p(Y))
    return Y


def qlinear_conv2d(X, W, mult, bias=None, *, shape=None, pad=(0, 0), stride=(1, 1), x_zp=0, y_zp=0, relu=False,
                   pool=0, x_layout=LAYOUT_NCHW, y_layout=LAYOUT_NCHW, w_packed=False, kernel=None):
    N, Cin, H, Wd = shape if shape is not None else X.shape
    if w_packed:
        Cout, kH, kW = W.shape[0], kernel[0], kernel[1]
    else:
        Cout, kH, kW = W.shape[0], W.shape[2], W.shape[3]
    oH, oW = conv_out_hw(H, Wd, kH, kW, pad, stride)
    if pool == 2:
        oH, oW = oH // 2, oW // 2
    yshape = (N, oH, oW, Cout) if y_layout == LAYOUT_NHWC else (N, Cout, oH, oW)
    Y = torch.empty(yshape, dtype=torch.uint8, device=X.device)
    d = capi.QConv2dDesc(N, Cin, H, Wd, Cout, kH, kW, pad[0], pad[1], stride[0], stride[1], x_layout, y_layout,
                         int(w_packed), int(x_zp), int(y_zp), int(relu), pool)
    capi.call("sofie_cuda_qlinear_conv2d", _stream(), C.byref(d), _p(X), _p(W), _p(mult), _p(bias), _p(Y))
    return Y


def qconv2d_pack_i8(W):
    Cout, Cin, kH, kW = W.shape
    P = torch.empty((Cout, kH, kW, Cin), dtype=torch.int8, device=W.device)
    d = capi.QConv2dDesc(0, Cin, 1, 1, Cout, kH, kW, 0, 0, 1, 1, 0, 0, 0, 0, 0, 0, 0)
    capi.call("sofie_cuda_qconv2d_pack_i8", _stream(), C.byref(d), _p(W), _p(P))
    return P


def maxpool2d_u8(X, *, kernel=(2, 2), stride=(2, 2), layout=LAYOUT_NCHW, shape=None):
    N, Cc, H, W = shape if shape is not None else X.shape
    oH, oW = (H - kernel[0]) // stride[0] + 1, (W - kernel[1]) // stride[1] + 1
    yshape = (N, oH, oW, Cc) if layout == LAYOUT_NHWC else (N, Cc, oH, oW)
    Y = torch.empty(yshape, dtype=torch.uint8, device=X.device)
    capi.call("sofie_cuda_maxpool2d_u8", _stream(), _p(X), _p(Y), N, Cc, H, W, kernel[0], kernel[1], stride[0],
              stride[1], layout)
    return Y


# ---------------------------------------------------------------- FP8 --------------------------
def quantize_e4m3(X, scale):
    Y = torch.empty(X.shape, dtype=torch.uint8, device=X.device)
    if X.dtype == torch.float32:
        capi.call("sofie_cuda_quantize_e4m3_f32", _stream(), _p(X), _p(Y), X.numel(), float(scale))
    else:
        assert X.dtype in (torch.bfloat16, torch.uint16, torch.int16)
        capi.call("sofie_cuda_quantize_e4m3_bf16", _stream(), _p(X), _p(Y), X.numel(), float(scale))
    return Y


def cast_bf16_f32(X):
    Y = torch.empty(X.shape, dtype=torch.float32, device=X.device)
    capi.call("sofie_cuda_cast_bf16_f32", _stream(), _p(X), _p(Y), X.numel())
    return Y


def cast_f32_bf16(X):
    Y = torch.empty(X.shape, dtype=torch.bfloat16, device=X.device)
    capi.call("sofie_cuda_cast_f32_bf16", _stream(), _p(X), _p(Y), X.numel())
    return Y


def amax_f32(X):
    out = torch.empty(1, dtype=torch.float32, device=X.device)
    capi.call("sofie_cuda_amax_f32", _stream(), _p(X), X.numel(), _p(out))
    return out


def gemm_e4m3(A, W, bias=None, *, a_scale=1.0, w_scale=1.0, relu=False, q_scale=0.0, want_bf16=True):
    """A [M,K] and W [N,K] are uint8 tensors holding E4M3 codes. Returns (bf16 Y or None, E4M3 Yq or None)."""
    M, K = A.shape
    N = W.shape[0]
    Y = torch.empty((M, N), dtype=torch.bfloat16, device=A.device) if want_bf16 else None
    Yq = torch.empty((M, N), dtype=torch.uint8, device=A.device) if q_scale > 0 else None
    d = capi.Fp8GemmDesc(M, N, K, float(a_scale), float(w_scale), int(relu), float(q_scale))
    capi.call("sofie_cuda_gemm_e4m3", _stream(), C.byref(d), _p(A), _p(W), _p(bias), _p(Y), _p(Yq))
    return Y, Yq


def gemm_e4m3_f32(A, W, bias=None, *, a_scale=1.0, w_scale=1.0, relu=False):
    """The FP8 product with the bf16-rounded result written as float32 (Fp8Gemm + Cast in one pass)."""
    M, K = A.shape
    N = W.shape[0]
    Y = torch.empty((M, N), dtype=torch.float32, device=A.device)
    d = capi.Fp8GemmDesc(M, N, K, float(a_scale), float(w_scale), int(relu), 0.0)
    capi.call("sofie_cuda_gemm_e4m3_f32", _stream(), C.byref(d), _p(A), _p(W), _p(bias), _p(Y))
    return Y
