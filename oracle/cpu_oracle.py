"""ctypes binding of liboracle.so (oracle/sofie_oracle.c). TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this module; the
product never does. Arrays are numpy; every function returns a new array.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "sofie_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.oracle_e4m3_to_f32.restype = C.c_float
        _lib.oracle_e4m3_to_f32.argtypes = [C.c_uint8]
        _lib.oracle_f32_to_e4m3.restype = C.c_uint8
        _lib.oracle_f32_to_e4m3.argtypes = [C.c_float]
        _lib.oracle_f32_to_bf16.restype = C.c_uint16
        _lib.oracle_f32_to_bf16.argtypes = [C.c_float]
        _lib.oracle_bf16_to_f32.restype = C.c_float
        _lib.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return lib().oracle_num_threads()


def gemm_f32(A, B, C_=None, transA=0, transB=0, alpha=1.0, beta=1.0, relu=False):
    A, B = _f(A), _f(B)
    M = A.shape[1] if transA else A.shape[0]
    K = A.shape[0] if transA else A.shape[1]
    N = B.shape[0] if transB else B.shape[1]
    kind = 0
    if C_ is not None:
        C_ = _f(C_)
        kind = 1 if C_.size == N else 2
    Y = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32(C.c_int(transA), C.c_int(transB), C.c_int(M), C.c_int(N), C.c_int(K), C.c_float(alpha),
                          _ptr(A), _ptr(B), C.c_float(beta), _ptr(C_), C.c_int(kind), C.c_int(int(relu)), _ptr(Y))
    return Y


def conv2d_f32(X, W, bias=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), group=1, relu=False):
    X, W = _f(X), _f(W)
    N, Cin, H, Wd = X.shape
    Cout, _, kh, kw = W.shape
    oH = (H + 2 * pad[0] - (dil[0] * (kh - 1) + 1)) // stride[0] + 1
    oW = (Wd + 2 * pad[1] - (dil[1] * (kw - 1) + 1)) // stride[1] + 1
    if bias is not None:
        bias = _f(bias)
    Y = np.empty((N, Cout, oH, oW), np.float32)
    ints = [N, Cin, H, Wd, Cout, kh, kw, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1], group]
    lib().oracle_conv2d_f32(*[C.c_int(v) for v in ints], _ptr(X), _ptr(W), _ptr(bias), C.c_int(int(relu)), _ptr(Y))
    return Y


def conv_transpose2d_f32(X, W, bias=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0)):
    """X [N, C, H, W], W [C, Cout, kh, kw] (ONNX ConvTranspose, group 1) -> [N, Cout, oH, oW]."""
    X, W = _f(X), _f(W)
    N, Cin, H, Wd = X.shape
    _, Cout, kh, kw = W.shape
    oH = stride[0] * (H - 1) + dil[0] * (kh - 1) + 1 + out_pad[0] - 2 * pad[0]
    oW = stride[1] * (Wd - 1) + dil[1] * (kw - 1) + 1 + out_pad[1] - 2 * pad[1]
    if bias is not None:
        bias = _f(bias)
    Y = np.empty((N, Cout, oH, oW), np.float32)
    ints = [N, Cin, H, Wd, Cout, kh, kw, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1], out_pad[0], out_pad[1]]
    lib().oracle_conv_transpose2d_f32(*[C.c_int(v) for v in ints], _ptr(X), _ptr(W), _ptr(bias), _ptr(Y))
    return Y


def einsum_f32(equation, A, B):
    """Two-operand Einsum without ellipsis, e.g. "abc,abd->ad"."""
    from sofie_b200.ops import einsum_plan
    A, B = _f(A), _f(B)
    out_shape, n_out, n_sum, extent, sa, sb = einsum_plan(equation, A.shape, B.shape)
    Y = np.empty(out_shape, np.float32)
    arr = lambda v: (C.c_longlong * 8)(*(list(v) + [0] * (8 - len(v))))
    lib().oracle_einsum_f32(C.c_int(n_out), C.c_int(n_sum), arr(extent), arr(sa), arr(sb), _ptr(A), _ptr(B), _ptr(Y))
    return Y


def relu_f32(X):
    X = _f(X)
    Y = np.empty_like(X)
    lib().oracle_relu_f32(_ptr(X), C.c_size_t(X.size), _ptr(Y))
    return Y


def pool2d_f32(X, mode=0, kernel=(2, 2), stride=(2, 2), pads=(0, 0, 0, 0), count_include_pad=0):
    X = _f(X)
    N, Cc, H, W = X.shape
    oH = -(-(H + pads[0] + pads[2] - kernel[0] + 1) // stride[0])
    oW = -(-(W + pads[1] + pads[3] - kernel[1] + 1) // stride[1])
    Y = np.empty((N, Cc, oH, oW), np.float32)
    p = (C.c_int * 4)(*pads)
    lib().oracle_pool2d_f32(C.c_int(mode), C.c_size_t(N * Cc), C.c_int(H), C.c_int(W), C.c_int(kernel[0]),
                            C.c_int(kernel[1]), p, C.c_int(stride[0]), C.c_int(stride[1]),
                            C.c_int(count_include_pad), _ptr(X), _ptr(Y))
    return Y


def conv3d_f32(X, W, bias=None, pad=(0, 0, 0), stride=(1, 1, 1), dil=(1, 1, 1), group=1, relu=False):
    """3-D convolution as the reference computes it (ROperator_Conv.hxx with fDim == 3: UTILITY::Im2col_3d, SOFIE_common.hxx:521-573,
    then one sgemm_ per image and group; bias added afterwards): X [N, C, D, H, W], W [Cout, C/group, kD, kH, kW].
    numpy restatement: for every filter tap the shifted, strided view of the zero-padded input times that tap's weights, summed in
    (ic, kd, kh, kw) order in float32."""
    X, W = _f(X), _f(W)
    N, Cin, D, H, Wd = X.shape
    Cout, cin_g, kD, kH, kW = W.shape
    assert cin_g * group == Cin and Cout % group == 0
    o = [(e + 2 * pad[i] - (dil[i] * (k - 1) + 1)) // stride[i] + 1 for i, (e, k) in enumerate(((D, kD), (H, kH), (Wd, kW)))]
    Xp = np.zeros((N, Cin, D + 2 * pad[0], H + 2 * pad[1], Wd + 2 * pad[2]), np.float32)
    Xp[:, :, pad[0]:pad[0] + D, pad[1]:pad[1] + H, pad[2]:pad[2] + Wd] = X
    Y = np.zeros((N, Cout, *o), np.float32)
    cout_g = Cout // group
    for g in range(group):
        for ic in range(cin_g):
            for a in range(kD):
                for b in range(kH):
                    for c in range(kW):
                        v = Xp[:, g * cin_g + ic,
                               a * dil[0]:a * dil[0] + (o[0] - 1) * stride[0] + 1:stride[0],
                               b * dil[1]:b * dil[1] + (o[1] - 1) * stride[1] + 1:stride[1],
                               c * dil[2]:c * dil[2] + (o[2] - 1) * stride[2] + 1:stride[2]]
                        w = W[g * cout_g:(g + 1) * cout_g, ic, a, b, c]
                        Y[:, g * cout_g:(g + 1) * cout_g] += v[:, None] * w[None, :, None, None, None]
    if bias is not None:
        Y += _f(bias)[None, :, None, None, None]
    if relu:
        Y = np.where(Y > 0, Y, np.float32(0)).astype(np.float32)
    return Y


def pool3d_f32(X, mode=0, kernel=(2, 2, 2), stride=(2, 2, 2), pads=(0, 0, 0, 0, 0, 0), count_include_pad=0):
    """MaxPool (mode 0) / AveragePool (mode 1) of [N, C, D, H, W] (reference: the fDim == 3 loops of ROperator_Pool.hxx:266-476, output
    extent :172-197); pads = (d, h, w begin, d, h, w end). A maximum starts at -inf and takes v only when v > max (a NaN never wins);
    an average adds the window's values in (d, h, w) order and divides by the number of values inside the tensor, or by the window
    size with count_include_pad (or without padding)."""
    X = _f(X)
    N, Cc, D, H, W = X.shape
    o = [-(-(e + pads[i] + pads[i + 3] - kernel[i] + 1) // stride[i]) for i, e in enumerate((D, H, W))]
    Y = np.empty((N, Cc, *o), np.float32)
    padded = any(pads)
    for od in range(o[0]):
        for oh in range(o[1]):
            for ow in range(o[2]):
                d0, h0, w0 = od * stride[0] - pads[0], oh * stride[1] - pads[1], ow * stride[2] - pads[2]
                val = np.full((N, Cc), -np.inf if mode == 0 else 0.0, np.float32)
                count = 0
                for a in range(max(d0, 0), min(d0 + kernel[0], D)):
                    for b in range(max(h0, 0), min(h0 + kernel[1], H)):
                        for c in range(max(w0, 0), min(w0 + kernel[2], W)):
                            v = X[:, :, a, b, c]
                            if mode == 0:
                                val = np.where(v > val, v, val)
                            else:
                                val = (val + v).astype(np.float32)
                                count += 1
                if mode == 1:
                    n = kernel[0] * kernel[1] * kernel[2] if (count_include_pad or not padded) else count
                    val = (val / np.float32(n)).astype(np.float32)
                Y[:, :, od, oh, ow] = val
    return Y


UNARY_OPS = {"Sigmoid": 0, "Tanh": 1, "LeakyRelu": 2, "Selu": 3, "Elu": 4, "Neg": 5, "Exp": 6, "Log": 7, "Sqrt": 8,
             "Reciprocal": 9, "Abs": 10, "Erf": 11, "Swish": 12, "Cos": 13, "Sin": 14}
BINARY_OPS = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3}


def unary_f32(X, op, alpha=0.0):
    X = _f(X)
    Y = np.empty_like(X)
    lib().oracle_unary_f32(C.c_int(UNARY_OPS[op]), C.c_float(alpha), _ptr(X), _ptr(Y), C.c_size_t(X.size))
    return Y


def broadcast_strides(a_shape, b_shape):
    """(output shape, a strides, b strides) of numpy-style broadcasting, padded to rank 4, in elements."""
    out = np.broadcast_shapes(tuple(a_shape), tuple(b_shape))
    if len(out) > 4:
        raise ValueError("binary operators are built for rank <= 4")

    def strides(shape):
        shape = (1,) * (len(out) - len(shape)) + tuple(shape)
        st, dense = [], 1
        for d in reversed(shape):
            st.append(0 if d == 1 else dense)
            dense *= d
        st = list(reversed(st))
        return [0] * (4 - len(out)) + [0 if o != d and d == 1 else s for s, d, o in zip(st, shape, out)]

    return out, [1] * (4 - len(out)) + list(out), strides(a_shape), strides(b_shape)


def binary_f32(A, B, op):
    A, B = _f(A), _f(B)
    out, shape4, sa, sb = broadcast_strides(A.shape, B.shape)
    Y = np.empty(out, np.float32)
    i64 = C.c_int64 * 4
    lib().oracle_binary_f32(C.c_int(BINARY_OPS[op]), i64(*shape4), i64(*sa), i64(*sb), _ptr(A), _ptr(B), _ptr(Y))
    return Y


def batchnorm_f32(X, scale, bias, mean, var, epsilon=1e-5, relu=False):
    X, scale, bias, mean, var = _f(X), _f(scale), _f(bias), _f(mean), _f(var)
    N, Cc = X.shape[0], X.shape[1]
    HW = int(np.prod(X.shape[2:], dtype=np.int64))
    Y = np.empty_like(X)
    lib().oracle_batchnorm_f32(C.c_int(N), C.c_int(Cc), C.c_int(HW), C.c_float(epsilon), C.c_int(int(relu)), _ptr(X), _ptr(scale),
                               _ptr(bias), _ptr(mean), _ptr(var), _ptr(Y))
    return Y


def batchnorm_folded_scale(scale, var, epsilon=1e-5):
    """scale * (1 / sqrt(var + epsilon)) with the roundings of the reference's Initialize."""
    v = (_f(var) + np.float32(epsilon)).astype(np.float32)
    inv = (1.0 / np.sqrt(v.astype(np.float64))).astype(np.float32)
    return (_f(scale) * inv).astype(np.float32)


def softmax_f32(X, axis=-1):
    X = _f(X)
    axis = axis % X.ndim
    outer = int(np.prod(X.shape[:axis], dtype=np.int64))
    inner = int(np.prod(X.shape[axis + 1:], dtype=np.int64))
    Y = np.empty_like(X)
    lib().oracle_softmax_f32(C.c_size_t(outer), C.c_size_t(X.shape[axis]), C.c_size_t(inner), _ptr(X), _ptr(Y))
    return Y


def requant_multiplier(a_scale, w_scale, y_scale):
    w_scale = _f(w_scale)
    m = np.empty_like(w_scale)
    lib().oracle_requant_multiplier(C.c_float(a_scale), _ptr(w_scale), C.c_int(w_scale.size), C.c_float(y_scale),
                                    _ptr(m))
    return m


def quantize_u8(X, scale, zp):
    X = _f(X)
    Y = np.empty(X.shape, np.uint8)
    lib().oracle_quantize_u8(_ptr(X), C.c_size_t(X.size), C.c_float(scale), C.c_int32(zp), _ptr(Y))
    return Y


def dequantize_u8(X, scale, zp):
    X = np.ascontiguousarray(X, np.uint8)
    Y = np.empty(X.shape, np.float32)
    lib().oracle_dequantize_u8(_ptr(X), C.c_size_t(X.size), C.c_float(scale), C.c_int32(zp), _ptr(Y))
    return Y


def qlinear_matmul(A, a_scale, a_zp, W, w_scale, y_scale, y_zp, bias=None, w_is_nk=True, relu=False):
    A = np.ascontiguousarray(A, np.uint8)
    W = np.ascontiguousarray(W, np.int8)
    w_scale = _f(w_scale)
    M, K = A.shape
    N = W.shape[0] if w_is_nk else W.shape[1]
    if bias is not None:
        bias = np.ascontiguousarray(bias, np.int32)
    Y = np.empty((M, N), np.uint8)
    lib().oracle_qlinear_matmul(C.c_int(M), C.c_int(N), C.c_int(K), _ptr(A), C.c_float(a_scale), C.c_int32(a_zp),
                                _ptr(W), C.c_int(int(w_is_nk)), _ptr(w_scale), _ptr(bias), C.c_float(y_scale),
                                C.c_int32(y_zp), C.c_int(int(relu)), _ptr(Y))
    return Y


def qlinear_conv2d(X, x_scale, x_zp, W, w_scale, y_scale, y_zp, bias=None, pad=(0, 0), stride=(1, 1), relu=False):
    X = np.ascontiguousarray(X, np.uint8)
    W = np.ascontiguousarray(W, np.int8)
    w_scale = _f(w_scale)
    N, Cin, H, Wd = X.shape
    Cout, _, kh, kw = W.shape
    oH = (H + 2 * pad[0] - kh) // stride[0] + 1
    oW = (Wd + 2 * pad[1] - kw) // stride[1] + 1
    if bias is not None:
        bias = np.ascontiguousarray(bias, np.int32)
    Y = np.empty((N, Cout, oH, oW), np.uint8)
    ints = [N, Cin, H, Wd, Cout, kh, kw, pad[0], pad[1], stride[0], stride[1]]
    lib().oracle_qlinear_conv2d(*[C.c_int(v) for v in ints], _ptr(X), C.c_float(x_scale), C.c_int32(x_zp), _ptr(W),
                                _ptr(w_scale), _ptr(bias), C.c_float(y_scale), C.c_int32(y_zp), C.c_int(int(relu)),
                                _ptr(Y))
    return Y


def maxpool2d_u8(X, kernel=(2, 2), stride=(2, 2)):
    X = np.ascontiguousarray(X, np.uint8)
    N, Cc, H, W = X.shape
    oH, oW = (H - kernel[0]) // stride[0] + 1, (W - kernel[1]) // stride[1] + 1
    Y = np.empty((N, Cc, oH, oW), np.uint8)
    lib().oracle_maxpool2d_u8(C.c_size_t(N * Cc), C.c_int(H), C.c_int(W), C.c_int(kernel[0]), C.c_int(kernel[1]),
                              C.c_int(stride[0]), C.c_int(stride[1]), _ptr(X), _ptr(Y))
    return Y


def quantize_e4m3(X, scale):
    X = _f(X)
    Y = np.empty(X.shape, np.uint8)
    lib().oracle_quantize_e4m3(_ptr(X), C.c_size_t(X.size), C.c_float(scale), _ptr(Y))
    return Y


def e4m3_table():
    return np.array([lib().oracle_e4m3_to_f32(i) for i in range(256)], np.float32)


def f32_to_bf16_bits(X):
    X = _f(X)
    return np.array([lib().oracle_f32_to_bf16(float(v)) for v in X.ravel()], np.uint16).reshape(X.shape)


def bf16_bits_to_f32(B):
    B = np.ascontiguousarray(B, np.uint16)
    return (B.astype(np.uint32) << 16).view(np.float32)


def gemm_e4m3(A, a_scale, W, w_scale, bias=None, relu=False):
    """A [M,K], W [N,K] uint8 E4M3 codes -> bf16 bits [M,N] (uint16)."""
    A = np.ascontiguousarray(A, np.uint8)
    W = np.ascontiguousarray(W, np.uint8)
    M, K = A.shape
    N = W.shape[0]
    if bias is not None:
        bias = _f(bias)
    Y = np.empty((M, N), np.uint16)
    lib().oracle_gemm_e4m3(C.c_int(M), C.c_int(N), C.c_int(K), _ptr(A), C.c_float(a_scale), _ptr(W),
                           C.c_float(w_scale), _ptr(bias), C.c_int(int(relu)), _ptr(Y))
    return Y
