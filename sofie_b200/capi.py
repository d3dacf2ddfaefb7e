"""ctypes binding of the C ABI declared in include/sofie_cuda.h.

This is the same set of entry points the code emitted by the C++ generator links against; the
Python tests and the benchmark call them directly. The binding fails loudly when the library is
missing or a call returns a non-zero status -- there is no CPU path behind it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import _build

i32, f32, vp, sz = C.c_int32, C.c_float, C.c_void_p, C.c_size_t

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_NOMEM, ERR_DEVICE = range(6)
LAYOUT_NCHW, LAYOUT_NHWC = 0, 1
ENGINE_NONE, ENGINE_SIMT, ENGINE_TCGEN05 = 0, 1, 2


class SofieCudaError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str):
        super().__init__(f"{what}: {detail} (status {status})")
        self.status = status


class GemmF32Desc(C.Structure):
    _fields_ = [("M", i32), ("N", i32), ("K", i32), ("transA", i32), ("transB", i32), ("alpha", f32), ("beta", f32),
                ("bias_kind", i32), ("relu", i32)]


class Conv2dDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("N", "C", "H", "W", "Cout", "kH", "kW", "pad_h", "pad_w", "stride_h", "stride_w",
                                   "dil_h", "dil_w", "group", "x_layout", "y_layout", "w_packed", "relu", "pool")]


class Pool2dDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("mode", "N", "C", "H", "W", "kH", "kW", "stride_h", "stride_w")] + \
               [("pads", i32 * 4), ("count_include_pad", i32), ("layout", i32)]


class Pool3dDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("mode", "N", "C", "D", "H", "W", "kD", "kH", "kW", "stride_d", "stride_h", "stride_w")] + \
               [("pads", i32 * 6), ("count_include_pad", i32)]


class Conv3dDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("N", "C", "D", "H", "W", "Cout", "kD", "kH", "kW", "pad_d", "pad_h", "pad_w", "stride_d", "stride_h",
                                   "stride_w", "dil_d", "dil_h", "dil_w", "group", "relu")]


class QGemmDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("M", "N", "K", "w_is_nk", "y_zp", "relu")]


class QConv2dDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("N", "C", "H", "W", "Cout", "kH", "kW", "pad_h", "pad_w", "stride_h", "stride_w",
                                   "x_layout", "y_layout", "w_packed", "x_zp", "y_zp", "relu", "pool")]


class ConvTranspose2dDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("N", "C", "H", "W", "Cout", "kH", "kW", "pad_h", "pad_w", "stride_h", "stride_w", "dil_h", "dil_w",
                                   "out_pad_h", "out_pad_w", "relu")]


class EinsumDesc(C.Structure):
    _fields_ = [("n_out", i32), ("n_sum", i32), ("extent", C.c_int64 * 8), ("a_stride", C.c_int64 * 8), ("b_stride", C.c_int64 * 8)]


class MlpDesc(C.Structure):
    _fields_ = [("M", i32), ("layers", i32), ("dims", i32 * 9), ("relu", i32 * 8), ("w_is_nk", i32 * 8)]


class BinaryDesc(C.Structure):
    _fields_ = [("op", i32), ("shape", C.c_int64 * 4), ("a_stride", C.c_int64 * 4), ("b_stride", C.c_int64 * 4)]


class BatchNormDesc(C.Structure):
    _fields_ = [(n, i32) for n in ("N", "C", "HW", "layout", "relu")]


class Fp8GemmDesc(C.Structure):
    _fields_ = [("M", i32), ("N", i32), ("K", i32), ("a_scale", f32), ("w_scale", f32), ("relu", i32),
                ("q_scale", f32)]


# name -> argument types, in the order of include/sofie_cuda.h. Everything returns int except
# the two string getters.
SIGNATURES = {
    "sofie_cuda_abi_version": [],
    "sofie_cuda_device_count": [C.POINTER(C.c_int)],
    "sofie_cuda_set_default_device": [C.c_int],
    "sofie_cuda_ctx_create": [C.POINTER(vp), C.c_int, sz],
    "sofie_cuda_ctx_destroy": [vp],
    "sofie_cuda_ctx_stream": [vp, C.POINTER(vp)],
    "sofie_cuda_ctx_device": [vp, C.POINTER(C.c_int)],
    "sofie_cuda_ctx_arena": [vp, sz, sz, C.POINTER(vp)],
    "sofie_cuda_ctx_alloc": [vp, sz, C.POINTER(vp)],
    "sofie_cuda_ctx_upload": [vp, vp, sz, C.POINTER(vp)],
    "sofie_cuda_ctx_h2d": [vp, vp, vp, sz],
    "sofie_cuda_ctx_d2h": [vp, vp, vp, sz],
    "sofie_cuda_ctx_fetch": [vp, vp, sz, C.POINTER(vp)],
    "sofie_cuda_ctx_sync": [vp],
    "sofie_cuda_ctx_check": [vp],
    "sofie_cuda_device_check": [C.c_int],
    "sofie_cuda_selftest_wait_timeout": [vp, C.c_int64, vp],
    "sofie_cuda_selftest_host_copy": [vp, vp, C.c_size_t, C.c_size_t, C.c_int, C.c_int],
    "sofie_cuda_ctx_timers": [vp, C.c_int],
    "sofie_cuda_ctx_mark": [vp, C.c_int],
    "sofie_cuda_ctx_timers_read": [vp, vp, C.c_int, C.POINTER(C.c_int)],
    "sofie_cuda_ctx_host_output": [vp, sz, C.POINTER(vp)],
    "sofie_cuda_ctx_h2d_part": [vp, vp, vp, sz, C.c_int],
    "sofie_cuda_ctx_wait_part": [vp, C.c_int],
    "sofie_cuda_ctx_graph_begin": [vp],
    "sofie_cuda_ctx_graph_end": [vp],
    "sofie_cuda_ctx_graph_launch": [vp],
    "sofie_cuda_ctx_graph_ready": [vp, C.POINTER(C.c_int)],
    "sofie_cuda_last_engine": [],
    "sofie_cuda_set_engine": [C.c_int],
    "sofie_cuda_gemm_f32": [vp, C.POINTER(GemmF32Desc), vp, vp, vp, vp],
    "sofie_cuda_gemm_f32_batched": [vp, C.POINTER(GemmF32Desc), vp, vp, vp, vp, i32, C.c_int64, C.c_int64, C.c_int64],
    "sofie_cuda_gemm_f32_splitk_static": [vp, C.POINTER(GemmF32Desc), vp, vp, vp, vp],
    "sofie_cuda_transpose_f32": [vp, vp, vp, i32, i32],
    "sofie_cuda_conv2d_f32": [vp, C.POINTER(Conv2dDesc), vp, vp, vp, vp],
    "sofie_cuda_conv2d_pack_f32": [vp, C.POINTER(Conv2dDesc), vp, vp],
    "sofie_cuda_conv_transpose2d_f32": [vp, C.POINTER(ConvTranspose2dDesc), vp, vp, vp, vp],
    "sofie_cuda_conv_transpose2d_f32_gemm": [vp, C.POINTER(ConvTranspose2dDesc), vp, vp, vp, vp, vp, C.c_size_t],
    "sofie_cuda_einsum_f32": [vp, C.POINTER(EinsumDesc), vp, vp, vp],
    "sofie_cuda_relu_f32": [vp, vp, vp, sz],
    "sofie_cuda_pool2d_f32": [vp, C.POINTER(Pool2dDesc), vp, vp],
    "sofie_cuda_pool3d_f32": [vp, C.POINTER(Pool3dDesc), vp, vp],
    "sofie_cuda_conv3d_f32": [vp, C.POINTER(Conv3dDesc), vp, vp, vp, vp],
    "sofie_cuda_softmax_f32": [vp, vp, vp, sz, sz, sz],
    "sofie_cuda_mlp_f32": [vp, C.POINTER(MlpDesc), vp, C.POINTER(vp), C.POINTER(vp), vp],
    "sofie_cuda_unary_f32": [vp, i32, f32, vp, vp, sz],
    "sofie_cuda_binary_f32": [vp, C.POINTER(BinaryDesc), vp, vp, vp],
    "sofie_cuda_batchnorm_f32": [vp, C.POINTER(BatchNormDesc), vp, vp, vp, vp, vp],
    "sofie_cuda_nchw_to_nhwc_f32": [vp, vp, vp, i32, i32, i32, i32],
    "sofie_cuda_nhwc_to_nchw_f32": [vp, vp, vp, i32, i32, i32, i32],
    "sofie_cuda_quantize_u8": [vp, vp, vp, sz, f32, i32],
    "sofie_cuda_dequantize_u8": [vp, vp, vp, sz, f32, i32],
    "sofie_cuda_qlinear_prepare": [vp, i32, i32, vp, i32, f32, i32, vp, f32, vp, vp, vp],
    "sofie_cuda_qlinear_matmul": [vp, C.POINTER(QGemmDesc), vp, vp, vp, vp, vp],
    "sofie_cuda_qlinear_matmul_f32": [vp, C.POINTER(QGemmDesc), vp, vp, vp, vp, f32, vp],
    "sofie_cuda_transpose_i8": [vp, vp, vp, i32, i32],
    "sofie_cuda_qlinear_conv2d": [vp, C.POINTER(QConv2dDesc), vp, vp, vp, vp, vp],
    "sofie_cuda_qconv2d_pack_i8": [vp, C.POINTER(QConv2dDesc), vp, vp],
    "sofie_cuda_maxpool2d_u8": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32],
    "sofie_cuda_nchw_to_nhwc_u8": [vp, vp, vp, i32, i32, i32, i32],
    "sofie_cuda_nhwc_to_nchw_u8": [vp, vp, vp, i32, i32, i32, i32],
    "sofie_cuda_quantize_e4m3_f32": [vp, vp, vp, sz, f32],
    "sofie_cuda_quantize_e4m3_bf16": [vp, vp, vp, sz, f32],
    "sofie_cuda_cast_bf16_f32": [vp, vp, vp, sz],
    "sofie_cuda_cast_f32_bf16": [vp, vp, vp, sz],
    "sofie_cuda_amax_f32": [vp, vp, sz, vp],
    "sofie_cuda_gemm_e4m3": [vp, C.POINTER(Fp8GemmDesc), vp, vp, vp, vp, vp],
    "sofie_cuda_gemm_e4m3_f32": [vp, C.POINTER(Fp8GemmDesc), vp, vp, vp, vp],
    "sofie_cuda_dynamic_quantize_e4m3_f32": [vp, vp, vp, sz, vp],
    "sofie_cuda_dynamic_quantize_e4m3_bf16": [vp, vp, vp, sz, vp],
    "sofie_cuda_gemm_e4m3_dynamic": [vp, C.POINTER(Fp8GemmDesc), vp, vp, vp, vp, vp, vp],
}
STRING_GETTERS = {"sofie_cuda_strerror": [C.c_int], "sofie_cuda_last_error": []}
SIZE_GETTERS = {"sofie_cuda_mlp_f32_smem": [C.POINTER(MlpDesc)],
                "sofie_cuda_conv_transpose2d_f32_gemm_scratch": [C.POINTER(ConvTranspose2dDesc)]}
MLP_MAX_LAYERS, MLP_MAX_WIDTH, MLP_MAX_SMEM = 8, 256, 200 * 1024

_lib = None


def library_path() -> Path:
    return _build.LIB


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load libSOFIE_cuda.so (building it in-tree first when it is absent or stale)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build() if build_if_missing else _build.LIB
    if not Path(path).exists():
        raise RuntimeError(f"{path} is missing: the CUDA back end was not built and there is no other back end")
    lib = C.CDLL(str(path))
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    for name, args in STRING_GETTERS.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_char_p
    for name, args in SIZE_GETTERS.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_size_t
    if lib.sofie_cuda_abi_version() != 1:
        raise RuntimeError("libSOFIE_cuda ABI version mismatch")
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != OK:
        lib = load()
        detail = lib.sofie_cuda_last_error().decode() or lib.sofie_cuda_strerror(status).decode()
        raise SofieCudaError(status, what, detail)


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise SofieCudaError on a non-zero status."""
    check(getattr(load(), name)(*args), name)
