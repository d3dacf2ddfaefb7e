"""GPU parity of the tcgen05 / TMEM / TMA GEMM kernels (engine forced to the tensor-core family, so a
shape the kernel does not take fails instead of silently running on CUDA cores).
fp32 (3xTF32): tensor-relative error <= 1e-5 against the oracle; int8: bit-exact; FP8: <= 2e-2."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import rel_err
from oracle import cpu_oracle as o
from sofie_b200 import capi, ops

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def umma_engine(cuda_device):
    ops.set_engine(capi.ENGINE_TCGEN05)
    yield
    ops.set_engine(0)
    ctx = C.c_void_p()
    capi.call("sofie_cuda_ctx_create", C.byref(ctx), 0, 0)
    try:
        capi.call("sofie_cuda_ctx_check", ctx)  # no kernel gave up on a wait
    finally:
        capi.call("sofie_cuda_ctx_destroy", ctx)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("M,N,K,bias,relu", [(128, 128, 32, 0, 0), (128, 128, 128, 1, 1), (1024, 128, 64, 1, 1),
                                             (1024, 10, 128, 1, 0), (300, 72, 260, 2, 1), (1, 7, 4, 0, 0),
                                             (256, 10, 4096, 1, 0), (513, 384, 1000, 1, 1), (4096, 256, 512, 1, 1)])
def test_gemm_f32_3xtf32(M, N, K, bias, relu):
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((N, K)).astype(np.float32)
    Cb = None if bias == 0 else rng.standard_normal((N,) if bias == 1 else (M, N)).astype(np.float32)
    ref = o.gemm_f32(A, B, Cb, transB=1, alpha=1.25, beta=0.5, relu=bool(relu))
    y = ops.gemm_f32(dev(A), dev(B), None if Cb is None else dev(Cb), transB=1, alpha=1.25, beta=0.5, relu=bool(relu))
    assert ops.last_engine() == capi.ENGINE_TCGEN05
    assert rel_err(y.cpu().numpy(), ref) <= 1e-5


def test_gemm_f32_shape_outside_tensor_core_kernel_is_refused_when_forced():
    A, B = torch.zeros((8, 6), device="cuda"), torch.zeros((4, 6), device="cuda")   # K*4 not a multiple of 16
    with pytest.raises(capi.SofieCudaError) as e:
        ops.gemm_f32(A, B, transB=1)
    assert e.value.status == capi.ERR_UNSUPPORTED
    ops.set_engine(0)  # automatic: the CUDA-core kernel takes it
    ops.gemm_f32(A, B, transB=1)
    assert ops.last_engine() == capi.ENGINE_SIMT


@pytest.mark.parametrize("M,N,K,relu,zp", [(128, 32, 128, 0, 128), (8192 // 8, 1024, 512, 0, 128), (100, 40, 48, 1, 3),
                                           (700, 256, 2048, 1, 0), (257, 2, 256, 0, 128), (130, 1000, 1024, 0, 128)])
def test_qlinear_matmul_tcgen05_bit_exact(M, N, K, relu, zp):
    rng = np.random.default_rng(N + K)
    A = rng.integers(0, 256, (M, K)).astype(np.uint8)
    W = rng.integers(-127, 128, (N, K)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, N).astype(np.float32)
    y_scale = 0.02 * np.sqrt(K) * 0.3
    ref = o.qlinear_matmul(A, 0.02, zp, W, ws, y_scale, 128, w_is_nk=True, relu=bool(relu))
    mult, corr = ops.qlinear_prepare(W, True, 0.02, zp, ws, y_scale, None, "cuda")
    y = ops.qlinear_matmul(dev(A), dev(W), mult, corr, w_is_nk=True, y_zp=128, relu=bool(relu)).cpu().numpy()
    assert ops.last_engine() == capi.ENGINE_TCGEN05
    assert np.array_equal(y, ref)
    assert len(np.unique(ref)) > 20


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (70, 45, 144), (1000, 512, 4096), (256, 4096, 512)])
def test_gemm_e4m3_tcgen05(M, N, K):
    rng = np.random.default_rng(K + M)
    X = rng.standard_normal((M, K)).astype(np.float32)
    Wf = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    sa, sw = float(np.abs(X).max() / 448), float(np.abs(Wf).max() / 448)
    Aq, Wq = o.quantize_e4m3(X, sa), o.quantize_e4m3(Wf, sw)
    ref = o.bf16_bits_to_f32(o.gemm_e4m3(Aq, sa, Wq, sw, bias, relu=True))
    Y, Yq = ops.gemm_e4m3(dev(Aq), dev(Wq), dev(bias), a_scale=sa, w_scale=sw, relu=True, q_scale=0.01)
    assert ops.last_engine() == capi.ENGINE_TCGEN05
    y = Y.float().cpu().numpy()
    assert rel_err(y, ref) <= 2e-2
    assert rel_err(y, ref) <= 8e-3
    assert np.array_equal(Yq.cpu().numpy(), o.quantize_e4m3(y, 0.01))


def test_tensor_core_and_cuda_core_kernels_agree():
    rng = np.random.default_rng(11)
    A = rng.standard_normal((640, 256)).astype(np.float32)
    B = rng.standard_normal((192, 256)).astype(np.float32)
    y_tc = ops.gemm_f32(dev(A), dev(B), transB=1).cpu().numpy()
    ops.set_engine(capi.ENGINE_SIMT)
    y_cc = ops.gemm_f32(dev(A), dev(B), transB=1).cpu().numpy()
    assert rel_err(y_tc, y_cc) <= 1e-5
