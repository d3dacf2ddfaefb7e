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


# Shapes with at least 296 tiles of 256 x 256 run on CTA pairs (cta_group::2); ragged M and N included.
@pytest.mark.parametrize("M,N,K,relu,zp", [(19000, 1000, 256, 1, 128), (2048 * 19, 512, 128, 0, 7)])
def test_qlinear_matmul_pair_kernel_bit_exact(M, N, K, relu, zp):
    rng = np.random.default_rng(M + N + K)
    A = rng.integers(0, 256, (M, K)).astype(np.uint8)
    W = rng.integers(-127, 128, (N, K)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, N).astype(np.float32)
    y_scale = 0.02 * np.sqrt(K) * 0.3
    ref = o.qlinear_matmul(A, 0.02, zp, W, ws, y_scale, 128, w_is_nk=True, relu=bool(relu))
    mult, corr = ops.qlinear_prepare(W, True, 0.02, zp, ws, y_scale, None, "cuda")
    for _ in range(2):  # a second launch reuses the barriers' initial state and TMEM
        y = ops.qlinear_matmul(dev(A), dev(W), mult, corr, w_is_nk=True, y_zp=128, relu=bool(relu)).cpu().numpy()
        assert ops.last_engine() == capi.ENGINE_TCGEN05
        assert np.array_equal(y, ref)
    assert len(np.unique(ref)) > 20


def test_gemm_e4m3_pair_kernel():
    M, N, K = 19200, 1024, 256
    rng = np.random.default_rng(3)
    X = rng.standard_normal((M, K)).astype(np.float32)
    Wf = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    sa, sw = float(np.abs(X).max() / 448), float(np.abs(Wf).max() / 448)
    Aq, Wq = o.quantize_e4m3(X, sa), o.quantize_e4m3(Wf, sw)
    ref = o.bf16_bits_to_f32(o.gemm_e4m3(Aq, sa, Wq, sw, bias, relu=True))
    Y, Yq = ops.gemm_e4m3(dev(Aq), dev(Wq), dev(bias), a_scale=sa, w_scale=sw, relu=True, q_scale=0.01)
    y = Y.float().cpu().numpy()
    assert rel_err(y, ref) <= 8e-3
    assert np.array_equal(Yq.cpu().numpy(), o.quantize_e4m3(y, 0.01))


# ------------------------------------------------------------------------------------ implicit-GEMM convolution
CONV_TC = [
    # N, C, H, W, Cout, relu, pool
    (4, 16, 32, 32, 32, 1, 2), (6, 32, 16, 16, 64, 1, 2), (5, 64, 8, 8, 128, 1, 0), (5, 64, 8, 8, 128, 0, 2),
    (3, 8, 16, 24, 20, 1, 0), (2, 32, 64, 64, 64, 1, 2), (300, 16, 32, 32, 32, 1, 2), (1, 128, 8, 16, 16, 0, 0),
    # haloed-patch kernel: channels streamed in plane groups, partial channel chunks, wide tiles
    (2, 64, 16, 16, 32, 0, 0), (2, 16, 48, 40, 48, 1, 2), (2, 32, 32, 16, 128, 1, 2), (3, 16, 16, 8, 8, 0, 2),
]


@pytest.mark.parametrize("case", CONV_TC)
def test_conv3x3_f32_tcgen05(case):
    N, C, H, W, Cout, relu, pool = case
    rng = np.random.default_rng(sum(case))
    X = rng.standard_normal((N, C, H, W)).astype(np.float32)
    Wt = (rng.standard_normal((Cout, C, 3, 3)) * 0.2).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32)
    ref = o.conv2d_f32(X, Wt, b, pad=(1, 1), relu=bool(relu))
    if pool:
        ref = o.pool2d_f32(ref, 0, (2, 2), (2, 2))
    y = ops.conv2d_f32(dev(X.transpose(0, 2, 3, 1)), ops.conv2d_pack_f32(dev(Wt)), dev(b), shape=X.shape, pad=(1, 1),
                       relu=bool(relu), pool=pool, x_layout=1, y_layout=1, w_packed=True, kernel=(3, 3))
    assert ops.last_engine() == capi.ENGINE_TCGEN05
    assert rel_err(y.cpu().numpy().transpose(0, 3, 1, 2), ref) <= 1e-5


@pytest.mark.parametrize("case", [(3, 32, 32, 32, 64, 1, 2), (7, 64, 16, 16, 64, 1, 2), (9, 64, 8, 8, 128, 1, 2), (2, 32, 16, 16, 40, 0, 0),
                                  (130, 32, 32, 32, 64, 1, 2), (3, 128, 16, 16, 128, 1, 2), (2, 256, 16, 16, 32, 0, 0),
                                  (2, 128, 32, 16, 64, 1, 0), (5, 32, 16, 16, 24, 1, 2),
                                  # pooled-window kernel (32 x 16 tiles, pooling in tensor memory): two K steps per tap, 32 and 48
                                  # output channels, no Relu, several tiles per image in both directions, more tiles than SMs
                                  (2, 64, 32, 32, 64, 1, 2), (2, 32, 64, 48, 32, 0, 2), (3, 64, 32, 16, 48, 1, 2), (40, 32, 64, 32, 16, 1, 2),
                                  # lines of eight pixels with more tiles than SMs (per-tap kernel with resident weights): two images per
                                  # tile, one image per tile, 32-byte pixels
                                  (301, 64, 8, 8, 128, 1, 2), (310, 64, 8, 8, 72, 0, 0), (160, 64, 16, 8, 64, 1, 2), (300, 32, 8, 8, 32, 1, 0)])
def test_qlinear_conv3x3_tcgen05_bit_exact(case):
    N, C, H, W, Cout, relu, pool = case
    rng = np.random.default_rng(sum(case))
    X = (rng.integers(0, 256, (N, C, H, W)) * (rng.random((N, C, H, W)) < 0.4)).astype(np.uint8)
    Wt = rng.integers(-127, 128, (Cout, C, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, Cout).astype(np.float32)
    bias = rng.integers(-1000, 1000, Cout).astype(np.int32)
    y_scale = 0.05 * 0.005 * 127 * 80 * np.sqrt(C * 9) / 100
    ref = o.qlinear_conv2d(X, 0.05, 0, Wt, ws, y_scale, 3, bias=bias, pad=(1, 1), relu=bool(relu))
    if pool:
        ref = o.maxpool2d_u8(ref)
    mult = dev(o.requant_multiplier(0.05, ws, y_scale))
    y = ops.qlinear_conv2d(dev(X.transpose(0, 2, 3, 1)), ops.qconv2d_pack_i8(dev(Wt)), mult, dev(bias), shape=X.shape, pad=(1, 1),
                           x_zp=0, y_zp=3, relu=bool(relu), pool=pool, x_layout=1, y_layout=1, w_packed=True, kernel=(3, 3))
    assert ops.last_engine() == capi.ENGINE_TCGEN05
    assert np.array_equal(y.cpu().numpy().transpose(0, 3, 1, 2), ref)
    assert len(np.unique(ref)) > 20


@pytest.mark.parametrize("case", [(3, 64, 64, 32, 1, 0), (2, 32, 48, 16, 0, 7), (5, 96, 32, 64, 1, 0), (150, 64, 64, 32, 1, 3), (1, 32, 16, 48, 1, 200)])
def test_qlinear_first_layer_pooled_tcgen05_bit_exact(case):
    """One input channel, 3x3 / pad 1, Relu or not, MaxPool 2x2 fused: the tensor-core first-layer kernel (operand rows built
    from the staged image rows, pooling in tensor memory) against the oracle, NCHW input as the Session hands it over."""
    N, H, W, Cout, relu, y_zp = case
    ops.set_engine(0)
    rng = np.random.default_rng(sum(case))
    X = (rng.integers(0, 256, (N, 1, H, W)) * (rng.random((N, 1, H, W)) < 0.3)).astype(np.uint8)
    X[0, 0, 0, :] = 255
    X[0, 0, :, -1] = 255                       # bright borders next to the padding
    Wt = rng.integers(-127, 128, (Cout, 1, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, Cout).astype(np.float32)
    bias = rng.integers(-300, 300, Cout).astype(np.int32)
    y_scale = 0.03 * 0.005 * 127 * 6
    ref = o.maxpool2d_u8(o.qlinear_conv2d(X, 0.03, 0, Wt, ws, y_scale, y_zp, bias=bias, pad=(1, 1), relu=bool(relu)))
    mult = dev(o.requant_multiplier(0.03, ws, y_scale))
    y = ops.qlinear_conv2d(dev(X), dev(Wt), mult, dev(bias), shape=X.shape, pad=(1, 1), x_zp=0, y_zp=y_zp, relu=bool(relu), pool=2,
                           x_layout=0, y_layout=1, w_packed=False)
    assert ops.last_engine() == capi.ENGINE_TCGEN05
    assert np.array_equal(y.cpu().numpy().transpose(0, 3, 1, 2), ref)
    assert len(np.unique(ref)) > 20


@pytest.mark.parametrize("case", [(3, 32, 32, 32, 64), (2, 64, 16, 16, 64), (4, 1, 32, 32, 16), (2, 64, 8, 8, 128), (2, 64, 32, 32, 32)])
def test_qconv_pool_with_negative_multipliers(case):
    """A negative requantisation multiplier makes the requantisation decreasing in the accumulator, so the
    kernels must not pool the raw accumulators first; they detect it and pool the finished values."""
    N, C, H, W, Cout = case
    if C <= 4:
        ops.set_engine(0)  # the first-layer kernel is a CUDA-core kernel; this file forces tcgen05 otherwise
    rng = np.random.default_rng(sum(case))
    X = rng.integers(0, 256, (N, C, H, W)).astype(np.uint8)
    Wt = rng.integers(-127, 128, (Cout, C, 3, 3)).astype(np.int8)
    ws = (rng.uniform(0.001, 0.01, Cout) * rng.choice([-1.0, 1.0], Cout)).astype(np.float32)
    assert (ws < 0).any() and (ws > 0).any()
    y_scale = 0.02 * 0.005 * 128 * 3 * np.sqrt(C)
    ref = o.maxpool2d_u8(o.qlinear_conv2d(X, 0.02, 0, Wt, ws, y_scale, 100, pad=(1, 1), relu=False))
    mult = dev(o.requant_multiplier(0.02, ws, y_scale))
    y = ops.qlinear_conv2d(dev(X.transpose(0, 2, 3, 1)), ops.qconv2d_pack_i8(dev(Wt)), mult, None, shape=X.shape, pad=(1, 1),
                           x_zp=0, y_zp=100, relu=False, pool=2, x_layout=1, y_layout=1, w_packed=True, kernel=(3, 3)).cpu().numpy()
    assert np.array_equal(y.transpose(0, 3, 1, 2), ref)
    assert len(np.unique(ref)) > 20
