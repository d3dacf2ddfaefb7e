"""GPU parity of every operator of the dense-contraction path, through the C ABI, against the CPU
oracle and the reference's golden vectors. The contractions run here on the CUDA-core kernels
(engine forced); the tcgen05 kernels have their own file.
Tolerances: fp32 1e-5 (tensor-relative, helpers.rel_err), int8 bit-exact, FP8 2e-2."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import CudaBackend, FIXTURE_CASES, load_fixtures, rel_err, run_fixture
from oracle import cpu_oracle as o
from sofie_b200 import capi, ops

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5


@pytest.fixture(autouse=True)
def simt_engine(cuda_device):
    ops.set_engine(capi.ENGINE_SIMT)
    yield
    ops.set_engine(0)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("name", FIXTURE_CASES)
def test_reference_golden_vectors(name):
    manifest, arrays = load_fixtures()
    y = run_fixture(name, manifest, arrays, CudaBackend())
    exp = arrays[f"{name}/expected"]
    assert y.shape == exp.shape
    assert np.abs(y - exp).max() <= 1e-3  # the reference's own tolerance for these vectors


@pytest.mark.parametrize("M,N,K,tA,tB,bias", [(1, 1, 1, 0, 0, 0), (37, 29, 53, 0, 0, 1), (64, 128, 64, 0, 1, 1),
                                              (130, 70, 257, 1, 1, 2), (5, 300, 17, 1, 0, 0), (1024, 10, 128, 0, 1, 1),
                                              (256, 10, 4096, 0, 1, 1),
                                              # skinny shapes of the split-K kernel: ragged K, both B layouts, full bias
                                              (24, 10, 4096, 0, 1, 1), (100, 16, 1500, 0, 0, 2), (300, 7, 2050, 0, 1, 2),
                                              (129, 16, 1025, 0, 0, 1), (640, 1, 8192, 0, 1, 0),
                                              # one-launch row-block kernel: rows not a multiple of 4, every bias kind, widest N
                                              (2, 10, 1024, 0, 1, 2), (1027, 16, 4096, 0, 1, 1), (2048, 3, 1028, 0, 1, 0)])
def test_gemm_f32(M, N, K, tA, tB, bias):
    rng = np.random.default_rng(M * 7 + N)
    A = rng.standard_normal((K, M) if tA else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if tB else (K, N)).astype(np.float32)
    Cb = None if bias == 0 else rng.standard_normal((N,) if bias == 1 else (M, N)).astype(np.float32)
    ref = o.gemm_f32(A, B, Cb, transA=tA, transB=tB, alpha=0.75, beta=1.5, relu=True)
    y = ops.gemm_f32(dev(A), dev(B), None if Cb is None else dev(Cb), transA=tA, transB=tB, alpha=0.75, beta=1.5,
                     relu=True).cpu().numpy()
    assert ops.last_engine() == capi.ENGINE_SIMT
    assert rel_err(y, ref) <= FP32_TOL


def _mlp_reference(x, Ws, Bs, relu, nk):
    for W, b, r, t in zip(Ws, Bs, relu, nk):
        x = o.gemm_f32(x, W, b, transB=int(t), relu=bool(r))
    return x


@pytest.mark.parametrize("M,dims,relu,nk,bias", [
    (1024, (64, 128, 128, 10), (1, 1, 0), (1, 1, 1), (1, 1, 1)),      # the three-layer perceptron configuration
    (1, (7, 5), (0,), (1,), (0,)),                                    # one row, one layer, no bias
    (33, (19, 45, 3), (1, 1), (0, 1), (1, 0)),                        # ragged rows and widths, both weight layouts
    (257, (256, 96, 1), (0, 1), (1, 0), (1, 1)),                      # the widest layer the kernel takes
    (300, (150, 100, 7), (1, 0), (1, 1), (1, 1)),                     # widths that are not multiples of 4: element-wise staging
    (20000, (64, 128, 128, 10), (1, 1, 0), (1, 1, 1), (1, 1, 1)),     # several tiles per block: the input prefetch
    (5000, (32, 64, 32, 64, 32, 64, 32, 64, 8), (1, 0, 1, 0, 1, 0, 1, 1), (1, 0, 1, 0, 1, 0, 1, 0), (1,) * 8),  # eight layers, more tiles than SMs
    (96, (100, 33, 200), (1, 0), (0, 0), (0, 1)),
    # widths the tensor-core chain takes: weights stored [K,N], a K that ends in a partial stage (40 = 32 + 8), four layers,
    # a last slab of one row, an output narrower than its 16-column chunk, no bias
    (300, (40, 48, 16), (1, 0), (0, 1), (1, 1)),
    (129, (8, 16, 128, 32, 3), (1, 1, 0, 1), (1, 0, 1, 0), (0, 1, 0, 1)),
    (1, (128, 128), (1,), (1,), (0,)),
    (19000, (24, 112, 5), (1, 0), (1, 1), (1, 1)),                     # more slabs than SMs
])
@pytest.mark.parametrize("engine", ["auto", "tcgen05"])
def test_mlp_f32_fused_chain(M, dims, relu, nk, bias, engine):
    tensor_shape = (len(dims) <= 5 and all(k % 8 == 0 and k <= 128 for k in dims[:-1]) and all(n <= 128 for n in dims[1:])
                    and all(n % 16 == 0 for n in dims[1:-1]))
    if engine == "tcgen05" and not tensor_shape:
        pytest.skip("widths outside the tensor-core chain")
    capi.call("sofie_cuda_set_engine", capi.ENGINE_TCGEN05 if engine == "tcgen05" else 0)
    rng = np.random.default_rng(M + len(dims))
    x = rng.standard_normal((M, dims[0])).astype(np.float32)
    Ws, Bs = [], []
    for l in range(len(dims) - 1):
        K, N = dims[l], dims[l + 1]
        Ws.append((rng.standard_normal((N, K) if nk[l] else (K, N)) / np.sqrt(K)).astype(np.float32))
        Bs.append(rng.standard_normal(N).astype(np.float32) if bias[l] else None)
    ref = _mlp_reference(x, Ws, Bs, relu, nk)
    try:
        y = ops.mlp_f32(dev(x), [dev(W) for W in Ws], [None if b is None else dev(b) for b in Bs], relu, nk).cpu().numpy()
        used = ops.last_engine()
    finally:
        capi.call("sofie_cuda_set_engine", 0)
    assert used == (capi.ENGINE_TCGEN05 if engine == "tcgen05" else capi.ENGINE_SIMT)
    assert y.shape == ref.shape and rel_err(y, ref) <= FP32_TOL


def test_mlp_f32_limits_and_empty_batch():
    W = torch.zeros((8, 300), device="cuda")
    with pytest.raises(capi.SofieCudaError) as e:
        ops.mlp_f32(torch.zeros((4, 300), device="cuda"), [W], [None], [0], [1])       # wider than the kernel takes
    assert e.value.status == capi.ERR_UNSUPPORTED
    Ws = [torch.zeros((256, 256), device="cuda") for _ in range(4)]
    with pytest.raises(capi.SofieCudaError) as e:
        ops.mlp_f32(torch.zeros((4, 256), device="cuda"), Ws, [None] * 4, [0] * 4, [1] * 4)  # weights beyond shared memory
    assert e.value.status == capi.ERR_UNSUPPORTED
    y = ops.mlp_f32(torch.zeros((0, 300 - 44), device="cuda"), [torch.zeros((8, 256), device="cuda")], [None], [0], [1])
    assert y.shape == (0, 8)


def test_gemm_empty_batch_and_bad_arguments():
    B = torch.zeros((4, 8), device="cuda")
    y = ops.gemm_f32(torch.zeros((0, 8), device="cuda"), B, transB=1)
    assert y.shape == (0, 4)
    with pytest.raises(capi.SofieCudaError) as e:
        d = capi.GemmF32Desc(4, 4, 4, 0, 0, 1.0, 1.0, 1, 0)  # bias_kind set, C NULL
        capi.call("sofie_cuda_gemm_f32", None, d, B.data_ptr(), B.data_ptr(), None, B.data_ptr())
    assert e.value.status == capi.ERR_INVALID


CONV_CASES = [
    # N, C, H, W, Cout, k, pad, stride, dil, group
    (2, 3, 9, 8, 4, (3, 3), (1, 1), (1, 1), (1, 1), 1),
    (1, 1, 5, 5, 1, (3, 3), (0, 0), (1, 1), (1, 1), 1),
    (3, 4, 11, 9, 6, (3, 3), (1, 1), (2, 1), (1, 1), 2),
    (2, 3, 12, 12, 5, (5, 5), (2, 2), (1, 1), (1, 1), 1),
    (2, 8, 10, 10, 20, (3, 3), (2, 2), (1, 1), (2, 2), 1),
    (2, 6, 7, 7, 6, (1, 1), (0, 0), (1, 1), (1, 1), 6),
    (4, 16, 32, 32, 32, (3, 3), (1, 1), (1, 1), (1, 1), 1),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv2d_f32_nchw(case):
    N, C, H, W, Cout, k, pad, stride, dil, group = case
    rng = np.random.default_rng(sum(case[:5]))
    X = rng.standard_normal((N, C, H, W)).astype(np.float32)
    Wt = rng.standard_normal((Cout, C // group, *k)).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32)
    ref = o.conv2d_f32(X, Wt, b, pad=pad, stride=stride, dil=dil, group=group)
    y = ops.conv2d_f32(dev(X), dev(Wt), dev(b), pad=pad, stride=stride, dil=dil, group=group).cpu().numpy()
    assert rel_err(y, ref) <= FP32_TOL
    y2 = ops.conv2d_f32(dev(X), dev(Wt), None, pad=pad, stride=stride, dil=dil, group=group).cpu().numpy()
    assert rel_err(y2, o.conv2d_f32(X, Wt, None, pad=pad, stride=stride, dil=dil, group=group)) <= FP32_TOL


@pytest.mark.parametrize("x_nhwc,y_nhwc,packed,relu,pool", [(0, 1, 0, 1, 0), (1, 1, 1, 1, 2), (1, 0, 1, 0, 2),
                                                           (0, 0, 0, 1, 2), (1, 1, 0, 0, 0)])
def test_conv2d_f32_layouts_and_fusion(x_nhwc, y_nhwc, packed, relu, pool):
    rng = np.random.default_rng(5)
    N, C, H, W, Cout = 3, 16, 10, 14, 24   # odd pooled extents are covered by H=10 -> 5
    X = rng.standard_normal((N, C, H, W)).astype(np.float32)
    Wt = rng.standard_normal((Cout, C, 3, 3)).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32)
    ref = o.conv2d_f32(X, Wt, b, pad=(1, 1), relu=bool(relu))
    if pool:
        ref = o.pool2d_f32(ref, 0, (2, 2), (2, 2))
    Xd = dev(X.transpose(0, 2, 3, 1)) if x_nhwc else dev(X)
    Wd = ops.conv2d_pack_f32(dev(Wt)) if packed else dev(Wt)
    y = ops.conv2d_f32(Xd, Wd, dev(b), shape=(N, C, H, W), pad=(1, 1), relu=bool(relu), pool=pool, x_layout=x_nhwc,
                       y_layout=y_nhwc, w_packed=bool(packed), kernel=(3, 3)).cpu().numpy()
    if y_nhwc:
        y = y.transpose(0, 3, 1, 2)
    assert rel_err(y, ref) <= FP32_TOL


@pytest.mark.parametrize("case", [
    # N, C, H, W, Cout, k, pad, stride, dil, out_pad, bias, relu
    (2, 3, 5, 6, 4, (3, 3), (0, 0), (1, 1), (1, 1), (0, 0), True, False),
    (1, 1, 3, 3, 2, (3, 3), (0, 0), (1, 1), (1, 1), (0, 0), False, False),
    (3, 8, 7, 5, 6, (2, 2), (0, 0), (2, 2), (1, 1), (0, 0), True, True),
    (2, 6, 9, 9, 3, (3, 3), (1, 1), (2, 2), (1, 1), (1, 1), True, False),      # the usual 2x upsampling layer
    (2, 5, 6, 4, 7, (3, 2), (1, 0), (3, 2), (2, 1), (2, 1), False, False),     # dilation, output_padding, Cout not a multiple of 4
    (1, 4, 1, 17, 5, (1, 5), (0, 2), (1, 3), (1, 1), (0, 0), True, False),     # a 1-D transposed convolution
    (4, 32, 16, 16, 16, (4, 4), (1, 1), (2, 2), (1, 1), (0, 0), True, True),
])
def test_conv_transpose2d_f32(case):
    N, Cin, H, W, Cout, k, pad, stride, dil, out_pad, bias, relu = case
    rng = np.random.default_rng(N * 100 + Cin)
    X = rng.standard_normal((N, Cin, H, W)).astype(np.float32)
    Wt = (rng.standard_normal((Cin, Cout) + k) / np.sqrt(Cin * k[0] * k[1])).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32) if bias else None
    ref = o.conv_transpose2d_f32(X, Wt, b, pad=pad, stride=stride, dil=dil, out_pad=out_pad)
    if relu:
        ref = o.relu_f32(ref)
    y = ops.conv_transpose2d_f32(dev(X), dev(Wt), None if b is None else dev(b), pad=pad, stride=stride, dil=dil, out_pad=out_pad,
                                 relu=relu).cpu().numpy()
    assert y.shape == ref.shape and rel_err(y, ref) <= FP32_TOL


@pytest.mark.parametrize("case", [
    # N, C, H, W, Cout, k, pad, stride, dil, out_pad, bias, relu
    (4, 32, 16, 16, 16, (4, 4), (1, 1), (2, 2), (1, 1), (0, 0), True, True),       # the usual 2x upsampling layer of a decoder
    (2, 16, 7, 5, 6, (3, 2), (1, 0), (3, 2), (2, 1), (2, 1), False, False),        # dilation, output_padding, Cout not a multiple of 4
    (3, 64, 8, 8, 32, (2, 2), (0, 0), (2, 2), (1, 1), (0, 0), True, False),        # stride = kernel: every output has one tap
    (1, 20, 1, 33, 8, (1, 5), (0, 2), (1, 3), (1, 1), (0, 0), True, True),         # 1-D, C not a multiple of 8 (the GEMM's own fallback)
    (5, 128, 12, 12, 64, (3, 3), (1, 1), (1, 1), (1, 1), (0, 0), True, False),     # stride 1: nine taps per output
])
def test_conv_transpose2d_f32_product_form(case):
    """The entry point that lowers to one GEMM over all images plus a gather (the reference's own lowering, on the tensor cores)."""
    N, Cin, H, W, Cout, k, pad, stride, dil, out_pad, bias, relu = case
    rng = np.random.default_rng(N * 100 + Cin)
    X = rng.standard_normal((N, Cin, H, W)).astype(np.float32)
    Wt = (rng.standard_normal((Cin, Cout) + k) / np.sqrt(Cin * k[0] * k[1])).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32) if bias else None
    ref = o.conv_transpose2d_f32(X, Wt, b, pad=pad, stride=stride, dil=dil, out_pad=out_pad)
    if relu:
        ref = o.relu_f32(ref)
    capi.call("sofie_cuda_set_engine", 0)
    y = ops.conv_transpose2d_f32(dev(X), dev(Wt), None if b is None else dev(b), pad=pad, stride=stride, dil=dil, out_pad=out_pad,
                                 relu=relu, product_form=True).cpu().numpy()
    assert y.shape == ref.shape and rel_err(y, ref) <= FP32_TOL
    if Cin % 8 == 0 and N * H * W >= 128:
        assert ops.last_engine() == capi.ENGINE_TCGEN05


def test_conv_transpose2d_product_form_limits():
    lib = capi.load()
    small = capi.ConvTranspose2dDesc(1, 8, 4, 4, 4, 3, 3, 0, 0, 1, 1, 1, 1, 0, 0, 0)       # fewer than 16 input channels
    assert lib.sofie_cuda_conv_transpose2d_f32_gemm_scratch(C.byref(small)) == 0
    x = torch.zeros(4096, device="cuda")
    p = C.c_void_p(x.data_ptr())
    assert lib.sofie_cuda_conv_transpose2d_f32_gemm(None, C.byref(small), p, p, None, p, p, 16384) == capi.ERR_UNSUPPORTED
    d = capi.ConvTranspose2dDesc(1, 16, 4, 4, 4, 3, 3, 0, 0, 1, 1, 1, 1, 0, 0, 0)
    need = lib.sofie_cuda_conv_transpose2d_f32_gemm_scratch(C.byref(d))
    assert need == 4 * (256 + 576 + 576)                                           # 16*16 input, 9*4*16 filter, 16*36 product floats
    assert lib.sofie_cuda_conv_transpose2d_f32_gemm(None, C.byref(d), p, p, None, p, p, need - 1) == capi.ERR_INVALID
    assert b"needed" in lib.sofie_cuda_last_error()


def test_conv_transpose2d_empty_batch_and_bad_arguments():
    Wt = torch.zeros((3, 2, 3, 3), device="cuda")
    assert ops.conv_transpose2d_f32(torch.zeros((0, 3, 4, 4), device="cuda"), Wt).shape == (0, 2, 6, 6)
    with pytest.raises(capi.SofieCudaError) as e:   # the pads eat the whole output
        ops.conv_transpose2d_f32(torch.zeros((1, 3, 1, 1), device="cuda"), Wt, pad=(2, 2))
    assert e.value.status == capi.ERR_INVALID
    with pytest.raises(capi.SofieCudaError) as e:   # output_padding not below the stride
        ops.conv_transpose2d_f32(torch.zeros((1, 3, 4, 4), device="cuda"), Wt, stride=(2, 2), out_pad=(2, 0))
    assert e.value.status == capi.ERR_INVALID


@pytest.mark.parametrize("eq,sa,sb", [("abc,abd->ad", (2, 2, 3), (2, 2, 3)), ("abcd,abed->abce", (2, 1, 2, 3), (2, 1, 3, 3)), ("i,i->", (3,), (3,)),
                                      ("bij,bjk->bik", (5, 33, 17), (5, 17, 9)), ("ij,kj->ik", (40, 50), (60, 50)), ("ab,cd->acbd", (2, 3), (4, 5)),
                                      ("bhqd,bhkd->bhqk", (2, 3, 16, 8), (2, 3, 12, 8)), ("ij,ij", (7, 9), (7, 9))])
def test_einsum_f32(eq, sa, sb):
    rng = np.random.default_rng(len(eq))
    A, B = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
    ref = o.einsum_f32(eq, A, B)
    y = ops.einsum_f32(eq, dev(A), dev(B)).cpu().numpy()
    assert y.shape == ref.shape and rel_err(y, ref) <= FP32_TOL
    full = eq if "->" in eq else eq + "->"
    assert rel_err(ref, np.einsum(full, A.astype(np.float64), B.astype(np.float64)).astype(np.float32)) <= FP32_TOL


def test_relu_nan_negzero_and_ragged_sizes():
    for n in (0, 1, 3, 4, 5, 1023, 4099):
        x = np.random.default_rng(n).standard_normal(n).astype(np.float32)
        if n > 3:
            x[1], x[2], x[3] = np.nan, -0.0, -np.inf
        y = ops.relu_f32(dev(x)).cpu().numpy() if n else np.zeros(0, np.float32)
        ref = o.relu_f32(x) if n else y
        assert np.array_equal(y.view(np.uint32), ref.view(np.uint32))
    # unaligned pointers take the scalar path
    x = torch.randn(1001, device="cuda")
    assert torch.equal(ops.relu_f32(x[1:].contiguous()), torch.clamp_min(x[1:], 0))


@pytest.mark.parametrize("mode,k,s,pads,cip", [(0, (2, 2), (2, 2), (0, 0, 0, 0), 0), (0, (3, 2), (1, 1), (0, 0, 0, 0), 0),
                                               (0, (3, 3), (2, 2), (1, 1, 1, 1), 0), (1, (3, 2), (2, 1), (0, 0, 0, 0), 0),
                                               (1, (3, 3), (1, 1), (1, 1, 1, 1), 0), (1, (3, 3), (1, 1), (1, 1, 1, 1), 1)])
def test_pool2d_f32(mode, k, s, pads, cip):
    rng = np.random.default_rng(3)
    X = rng.standard_normal((2, 5, 9, 10)).astype(np.float32)
    ref = o.pool2d_f32(X, mode, k, s, pads, cip)
    y = ops.pool2d_f32(dev(X), mode=mode, kernel=k, stride=s, pads=pads, count_include_pad=cip).cpu().numpy()
    assert rel_err(y, ref) <= 1e-6
    y2 = ops.pool2d_f32(dev(X.transpose(0, 2, 3, 1)), mode=mode, kernel=k, stride=s, pads=pads, count_include_pad=cip,
                        layout=1, shape=X.shape).cpu().numpy().transpose(0, 3, 1, 2)
    assert rel_err(y2, ref) <= 1e-6


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("shape", [(3, 5, 8, 12), (2, 16, 64, 64), (1, 4, 2, 4), (2, 3, 6, 10)])
def test_pool2d_f32_window_2x2_stride_2(mode, shape):
    """The window every configuration pools with has kernels of its own (16-byte accesses) in both layouts; the last shape
    (W not a multiple of 4, C not a multiple of 4) stays on the general kernel."""
    X = np.random.default_rng(sum(shape)).standard_normal(shape).astype(np.float32)
    X[0, 0, 0, 0] = np.nan                                           # a NaN never wins a maximum (v > m is false), as in the reference
    ref = o.pool2d_f32(X, mode, (2, 2), (2, 2), (0, 0, 0, 0), 0)
    y = ops.pool2d_f32(dev(X), mode=mode).cpu().numpy()
    np.testing.assert_array_equal(y, ref)                            # exact; a NaN average is a NaN on both sides
    y2 = ops.pool2d_f32(dev(X.transpose(0, 2, 3, 1)), mode=mode, layout=1, shape=X.shape).cpu().numpy().transpose(0, 3, 1, 2)
    np.testing.assert_array_equal(y2, ref)


@pytest.mark.parametrize("stride,pad,dil,group,relu,bias", [((1, 1, 1), (1, 1, 1), (1, 1, 1), 1, True, True),
                                                            ((2, 1, 1), (1, 0, 2), (1, 2, 1), 2, False, True),
                                                            ((1, 2, 3), (0, 0, 0), (1, 1, 1), 4, False, False)])
def test_conv3d_f32(stride, pad, dil, group, relu, bias):
    rng = np.random.default_rng(21)
    X = rng.standard_normal((3, 4, 5, 6, 7)).astype(np.float32)
    W = (rng.standard_normal((8, 4 // group, 3, 2, 3)) / 6).astype(np.float32)
    b = rng.standard_normal(8).astype(np.float32) if bias else None
    ref = o.conv3d_f32(X, W, b, pad=pad, stride=stride, dil=dil, group=group, relu=relu)
    y = ops.conv3d_f32(dev(X), dev(W), None if b is None else dev(b), pad=pad, stride=stride, dil=dil, group=group, relu=relu).cpu().numpy()
    assert y.shape == ref.shape and rel_err(y, ref) <= FP32_TOL
    assert ops.conv3d_f32(torch.zeros((0, 4, 5, 6, 7), device="cuda"), dev(W), group=group).shape[0] == 0
    with pytest.raises(capi.SofieCudaError):                                        # kernel larger than the padded input
        ops.conv3d_f32(torch.zeros((1, 4, 1, 1, 1), device="cuda"), dev(W), group=group)


@pytest.mark.parametrize("mode,k,s,pads,cip", [(0, (2, 2, 2), (2, 2, 2), (0,) * 6, 0), (0, (3, 2, 2), (1, 2, 1), (1, 0, 1, 0, 1, 0), 0),
                                               (1, (2, 2, 2), (2, 2, 2), (0,) * 6, 0), (1, (3, 3, 3), (2, 2, 2), (1,) * 6, 0),
                                               (1, (3, 3, 3), (2, 2, 2), (1,) * 6, 1)])
def test_pool3d_f32(mode, k, s, pads, cip):
    X = np.random.default_rng(22).standard_normal((2, 3, 6, 5, 7)).astype(np.float32)
    ref = o.pool3d_f32(X, mode, k, s, pads, cip)
    y = ops.pool3d_f32(dev(X), mode=mode, kernel=k, stride=s, pads=pads, count_include_pad=cip).cpu().numpy()
    assert y.shape == ref.shape and rel_err(y, ref) <= 1e-6


@pytest.mark.parametrize("shape,axis", [((3,), 0), ((1, 3), 1), ((2, 3, 4), 1), ((2, 3, 4, 2), -2), ((64, 10), -1),
                                        ((5, 1000), 1), ((4, 7, 33), 0),
                                        ((1000, 10), 1), ((257, 32), 1), ((300, 1), 1),      # short rows: 256 rows per block, a ragged last block
                                        ((9, 36), 1), ((70, 256), 1), ((33, 1024), 1), ((5, 2048), 1),  # rows kept in registers
                                        ((3, 2052), 1), ((6, 1001), 1), ((4, 4096), 1)])     # longer or not a multiple of 4: re-read
def test_softmax_f32(shape, axis):
    X = np.random.default_rng(1).standard_normal(shape).astype(np.float32) * 3
    y = ops.softmax_f32(dev(X), axis).cpu().numpy()
    assert np.abs(y - o.softmax_f32(X, axis)).max() <= 1e-6
    # a view that starts 4 bytes into its buffer (not 16-byte aligned) takes the element-wise kernels
    if len(shape) == 2 and axis == 1:
        buf = torch.zeros(X.size + 1, device="cuda")
        buf[1:] = dev(X).flatten()
        y = ops.softmax_f32(buf[1:].view(shape), axis).cpu().numpy()
        assert np.abs(y - o.softmax_f32(X, axis)).max() <= 1e-6


def test_layout_round_trips():
    X = np.random.default_rng(2).standard_normal((3, 5, 7, 9)).astype(np.float32)
    nhwc = ops.nchw_to_nhwc(dev(X))
    assert np.array_equal(nhwc.cpu().numpy(), X.transpose(0, 2, 3, 1))
    assert np.array_equal(ops.nhwc_to_nchw(nhwc).cpu().numpy(), X)
    for shape in ((2, 4, 3, 5), (3, 16, 8, 8), (1, 64, 5, 7), (2, 68, 4, 4)):   # few channels, a multiple of 4: one thread per pixel
        X = np.random.default_rng(4).standard_normal(shape).astype(np.float32)
        nhwc = ops.nchw_to_nhwc(dev(X))
        assert np.array_equal(nhwc.cpu().numpy(), X.transpose(0, 2, 3, 1))
        assert np.array_equal(ops.nhwc_to_nchw(nhwc).cpu().numpy(), X)
    U = np.random.default_rng(2).integers(0, 256, (2, 33, 6, 5)).astype(np.uint8)
    assert np.array_equal(ops.nhwc_to_nchw(ops.nchw_to_nhwc(dev(U))).cpu().numpy(), U)
    Wm = np.random.default_rng(2).standard_normal((45, 70)).astype(np.float32)
    assert np.array_equal(ops.transpose2d(dev(Wm)).cpu().numpy(), Wm.T)


# ------------------------------------------------------------------------------------ int8
def test_quantize_dequantize_u8_bit_exact():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(10007) * 2, np.arange(-300, 300) * 0.01, [1e9, -1e9, 0.01, 0.03, -0.01]]).astype(np.float32)
    for scale, zp in ((0.02, 128), (8 / 255, 0), (0.5, 255)):
        q = ops.quantize_u8(dev(x), scale, zp).cpu().numpy()
        assert np.array_equal(q, o.quantize_u8(x, scale, zp))
        d = ops.dequantize_u8(dev(q), scale, zp).cpu().numpy()
        assert np.array_equal(d.view(np.uint32), o.dequantize_u8(q, scale, zp).view(np.uint32))
        # a view that starts 4 bytes into the buffer: not 16-byte aligned, the element-wise kernel takes it
        q1 = ops.quantize_u8(dev(x)[1:], scale, zp).cpu().numpy()
        assert np.array_equal(q1, o.quantize_u8(x[1:], scale, zp))


@pytest.mark.parametrize("M,N,K,relu,zp", [(64, 256, 512, 0, 128), (100, 40, 64, 1, 7), (8192, 256, 1024, 0, 128)])
def test_qlinear_matmul_float_output_equals_matmul_then_dequantize(M, N, K, relu, zp):
    rng = np.random.default_rng(N)
    A = dev(rng.integers(0, 256, (M, K), dtype=np.uint8))
    Wnk = rng.integers(-127, 128, (N, K), dtype=np.int8)
    w_scale = rng.uniform(0.001, 0.01, N).astype(np.float32)
    mult, corr = ops.qlinear_prepare(Wnk, True, 0.02, 128, w_scale, 0.05, None, "cuda")
    W = dev(Wnk)
    for engine in (1, 2):
        ops.set_engine(engine)
        try:
            q = ops.qlinear_matmul(A, W, mult, corr, w_is_nk=True, y_zp=zp, relu=bool(relu))
            yf = ops.qlinear_matmul_f32(A, W, mult, corr, 0.037, w_is_nk=True, y_zp=zp, relu=bool(relu))
        except capi.SofieCudaError as e:
            assert engine == 2 and e.status == capi.ERR_UNSUPPORTED
            continue
        finally:
            ops.set_engine(0)
        assert torch.equal(yf.view(torch.int32), ops.dequantize_u8(q, 0.037, zp).view(torch.int32))


def test_quantize_u8_rounding_boundaries_bit_exact():
    """The kernel multiplies by 1 / scale and falls back to the exact division near a half-integer quotient: inputs on and
    one ulp either side of every tie, across scales whose reciprocal is not exact, must still match the divided value."""
    rng = np.random.default_rng(1)
    for scale in (0.02, 8 / 255, 0.5, 0.0173, 1e-3, 3.7, 1e-38):
        s32 = np.float32(scale)
        ties = ((np.arange(-300, 300) + 0.5) * np.float64(s32)).astype(np.float32)
        x = np.concatenate([ties, np.nextafter(ties, np.float32(np.inf)), np.nextafter(ties, np.float32(-np.inf)),
                            (rng.standard_normal(50000) * 100 * scale).astype(np.float32),
                            np.array([0.0, -0.0, np.inf, -np.inf, 3e38, -3e38, 1e-45, 1e-39], np.float32)])
        for zp in (0, 128, 255):
            q = ops.quantize_u8(dev(x), float(s32), zp).cpu().numpy()
            assert np.array_equal(q, o.quantize_u8(x, float(s32), zp)), (scale, zp)


@pytest.mark.parametrize("M,N,K,nk,relu,zp", [(8, 16, 32, 1, 0, 128), (100, 37, 77, 0, 1, 128), (64, 256, 512, 1, 0, 0),
                                              (33, 1000, 129, 0, 0, 7)])
def test_qlinear_matmul_bit_exact(M, N, K, nk, relu, zp):
    rng = np.random.default_rng(N)
    A = rng.integers(0, 256, (M, K)).astype(np.uint8)
    W = rng.integers(-127, 128, (N, K) if nk else (K, N)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, N).astype(np.float32)
    y_scale = 0.02 * np.sqrt(K) * 0.3
    ref = o.qlinear_matmul(A, 0.02, zp, W, ws, y_scale, 128, w_is_nk=bool(nk), relu=bool(relu))
    mult, corr = ops.qlinear_prepare(W, bool(nk), 0.02, zp, ws, y_scale, None, "cuda")
    assert np.array_equal(mult.cpu().numpy().view(np.uint32), o.requant_multiplier(0.02, ws, y_scale).view(np.uint32))
    y = ops.qlinear_matmul(dev(A), dev(W), mult, corr, w_is_nk=bool(nk), y_zp=128, relu=bool(relu)).cpu().numpy()
    assert np.array_equal(y, ref)
    assert len(np.unique(ref)) > 20  # the case is not degenerate


@pytest.mark.parametrize("x_nhwc,y_nhwc,packed,pool,x_zp", [(0, 0, 0, 0, 0), (0, 1, 0, 2, 0), (1, 1, 1, 2, 0), (1, 0, 1, 0, 3),
                                                           (0, 0, 0, 2, 128)])
def test_qlinear_conv2d_bit_exact(x_nhwc, y_nhwc, packed, pool, x_zp):
    rng = np.random.default_rng(9)
    N, C, H, W, Cout = 2, 8, 12, 10, 20
    X = rng.integers(0, 256, (N, C, H, W)).astype(np.uint8)
    Wt = rng.integers(-127, 128, (Cout, C, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, Cout).astype(np.float32)
    bias = rng.integers(-1000, 1000, Cout).astype(np.int32)
    ref = o.qlinear_conv2d(X, 0.05, x_zp, Wt, ws, 2.0, 10, bias=bias, pad=(1, 1), relu=True)
    if pool:
        ref = o.maxpool2d_u8(ref)
    mult = dev(o.requant_multiplier(0.05, ws, 2.0))
    Xd = dev(X.transpose(0, 2, 3, 1)) if x_nhwc else dev(X)
    Wd = ops.qconv2d_pack_i8(dev(Wt)) if packed else dev(Wt)
    y = ops.qlinear_conv2d(Xd, Wd, mult, dev(bias), shape=X.shape, pad=(1, 1), x_zp=x_zp, y_zp=10, relu=True, pool=pool,
                           x_layout=x_nhwc, y_layout=y_nhwc, w_packed=bool(packed), kernel=(3, 3)).cpu().numpy()
    if y_nhwc:
        y = y.transpose(0, 3, 1, 2)
    assert np.array_equal(y, ref)
    assert len(np.unique(ref)) > 20


# ------------------------------------------------------------------------------------ elementwise family
@pytest.mark.parametrize("op,alpha", [("Sigmoid", 0), ("Tanh", 0), ("LeakyRelu", 0.1), ("Selu", 0), ("Elu", 1.0), ("Elu", 0.5), ("Neg", 0),
                                      ("Exp", 0), ("Log", 0), ("Sqrt", 0), ("Reciprocal", 0), ("Abs", 0)])
def test_unary_f32(op, alpha):
    rng = np.random.default_rng(len(op))
    for n in (0, 1, 5, 4099, 1 << 18):
        x = (rng.standard_normal(n) * 3).astype(np.float32)
        if op in ("Log", "Sqrt"):
            x = np.abs(x) + np.float32(1e-3)
        y = ops.unary_f32(dev(x), op, alpha).cpu().numpy()
        ref = o.unary_f32(x, op, alpha)
        assert rel_err(y, ref) <= FP32_TOL
        # device and libm transcendental functions agree to a few ulp; exp(x) - 1 (Selu, Elu) turns an ulp of
        # exp(x) near 1 into an absolute error of about 1e-7
        assert np.allclose(y, ref, rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("sa,sb", [((6, 5, 4, 3), (6, 5, 4, 3)), ((6, 5, 4, 3), (3,)), ((6, 5, 4, 3), (5, 1, 1)), ((5, 1, 3), (6, 1, 4, 1)),
                                   ((1,), (7, 9)), ((1025, 33), (1025, 1)), ((0, 4), (4,))])
@pytest.mark.parametrize("op", ["Add", "Sub", "Mul", "Div"])
def test_binary_f32_broadcast(sa, sb, op):
    rng = np.random.default_rng(len(sa) * 10 + len(sb))
    a = rng.standard_normal(sa).astype(np.float32)
    b = (rng.standard_normal(sb) + 3).astype(np.float32)
    y = ops.binary_f32(dev(a), dev(b), op).cpu().numpy()
    ref = o.binary_f32(a, b, op)
    assert y.shape == ref.shape
    assert np.array_equal(y, ref)  # one IEEE operation per element: bit-exact
    assert np.array_equal(ref, {"Add": a + b, "Sub": a - b, "Mul": a * b, "Div": a / b}[op])


@pytest.mark.parametrize("shape,layout,relu", [((4, 16, 8, 8), 0, 0), ((4, 16, 8, 8), 1, 1), ((3, 5), 0, 1), ((2, 7, 9), 0, 0)])
def test_batchnorm_f32(shape, layout, relu):
    rng = np.random.default_rng(sum(shape))
    Cc = shape[1]
    x = rng.standard_normal(shape).astype(np.float32)
    scale, bias, mean = (rng.standard_normal(Cc).astype(np.float32) for _ in range(3))
    var = rng.uniform(0.5, 2.0, Cc).astype(np.float32)
    ref = o.batchnorm_f32(x, scale, bias, mean, var, 1e-5, bool(relu))
    folded = o.batchnorm_folded_scale(scale, var, 1e-5)
    HW = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    xd = dev(x.transpose(0, 2, 3, 1)) if layout else dev(x)
    y = ops.batchnorm_f32(xd, dev(folded), dev(bias), dev(mean), shape[0], Cc, HW, layout=layout, relu=bool(relu)).cpu().numpy()
    if layout:
        y = y.transpose(0, 3, 1, 2)
    assert np.array_equal(y, ref)  # same three roundings per element


FIRST_LAYER = [
    # N, C, H, W, Cout, x_nhwc, y_nhwc, packed, relu, pool, x_zp
    (5, 1, 64, 64, 32, 0, 1, 1, 1, 2, 0), (3, 3, 32, 32, 16, 0, 1, 1, 1, 0, 0), (2, 1, 20, 36, 12, 0, 0, 0, 1, 2, 7),
    (2, 4, 17, 33, 64, 1, 1, 1, 0, 0, 128), (3, 2, 34, 18, 20, 1, 0, 0, 1, 2, 0), (1, 3, 8, 8, 5, 0, 1, 0, 0, 2, 3),
    # one channel with the pool fused and a width that is a multiple of 4: the specialised row-word kernel
    (3, 1, 30, 68, 24, 1, 1, 1, 0, 2, 128), (2, 1, 66, 100, 9, 0, 1, 0, 1, 2, 200), (1, 1, 4, 4, 8, 0, 0, 1, 1, 2, 1),
    # ... and a width that is not: the general kernel
    (2, 1, 22, 34, 16, 0, 1, 1, 1, 2, 5),
]


@pytest.mark.parametrize("case", FIRST_LAYER)
def test_first_layer_qconv_bit_exact(case):
    N, C, H, W, Cout, x_nhwc, y_nhwc, packed, relu, pool, x_zp = case
    rng = np.random.default_rng(sum(case))
    X = rng.integers(0, 256, (N, C, H, W)).astype(np.uint8)
    Wt = rng.integers(-127, 128, (Cout, C, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, Cout).astype(np.float32)
    bias = rng.integers(-1000, 1000, Cout).astype(np.int32)
    y_scale = 0.05 * 0.005 * 128 * 3 * np.sqrt(C)
    ref = o.qlinear_conv2d(X, 0.05, x_zp, Wt, ws, y_scale, 10, bias=bias, pad=(1, 1), relu=bool(relu))
    if pool:
        ref = o.maxpool2d_u8(ref)
    mult = dev(o.requant_multiplier(0.05, ws, y_scale))
    Xd = dev(X.transpose(0, 2, 3, 1)) if x_nhwc else dev(X)
    Wd = ops.qconv2d_pack_i8(dev(Wt)) if packed else dev(Wt)
    y = ops.qlinear_conv2d(Xd, Wd, mult, dev(bias), shape=X.shape, pad=(1, 1), x_zp=x_zp, y_zp=10, relu=bool(relu), pool=pool,
                           x_layout=x_nhwc, y_layout=y_nhwc, w_packed=bool(packed), kernel=(3, 3)).cpu().numpy()
    if y_nhwc:
        y = y.transpose(0, 3, 1, 2)
    assert np.array_equal(y, ref)
    assert len(np.unique(ref)) > 20


@pytest.mark.parametrize("case", FIRST_LAYER)
def test_first_layer_conv_f32(case):
    N, C, H, W, Cout, x_nhwc, y_nhwc, packed, relu, pool, _ = case
    rng = np.random.default_rng(sum(case) + 1)
    X = rng.standard_normal((N, C, H, W)).astype(np.float32)
    Wt = rng.standard_normal((Cout, C, 3, 3)).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32)
    ref = o.conv2d_f32(X, Wt, b, pad=(1, 1), relu=bool(relu))
    if pool:
        ref = o.pool2d_f32(ref, 0, (2, 2), (2, 2))
    Xd = dev(X.transpose(0, 2, 3, 1)) if x_nhwc else dev(X)
    Wd = ops.conv2d_pack_f32(dev(Wt)) if packed else dev(Wt)
    y = ops.conv2d_f32(Xd, Wd, dev(b), shape=(N, C, H, W), pad=(1, 1), relu=bool(relu), pool=pool, x_layout=x_nhwc,
                       y_layout=y_nhwc, w_packed=bool(packed), kernel=(3, 3)).cpu().numpy()
    if y_nhwc:
        y = y.transpose(0, 3, 1, 2)
    assert rel_err(y, ref) <= FP32_TOL


def test_maxpool2d_u8():
    X = np.random.default_rng(4).integers(0, 256, (3, 6, 9, 8)).astype(np.uint8)
    assert np.array_equal(ops.maxpool2d_u8(dev(X)).cpu().numpy(), o.maxpool2d_u8(X))
    y = ops.maxpool2d_u8(dev(X.transpose(0, 2, 3, 1)), layout=1, shape=X.shape).cpu().numpy().transpose(0, 3, 1, 2)
    assert np.array_equal(y, o.maxpool2d_u8(X))


# ------------------------------------------------------------------------------------ FP8 / bf16
def test_e4m3_and_bf16_conversions_bit_exact():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(50000) * 50, rng.standard_normal(5000) * 0.01,
                        [0, -0.0, 448, 449, 464, 465, 1e6, -1e6, 2 ** -9, 2 ** -10, 1.5 * 2 ** -10, 0.0175]]).astype(np.float32)
    for scale in (1.0, 0.37):
        assert np.array_equal(ops.quantize_e4m3(dev(x), scale).cpu().numpy(), o.quantize_e4m3(x, scale))
    b = ops.cast_f32_bf16(dev(x))
    assert np.array_equal(b.view(torch.int16).cpu().numpy().view(np.uint16), o.f32_to_bf16_bits(x))
    assert np.array_equal(ops.cast_bf16_f32(b.view(torch.int16)).cpu().numpy(), o.bf16_bits_to_f32(o.f32_to_bf16_bits(x)))
    assert np.array_equal(ops.quantize_e4m3(b.view(torch.int16), 0.37).cpu().numpy(),
                          o.quantize_e4m3(o.bf16_bits_to_f32(o.f32_to_bf16_bits(x)), 0.37))
    assert float(ops.amax_f32(dev(x)).cpu()) == np.abs(x).max()


@pytest.mark.parametrize("M,N,K", [(16, 32, 64), (70, 45, 130), (128, 256, 512)])
def test_gemm_e4m3(M, N, K):
    rng = np.random.default_rng(K)
    X = rng.standard_normal((M, K)).astype(np.float32)
    Wf = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    sa, sw = float(np.abs(X).max() / 448), float(np.abs(Wf).max() / 448)
    Aq, Wq = o.quantize_e4m3(X, sa), o.quantize_e4m3(Wf, sw)
    ref = o.bf16_bits_to_f32(o.gemm_e4m3(Aq, sa, Wq, sw, bias, relu=True))
    Y, Yq = ops.gemm_e4m3(dev(Aq), dev(Wq), dev(bias), a_scale=sa, w_scale=sw, relu=True, q_scale=0.01)
    y = Y.float().cpu().numpy()
    assert rel_err(y, ref) <= 2e-2
    assert rel_err(y, ref) <= 8e-3  # one bf16 ulp: the accumulation itself is fp32
    # the fused quantised output is exactly the quantisation of the bf16 output
    assert np.array_equal(Yq.cpu().numpy(), o.quantize_e4m3(y, 0.01))


# ------------------------------------------------------------------------------------ context
@pytest.mark.parametrize("M,N,K,bias,relu", [(64, 96, 128, True, True), (130, 70, 48, False, False), (256, 512, 1024, True, False)])
def test_gemm_e4m3_float_output_equals_gemm_then_cast(M, N, K, bias, relu):
    rng = np.random.default_rng(M + N)
    A = torch.from_numpy(rng.integers(0, 256, (M, K), dtype=np.uint8)).cuda()
    W = torch.from_numpy(rng.integers(0, 256, (N, K), dtype=np.uint8)).cuda()
    # keep NaN codes (0x7F / 0xFF) out of the operands
    A[(A & 0x7F) == 0x7F] = 0
    W[(W & 0x7F) == 0x7F] = 0
    b = dev(rng.standard_normal(N).astype(np.float32)) if bias else None
    for engine in (0, 1, 2):     # automatic, CUDA cores, tensor cores (shapes the tensor-core kernel refuses fall through)
        ops.set_engine(engine)
        try:
            y16, _ = ops.gemm_e4m3(A, W, b, a_scale=0.01, w_scale=0.02, relu=relu)
            y32 = ops.gemm_e4m3_f32(A, W, b, a_scale=0.01, w_scale=0.02, relu=relu)
        except capi.SofieCudaError as e:
            assert engine == 2 and e.status == capi.ERR_UNSUPPORTED
            continue
        finally:
            ops.set_engine(0)
        assert torch.equal(y32.view(torch.int32), ops.cast_bf16_f32(y16.view(torch.int16)).view(torch.int32))


def test_context_arena_upload_copy_and_graph():
    import ctypes as C
    lib = capi.load()
    ctx = C.c_void_p()
    capi.call("sofie_cuda_ctx_create", C.byref(ctx), 0, 1 << 20)
    try:
        p = C.c_void_p()
        capi.call("sofie_cuda_ctx_arena", ctx, 256, 4096, C.byref(p))
        assert lib.sofie_cuda_ctx_arena(ctx, 100, 16, C.byref(p)) == capi.ERR_INVALID      # misaligned
        assert lib.sofie_cuda_ctx_arena(ctx, 1 << 20, 256, C.byref(p)) == capi.ERR_NOMEM    # out of range
        A = np.random.default_rng(0).standard_normal((64, 32)).astype(np.float32)
        Wm = np.random.default_rng(1).standard_normal((16, 32)).astype(np.float32)
        dW, dA, dY = C.c_void_p(), C.c_void_p(), C.c_void_p()
        capi.call("sofie_cuda_ctx_upload", ctx, Wm.ctypes.data_as(C.c_void_p), Wm.nbytes, C.byref(dW))
        capi.call("sofie_cuda_ctx_arena", ctx, 0, A.nbytes, C.byref(dA))
        capi.call("sofie_cuda_ctx_arena", ctx, 8192, 64 * 16 * 4, C.byref(dY))
        stream = C.c_void_p()
        capi.call("sofie_cuda_ctx_stream", ctx, C.byref(stream))
        d = capi.GemmF32Desc(64, 16, 32, 0, 1, 1.0, 0.0, 0, 1)
        capi.call("sofie_cuda_ctx_h2d", ctx, dA, A.ctypes.data_as(C.c_void_p), A.nbytes)
        # warm-up launch outside capture, then capture and replay
        capi.call("sofie_cuda_gemm_f32", stream, C.byref(d), dA, dW, None, dY)
        capi.call("sofie_cuda_ctx_graph_begin", ctx)
        capi.call("sofie_cuda_gemm_f32", stream, C.byref(d), dA, dW, None, dY)
        capi.call("sofie_cuda_ctx_graph_end", ctx)
        ready = C.c_int()
        capi.call("sofie_cuda_ctx_graph_ready", ctx, C.byref(ready))
        assert ready.value == 1
        A2 = (A * 2).astype(np.float32)
        capi.call("sofie_cuda_ctx_h2d", ctx, dA, A2.ctypes.data_as(C.c_void_p), A2.nbytes)
        capi.call("sofie_cuda_ctx_graph_launch", ctx)
        Y = np.empty((64, 16), np.float32)
        capi.call("sofie_cuda_ctx_d2h", ctx, Y.ctypes.data_as(C.c_void_p), dY, Y.nbytes)
        assert rel_err(Y, o.gemm_f32(A2, Wm, transB=1, relu=True)) <= FP32_TOL
        capi.call("sofie_cuda_ctx_check", ctx)
    finally:
        capi.call("sofie_cuda_ctx_destroy", ctx)


def test_many_contexts_one_after_another_share_the_splitk_scratch_pool():
    """Each context's stream borrows a split-K scratch buffer from a pool of 16 and gives it back when the
    context is destroyed: far more than 16 contexts can come and go, and 16 can be alive at once."""
    import ctypes as C
    A = np.random.default_rng(3).standard_normal((24, 2050)).astype(np.float32)
    Wm = np.random.default_rng(4).standard_normal((10, 2050)).astype(np.float32)
    ref = o.gemm_f32(A, Wm, transB=1)
    d = capi.GemmF32Desc(24, 10, 2050, 0, 1, 1.0, 0.0, 0, 0)  # K not a multiple of 4: the split-K pair, not the one-launch kernel

    def run(ctx):
        dW, dA, dY, stream = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        capi.call("sofie_cuda_ctx_upload", ctx, Wm.ctypes.data_as(C.c_void_p), Wm.nbytes, C.byref(dW))
        capi.call("sofie_cuda_ctx_arena", ctx, 0, A.nbytes, C.byref(dA))
        capi.call("sofie_cuda_ctx_arena", ctx, 1 << 18, 24 * 10 * 4, C.byref(dY))
        capi.call("sofie_cuda_ctx_stream", ctx, C.byref(stream))
        capi.call("sofie_cuda_ctx_h2d", ctx, dA, A.ctypes.data_as(C.c_void_p), A.nbytes)
        capi.call("sofie_cuda_gemm_f32", stream, C.byref(d), dA, dW, None, dY)
        Y = np.empty((24, 10), np.float32)
        capi.call("sofie_cuda_ctx_d2h", ctx, Y.ctypes.data_as(C.c_void_p), dY, Y.nbytes)
        assert rel_err(Y, ref) <= FP32_TOL

    for _ in range(40):
        ctx = C.c_void_p()
        capi.call("sofie_cuda_ctx_create", C.byref(ctx), 0, 1 << 19)
        try:
            run(ctx)
        finally:
            capi.call("sofie_cuda_ctx_destroy", ctx)
    alive = []
    try:
        for _ in range(15):   # the test session's own stream may hold one buffer of the pool
            ctx = C.c_void_p()
            capi.call("sofie_cuda_ctx_create", C.byref(ctx), 0, 1 << 19)
            alive.append(ctx)
            run(ctx)
    finally:
        for ctx in alive:
            capi.call("sofie_cuda_ctx_destroy", ctx)
