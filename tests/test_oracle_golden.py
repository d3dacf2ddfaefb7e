"""Pins the CPU oracle: it must reproduce every golden vector the reference's own tests hold for
the dense-contraction path (reference: src/SOFIE_core/test/TestCustomModelsFromONNX.cxx:330-391,
693-712,860-967,1028-1115,1966-2045,3028-3044) within the reference's tolerance of 1e-3."""
import numpy as np
import pytest

from helpers import FIXTURE_CASES, OracleBackend, load_fixtures, run_fixture


@pytest.mark.parametrize("name", FIXTURE_CASES)
def test_oracle_reproduces_reference_golden(name):
    manifest, arrays = load_fixtures()
    y = run_fixture(name, manifest, arrays, OracleBackend())
    exp = arrays[f"{name}/expected"]
    assert y.shape == exp.shape
    assert np.abs(y - exp).max() <= manifest[name]["tolerance"]


@pytest.mark.parametrize("stride,pad,dil,out_pad", [((1, 1), (0, 0), (1, 1), (0, 0)), ((2, 2), (1, 1), (1, 1), (1, 1)),
                                                    ((3, 2), (1, 0), (2, 1), (2, 1)), ((2, 1), (0, 2), (1, 2), (0, 0))])
def test_conv_transpose_oracle_against_an_independent_implementation(stride, pad, dil, out_pad):
    """The restated ConvTranspose (reference: filter GEMM + col2im) against torch's CPU operator, beyond the
    un-strided, un-padded shapes the reference's own fixtures cover."""
    import torch
    from oracle import cpu_oracle as o
    rng = np.random.default_rng(7)
    X = rng.standard_normal((2, 5, 6, 7)).astype(np.float32)
    W = rng.standard_normal((5, 4, 3, 3)).astype(np.float32)
    b = rng.standard_normal(4).astype(np.float32)
    y = o.conv_transpose2d_f32(X, W, b, pad=pad, stride=stride, dil=dil, out_pad=out_pad)
    ref = torch.nn.functional.conv_transpose2d(torch.from_numpy(X), torch.from_numpy(W), torch.from_numpy(b), stride=stride,
                                               padding=pad, output_padding=out_pad, dilation=dil).numpy()
    assert y.shape == ref.shape and np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("stride,pad,dil,group", [((1, 1, 1), (0, 0, 0), (1, 1, 1), 1), ((2, 1, 1), (1, 0, 2), (1, 2, 1), 2),
                                                  ((1, 2, 3), (1, 1, 1), (1, 1, 1), 4)])
def test_conv3d_oracle_against_an_independent_implementation(stride, pad, dil, group):
    """The restated 3-D convolution (reference: Im2col_3d + sgemm_ per image and group) against torch's CPU operator: the
    reference's own test of this operator (TestSofieModels.cxx, Conv3d) compares with PyTorch in the same way."""
    import torch
    from oracle import cpu_oracle as o
    rng = np.random.default_rng(11)
    X = rng.standard_normal((2, 4, 5, 6, 7)).astype(np.float32)
    W = rng.standard_normal((8, 4 // group, 3, 2, 3)).astype(np.float32)
    b = rng.standard_normal(8).astype(np.float32)
    y = o.conv3d_f32(X, W, b, pad=pad, stride=stride, dil=dil, group=group)
    ref = torch.nn.functional.conv3d(torch.from_numpy(X), torch.from_numpy(W), torch.from_numpy(b), stride=stride, padding=pad,
                                     dilation=dil, groups=group).numpy()
    assert y.shape == ref.shape and np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()


def test_pool3d_oracle_against_an_independent_implementation():
    import torch
    from oracle import cpu_oracle as o
    X = np.random.default_rng(12).standard_normal((2, 3, 6, 5, 7)).astype(np.float32)
    y = o.pool3d_f32(X, 0, (3, 2, 2), (1, 2, 1), (1, 0, 1, 0, 1, 0))
    padded = torch.nn.functional.pad(torch.from_numpy(X), (1, 0, 0, 1, 1, 0), value=float("-inf"))
    assert np.array_equal(y, torch.nn.functional.max_pool3d(padded, (3, 2, 2), (1, 2, 1)).numpy())
    y = o.pool3d_f32(X, 1, (2, 2, 2), (2, 2, 2))
    assert np.abs(y - torch.nn.functional.avg_pool3d(torch.from_numpy(X), 2, 2).numpy()).max() <= 1e-6
    y = o.pool3d_f32(X, 1, (3, 3, 3), (2, 2, 2), (1, 1, 1, 1, 1, 1), count_include_pad=0)
    ref = torch.nn.functional.avg_pool3d(torch.from_numpy(X), 3, 2, padding=1, count_include_pad=False).numpy()
    assert y.shape == ref.shape and np.abs(y - ref).max() <= 1e-6
