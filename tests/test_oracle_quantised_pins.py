"""Independent pins for the part of the oracle the reference cannot pin (it has no quantised operators).

oracle/sofie_oracle.c restates the ONNX definitions of QuantizeLinear, QLinearMatMul, QLinearConv and the E4M3 /
bfloat16 conversions. Here the same definitions are written a second time, in numpy (int64 accumulation, float32
requantisation) and through ml_dtypes' float8_e4m3fn / bfloat16, without looking at the C code's structure: a shared
misreading of a definition (border zero point, tie rounding, the order of saturation and zero point) would have to
be made twice, in two languages, to pass."""
import ml_dtypes
import numpy as np
import pytest

from oracle import cpu_oracle as o


# ---------------------------------------------------------------------------------------- numpy restatements
def np_requant(acc, mult, y_zp, relu):
    v = acc.astype(np.float32) * mult.astype(np.float32)          # (float)int32, one float32 product
    q = np.rint(v).astype(np.int64) + y_zp                         # round half to even, then the zero point
    q = np.clip(q, 0, 255)                                         # saturate to uint8
    if relu:
        q = np.maximum(q, y_zp)                                    # Relu of a quantised tensor
    return q.astype(np.uint8)


def np_multiplier(a_scale, w_scale, y_scale):
    return (np.float32(a_scale) * w_scale.astype(np.float32)) / np.float32(y_scale)


def np_qlinear_matmul(A, a_scale, a_zp, W_kn, w_scale, y_scale, y_zp, bias=None, relu=False):
    acc = (A.astype(np.int64) - a_zp) @ W_kn.astype(np.int64)
    if bias is not None:
        acc = acc + bias.astype(np.int64)
    assert np.abs(acc).max() < 2 ** 31
    return np_requant(acc, np_multiplier(a_scale, w_scale, y_scale)[None, :], y_zp, relu)


def np_qlinear_conv2d(X, x_scale, x_zp, W, w_scale, y_scale, y_zp, bias=None, pad=(0, 0), stride=(1, 1), relu=False):
    n, c, h, w = X.shape
    co, _, kh, kw = W.shape
    xp = np.zeros((n, c, h + 2 * pad[0], w + 2 * pad[1]), np.int64)       # padding is the real value 0 = code x_zp
    xp[:, :, pad[0]:pad[0] + h, pad[1]:pad[1] + w] = X.astype(np.int64) - x_zp
    win = np.lib.stride_tricks.sliding_window_view(xp, (kh, kw), axis=(2, 3))[:, :, ::stride[0], ::stride[1]]
    acc = np.einsum("nchwij,ocij->nohw", win, W.astype(np.int64))
    if bias is not None:
        acc = acc + bias.astype(np.int64)[None, :, None, None]
    return np_requant(acc, np_multiplier(x_scale, w_scale, y_scale)[None, :, None, None], y_zp, relu)


# ---------------------------------------------------------------------------------------- int8
@pytest.mark.parametrize("a_zp,y_zp,relu,with_bias", [(128, 128, False, False), (0, 0, True, True), (3, 250, False, True), (255, 0, True, False), (17, 99, True, True)])
def test_qlinear_matmul_against_numpy_int64(a_zp, y_zp, relu, with_bias):
    rng = np.random.default_rng(100 + a_zp + y_zp)
    M, K, N = 37, 300, 29
    A = rng.integers(0, 256, (M, K)).astype(np.uint8)
    A[0], A[1] = 0, 255                                                   # extreme rows: saturation both ways
    W = rng.integers(-128, 128, (K, N)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, N).astype(np.float32)
    ws[::7] *= -1                                                         # negative multipliers are legal
    bias = rng.integers(-50000, 50000, N).astype(np.int32) if with_bias else None
    ref = np_qlinear_matmul(A, 0.02, a_zp, W, ws, 0.05, y_zp, bias, relu)
    got = o.qlinear_matmul(A, 0.02, a_zp, W, ws, 0.05, y_zp, bias=bias, w_is_nk=False, relu=relu)
    assert np.array_equal(got, ref)
    got_nk = o.qlinear_matmul(A, 0.02, a_zp, np.ascontiguousarray(W.T), ws, 0.05, y_zp, bias=bias, w_is_nk=True, relu=relu)
    assert np.array_equal(got_nk, ref)
    assert ref.min() == (y_zp if relu else 0) and ref.max() == 255        # both ends of the range are reached
    assert np.array_equal(o.requant_multiplier(0.02, ws, 0.05).view(np.uint32), np_multiplier(0.02, ws, 0.05).view(np.uint32))


def test_requantisation_ties_round_to_even_and_saturate():
    # one weight of +-1 and a multiplier of 0.5 / 0.25 put every second / fourth accumulator on a tie
    A = np.arange(256, dtype=np.uint8)[:, None]
    W = np.array([[1, -1, 1, -1]], np.int8)
    ws = np.array([0.5, 0.5, 0.25, 0.25], np.float32)
    for a_zp, y_zp in ((0, 0), (128, 128), (100, 7)):
        ref = np_qlinear_matmul(A, 1.0, a_zp, W, ws, 1.0, y_zp)
        got = o.qlinear_matmul(A, 1.0, a_zp, W, ws, 1.0, y_zp, w_is_nk=False)
        assert np.array_equal(got, ref)
    # spelled out for zero points 0: 0.5 -> 0, 1.5 -> 2, 2.5 -> 2, 3.5 -> 4 (half to even, not half up)
    got = o.qlinear_matmul(A, 1.0, 0, W, ws, 1.0, 0, w_is_nk=False)
    assert got[[1, 3, 5, 7], 0].tolist() == [0, 2, 2, 4] and got[[2, 6, 10], 2].tolist() == [0, 2, 2]
    assert got[:, 1].max() == 0                                           # negative products saturate at 0


@pytest.mark.parametrize("x_zp,y_zp,pad,stride,relu,with_bias", [(0, 0, (1, 1), (1, 1), True, False), (128, 128, (1, 1), (1, 1), False, True),
                                                               (37, 5, (2, 1), (2, 2), True, True), (255, 200, (0, 0), (1, 2), False, False)])
def test_qlinear_conv_against_numpy_int64_with_borders(x_zp, y_zp, pad, stride, relu, with_bias):
    rng = np.random.default_rng(7 + x_zp)
    X = rng.integers(0, 256, (3, 5, 9, 8)).astype(np.uint8)
    X[0, :, 0, :] = 255                                                   # a bright border row next to the padding
    W = rng.integers(-128, 128, (6, 5, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.0005, 0.004, 6).astype(np.float32)
    ws[2] *= -1
    bias = rng.integers(-20000, 20000, 6).astype(np.int32) if with_bias else None
    ref = np_qlinear_conv2d(X, 0.03, x_zp, W, ws, 0.08, y_zp, bias, pad, stride, relu)
    got = o.qlinear_conv2d(X, 0.03, x_zp, W, ws, 0.08, y_zp, bias=bias, pad=pad, stride=stride, relu=relu)
    assert got.shape == ref.shape and np.array_equal(got, ref)
    # the border matters: treating padded taps as code 0 instead of code x_zp changes the result when x_zp != 0
    if x_zp and any(pad):
        wrong = np_qlinear_conv2d(X, 0.03, 0, W, ws, 0.08, y_zp, bias, pad, stride, relu)
        assert not np.array_equal(wrong, ref)


def test_quantize_and_dequantize_u8_against_numpy():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 3, (np.arange(-600, 600, dtype=np.float32) + 0.5) * np.float32(0.02),
                        np.array([1e30, -1e30, 0.0, -0.0], np.float32)])
    for scale, zp in ((0.02, 128), (8.0 / 255.0, 0), (0.5, 255)):
        ref = np.clip(np.rint(x / np.float32(scale)).astype(np.float64) + zp, 0, 255).astype(np.uint8)
        assert np.array_equal(o.quantize_u8(x, scale, zp), ref)
        codes = np.arange(256, dtype=np.uint8)
        deq = (codes.astype(np.int32) - zp).astype(np.float32) * np.float32(scale)
        assert np.array_equal(o.dequantize_u8(codes, scale, zp).view(np.uint32), deq.view(np.uint32))


def test_maxpool_u8_against_numpy():
    X = np.random.default_rng(2).integers(0, 256, (2, 3, 8, 6)).astype(np.uint8)
    ref = X.reshape(2, 3, 4, 2, 3, 2).max(axis=(3, 5))
    assert np.array_equal(o.maxpool2d_u8(X), ref)


# ---------------------------------------------------------------------------------------- E4M3 and bfloat16
def test_e4m3_decode_table_against_ml_dtypes():
    ref = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    got = o.e4m3_table()
    finite = ~np.isnan(ref)
    assert finite.sum() == 254 and np.array_equal(got[finite].view(np.uint32), ref[finite].view(np.uint32))
    assert np.abs(ref[finite]).max() == 448.0


def test_e4m3_quantisation_against_ml_dtypes():
    rng = np.random.default_rng(11)
    # dense in value (every decade of the E4M3 range, subnormals included), plus every representable value, every midpoint
    # between neighbours (the ties) and values just off them
    table = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    pos = np.sort(table[:0x7F])
    mids = (pos[:-1] + pos[1:]) / 2
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-4, 3, 200000).astype(np.float32),
                        pos, -pos, mids, -mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)),
                        np.array([448.0, 463.9, 464.0, 480.0, 1e6, -1e6, 0.0, -0.0, 2.0 ** -10, 2.0 ** -11], np.float32)]).astype(np.float32)
    for scale in (1.0, 0.0371, 3.5):
        v = x / np.float32(scale)
        ref = v.astype(ml_dtypes.float8_e4m3fn)
        got = o.quantize_e4m3(x, scale)
        finite = ~np.isnan(ref.astype(np.float32))
        assert np.array_equal(got[finite], ref.view(np.uint8)[finite])       # round to nearest even, identical codes
        # beyond the largest finite value ml_dtypes yields NaN (E4M3FN has no infinity); the quantiser saturates instead
        over = ~finite
        assert over.any() and np.array_equal(got[over], np.where(v[over] > 0, 0x7E, 0xFE).astype(np.uint8))
        assert np.abs(v[over]).min() >= 464.0


def test_bf16_rounding_against_ml_dtypes_over_every_pattern():
    hi = np.arange(65536, dtype=np.uint32) << 16
    # every bfloat16 pattern exactly, and around it: just above, just below a tie, the tie, just above the tie, the top
    for low in (0x0000, 0x0001, 0x7FFF, 0x8000, 0x8001, 0xFFFF):
        x = (hi | low).view(np.float32)
        ref = x.astype(ml_dtypes.bfloat16).view(np.uint16)
        got = o.f32_to_bf16_bits(x)
        ok = ~np.isnan(x)
        assert np.array_equal(got[ok], ref[ok]), hex(low)
        assert np.all(np.isnan(o.bf16_bits_to_f32(got[~ok])))                # a NaN stays a NaN
    back = o.bf16_bits_to_f32(np.arange(65536, dtype=np.uint16))
    assert np.array_equal(back.view(np.uint32), hi)


def test_fp8_gemm_against_ml_dtypes_and_float64():
    rng = np.random.default_rng(21)
    M, K, N = 24, 160, 40
    A = (rng.standard_normal((M, K)) * 1.5).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    sa, sw = float(np.abs(A).max() / 448), float(np.abs(W).max() / 448)
    Aq, Wq = o.quantize_e4m3(A, sa), o.quantize_e4m3(W, sw)
    dq = lambda c: c.view(ml_dtypes.float8_e4m3fn).astype(np.float64)
    y = dq(Aq) @ dq(Wq).T * (np.float32(sa) * np.float32(sw)).astype(np.float64) + bias
    y = np.maximum(y, 0)
    ref = y.astype(np.float32).astype(ml_dtypes.bfloat16).astype(np.float32)
    got = o.bf16_bits_to_f32(o.gemm_e4m3(Aq, sa, Wq, sw, bias, relu=True))
    # both are bf16 values of the same sums; they may differ by one bf16 step where the fp32 and fp64 sums straddle a tie
    assert np.abs(got - ref).max() <= 2.0 ** -7 * np.abs(ref).max()
    assert (got == ref).mean() > 0.98
