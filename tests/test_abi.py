"""The C-ABI library loads without a GPU and exports exactly what include/sofie_cuda.h declares."""
import ctypes as C
import re
from pathlib import Path

import pytest

from sofie_b200 import capi

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "sofie_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sofie_cuda_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = capi.load()
    names = declared_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in sofie_cuda.h but not exported by libSOFIE_cuda.so"
    bound = set(capi.SIGNATURES) | set(capi.STRING_GETTERS) | set(capi.SIZE_GETTERS)
    assert bound == set(names), sorted(bound ^ set(names))


def test_struct_sizes_match_header():
    # all descriptor fields are 4 bytes wide, so the size is 4 * number of fields
    assert C.sizeof(capi.GemmF32Desc) == 9 * 4
    assert C.sizeof(capi.Conv2dDesc) == 19 * 4
    assert C.sizeof(capi.Pool2dDesc) == 15 * 4
    assert C.sizeof(capi.QGemmDesc) == 6 * 4
    assert C.sizeof(capi.QConv2dDesc) == 18 * 4
    assert C.sizeof(capi.Fp8GemmDesc) == 7 * 4
    assert C.sizeof(capi.MlpDesc) == (2 + 9 + 8 + 8) * 4


def test_fused_mlp_shared_memory_arithmetic():
    from sofie_b200 import ops
    # 64 -> 128 -> 128 -> 10: padded weight rows (68, 132, 132 floats), biases, one input tile and two activation tiles of 32 rows
    d = ops.mlp_desc(0, [64, 128, 128, 10], [1, 1, 0], [1, 1, 1])
    want = 4 * (128 * 68 + 128 + 128 * 132 + 128 + 32 * 132 + 32 + 32 * 68 + 2 * 32 * 132)
    assert capi.load().sofie_cuda_mlp_f32_smem(C.byref(d)) == want
    assert ops.mlp_fits([64, 128, 128, 10]) and ops.mlp_fits([256, 96, 1])
    assert not ops.mlp_fits([256, 256, 8]) and not ops.mlp_fits([300, 8]) and not ops.mlp_fits([8] * 10)


def test_status_strings_and_argument_errors():
    lib = capi.load()
    assert lib.sofie_cuda_strerror(0) == b"success"
    assert lib.sofie_cuda_strerror(1) == b"invalid argument"
    assert lib.sofie_cuda_abi_version() == 1
    # NULL descriptor: rejected before anything touches a device
    rc = lib.sofie_cuda_gemm_f32(None, None, None, None, None, None)
    assert rc == capi.ERR_INVALID
    assert b"NULL" in lib.sofie_cuda_last_error()
    d = capi.GemmF32Desc(0, 4, 4, 0, 0, 1.0, 1.0, 0, 0)   # an empty batch is not an error
    assert lib.sofie_cuda_gemm_f32(None, C.byref(d), None, None, None, None) == capi.OK
    d = capi.GemmF32Desc(4, 0, 4, 0, 0, 1.0, 1.0, 0, 0)
    rc = lib.sofie_cuda_gemm_f32(None, C.byref(d), C.c_void_p(16), C.c_void_p(16), None, C.c_void_p(16))
    assert rc == capi.ERR_INVALID
    with pytest.raises(capi.SofieCudaError):
        capi.call("sofie_cuda_set_engine", 7)


def test_no_gpu_means_loud_failure_not_cpu_fallback():
    """Without a device the context cannot be created; nothing computes on the CPU instead."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = capi.load()
    ctx = C.c_void_p()
    rc = lib.sofie_cuda_ctx_create(C.byref(ctx), 0, 1 << 20)
    assert rc != capi.OK and not ctx.value
    import mirror_session as runner
    from sofie_b200 import configs
    m, _ = configs.mlp_f32(batch=4)
    with pytest.raises(RuntimeError):
        runner.Session(m)


@pytest.mark.parametrize("threads", [1, 2, 4, 7])
def test_threaded_host_copy_moves_every_byte(threads):
    """The copy that carries pageable inputs into the staging ring, run on plain host memory: chunk sizes below and above the 4 MB
    from which the helper threads join in, lengths that are no multiple of a page or of the thread count, many chunks in a row
    (the helpers spin between chunks, then sleep), and a pool that is created and destroyed per call."""
    import numpy as np
    capi.load()
    rng = np.random.default_rng(threads)
    for nbytes, chunk, repeats in ((0, 1 << 20, 1), (1, 8 << 20, 1), (4095, 8 << 20, 2), ((4 << 20) - 1, 8 << 20, 1), (4 << 20, 8 << 20, 1),
                                   ((4 << 20) + 1, 8 << 20, 3), ((33 << 20) + 7, 8 << 20, 2), ((24 << 20) + 4097, (5 << 20) + 13, 1)):
        src = rng.integers(0, 256, nbytes, dtype=np.uint8)
        dst = np.zeros(nbytes + 64, np.uint8)
        dst[nbytes:] = 0xA5                                     # canary behind the destination
        capi.call("sofie_cuda_selftest_host_copy", dst.ctypes.data, src.ctypes.data, nbytes, chunk, threads, repeats)
        assert np.array_equal(dst[:nbytes], src), (nbytes, chunk)
        assert (dst[nbytes:] == 0xA5).all()
    with pytest.raises(RuntimeError):
        capi.call("sofie_cuda_selftest_host_copy", 0, 0, 16, 1 << 20, 1, 1)
    with pytest.raises(RuntimeError):
        capi.call("sofie_cuda_selftest_host_copy", dst.ctypes.data, src.ctypes.data, 16, 1 << 20, 0, 1)
