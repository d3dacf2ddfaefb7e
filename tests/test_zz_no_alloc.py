"""The allocation-free skinny GEMM entry point (sofie_cuda_gemm_f32_splitk_static), called through
the C ABI, against the regular entry point (sofie_cuda_gemm_f32) on the same inputs.

Who needs it: callers that may not allocate device memory when the call happens -- a serving
process whose own pool already holds all free device memory, or code running while a CUDA graph
is being captured in global mode, where cudaMalloc fails. The regular entry point takes its
partial-sum buffer from the CUDA allocator on first use of a stream; this one uses a fixed array
inside the library. Collected last on purpose (file name), so a run that stops at the first failure
has already run every other test; it passes alone in a fresh process as well."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import rel_err
from oracle import cpu_oracle as o
from sofie_b200 import capi

pytestmark = pytest.mark.gpu


def _run(entry, d, A, B, Cb, Y):
    capi.call(entry, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(d), C.c_void_p(A.data_ptr()),
              C.c_void_p(B.data_ptr()), C.c_void_p(Cb.data_ptr()), C.c_void_p(Y.data_ptr()))


def test_static_scratch_gemm_matches_regular_entry_point_twice(cuda_device):
    capi.call("sofie_cuda_set_engine", 0)
    M, N, K = 256, 10, 4096
    d = capi.GemmF32Desc(M, N, K, 0, 1, 1.0, 1.0, 1, 1)
    for call in range(2):  # two calls in a row: the second must not see anything of the first
        rng = np.random.default_rng(100 + call)
        A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
        B = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32)).cuda()
        Cb = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).cuda()
        y_static = torch.full((M, N), float("nan"), device="cuda")
        y_regular = torch.full((M, N), float("nan"), device="cuda")
        _run("sofie_cuda_gemm_f32_splitk_static", d, A, B, Cb, y_static)
        _run("sofie_cuda_gemm_f32", d, A, B, Cb, y_regular)
        torch.cuda.synchronize()
        assert rel_err(y_static.cpu().numpy(), y_regular.cpu().numpy()) <= 1e-5
        ref = o.gemm_f32(A.cpu().numpy(), B.cpu().numpy(), Cb.cpu().numpy(), transB=1, relu=True)
        assert rel_err(y_static.cpu().numpy(), ref) <= 1e-5


@pytest.mark.parametrize("M,N,K,transB", [(37, 10, 4098, 1), (256, 16, 2048, 0), (101, 3, 1030, 0)])
def test_static_scratch_gemm_other_staging_paths_and_no_allocation(M, N, K, transB, cuda_device):
    """Weights stored [K,N], a K that is not a multiple of 4 and a row count that is not a multiple of 8 take the entry point's
    other staging paths; and the property it is named for: once the first call on the device has looked up the array's
    address, a call leaves the amount of free device memory exactly as it found it."""
    capi.call("sofie_cuda_set_engine", 0)
    rng = np.random.default_rng(M + K)
    A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    Bh = rng.standard_normal((N, K) if transB else (K, N)).astype(np.float32)
    B = torch.from_numpy(Bh).cuda()
    Cb = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).cuda()
    d = capi.GemmF32Desc(M, N, K, 0, transB, 1.0, 1.0, 1, 0)
    y = [torch.full((M, N), float("nan"), device="cuda") for _ in range(2)]
    y_regular = torch.full((M, N), float("nan"), device="cuda")
    _run("sofie_cuda_gemm_f32_splitk_static", d, A, B, Cb, y[0])      # may be the first call on this device: it takes the symbol's address
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    _run("sofie_cuda_gemm_f32_splitk_static", d, A, B, Cb, y[1])
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before                # nothing was allocated (or freed) by the call
    _run("sofie_cuda_gemm_f32", d, A, B, Cb, y_regular)
    torch.cuda.synchronize()
    ref = o.gemm_f32(A.cpu().numpy(), Bh, Cb.cpu().numpy(), transB=transB)
    for out in y:
        assert rel_err(out.cpu().numpy(), y_regular.cpu().numpy()) <= 1e-5
        assert rel_err(out.cpu().numpy(), ref) <= 1e-5


def test_static_scratch_gemm_rejects_what_it_cannot_hold(cuda_device):
    lib = capi.load()
    x = torch.zeros(16, device="cuda")
    p = C.c_void_p(x.data_ptr())
    # more outputs than the static scratch is sized for
    d = capi.GemmF32Desc(4096, 16, 2048, 0, 1, 1.0, 0.0, 0, 0)
    assert lib.sofie_cuda_gemm_f32_splitk_static(None, C.byref(d), p, p, None, p) == capi.ERR_INVALID
    assert b"exceed" in lib.sofie_cuda_last_error()
    # outside the split-K shape class
    d = capi.GemmF32Desc(64, 64, 2048, 0, 1, 1.0, 0.0, 0, 0)
    assert lib.sofie_cuda_gemm_f32_splitk_static(None, C.byref(d), p, p, None, p) == capi.ERR_UNSUPPORTED
