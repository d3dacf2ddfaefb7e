"""Context services on the GPU: the per-context status word with a bounded wait that is made to run out (the kernel
ends by itself, reports once, and the context keeps computing), the per-operator device timers of the emitted
Launch(), Session::RunResident, and two Sessions that do not see each other's failures."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import run_model
from sofie_b200 import capi, configs, generated

pytestmark = pytest.mark.gpu


def _ctx(arena=1 << 20):
    ctx = C.c_void_p()
    capi.call("sofie_cuda_ctx_create", C.byref(ctx), 0, arena)
    stream = C.c_void_p()
    capi.call("sofie_cuda_ctx_stream", ctx, C.byref(stream))
    return ctx, stream


def test_bounded_wait_runs_out_reports_once_and_the_context_stays_usable(cuda_device):
    a, sa = _ctx()
    b, sb = _ctx()
    try:
        flag = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        # a barrier nothing arrives on, a limit of 200 000 SM clocks (about 0.1 ms): the kernel gives up and returns
        capi.call("sofie_cuda_selftest_wait_timeout", sa, 200_000, C.c_void_p(flag.data_ptr()))
        with pytest.raises(capi.SofieCudaError) as e:
            capi.call("sofie_cuda_ctx_check", a)
        assert e.value.status == capi.ERR_DEVICE and "0x1ff" in str(e.value) and "0x7e57" in str(e.value)
        assert int(flag.item()) == 1                    # the kernel went through its normal exit (tensor memory released)
        capi.call("sofie_cuda_ctx_check", a)            # reported once, then clear
        capi.call("sofie_cuda_ctx_check", b)            # the other context never saw it
        # the context still computes: a tensor-core GEMM on the same stream, then a clean check
        rng = np.random.default_rng(3)
        A = rng.standard_normal((256, 512)).astype(np.float32)
        B = rng.standard_normal((64, 512)).astype(np.float32)
        dA, dB = torch.from_numpy(A).to(cuda_device), torch.from_numpy(B).to(cuda_device)
        dY = torch.empty(256, 64, device=cuda_device)
        d = capi.GemmF32Desc(256, 64, 512, 0, 1, 1.0, 0.0, 0, 0)
        torch.cuda.synchronize()
        capi.call("sofie_cuda_gemm_f32", sa, C.byref(d), C.c_void_p(dA.data_ptr()), C.c_void_p(dB.data_ptr()), None, C.c_void_p(dY.data_ptr()))
        capi.call("sofie_cuda_ctx_check", a)
        ref = A.astype(np.float64) @ B.astype(np.float64).T
        assert np.abs(dY.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
        # a limit outside the self test's range is refused before anything is launched
        with pytest.raises(capi.SofieCudaError):
            capi.call("sofie_cuda_selftest_wait_timeout", sa, 10**12, None)
    finally:
        capi.call("sofie_cuda_ctx_destroy", a)
        capi.call("sofie_cuda_ctx_destroy", b)


def test_fetch_reports_a_kernel_that_gave_up(cuda_device):
    ctx, stream = _ctx()
    try:
        buf = C.c_void_p()
        capi.call("sofie_cuda_ctx_arena", ctx, 0, 1024, C.byref(buf))
        capi.call("sofie_cuda_selftest_wait_timeout", stream, 100_000, None)
        host = C.c_void_p()
        with pytest.raises(capi.SofieCudaError) as e:   # what the emitted infer() turns into std::runtime_error
            capi.call("sofie_cuda_ctx_fetch", ctx, buf, 1024, C.byref(host))
        assert e.value.status == capi.ERR_DEVICE
        capi.call("sofie_cuda_ctx_fetch", ctx, buf, 1024, C.byref(host))
    finally:
        capi.call("sofie_cuda_ctx_destroy", ctx)


def test_copies_are_refused_during_a_graph_capture(cuda_device):
    ctx, _ = _ctx()
    try:
        buf = C.c_void_p()
        capi.call("sofie_cuda_ctx_arena", ctx, 0, 1024, C.byref(buf))
        src = np.zeros(256, np.float32)
        capi.call("sofie_cuda_ctx_graph_begin", ctx)
        for name, args in (("sofie_cuda_ctx_h2d", (ctx, buf, src.ctypes.data_as(C.c_void_p), 1024)),
                           ("sofie_cuda_ctx_d2h", (ctx, src.ctypes.data_as(C.c_void_p), buf, 1024)),
                           ("sofie_cuda_ctx_check", (ctx,))):
            with pytest.raises(capi.SofieCudaError) as e:
                capi.call(name, *args)
            assert e.value.status == capi.ERR_INVALID
        capi.call("sofie_cuda_ctx_graph_end", ctx)
    finally:
        capi.call("sofie_cuda_ctx_destroy", ctx)


def test_operator_timers_and_run_resident_of_the_emitted_session(cuda_device, monkeypatch):
    m, x = configs.cnn_f32(batch=32)
    ref = run_model.run(m, x).ravel()
    plain = generated.session_from_model(m, "c2_b32_timers")
    y0 = plain.infer(x)
    n = C.c_int(-1)
    capi.call("sofie_cuda_ctx_timers_read", plain.ctx, None, 0, C.byref(n))
    assert n.value == 0                                     # timers are off unless asked for
    monkeypatch.setenv("SOFIE_CUDA_TIMERS", "1")
    timed = generated.session_from_model(m, "c2_b32_timers")
    monkeypatch.delenv("SOFIE_CUDA_TIMERS")
    plan = generated.launch_plan(timed.hxx)
    assert [p["calls"] for p in plan] == [["sofie_cuda_conv2d_f32"]] * 3 + [[], ["sofie_cuda_gemm_f32"]]   # Flatten is an alias
    assert sum(p["flops"] for p in plan) == m.flops_per_sample * 32
    ms = (C.c_float * len(plan))()
    for _ in range(3):                                      # eager pass, capturing pass, graph replay
        y = timed.infer(x)
        capi.call("sofie_cuda_ctx_timers_read", timed.ctx, ms, len(plan), C.byref(n))
        assert n.value == len(plan) and all(0.0 <= t < 50.0 for t in ms)
        assert np.array_equal(y, y0)
    assert np.abs(y0 - ref).max() <= 1e-5 * np.abs(ref).max()
    # RunResident: the kernels again on the input the last infer() left on the device, no copies
    stream = C.c_void_p()
    capi.call("sofie_cuda_ctx_stream", plain.ctx, C.byref(stream))
    plain.run_resident()
    plain.run_resident()
    capi.call("sofie_cuda_ctx_check", plain.ctx)
    assert np.array_equal(plain.infer(x), y0)
